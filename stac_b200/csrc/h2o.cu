// H2O heavy-hitter bookkeeping on the hot cache: score update, keep-set selection and the
// gather-compaction of the cache.
//
// Replaces stac/h2o.py:177-216 (_update_scores), stac/h2o.py:244-354 (_parallel_prune_kv:
// index_select + torch.topk + cat + torch.sort over [L*H, T]) and stac/h2o.py:356-436 with
// stac/stac_voxel.py:409-419 (six torch.gather compactions with full-size temporaries).
#include "common.cuh"
#include "stac_internal.h"

namespace stac {
namespace {

// score = colsum * T_live / Tq; new tail is written, the old prefix decays:
// score = score * temperature + s (two roundings, as mul_ then add_), count += 1.
__global__ void scores_update_kernel(const float* __restrict__ colsum, long long colsum_stride,
                                     float* __restrict__ scores, float* __restrict__ counts, long long row_stride,
                                     int H, int T_live, int old_T, float t_live_f, float tq_f, float temperature) {
  grid_dep_wait();   // launched with programmatic serialization behind the column-sum kernel
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  const int h = blockIdx.y;
  if (t >= T_live) return;
  const float s = __fdiv_rn(__fmul_rn(colsum[h * colsum_stride + t], t_live_f), tq_f);
  const long long o = h * row_stride + t;
  if (t >= old_T) {
    scores[o] = s;
  } else {
    scores[o] = __fadd_rn(__fmul_rn(scores[o], temperature), s);
  }
  counts[o] = __fadd_rn(counts[o], 1.0f);
}

__device__ __forceinline__ unsigned int float_key(float f) {
  const unsigned int u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// Block-wide exclusive scan of one int per thread (1024 threads); returns the exclusive
// prefix and leaves the block total in *total_out (shared).
__device__ __forceinline__ int block_scan_1024(int v, int* warp_sums, int* total_out) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  if (lane == 31) warp_sums[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int w = warp_sums[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, w, o);
      if (lane >= o) w += t;
    }
    warp_sums[lane] = w;
  }
  __syncthreads();
  const int excl = (warp > 0 ? warp_sums[warp - 1] : 0) + incl - v;
  if (threadIdx.x == 0) *total_out = warp_sums[31];
  __syncthreads();
  return excl;
}

// One CTA per (layer, head) row.  Positions flagged in `is_base` (pinned and recent tokens)
// are always kept; of the others the `k` highest scores are kept (ties: lower position
// first).  Emits the kept positions and the dropped positions, both ascending.
// (two CTAs per SM: 384 rows run in two waves instead of three)
__global__ void __launch_bounds__(1024, 2)
h2o_select_kernel(const float* __restrict__ scores, long long row_stride, const unsigned char* __restrict__ is_base,
                  int T, int n_keep, int* __restrict__ keep_idx, int* __restrict__ drop_idx) {
  grid_dep_wait();   // launched with programmatic serialization behind the previous kernel in the stream
  extern __shared__ unsigned int keys[];
  __shared__ int hist[256];
  __shared__ int warp_sums[32];
  __shared__ int sh_total;
  __shared__ unsigned int sh_prefix;
  __shared__ int sh_remaining;
  const int row = blockIdx.x;
  const float* srow = scores + row * row_stride;
  // four independent loads per thread in flight
  for (int base = 0; base < T; base += 4 * 1024) {
    float sc[4];
    unsigned char bs[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int t = base + j * 1024 + static_cast<int>(threadIdx.x);
      sc[j] = t < T ? srow[t] : 0.f;
      bs[j] = t < T ? is_base[t] : static_cast<unsigned char>(0);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int t = base + j * 1024 + static_cast<int>(threadIdx.x);
      if (t < T) keys[t] = bs[j] ? 0xFFFFFFFFu : float_key(sc[j]);
    }
  }
  if (threadIdx.x == 0) {
    sh_prefix = 0;
    sh_remaining = n_keep;
  }
  __syncthreads();
  // radix select: find the n_keep-th largest key, 8 bits at a time from the top
  for (int shift = 24; shift >= 0; shift -= 8) {
    if (threadIdx.x < 256) hist[threadIdx.x] = 0;
    __syncthreads();
    const unsigned int prefix = sh_prefix;
    const unsigned int hi_mask = shift == 24 ? 0u : (0xFFFFFFFFu << (shift + 8));
    for (int t = threadIdx.x; t < T; t += blockDim.x) {
      const unsigned int k = keys[t];
      if ((k & hi_mask) == prefix) {
        // scores of one row share their exponent: most keys fall into a few bins of the upper
        // digits, so a counter is bumped once per warp and distinct digit, not once per lane
        const unsigned int bin = (k >> shift) & 255u;
        const unsigned int peers = __match_any_sync(__activemask(), bin);
        if ((peers & ((1u << (threadIdx.x & 31)) - 1u)) == 0u) atomicAdd(&hist[bin], __popc(peers));
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int remaining = sh_remaining;
      int d = 255;
      for (; d > 0; --d) {
        if (hist[d] >= remaining) break;
        remaining -= hist[d];
      }
      sh_prefix = prefix | (static_cast<unsigned int>(d) << shift);
      sh_remaining = remaining;
    }
    __syncthreads();
  }
  const unsigned int tau = sh_prefix;   // the n_keep-th largest key
  const int need_eq = sh_remaining;     // how many keys equal to tau are kept
  __shared__ int eq_carry, keep_carry, drop_carry;
  if (threadIdx.x == 0) {
    eq_carry = 0;
    keep_carry = 0;
    drop_carry = 0;
  }
  __syncthreads();
  int* krow = keep_idx + static_cast<long long>(row) * n_keep;
  int* drow = drop_idx + static_cast<long long>(row) * (T - n_keep);
  // four consecutive positions per thread: two block scans per 4096 positions
  for (int base = 0; base < T; base += 4096) {
    const int t0 = base + static_cast<int>(threadIdx.x) * 4;
    unsigned int k[4];
    int eq[4], keep[4];
    int n_eq = 0, n_keep_here = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const bool in = t0 + j < T;
      k[j] = in ? keys[t0 + j] : 0u;
      eq[j] = (in && k[j] == tau) ? 1 : 0;
      n_eq += eq[j];
    }
    int eq_rank = eq_carry + block_scan_1024(n_eq, warp_sums, &sh_total);
    const int eq_total = sh_total;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const bool in = t0 + j < T;
      keep[j] = (in && (k[j] > tau || (eq[j] && eq_rank < need_eq))) ? 1 : 0;
      eq_rank += eq[j];
      n_keep_here += keep[j];
    }
    int keep_rank = keep_carry + block_scan_1024(n_keep_here, warp_sums, &sh_total);
    const int keep_total = sh_total;
    // positions before this thread's in the block that are not kept (they are all inside the row
    // whenever this thread has a position inside it)
    int drop_rank = drop_carry + (static_cast<int>(threadIdx.x) * 4 - (keep_rank - keep_carry));
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (t0 + j < T) {
        if (keep[j]) krow[keep_rank++] = t0 + j;
        else drow[drop_rank++] = t0 + j;
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      eq_carry += eq_total;
      keep_carry += keep_total;
      drop_carry += min(4096, T - base) - keep_total;
    }
    __syncthreads();
  }
}

// Gather-compaction into a second set of buffers: dst[row, j] = src[row, keep[row, j]].
// K and V move as 16-byte vectors, eight threads per 128-byte (bf16) or sixteen per 256-byte
// (fp32) row.
__global__ void compact_kv_kernel(const int* __restrict__ keep_idx, int n_keep, const uint4* __restrict__ k_src,
                                  const uint4* __restrict__ v_src, uint4* __restrict__ k_dst,
                                  uint4* __restrict__ v_dst, long long row_stride_vec, int vec_per_token) {
  grid_dep_wait();   // launched with programmatic serialization behind the previous kernel in the stream
  const long long gid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int row = blockIdx.y;
  const long long tok = gid / vec_per_token;
  const int part = static_cast<int>(gid % vec_per_token);
  if (tok >= n_keep) return;
  const int src = keep_idx[static_cast<long long>(row) * n_keep + tok];
  const long long so = row * row_stride_vec + static_cast<long long>(src) * vec_per_token + part;
  const long long dof = row * row_stride_vec + tok * vec_per_token + part;
  k_dst[dof] = k_src[so];
  v_dst[dof] = v_src[so];
}

__global__ void compact_meta_kernel(const int* __restrict__ keep_idx, int n_keep, int T_buf,
                                    const long long* __restrict__ ti_src, long long* __restrict__ ti_dst,
                                    const float* __restrict__ s_src, float* __restrict__ s_dst,
                                    const float* __restrict__ c_src, float* __restrict__ c_dst,
                                    const int* __restrict__ vx_src, int* __restrict__ vx_dst) {
  grid_dep_wait();   // launched with programmatic serialization behind the previous kernel in the stream
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  const int row = blockIdx.y;
  if (j >= T_buf) return;
  const long long o = static_cast<long long>(row) * T_buf + j;
  if (j < n_keep) {
    const long long s = static_cast<long long>(row) * T_buf + keep_idx[static_cast<long long>(row) * n_keep + j];
    ti_dst[o] = ti_src[s];
    s_dst[o] = s_src[s];
    c_dst[o] = c_src[s];
    if (vx_src != nullptr) vx_dst[o] = vx_src[s];
  } else {
    ti_dst[o] = -1;
    s_dst[o] = 0.f;
    c_dst[o] = 0.f;
    if (vx_dst != nullptr) vx_dst[o] = -1;
  }
}

// New K/V rows of one layer into the tail of the hot cache plus their global token ids, one
// launch instead of three strided copies (stac/kv_manager.py:285-305).
__global__ void append_kv_kernel(const uint4* __restrict__ k, const uint4* __restrict__ v, long long k_head_stride_vec,
                                 long long k_row_stride_vec, long long v_head_stride_vec, long long v_row_stride_vec,
                                 uint4* __restrict__ k_cache, uint4* __restrict__ v_cache,
                                 long long cache_head_stride_vec, long long* __restrict__ token_idx,
                                 long long idx_head_stride, int T_new, int old_T, long long first_id,
                                 int vec_per_token) {
  grid_dep_wait();   // launched with programmatic serialization: whatever produced k and v is complete now
  const int h = blockIdx.y;
  const long long total = static_cast<long long>(T_new) * vec_per_token;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long g0 = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  // four 16-byte vectors of K and of V per thread, all loads before the stores
  uint4 kv[4], vv[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const long long gid = g0 + j * stride;
    if (gid < total) {
      const long long t = gid / vec_per_token;
      const int part = static_cast<int>(gid - t * vec_per_token);
      kv[j] = k[h * k_head_stride_vec + t * k_row_stride_vec + part];
      vv[j] = v[h * v_head_stride_vec + t * v_row_stride_vec + part];
    }
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const long long gid = g0 + j * stride;
    if (gid < total) {
      const long long t = gid / vec_per_token;
      const int part = static_cast<int>(gid - t * vec_per_token);
      const long long dst = h * cache_head_stride_vec + (old_T + t) * vec_per_token + part;
      k_cache[dst] = kv[j];
      v_cache[dst] = vv[j];
      if (part == 0) token_idx[h * idx_head_stride + old_T + t] = first_id + t;
    }
  }
}

// The epilogue of the attention layer's QKV projection fused with append_kv
// (causalvggt/layers/attention.py:119-128 and :141): one warp per (token, head) takes the three
// 64-value rows q, k, v of the projection output, applies LayerNorm over the head dimension to
// q and k (fp32: mean, biased variance, eps, affine), the 2-D rotary embedding (dims 0..31 turn
// with the token's y position, dims 32..63 with its x position; 16 frequencies each, rotate-half
// form, cos / sin read from the caller's tables), rounds to bf16 and writes q to the query
// tensor and k, v straight into the cache tail together with the token id.  Lane l holds dims l
// and 32 + l; the rotation partner of dim l inside its half is dim l ^ 16, i.e. lane l ^ 16.
__global__ void __launch_bounds__(256) qkv_epilogue_kernel(
    const __nv_bfloat16* __restrict__ qkv, long long token_stride, int H, const float* __restrict__ q_w,
    const float* __restrict__ q_b, const float* __restrict__ k_w, const float* __restrict__ k_b, float eps,
    const long long* __restrict__ pos, const float* __restrict__ cos_tab, const float* __restrict__ sin_tab,
    int n_pos, __nv_bfloat16* __restrict__ q_out, long long q_row_stride, __nv_bfloat16* __restrict__ k_cache,
    __nv_bfloat16* __restrict__ v_cache, long long cache_head_stride, long long* __restrict__ token_idx,
    long long idx_head_stride, int T_new, int old_T, long long first_id) {
  grid_dep_wait();   // launched with programmatic serialization: the projection that wrote qkv is complete now
  const int lane = threadIdx.x & 31;
  const long long w = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (w >= static_cast<long long>(T_new) * H) return;
  const int t = static_cast<int>(w / H), h = static_cast<int>(w - static_cast<long long>(t) * H);
  const __nv_bfloat16* src = qkv + t * token_stride + h * 64;
  float c_y = 1.f, s_y = 0.f, c_x = 1.f, s_x = 0.f;
  if (cos_tab != nullptr) {
    long long py = pos[2 * t], px = pos[2 * t + 1];
    py = py < 0 ? 0 : (py >= n_pos ? n_pos - 1 : py);
    px = px < 0 ? 0 : (px >= n_pos ? n_pos - 1 : px);
    const int f = lane & 15;
    c_y = cos_tab[py * 16 + f]; s_y = sin_tab[py * 16 + f];
    c_x = cos_tab[px * 16 + f]; s_x = sin_tab[px * 16 + f];
  }
  const float sign = (lane < 16) ? -1.f : 1.f;     // rotate-half: (-x2, x1)
  auto norm_rope = [&](int which, const float* wgt, const float* bia, float& a, float& b) {
    a = __bfloat162float(src[which * H * 64 + lane]);
    b = __bfloat162float(src[which * H * 64 + 32 + lane]);
    if (wgt != nullptr) {
      float sum = a + b;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      const float mean = sum * (1.f / 64.f);
      const float da = a - mean, db = b - mean;
      float sq = da * da + db * db;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
      const float rstd = rsqrtf(sq * (1.f / 64.f) + eps);
      a = da * rstd * wgt[lane] + bia[lane];
      b = db * rstd * wgt[32 + lane] + bia[32 + lane];
    }
    if (cos_tab != nullptr) {
      const float pa = __shfl_xor_sync(0xffffffffu, a, 16), pb = __shfl_xor_sync(0xffffffffu, b, 16);
      a = a * c_y + sign * pa * s_y;
      b = b * c_x + sign * pb * s_x;
    }
  };
  float qa, qb, ka, kb;
  norm_rope(0, q_w, q_b, qa, qb);
  norm_rope(1, k_w, k_b, ka, kb);
  __nv_bfloat16* qd = q_out + t * q_row_stride + h * 64;
  qd[lane] = __float2bfloat16_rn(qa);
  qd[32 + lane] = __float2bfloat16_rn(qb);
  const long long dst = h * cache_head_stride + static_cast<long long>(old_T + t) * 64;
  k_cache[dst + lane] = __float2bfloat16_rn(ka);
  k_cache[dst + 32 + lane] = __float2bfloat16_rn(kb);
  v_cache[dst + lane] = src[2 * H * 64 + lane];
  v_cache[dst + 32 + lane] = src[2 * H * 64 + 32 + lane];
  if (lane == 0) token_idx[h * idx_head_stride + old_T + t] = first_id + t;
}

}  // namespace
}  // namespace stac

extern "C" {

int stac_qkv_epilogue_append(const void* qkv, int64_t qkv_token_stride, const float* q_norm_w, const float* q_norm_b,
                             const float* k_norm_w, const float* k_norm_b, float eps, const int64_t* pos,
                             const float* cos_table, const float* sin_table, int n_pos, void* q_out,
                             int64_t q_out_row_stride, void* k_cache, void* v_cache, int64_t cache_head_stride,
                             int64_t* token_idx, int64_t idx_head_stride, int H, int T_new, int old_T,
                             int64_t first_token_id, stac_stream_t stream) {
  if (qkv == nullptr || q_out == nullptr || k_cache == nullptr || v_cache == nullptr || token_idx == nullptr ||
      H <= 0 || T_new < 0 || old_T < 0)
    return STAC_ERR_BAD_ARG;
  if ((q_norm_w == nullptr) != (q_norm_b == nullptr) || (k_norm_w == nullptr) != (k_norm_b == nullptr))
    return STAC_ERR_BAD_ARG;
  if (cos_table != nullptr && (sin_table == nullptr || pos == nullptr || n_pos <= 0)) return STAC_ERR_BAD_ARG;
  if (T_new == 0) return STAC_OK;
  const long long warps = static_cast<long long>(T_new) * H;
  const unsigned blocks = static_cast<unsigned>((warps * 32 + 255) / 256);
  if (stac::launch_behind(stac::qkv_epilogue_kernel, dim3(blocks), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream),
      static_cast<const __nv_bfloat16*>(qkv), qkv_token_stride, H, q_norm_w, q_norm_b, k_norm_w, k_norm_b, eps,
      reinterpret_cast<const long long*>(pos), cos_table, sin_table, n_pos, static_cast<__nv_bfloat16*>(q_out),
      q_out_row_stride, static_cast<__nv_bfloat16*>(k_cache), static_cast<__nv_bfloat16*>(v_cache), cache_head_stride,
      reinterpret_cast<long long*>(token_idx), idx_head_stride, T_new, old_T, first_token_id) != cudaSuccess)
    return STAC_ERR_CUDA;
  return STAC_OK;
}

int stac_append_kv(const void* k, const void* v, int64_t k_head_stride, int64_t k_row_stride, int64_t v_head_stride,
                   int64_t v_row_stride, void* k_cache, void* v_cache, int64_t cache_head_stride, int64_t* token_idx,
                   int64_t idx_head_stride, int H, int T_new, int old_T, int64_t first_token_id, int head_dim,
                   int elem_bytes, stac_stream_t stream) {
  if (k == nullptr || v == nullptr || k_cache == nullptr || v_cache == nullptr || token_idx == nullptr || H <= 0 ||
      T_new < 0 || old_T < 0)
    return STAC_ERR_BAD_ARG;
  const int token_bytes = head_dim * elem_bytes;
  if (token_bytes % 16 != 0) return STAC_ERR_BAD_ARG;
  const int epv = 16 / elem_bytes;  // elements per 16-byte vector
  if ((k_head_stride % epv) || (k_row_stride % epv) || (v_head_stride % epv) || (v_row_stride % epv) ||
      (cache_head_stride % epv))
    return STAC_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(k_cache) |
       reinterpret_cast<uintptr_t>(v_cache)) & 15)
    return STAC_ERR_BAD_ARG;
  if (T_new == 0) return STAC_OK;
  const int vpt = token_bytes / 16;
  const long long total = static_cast<long long>(T_new) * vpt;
  dim3 grid(static_cast<unsigned>((total + 4 * 256 - 1) / (4 * 256)), H);   // four vectors per thread
  if (stac::launch_behind(stac::append_kv_kernel, grid, dim3(256), 0, reinterpret_cast<cudaStream_t>(stream),
      static_cast<const uint4*>(k), static_cast<const uint4*>(v), k_head_stride / epv, k_row_stride / epv,
      v_head_stride / epv, v_row_stride / epv, static_cast<uint4*>(k_cache), static_cast<uint4*>(v_cache),
      cache_head_stride / epv, reinterpret_cast<long long*>(token_idx), idx_head_stride, T_new, old_T, first_token_id,
      vpt) != cudaSuccess)
    return STAC_ERR_CUDA;
  return STAC_OK;
}

int stac_scores_update(const float* colsum, int64_t colsum_head_stride, float* scores, float* counts,
                       int64_t row_stride, int H, int T_live, int old_T, int Tq, float temperature,
                       stac_stream_t stream) {
  if (colsum == nullptr || scores == nullptr || counts == nullptr || H <= 0 || T_live < 0 || old_T < 0 || Tq <= 0)
    return STAC_ERR_BAD_ARG;
  if (T_live == 0) return STAC_OK;
  dim3 grid((T_live + 255) / 256, H);
  if (stac::launch_behind(stac::scores_update_kernel, grid, dim3(256), 0, reinterpret_cast<cudaStream_t>(stream),
                          colsum, colsum_head_stride, scores, counts, row_stride, H, T_live, old_T,
                          static_cast<float>(T_live), static_cast<float>(Tq), temperature) != cudaSuccess)
    return STAC_ERR_CUDA;
  return STAC_OK;
}

int stac_h2o_select(const float* scores, int64_t row_stride, int n_rows, const uint8_t* is_base, int T, int n_keep,
                    int* keep_idx, int* drop_idx, stac_stream_t stream) {
  if (scores == nullptr || is_base == nullptr || keep_idx == nullptr || (drop_idx == nullptr && n_keep < T) ||
      n_rows <= 0 || T <= 0 || n_keep <= 0 || n_keep > T)
    return STAC_ERR_BAD_ARG;
  const int smem = T * 4;
  if (smem > 200 * 1024) return STAC_ERR_CAPACITY;
  int dev = 0;
  if (stac::current_device(&dev) != STAC_OK) return STAC_ERR_CUDA;
  static stac::PerDeviceFlag attr_done;   // the shared-memory opt-in is made once per device
  if (attr_done.needs_setup(dev)) {
    if (cudaFuncSetAttribute(stac::h2o_select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) !=
        cudaSuccess)
      return STAC_ERR_CUDA;
    attr_done.mark(dev);
  }
  if (stac::launch_behind(stac::h2o_select_kernel, dim3(n_rows), dim3(1024), smem, reinterpret_cast<cudaStream_t>(stream),
                          scores, row_stride, is_base, T, n_keep, keep_idx, drop_idx) != cudaSuccess)
    return STAC_ERR_CUDA;
  return cudaGetLastError() == cudaSuccess ? STAC_OK : STAC_ERR_CUDA;
}

int stac_compact(const int* keep_idx, int n_rows, int n_keep, int T_buf, int head_dim, int elem_bytes,
                 const void* k_src, const void* v_src, void* k_dst, void* v_dst, const int64_t* ti_src,
                 int64_t* ti_dst, const float* s_src, float* s_dst, const float* c_src, float* c_dst,
                 const int* vx_src, int* vx_dst, stac_stream_t stream) {
  if (keep_idx == nullptr || k_src == nullptr || v_src == nullptr || k_dst == nullptr || v_dst == nullptr ||
      ti_src == nullptr || ti_dst == nullptr || s_src == nullptr || s_dst == nullptr || c_src == nullptr ||
      c_dst == nullptr || n_rows <= 0 || n_keep < 0 || n_keep > T_buf)
    return STAC_ERR_BAD_ARG;
  if ((vx_src == nullptr) != (vx_dst == nullptr)) return STAC_ERR_BAD_ARG;
  const int token_bytes = head_dim * elem_bytes;
  if (token_bytes % 16 != 0 || (elem_bytes != 2 && elem_bytes != 4)) return STAC_ERR_BAD_ARG;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int vpt = token_bytes / 16;
  if (n_keep > 0) {
    const long long total = static_cast<long long>(n_keep) * vpt;
    dim3 grid(static_cast<unsigned>((total + 255) / 256), n_rows);
    if (stac::launch_behind(stac::compact_kv_kernel, grid, dim3(256), 0, st, keep_idx, n_keep,
                            static_cast<const uint4*>(k_src), static_cast<const uint4*>(v_src),
                            static_cast<uint4*>(k_dst), static_cast<uint4*>(v_dst),
                            static_cast<long long>(T_buf) * vpt, vpt) != cudaSuccess)
      return STAC_ERR_CUDA;
  }
  dim3 grid_m((T_buf + 255) / 256, n_rows);
  if (stac::launch_behind(stac::compact_meta_kernel, grid_m, dim3(256), 0, st, keep_idx, n_keep, T_buf,
                          reinterpret_cast<const long long*>(ti_src), reinterpret_cast<long long*>(ti_dst), s_src,
                          s_dst, c_src, c_dst, vx_src, vx_dst) != cudaSuccess)
    return STAC_ERR_CUDA;
  return cudaGetLastError() == cudaSuccess ? STAC_OK : STAC_ERR_CUDA;
}

}  // extern "C"
