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
__global__ void __launch_bounds__(1024, 1)
h2o_select_kernel(const float* __restrict__ scores, long long row_stride, const unsigned char* __restrict__ is_base,
                  int T, int n_keep, int* __restrict__ keep_idx, int* __restrict__ drop_idx) {
  extern __shared__ unsigned int keys[];
  __shared__ int hist[256];
  __shared__ int warp_sums[32];
  __shared__ int sh_total;
  __shared__ unsigned int sh_prefix;
  __shared__ int sh_remaining;
  const int row = blockIdx.x;
  const float* srow = scores + row * row_stride;
  for (int t = threadIdx.x; t < T; t += blockDim.x) keys[t] = is_base[t] ? 0xFFFFFFFFu : float_key(srow[t]);
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
      if ((k & hi_mask) == prefix) atomicAdd(&hist[(k >> shift) & 255], 1);
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
  for (int base = 0; base < T; base += blockDim.x) {
    const int t = base + threadIdx.x;
    const bool in = t < T;
    const unsigned int k = in ? keys[t] : 0u;
    const int eq = (in && k == tau) ? 1 : 0;
    const int eq_rank = eq_carry + block_scan_1024(eq, warp_sums, &sh_total);
    const int eq_total = sh_total;
    const int keep = (in && (k > tau || (eq && eq_rank < need_eq))) ? 1 : 0;
    const int keep_rank = keep_carry + block_scan_1024(keep, warp_sums, &sh_total);
    const int keep_total = sh_total;
    if (in) {
      if (keep) krow[keep_rank] = t;
      else drow[drop_carry + (threadIdx.x - (keep_rank - keep_carry))] = t;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      eq_carry += eq_total;
      keep_carry += keep_total;
      drop_carry += min(static_cast<int>(blockDim.x), T - base) - keep_total;
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
  const long long gid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int h = blockIdx.y;
  const long long t = gid / vec_per_token;
  const int part = static_cast<int>(gid % vec_per_token);
  if (t >= T_new) return;
  const long long dst = h * cache_head_stride_vec + (old_T + t) * vec_per_token + part;
  k_cache[dst] = k[h * k_head_stride_vec + t * k_row_stride_vec + part];
  v_cache[dst] = v[h * v_head_stride_vec + t * v_row_stride_vec + part];
  if (part == 0) token_idx[h * idx_head_stride + old_T + t] = first_id + t;
}

}  // namespace
}  // namespace stac

extern "C" {

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
  dim3 grid(static_cast<unsigned>((total + 255) / 256), H);
  stac::append_kv_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(k), static_cast<const uint4*>(v), k_head_stride / epv, k_row_stride / epv,
      v_head_stride / epv, v_row_stride / epv, static_cast<uint4*>(k_cache), static_cast<uint4*>(v_cache),
      cache_head_stride / epv, reinterpret_cast<long long*>(token_idx), idx_head_stride, T_new, old_T, first_token_id,
      vpt);
  return cudaGetLastError() == cudaSuccess ? STAC_OK : STAC_ERR_CUDA;
}

int stac_scores_update(const float* colsum, int64_t colsum_head_stride, float* scores, float* counts,
                       int64_t row_stride, int H, int T_live, int old_T, int Tq, float temperature,
                       stac_stream_t stream) {
  if (colsum == nullptr || scores == nullptr || counts == nullptr || H <= 0 || T_live < 0 || old_T < 0 || Tq <= 0)
    return STAC_ERR_BAD_ARG;
  if (T_live == 0) return STAC_OK;
  dim3 grid((T_live + 255) / 256, H);
  stac::scores_update_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      colsum, colsum_head_stride, scores, counts, row_stride, H, T_live, old_T, static_cast<float>(T_live),
      static_cast<float>(Tq), temperature);
  return cudaGetLastError() == cudaSuccess ? STAC_OK : STAC_ERR_CUDA;
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
  stac::h2o_select_kernel<<<n_rows, 1024, smem, reinterpret_cast<cudaStream_t>(stream)>>>(
      scores, row_stride, is_base, T, n_keep, keep_idx, drop_idx);
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
    stac::compact_kv_kernel<<<grid, 256, 0, st>>>(keep_idx, n_keep, static_cast<const uint4*>(k_src),
                                                 static_cast<const uint4*>(v_src), static_cast<uint4*>(k_dst),
                                                 static_cast<uint4*>(v_dst),
                                                 static_cast<long long>(T_buf) * vpt, vpt);
  }
  dim3 grid_m((T_buf + 255) / 256, n_rows);
  stac::compact_meta_kernel<<<grid_m, 256, 0, st>>>(keep_idx, n_keep, T_buf,
                                                   reinterpret_cast<const long long*>(ti_src),
                                                   reinterpret_cast<long long*>(ti_dst), s_src, s_dst, c_src, c_dst,
                                                   vx_src, vx_dst);
  return cudaGetLastError() == cudaSuccess ? STAC_OK : STAC_ERR_CUDA;
}

}  // extern "C"
