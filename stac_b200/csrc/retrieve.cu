// Pivot retrieval: for every pool head, the pivots of the queried voxels ordered by weight W
// (descending), the first R of them copied out with bias log C.
//
// Replaces VoxelKVMerger.retrieve on the reference's Python path (stac/merger.py:1377-1482:
// gather of all [H, Q*P] pivots, argsort by W, three more gathers, index_put compaction) and
// MergerWrapper.retrieve_seg with its torch sort (merger-cuda/csrc/merger_wrapper.cu:3148-3221).
//
// retrieve_select_kernel  one CTA per head: radix select of the weight threshold over the
//                         (voxel, slot) candidates of the queried voxels, the candidates at or
//                         above it collected in shared memory and sorted (64-bit keys = weight
//                         bits | inverted candidate index, so equal weights resolve to the
//                         earlier candidate); writes their order.
// retrieve_gather_kernel  copies K/V of the selected pivots with 16-byte vectors, writes mask
//                         and bias, zero-fills the padding.
#include "common.cuh"
#include "stac_internal.h"

namespace stac {
namespace {

constexpr int kSelCap = 8192;     // shared-memory candidate buffer (64-bit keys)
constexpr int kSelThreads = 512;
constexpr int kSelBins = 8192;    // counters of one radix digit (13 + 11 + 8 bits, most significant first)
constexpr int kSelUnroll = 2;     // queried voxels per thread in flight

__device__ __forceinline__ unsigned int wkey(float f) {
  const unsigned int u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ void bitonic_desc(unsigned long long* a, int n) {
  for (int k = 2; k <= n; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int ixj = i ^ j;
        if (ixj > i) {
          const unsigned long long x = a[i], y = a[ixj];
          const bool desc = (i & k) == 0;
          if ((x < y) == desc) {
            a[i] = y;
            a[ixj] = x;
          }
        }
      }
      __syncthreads();
    }
  }
}

struct RetrieveParams {
  int heads, D, P, voxel_cap, voxel_used, R;
  const int* query_ids;    // ascending voxel ids
  const int* query_count;  // device scalar
  const int* piv_row_seg;
  const int* piv_row_cnt;
  const void* piv_K;
  const void* piv_V;
  const float* piv_W;
  const float* piv_C;
  int* sel;        // [heads][R] candidate index q*P + slot, -1 = padding
  void* out_K;     // [heads][R][D]
  void* out_V;
  unsigned char* out_mask;  // [heads][R]
  float* out_bias;          // [heads][R]
  int* out_idx;             // [heads][R][2] (voxel, slot) or nullptr
};

// Calls f(weight key, candidate index) for every pivot of the queried voxels of head h: one
// pass over the candidates, kSelUnroll voxels per thread in flight.  Every thread of the CTA
// must call it (no barrier inside).
template <typename F>
__device__ __forceinline__ void for_each_candidate(const RetrieveParams& p, int h, int Q, F f) {
  for (int base = 0; base < Q; base += kSelThreads * kSelUnroll) {
    int n[kSelUnroll];
    long long r[kSelUnroll];
#pragma unroll
    for (int u = 0; u < kSelUnroll; ++u) {
      const int q = base + u * kSelThreads + threadIdx.x;
      n[u] = 0;
      r[u] = 0;
      if (q < Q) {
        const int v = p.query_ids[q];
        if (v >= 0 && v < p.voxel_used) {
          r[u] = static_cast<long long>(h) * p.voxel_cap + v;
          n[u] = min(p.piv_row_cnt[r[u]], 4);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kSelUnroll; ++u) {
      const int q = base + u * kSelThreads + threadIdx.x;
      int seg[4];
#pragma unroll
      for (int s = 0; s < 4; ++s) seg[s] = s < n[u] ? p.piv_row_seg[r[u] * p.P + s] : 0;
      float w[4];
#pragma unroll
      for (int s = 0; s < 4; ++s) w[s] = s < n[u] ? p.piv_W[seg[s]] : 0.f;
#pragma unroll
      for (int s = 0; s < 4; ++s)
        if (s < n[u]) f(wkey(w[s]), static_cast<unsigned int>(q * p.P + s));
    }
  }
}

// Shared-memory counters are bumped once per warp and distinct value, not once per lane: the
// weights of one head fall into few histogram bins (their exponents are alike), and the lanes of
// a warp would otherwise queue up on the same word.
__device__ __forceinline__ void hist_add(int* hist, unsigned int bin) {
  const unsigned int m = __activemask();
  const unsigned int peers = __match_any_sync(m, bin);
  const unsigned int lane = threadIdx.x & 31;
  if ((peers & ((1u << lane) - 1u)) == 0u) atomicAdd(&hist[bin], __popc(peers));
}
// One slot of a shared list per calling lane (slots of one warp are consecutive).
__device__ __forceinline__ int list_push(int* counter) {
  const unsigned int m = __activemask();
  const unsigned int lane = threadIdx.x & 31;
  const int leader = __ffs(m) - 1;
  int base = 0;
  if (static_cast<int>(lane) == leader) base = atomicAdd(counter, __popc(m));
  base = __shfl_sync(m, base, leader);
  return base + __popc(m & ((1u << lane) - 1u));
}

// Top R candidates of one head by (weight desc, candidate index asc).  A radix select on the
// weight key finds the threshold digit by digit (13 + 11 + 8 bits, one pass over the candidates
// per digit) and stops as soon as the candidates at or above the current prefix fit the
// shared-memory buffer, which is then sorted; with the usual spread of weights that is after the
// first digit, i.e. two passes.  Only when more than kSelCap - R candidates share one exact
// weight is the last group taken in candidate order by an ordered pass.
__global__ void __launch_bounds__(kSelThreads, 3) retrieve_select_kernel(const RetrieveParams p) {
  grid_dep_wait();   // launched with programmatic serialization behind the previous kernel in the stream
  // kSelCap keys; the digit counters live in the same 64 KB (they are dead once the threshold is
  // known and the keys are collected), so three CTAs fit one SM and 384 heads run in one wave
  extern __shared__ unsigned long long cand[];
  int* hist = reinterpret_cast<int*>(cand);
  static_assert(kSelBins * 4 <= kSelCap * 8, "digit counters must fit the candidate buffer");
  __shared__ int warp_sums[kSelThreads / 32];
  __shared__ int sh_count, sh_bin, sh_above, sh_ties;
  const int h = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int Q = *p.query_count;
  const int R = p.R;
  // prefix of the threshold found so far: candidates with (key >> shift) > prefix are in for
  // certain, those with (key >> shift) == prefix are undecided
  unsigned int prefix = 0;
  int shift = 32, need = R;       // need = how many of the undecided ones are wanted
  bool take_all = false, ordered_ties = false;
  const int widths[3] = {13, 11, 8};
  for (int level = 0; level < 3; ++level) {
    const int width = widths[level];
    const int new_shift = shift - width;
    for (int i = threadIdx.x; i < kSelBins; i += kSelThreads) hist[i] = 0;
    __syncthreads();
    const unsigned int pf = prefix;
    const int sh_old = shift;
    for_each_candidate(p, h, Q, [&](unsigned int wk, unsigned int) {
      if (sh_old == 32 || (wk >> sh_old) == pf) hist_add(hist, (wk >> new_shift) & ((1u << width) - 1u));
    });
    __syncthreads();
    // the digit at which the count from the top reaches `need`
    if (warp == 0) {
      const int bins = 1 << width;
      int above = 0, found = -1, found_above = 0;
      for (int top = bins - 32; top >= 0 && found < 0; top -= 32) {
        const int b = top + (31 - lane);              // lane 0 holds the highest digit of the chunk
        const int c = hist[b];
        int incl = c;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int t = __shfl_up_sync(0xffffffffu, incl, o);
          if (lane >= o) incl += t;
        }
        const bool hit = above + incl >= need;
        const unsigned m = __ballot_sync(0xffffffffu, hit);
        if (m) {
          const int l = __ffs(m) - 1;
          found = top + (31 - l);
          found_above = above + __shfl_sync(0xffffffffu, incl - c, l);
        }
        above += __shfl_sync(0xffffffffu, incl, 31);
      }
      if (lane == 0) {
        sh_bin = found;                 // -1: fewer than `need` undecided candidates exist
        sh_above = found >= 0 ? found_above : above;
        sh_ties = found >= 0 ? hist[found] : 0;
      }
    }
    __syncthreads();
    if (sh_bin < 0) {
      take_all = true;                  // everything undecided is wanted
      break;
    }
    prefix = (prefix << width) | static_cast<unsigned int>(sh_bin);
    shift = new_shift;
    const int decided = (R - need) + sh_above;      // candidates strictly above the new prefix
    need -= sh_above;
    if (decided + sh_ties <= kSelCap) break;        // they all fit: sort settles the rest
    if (level == 2) ordered_ties = true;            // one exact weight, more copies than fit
    __syncthreads();
  }
  // ---- collect (the counters are no longer needed: their memory becomes the key buffer)
  __syncthreads();
  if (threadIdx.x == 0) sh_count = 0;
  __syncthreads();
  if (!ordered_ties) {
    const unsigned int pf = prefix;
    const int sh = shift;
    for_each_candidate(p, h, Q, [&](unsigned int wk, unsigned int idx) {
      if (take_all || sh == 32 || (wk >> sh) >= pf) {
        const int pos = list_push(&sh_count);
        if (pos < kSelCap) cand[pos] = (static_cast<unsigned long long>(wk) << 32) | (0xFFFFFFFFu - idx);
      }
    });
  } else {
    // weights above the threshold in any order, then the first `need` candidates that carry the
    // threshold weight itself, in candidate order (batches of one voxel per thread, block scan)
    const unsigned int T = prefix;
    for_each_candidate(p, h, Q, [&](unsigned int wk, unsigned int idx) {
      if (wk > T) {
        const int pos = list_push(&sh_count);
        cand[pos] = (static_cast<unsigned long long>(wk) << 32) | (0xFFFFFFFFu - idx);
      }
    });
    __syncthreads();
    int taken = 0;                    // ties accepted so far (same value in every thread)
    for (int base = 0; base < Q && taken < need; base += kSelThreads) {
      const int q = base + threadIdx.x;
      unsigned int mine[4];
      int n_mine = 0;
      if (q < Q) {
        const int v = p.query_ids[q];
        if (v >= 0 && v < p.voxel_used) {
          const long long r = static_cast<long long>(h) * p.voxel_cap + v;
          const int n = min(p.piv_row_cnt[r], 4);
          for (int s = 0; s < n; ++s)
            if (wkey(p.piv_W[p.piv_row_seg[r * p.P + s]]) == T) mine[n_mine++] = static_cast<unsigned int>(q * p.P + s);
        }
      }
      int incl = n_mine;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
      }
      if (lane == 31) warp_sums[warp] = incl;
      __syncthreads();
      if (warp == 0) {
        int w = lane < kSelThreads / 32 ? warp_sums[lane] : 0;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int t = __shfl_up_sync(0xffffffffu, w, o);
          if (lane >= o) w += t;
        }
        if (lane < kSelThreads / 32) warp_sums[lane] = w;
      }
      __syncthreads();
      const int off = taken + (warp > 0 ? warp_sums[warp - 1] : 0) + incl - n_mine;
      for (int s = 0; s < n_mine; ++s) {
        if (off + s < need) {
          const int pos = atomicAdd(&sh_count, 1);
          cand[pos] = (static_cast<unsigned long long>(T) << 32) | (0xFFFFFFFFu - mine[s]);
        }
      }
      taken += warp_sums[kSelThreads / 32 - 1];
      __syncthreads();
    }
  }
  __syncthreads();
  {
    const int cnt = min(sh_count, kSelCap);
    int np2 = 1;
    while (np2 < cnt) np2 <<= 1;
    for (int i = cnt + threadIdx.x; i < np2; i += blockDim.x) cand[i] = 0ull;
    __syncthreads();
    if (cnt > 1) bitonic_desc(cand, np2);
    const int keep = min(cnt, R);
    for (int i = threadIdx.x; i < R; i += blockDim.x) {
      int c = -1;
      if (i < keep) c = static_cast<int>(0xFFFFFFFFu - static_cast<unsigned int>(cand[i] & 0xFFFFFFFFull));
      p.sel[static_cast<long long>(h) * R + i] = c;
    }
  }
}

__global__ void retrieve_gather_kernel(const RetrieveParams p, int vec_per_token) {
  grid_dep_wait();   // launched with programmatic serialization behind the previous kernel in the stream
  const long long gid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int h = blockIdx.y;
  const long long tok = gid / vec_per_token;
  const int part = static_cast<int>(gid % vec_per_token);
  if (tok >= p.R) return;
  const long long o = static_cast<long long>(h) * p.R + tok;
  const int c = p.sel[o];
  uint4 kv = make_uint4(0, 0, 0, 0), vv = make_uint4(0, 0, 0, 0);
  int seg = -1, v = -1, slot = -1;
  if (c >= 0) {
    v = p.query_ids[c / p.P];
    slot = c % p.P;
    seg = p.piv_row_seg[(static_cast<long long>(h) * p.voxel_cap + v) * p.P + slot];
    kv = static_cast<const uint4*>(p.piv_K)[static_cast<long long>(seg) * vec_per_token + part];
    vv = static_cast<const uint4*>(p.piv_V)[static_cast<long long>(seg) * vec_per_token + part];
  }
  static_cast<uint4*>(p.out_K)[o * vec_per_token + part] = kv;
  static_cast<uint4*>(p.out_V)[o * vec_per_token + part] = vv;
  if (part == 0) {
    p.out_mask[o] = c >= 0 ? 1 : 0;
    p.out_bias[o] = c >= 0 ? logf(fmaxf(p.piv_C[seg], 1e-9f)) : -INFINITY;
    if (p.out_idx != nullptr) {
      p.out_idx[2 * o] = v;
      p.out_idx[2 * o + 1] = slot;
    }
  }
}

}  // namespace
}  // namespace stac

extern "C" {

int stac_retrieve(const stac_pool* pool, const int* query_ids, const int* query_count, int retrieve_size, int* sel,
                  void* out_K, void* out_V, uint8_t* out_mask, float* out_bias, int* out_idx, stac_stream_t stream) {
  if (pool == nullptr || query_ids == nullptr || query_count == nullptr || sel == nullptr || out_K == nullptr ||
      out_V == nullptr || out_mask == nullptr || out_bias == nullptr)
    return STAC_ERR_BAD_ARG;
  if (retrieve_size <= 0 || retrieve_size > stac::kSelCap || pool->pivot_cap > 4) return STAC_ERR_BAD_ARG;
  const int token_bytes = pool->head_dim * pool->elem_bytes;
  if (token_bytes % 16 != 0) return STAC_ERR_BAD_ARG;
  stac::RetrieveParams rp;
  rp.heads = pool->heads; rp.D = pool->head_dim; rp.P = pool->pivot_cap; rp.voxel_cap = pool->voxel_cap;
  rp.voxel_used = pool->voxel_used; rp.R = retrieve_size;
  rp.query_ids = query_ids; rp.query_count = query_count;
  rp.piv_row_seg = pool->piv_row_seg; rp.piv_row_cnt = pool->piv_row_cnt;
  rp.piv_K = pool->piv_K; rp.piv_V = pool->piv_V; rp.piv_W = pool->piv_W; rp.piv_C = pool->piv_C;
  rp.sel = sel; rp.out_K = out_K; rp.out_V = out_V; rp.out_mask = out_mask; rp.out_bias = out_bias;
  rp.out_idx = out_idx;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int dev = 0;
  if (stac::current_device(&dev) != STAC_OK) return STAC_ERR_CUDA;
  static stac::PerDeviceFlag attr_done;   // the shared-memory opt-in is made once per device
  const int smem = stac::kSelCap * 8;
  if (attr_done.needs_setup(dev)) {
    if (cudaFuncSetAttribute(stac::retrieve_select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) !=
        cudaSuccess)
      return STAC_ERR_CUDA;
    attr_done.mark(dev);
  }
  if (stac::launch_behind(stac::retrieve_select_kernel, dim3(pool->heads), dim3(stac::kSelThreads), smem, st, rp) != cudaSuccess)
    return STAC_ERR_CUDA;
  const int vpt = token_bytes / 16;
  const long long total = static_cast<long long>(retrieve_size) * vpt;
  dim3 grid(static_cast<unsigned>((total + 255) / 256), pool->heads);
  if (stac::launch_behind(stac::retrieve_gather_kernel, grid, dim3(256), 0, st, rp, vpt) != cudaSuccess) return STAC_ERR_CUDA;
  return cudaGetLastError() == cudaSuccess ? STAC_OK : STAC_ERR_CUDA;
}

}  // extern "C"
