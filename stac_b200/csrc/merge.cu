// Eviction into the voxel memory: deterministic segmented merge of evicted K/V into the
// per-(head, voxel) pools.
//
// Replaces VoxelKVMerger.insert_and_merge and its helpers on the reference's Python path
// (stac/merger.py:1157-1255 filter + stable sort by row, :765-918 order of operations,
// :586-760 token -> pivot merge, :408-461 full buffer -> one pivot, :462-582 pivot insert /
// victim re-merge) together with the Top-B append and the segment allocator
// (stac/allocator.py:559-723, :2237-2345, :2306-2319), and the merger-cuda pipeline that the
// reference uses on the GPU (merger-cuda/csrc/kernels/merger_kernels.cu).
//
// Every output is a pure function of the inputs: per-(head, voxel) work is done by one warp
// in token order, and everything that depends on an order across rows (which segment id a
// row gets, where its overflow lands, where freed ids go) is computed from exclusive scans
// over the rows in (head, voxel) order.  No floating-point atomics and no slot pops by
// atomics, so keys, slot maps and merged values repeat bit for bit from run to run.
//
// Kernels, in launch order:
//   sort_tokens_kernel   one CTA per pool head: list the head's valid evicted tokens followed
//                        by its carried overflow tokens, stable LSD radix sort by voxel id,
//                        emit the unique rows (CSR).
//   tokens_sim_kernel    token-parallel (eight lanes per token, 16-byte loads): cosine of every
//                        token with the pivots of its row, best pivot; rows in which a token
//                        reaches the merge threshold are queued for
//   rows_merge_kernel    one warp per queued row: fold those tokens into their pivots in token
//                        order (exp(sim) weights), publish the new pivot weights.
//   rows_rank_kernel     one thread per row: score gate of the row's pivots, selection, ranking of
//                        the buffered tokens + selected tokens by (score desc, arrival order),
//                        counts of new segments / overflow / full; rows with many tokens are
//                        queued for rows_rank_long_kernel (one warp per row, same result).
//   scan_heads_kernel /  exclusive scans of those counts, allocation plan (k ids from the top
//   scan_plan_kernel     of the free list, the rest fresh), capacity checks.
//   rows_phase_b1a_kernel one thread per row: hand out segment ids, publish occupancy, queue rows
//                        whose buffered tokens change column / whose buffer filled up.
//   rows_phase_b1m_kernel one warp per queued row: move buffered tokens to their new column
//                        (or to the overflow list), last column first, in place.
//   tokens_place_kernel  token-parallel 16-byte-vector copy of every selected token to its
//                        column's segment or overflow slot.
//   rows_phase_b2_kernel eight lanes per full row: turn the buffer into a pivot, insert it (folding
//                        the lowest-weight pivot into its nearest neighbour when the row is
//                        saturated), stage the freed segment ids.
//   finalize_kernel      append staged ids to the free list, publish counters.
#include <cuda_bf16.h>

#include "common.cuh"
#include "stac_internal.h"

namespace stac {
namespace {

constexpr int kMaxB = 8;
constexpr int kMaxP = 4;
constexpr unsigned kFull = 0xffffffffu;

// ------------------------------------------------------------------------------------ helpers
template <typename T> struct Elem;
template <> struct Elem<float> {
  static __device__ __forceinline__ float load(const float* p) { return *p; }
  static __device__ __forceinline__ float load_cg(const float* p) { return __ldcg(p); }
  static __device__ __forceinline__ void store(float* p, float v) { *p = v; }
  static __device__ __forceinline__ float round(float v) { return v; }
  static constexpr bool kIsBf16 = false;
};
template <> struct Elem<__nv_bfloat16> {
  static __device__ __forceinline__ float load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  static __device__ __forceinline__ float load_cg(const __nv_bfloat16* p) {
    const unsigned short u = __ldcg(reinterpret_cast<const unsigned short*>(p));
    return __uint_as_float(static_cast<unsigned int>(u) << 16);
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
  static __device__ __forceinline__ float round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
  static constexpr bool kIsBf16 = true;
};

// One slot of a global work list per calling lane: the lanes of a warp that push at the same time
// take consecutive slots with ONE atomic (the order of a list never reaches an output).
__device__ __forceinline__ int list_push(int* counter) {
  const unsigned m = __activemask();
  const unsigned lane = threadIdx.x & 31;
  const int leader = __ffs(m) - 1;
  int base = 0;
  if (static_cast<int>(lane) == leader) base = atomicAdd(counter, __popc(m));
  base = __shfl_sync(m, base, leader);
  return base + __popc(m & ((1u << lane) - 1u));
}

struct MergeParams {
  // geometry
  int heads, D, P, B, voxel_cap, voxel_used;
  float sim_thresh, replace_thresh, score_thresh;
  // evicted tokens: token j of head h lives at position pos = idx ? idx[h*n_new + j] : j
  const void* k_src;
  const void* v_src;
  const float* s_src;
  const int* vx_src;
  const int* idx;
  long long src_head_stride;   // elements between heads in k_src / v_src
  long long src_row_stride;    // elements between positions
  long long meta_head_stride;  // elements between heads in s_src / vx_src
  int n_new;                   // tokens per head
  // pools
  void* buf_K; void* buf_V; float* buf_S;
  int* buf_row_seg; int* buf_row_cnt; int* buf_free; int buf_cap;
  void* piv_K; void* piv_V; float* piv_W; float* piv_S; float* piv_C;
  int* piv_row_seg; int* piv_row_cnt; int piv_cap;
  // overflow lists
  const void* over_K_in; const void* over_V_in; const float* over_S_in; const int* over_hv_in;
  const int* over_start_in;  // [heads + 1]
  void* over_K_out; void* over_V_out; float* over_S_out; int* over_hv_out;
  int* over_start_out;
  int over_cap;
  int* meta;  // device ints, see STAC_META_*
  const int* voxel_count;  // device scalar or nullptr
  // scratch
  int ncap;            // per-head capacity of the token lists
  unsigned int* keys_a; unsigned int* keys_b;  // [heads][ncap]
  int* vals_a; int* vals_b;                    // [heads][ncap]
  int* n_tok;          // [heads]
  int* n_rows;         // [heads]
  int* row_vx;         // [heads][ncap]
  int* row_start;      // [heads][ncap + 1]
  int4* row_info;      // [heads][ncap]: add_cnt, over_cnt, flags, n_sel
  int4* row_pref;      // [heads][ncap]: exclusive prefixes inside the head
  int* old_dest;       // [heads][ncap][8] new rank of each buffered token (>= B: goes to the overflow list)
  int* tok_dest;       // [heads][ncap]
  float* tok_sim;      // [heads][ncap]
  float* tok_score;    // [heads][ncap]
  int4* head_tot;      // [heads]
  int4* head_base;     // [heads]
  int* plan;           // device ints, see kPlan*
  int* free_stage;     // [buf_cap]
  int2* defer_list;    // [heads*ncap] rows (head, row index) that need the warp-per-row phase A
  int2* full_list;     // [heads*ncap] rows whose buffer filled up in this call
  int2* move_list;     // [heads*ncap] rows in which buffered tokens change column
  int* tok_row;        // [heads][ncap] row index of each sorted token
  int* tok_best;       // [heads][ncap] index of the most similar pivot of the token's row
  int* row_flag;       // [heads][ncap] zero on entry: set once a token of the row merges into a pivot
  int2* merge_list;    // [heads*ncap] rows (head, row index) with at least one merging token
  int passes;          // radix passes (8 bits each)
  int* err;
};

enum { kPlanK = 0, kPlanFreeLen, kPlanBufTop, kPlanPivTop, kPlanTotalAdd, kPlanTotalFull, kPlanTotalOver,
       kPlanAnyValid, kPlanAbort, kPlanDeferCount, kPlanFullCount, kPlanMoveCount, kPlanShort, kPlanAvailBuf, kPlanAvailPiv,
       kPlanMergeCount, kPlanSize = 16 };

// Block-wide exclusive scan, 1024 threads.
__device__ __forceinline__ int block_scan(int v, int* warp_sums, int* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(kFull, incl, o);
    if (lane >= o) incl += t;
  }
  if (lane == 31) warp_sums[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int w = warp_sums[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(kFull, w, o);
      if (lane >= o) w += t;
    }
    warp_sums[lane] = w;
  }
  __syncthreads();
  const int excl = (warp > 0 ? warp_sums[warp - 1] : 0) + incl - v;
  if (threadIdx.x == 0) *total = warp_sums[31];
  __syncthreads();
  return excl;
}

// ------------------------------------------------------------------------------------ sort
__global__ void __launch_bounds__(1024, 2) sort_tokens_kernel(const MergeParams p) {
  grid_dep_wait();   // launched with programmatic serialization behind the previous kernel of the call
  __shared__ int hist[256 * 32];  // [digit][warp]
  __shared__ int warp_sums[32];
  __shared__ int sh_total;
  __shared__ int sh_carry;
  const int h = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  unsigned int* ka = p.keys_a + static_cast<long long>(h) * p.ncap;
  unsigned int* kb = p.keys_b + static_cast<long long>(h) * p.ncap;
  int* va = p.vals_a + static_cast<long long>(h) * p.ncap;
  int* vb = p.vals_b + static_cast<long long>(h) * p.ncap;

  // 1. valid evicted tokens in position order
  if (threadIdx.x == 0) sh_carry = 0;
  __syncthreads();
  // four consecutive positions per thread: one block scan per 4096 tokens, loads issued together
  for (int base = 0; base < p.n_new; base += 4096) {
    const int j0 = base + threadIdx.x * 4;
    int vxs[4];
    int sum = 0;
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const int j = j0 + t;
      int vx = -1;
      if (j < p.n_new) {
        const int pos = p.idx ? p.idx[static_cast<long long>(h) * p.n_new + j] : j;
        vx = p.vx_src[h * p.meta_head_stride + pos];
      }
      vxs[t] = (vx >= 0 && vx < p.voxel_used) ? vx : -1;
      sum += vxs[t] >= 0 ? 1 : 0;
    }
    int off = sh_carry + block_scan(sum, warp_sums, &sh_total);
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      if (vxs[t] >= 0) {
        ka[off] = static_cast<unsigned int>(vxs[t]);
        va[off] = j0 + t;
        ++off;
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) sh_carry += sh_total;
    __syncthreads();
  }
  const int n_valid = sh_carry;
  if (n_valid > 0 && threadIdx.x == 0) atomicOr(&p.plan[kPlanAnyValid], 1);
  // 2. carried overflow tokens of this head, in list order
  const int os = p.over_start_in[h], oe = p.over_start_in[h + 1];
  int n = n_valid + (oe - os);
  if (n > p.ncap) {
    if (threadIdx.x == 0) report_error(p.err, DEV_SORT_CAPACITY);
    n = p.ncap;
  }
  for (int o = os + threadIdx.x; o < oe; o += 1024) {
    const int dst = n_valid + (o - os);
    if (dst < n) {
      ka[dst] = static_cast<unsigned int>(p.over_hv_in[2 * o + 1]);
      va[dst] = ~o;
    }
  }
  __syncthreads();
  // 3. stable LSD radix sort by voxel id.  Each warp owns a contiguous chunk of the list so
  //    that (warp, position in chunk) preserves the input order.
  const int chunk = ((n + 31) / 32 + 31) / 32 * 32;  // items per warp, multiple of 32
  const int c0 = warp * chunk;
  const int c1 = min(n, c0 + chunk);
  unsigned int* kin = ka; int* vin = va; unsigned int* kout = kb; int* vout = vb;
  // A warp's chunk is read into registers once per pass when it is at most kRegIt * 32 items
  // (lists of up to 8192 tokens): one round trip to L2 per pass instead of one per 32 items in
  // each of the two loops.
  constexpr int kRegIt = 8;
  const bool in_regs = chunk <= 32 * kRegIt;
  for (int pass = 0; pass < p.passes; ++pass) {
    const int shift = pass * 8;
    for (int i = threadIdx.x; i < 256 * 32; i += 1024) hist[i] = 0;
    unsigned int kreg[kRegIt];
    int vreg[kRegIt];
    if (in_regs) {
#pragma unroll
      for (int t = 0; t < kRegIt; ++t) {
        const int i = c0 + t * 32 + lane;
        kreg[t] = i < c1 ? kin[i] : 0u;
        vreg[t] = i < c1 ? vin[i] : 0;
      }
    }
    __syncthreads();
    if (in_regs) {
#pragma unroll
      for (int t = 0; t < kRegIt; ++t) {
        const int base = c0 + t * 32;
        if (base < c1) {                                   // warp-uniform
          const bool in = base + lane < c1;
          const unsigned int d = in ? ((kreg[t] >> shift) & 255u) : (256u + lane);
          const unsigned int peers = __match_any_sync(kFull, d);
          if (in && (peers & ((1u << lane) - 1)) == 0) hist[d * 32 + warp] += __popc(peers);
          __syncwarp();
        }
      }
    } else {
      for (int base = c0; base < c1; base += 32) {
        const int i = base + lane;
        const bool in = i < c1;
        const unsigned int d = in ? ((kin[i] >> shift) & 255u) : (256u + lane);
        const unsigned int peers = __match_any_sync(kFull, d);
        if (in && (peers & ((1u << lane) - 1)) == 0) hist[d * 32 + warp] += __popc(peers);
        __syncwarp();
      }
    }
    __syncthreads();
    // exclusive scan of hist in (digit, warp) order: 8 consecutive entries per thread
    int loc[8];
    int sum = 0;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      loc[e] = hist[threadIdx.x * 8 + e];
      sum += loc[e];
    }
    int run = block_scan(sum, warp_sums, &sh_total);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      hist[threadIdx.x * 8 + e] = run;
      run += loc[e];
    }
    __syncthreads();
    auto scatter = [&](bool in, unsigned int key, int val) {
      const unsigned int d = in ? ((key >> shift) & 255u) : (256u + lane);
      const unsigned int peers = __match_any_sync(kFull, d);
      const unsigned int before = peers & ((1u << lane) - 1);
      if (in) {
        const int dst = hist[d * 32 + warp] + __popc(before);
        kout[dst] = key;
        vout[dst] = val;
      }
      __syncwarp();
      if (in && before == 0) hist[d * 32 + warp] += __popc(peers);
      __syncwarp();
    };
    if (in_regs) {
#pragma unroll
      for (int t = 0; t < kRegIt; ++t) {
        const int base = c0 + t * 32;
        if (base < c1) scatter(base + lane < c1, kreg[t], vreg[t]);
      }
    } else {
      for (int base = c0; base < c1; base += 32) {
        const int i = base + lane;
        const bool in = i < c1;
        scatter(in, in ? kin[i] : 0u, in ? vin[i] : 0);
      }
    }
    __syncthreads();
    unsigned int* tk = kin; kin = kout; kout = tk;
    int* tv = vin; vin = vout; vout = tv;
  }
  // 4. unique rows of the sorted list (kin / vin now hold the result)
  if (threadIdx.x == 0) sh_carry = 0;
  __syncthreads();
  int* rvx = p.row_vx + static_cast<long long>(h) * p.ncap;
  int* rst = p.row_start + static_cast<long long>(h) * (p.ncap + 1);
  for (int base = 0; base < n; base += 4096) {
    const int i0 = base + threadIdx.x * 4;
    unsigned int key[4];
    int hf[4];
    int sum = 0;
    const unsigned int prev = (i0 > 0 && i0 - 1 < n) ? kin[i0 - 1] : 0u;
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const int i = i0 + t;
      key[t] = i < n ? kin[i] : 0u;
      hf[t] = 0;
      if (i < n) hf[t] = (i == 0 || key[t] != (t == 0 ? prev : key[t - 1])) ? 1 : 0;
      sum += hf[t];
    }
    int r = sh_carry + block_scan(sum, warp_sums, &sh_total);    // rows that begin before this thread's tokens
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const int i = i0 + t;
      if (i < n) {
        if (hf[t]) {
          rvx[r] = static_cast<int>(key[t]);
          rst[r] = i;
        }
        p.tok_row[static_cast<long long>(h) * p.ncap + i] = r + hf[t] - 1;
        r += hf[t];
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) sh_carry += sh_total;
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    rst[sh_carry] = n;
    p.n_rows[h] = sh_carry;
    p.n_tok[h] = n;
  }
}

// ------------------------------------------------------------------------------------ token access
template <typename T, int EPL>
struct TokenReader {
  const MergeParams& p;
  int h, lane;
  __device__ TokenReader(const MergeParams& p_, int h_, int lane_) : p(p_), h(h_), lane(lane_) {}
  // code >= 0: evicted token index; code < 0: ~index into the carried overflow list
  __device__ __forceinline__ void load_k(int code, float (&k)[EPL]) const {
    const T* base;
    if (code >= 0) {
      const int pos = p.idx ? p.idx[static_cast<long long>(h) * p.n_new + code] : code;
      base = static_cast<const T*>(p.k_src) + h * p.src_head_stride + pos * p.src_row_stride;
    } else {
      base = static_cast<const T*>(p.over_K_in) + static_cast<long long>(~code) * p.D;
    }
#pragma unroll
    for (int e = 0; e < EPL; ++e) k[e] = Elem<T>::load(base + lane * EPL + e);
  }
  __device__ __forceinline__ void load_v(int code, float (&v)[EPL]) const {
    const T* base;
    if (code >= 0) {
      const int pos = p.idx ? p.idx[static_cast<long long>(h) * p.n_new + code] : code;
      base = static_cast<const T*>(p.v_src) + h * p.src_head_stride + pos * p.src_row_stride;
    } else {
      base = static_cast<const T*>(p.over_V_in) + static_cast<long long>(~code) * p.D;
    }
#pragma unroll
    for (int e = 0; e < EPL; ++e) v[e] = Elem<T>::load(base + lane * EPL + e);
  }
  __device__ __forceinline__ float load_s(int code) const {
    if (code >= 0) {
      const int pos = p.idx ? p.idx[static_cast<long long>(h) * p.n_new + code] : code;
      return p.s_src[h * p.meta_head_stride + pos];
    }
    return p.over_S_in[~code];
  }
};

// ------------------------------------------------------------------------------------ phase A
// Eight consecutive lanes work on one token: each holds eight of its 64 values (16 bytes of a
// bf16 row, 32 of an fp32 row).
template <typename T> struct Row8;
template <> struct Row8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* row, int sub, float (&x)[8]) {
    const uint4 u = reinterpret_cast<const uint4*>(row)[sub];
    x[0] = __uint_as_float(u.x << 16); x[1] = __uint_as_float(u.x & 0xffff0000u);
    x[2] = __uint_as_float(u.y << 16); x[3] = __uint_as_float(u.y & 0xffff0000u);
    x[4] = __uint_as_float(u.z << 16); x[5] = __uint_as_float(u.z & 0xffff0000u);
    x[6] = __uint_as_float(u.w << 16); x[7] = __uint_as_float(u.w & 0xffff0000u);
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* row, int sub, const float (&x)[8]) {
    uint4 u;
    u.x = pack_bf16x2(x[0], x[1]); u.y = pack_bf16x2(x[2], x[3]);
    u.z = pack_bf16x2(x[4], x[5]); u.w = pack_bf16x2(x[6], x[7]);
    reinterpret_cast<uint4*>(row)[sub] = u;
  }
};
template <> struct Row8<float> {
  static __device__ __forceinline__ void load(const float* row, int sub, float (&x)[8]) {
    const float4 a = reinterpret_cast<const float4*>(row)[2 * sub], b = reinterpret_cast<const float4*>(row)[2 * sub + 1];
    x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
  }
  static __device__ __forceinline__ void store(float* row, int sub, const float (&x)[8]) {
    reinterpret_cast<float4*>(row)[2 * sub] = make_float4(x[0], x[1], x[2], x[3]);
    reinterpret_cast<float4*>(row)[2 * sub + 1] = make_float4(x[4], x[5], x[6], x[7]);
  }
};

// sum over the eight lanes of a group (every lane gets it; same order in every group)
__device__ __forceinline__ float group8_sum(float v, unsigned gmask) {
  v += __shfl_xor_sync(gmask, v, 4);
  v += __shfl_xor_sync(gmask, v, 2);
  v += __shfl_xor_sync(gmask, v, 1);
  return v;
}

template <typename T>
__device__ __forceinline__ const T* token_row_ptr(const MergeParams& p, int h, int code, bool want_v) {
  if (code >= 0) {
    const int pos = p.idx ? p.idx[static_cast<long long>(h) * p.n_new + code] : code;
    return static_cast<const T*>(want_v ? p.v_src : p.k_src) + h * p.src_head_stride + pos * p.src_row_stride;
  }
  return static_cast<const T*>(want_v ? p.over_V_in : p.over_K_in) + static_cast<long long>(~code) * p.D;
}

__device__ __forceinline__ float token_score(const MergeParams& p, int h, int code) {
  if (code >= 0) {
    const int pos = p.idx ? p.idx[static_cast<long long>(h) * p.n_new + code] : code;
    return p.s_src[h * p.meta_head_stride + pos];
  }
  return p.over_S_in[~code];
}

// Tokens against the pivots of their row (stac/merger.py:586-660): cosine with every pivot key
// (both L2-normalised, norms clamped at 1e-6), clamped to [-1, 1]; the first largest wins.  All
// similarities are taken against the pivots as they are BEFORE this call's merges, as the
// reference's vectorised code does.
template <typename T>
__global__ void __launch_bounds__(256) tokens_sim_kernel(const MergeParams p) {
  grid_dep_wait();   // launched with programmatic serialization behind the previous kernel of the call
  const int h = blockIdx.y;
  if (p.plan[kPlanAnyValid] == 0) return;
  const int lane = threadIdx.x & 31, sub = threadIdx.x & 7;
  const unsigned gmask = 0xffu << (lane & 24);
  const int i = static_cast<int>((static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 3);
  if (i >= p.n_tok[h]) return;
  const long long hb = static_cast<long long>(h) * p.ncap;
  const int code = (((p.passes & 1) ? p.vals_b : p.vals_a) + hb)[i];
  const int ri = p.tok_row[hb + i];
  // the sorted key is the voxel id: no token -> row -> voxel hops before the row's pivots are known.
  // (Requesting the pivot segments and keys ahead of the pivot count, all four at once, measured
  // 10 % slower for the whole merge: more registers and loads for rows that hold no pivot.)
  const int vx = static_cast<int>((((p.passes & 1) ? p.keys_b : p.keys_a) + hb)[i]);
  const long long r = static_cast<long long>(h) * p.voxel_cap + vx;
  const int npiv = p.piv_row_cnt[r];
  if (sub == 0) p.tok_score[hb + i] = token_score(p, h, code);
  if (npiv == 0) {
    if (sub == 0) {
      p.tok_sim[hb + i] = -INFINITY;
      p.tok_best[hb + i] = 0;
    }
    return;
  }
  float k[8];
  Row8<T>::load(token_row_ptr<T>(p, h, code, false), sub, k);
  float kk = 0.f;
#pragma unroll
  for (int e = 0; e < 8; ++e) kk = fmaf(k[e], k[e], kk);
  float dot[kMaxP], pp[kMaxP];
#pragma unroll
  for (int q = 0; q < kMaxP; ++q) {
    dot[q] = pp[q] = 0.f;
    if (q < npiv) {
      const int seg = p.piv_row_seg[r * p.P + q];
      float pk[8];
      Row8<T>::load(static_cast<const T*>(p.piv_K) + static_cast<long long>(seg) * p.D, sub, pk);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        dot[q] = fmaf(k[e], pk[e], dot[q]);
        pp[q] = fmaf(pk[e], pk[e], pp[q]);
      }
    }
  }
  const float den_k = fmaxf(sqrtf(group8_sum(kk, gmask)), 1e-6f);
  float best_sim = -INFINITY;
  int best = 0;
#pragma unroll
  for (int q = 0; q < kMaxP; ++q) {
    if (q < npiv) {
      const float d = group8_sum(dot[q], gmask);
      const float den_p = fmaxf(sqrtf(group8_sum(pp[q], gmask)), 1e-6f);
      const float sim = fminf(1.f, fmaxf(-1.f, __fdiv_rn(d, __fmul_rn(den_k, den_p))));
      if (sim > best_sim) {
        best_sim = sim;
        best = q;
      }
    }
  }
  if (sub == 0) {
    p.tok_sim[hb + i] = best_sim;
    p.tok_best[hb + i] = best;
    if (best_sim >= p.sim_thresh && atomicExch(&p.row_flag[hb + ri], 1) == 0)
      p.merge_list[list_push(&p.plan[kPlanMergeCount])] = make_int2(h, ri);
  }
}

// Rows with merging tokens (one warp each, lane = two of the 64 values): the tokens whose best
// similarity reaches the threshold are folded into that pivot in token order with weights
// exp(sim): K <- (W K + sum a k) / (W + sum a), same for V, W += sum a, S += sum of the (clamped)
// scores, C += count; the result is stored in the pool dtype (stac/merger.py:660-760).
template <typename T, int EPL>
__global__ void __launch_bounds__(256) rows_merge_kernel(const MergeParams p) {
  grid_dep_wait();   // launched with programmatic serialization behind the previous kernel of the call
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  if (p.plan[kPlanAnyValid] == 0) return;
  const int n = p.plan[kPlanMergeCount];
  for (int w = blockIdx.x * warps_per_block + (threadIdx.x >> 5); w < n; w += gridDim.x * warps_per_block) {
    const int2 hr = p.merge_list[w];
    const int h = hr.x, ri = hr.y;
    const long long hb = static_cast<long long>(h) * p.ncap;
    const int vx = p.row_vx[hb + ri];
    const int* rst = p.row_start + static_cast<long long>(h) * (p.ncap + 1);
    const int s0 = rst[ri], s1 = rst[ri + 1];
    const int* codes = ((p.passes & 1) ? p.vals_b : p.vals_a) + hb;
    const long long r = static_cast<long long>(h) * p.voxel_cap + vx;
    const int npiv = p.piv_row_cnt[r];
    TokenReader<T, EPL> rd(p, h, lane);
    float accK[kMaxP][EPL], accV[kMaxP][EPL], accA[kMaxP], accS[kMaxP], accC[kMaxP];
#pragma unroll
    for (int q = 0; q < kMaxP; ++q) {
      accA[q] = accS[q] = accC[q] = 0.f;
#pragma unroll
      for (int e = 0; e < EPL; ++e) accK[q][e] = accV[q][e] = 0.f;
    }
    for (int i = s0; i < s1; ++i) {
      const float sim = p.tok_sim[hb + i];
      if (!(sim >= p.sim_thresh)) continue;
      const int best = p.tok_best[hb + i];
      const int code = codes[i];
      const float a = expf(sim);
      const float s_t = fmaxf(p.tok_score[hb + i], 1e-6f);
      float k[EPL], v[EPL];
      rd.load_k(code, k);
      rd.load_v(code, v);
#pragma unroll
      for (int q = 0; q < kMaxP; ++q) {
        if (q == best) {
#pragma unroll
          for (int e = 0; e < EPL; ++e) {
            accK[q][e] = __fadd_rn(accK[q][e], __fmul_rn(a, k[e]));
            accV[q][e] = __fadd_rn(accV[q][e], __fmul_rn(a, v[e]));
          }
          accA[q] = __fadd_rn(accA[q], a);
          accS[q] = __fadd_rn(accS[q], s_t);
          accC[q] = __fadd_rn(accC[q], 1.f);
        }
      }
    }
#pragma unroll
    for (int q = 0; q < kMaxP; ++q) {
      if (q < npiv && accA[q] > 0.f) {
        const int seg = p.piv_row_seg[r * p.P + q];
        T* kb = static_cast<T*>(p.piv_K) + static_cast<long long>(seg) * p.D;
        T* vb = static_cast<T*>(p.piv_V) + static_cast<long long>(seg) * p.D;
        const float W = p.piv_W[seg];
        const float denom = fmaxf(__fadd_rn(W, accA[q]), 1e-8f);
        const float fo = __fdiv_rn(W, denom), fn = __fdiv_rn(1.0f, denom);
#pragma unroll
        for (int e = 0; e < EPL; ++e) {
          const float ko = Elem<T>::load(kb + lane * EPL + e), vo = Elem<T>::load(vb + lane * EPL + e);
          Elem<T>::store(kb + lane * EPL + e, __fadd_rn(__fmul_rn(fo, ko), __fmul_rn(fn, accK[q][e])));
          Elem<T>::store(vb + lane * EPL + e, __fadd_rn(__fmul_rn(fo, vo), __fmul_rn(fn, accV[q][e])));
        }
        if (lane == 0) {
          p.piv_W[seg] = denom;
          p.piv_S[seg] = __fadd_rn(p.piv_S[seg], accS[q]);
          p.piv_C[seg] = __fadd_rn(p.piv_C[seg], accC[q]);
        }
      }
    }
    __syncwarp();
  }
}

// Score gate of a row with pivots (after this call's merges): mean score per merged token of
// the row's pivots times score_thresh (stac/merger.py:735-745).
__device__ __forceinline__ float row_gate(const MergeParams& p, long long r, int npiv) {
  float sumS = 0.f, sumC = 0.f;
  for (int q = 0; q < npiv; ++q) {
    const int seg = p.piv_row_seg[r * p.P + q];
    sumS = __fadd_rn(sumS, p.piv_S[seg]);
    sumC = __fadd_rn(sumC, p.piv_C[seg]);
  }
  return __fmul_rn(__fdiv_rn(sumS, fmaxf(sumC, 1e-6f)), p.score_thresh);
}

// Selection and ranking of one row by one warp (rows with many tokens).  A token of a row with
// pivots is selected for the buffer if it did not come close to a pivot (sim < replace) and its
// score passes the gate; every token of a row without pivots is selected.  Candidates = buffered
// tokens (in column order) then selected tokens (in list order), ranked by (score desc,
// candidate order); rank < B = new column, the rest overflows (stac/allocator.py:559-723).
__device__ __forceinline__ void rank_row_warp(const MergeParams& p, const int h, const int ri, const int lane) {
  const long long hb = static_cast<long long>(h) * p.ncap;
  const int vx = p.row_vx[hb + ri];
  const int* rst = p.row_start + static_cast<long long>(h) * (p.ncap + 1);
  const int s0 = rst[ri], s1 = rst[ri + 1];
  const long long r = static_cast<long long>(h) * p.voxel_cap + vx;
  const int npiv = p.piv_row_cnt[r];
  const int nbuf = p.buf_row_cnt[r];
  float* tsim = p.tok_sim + hb;
  float* tscore = p.tok_score + hb;
  int* tdest = p.tok_dest + hb;
  if (npiv > 0) {
    const float gate = row_gate(p, r, npiv);
    for (int i = s0 + lane; i < s1; i += 32) {
      const bool sel = (tsim[i] < p.replace_thresh) && (fmaxf(tscore[i], 1e-6f) > gate);
      tdest[i] = sel ? 0 : -1;
    }
  } else {
    for (int i = s0 + lane; i < s1; i += 32) tdest[i] = 0;
  }
  __syncwarp();
  // ---- rank existing buffer tokens and selected tokens by (score desc, arrival order)
  float ex_s = 0.f;
  if (lane < nbuf) ex_s = p.buf_S[p.buf_row_seg[r * p.B + lane]];
  int n_sel = 0;
  for (int base = s0; base < s1; base += 32) {
    const int i = base + lane;
    const bool sel = i < s1 && tdest[i] >= 0;
    n_sel += __popc(__ballot_sync(kFull, sel));
  }
  // existing tokens
  int ex_rank = 0;
  for (int c = 0; c < nbuf; ++c) {
    const float sc = __shfl_sync(kFull, ex_s, c);
    if (lane < nbuf && (sc > ex_s || (sc == ex_s && c < lane))) ++ex_rank;
  }
  for (int base = s0; base < s1; base += 32) {
    const int i = base + lane;
    const bool sel = i < s1 && tdest[i] >= 0;
    const float sc = sel ? tscore[i] : 0.f;
    const unsigned m = __ballot_sync(kFull, sel);
    for (unsigned mm = m; mm; mm &= mm - 1) {
      const int src = __ffs(mm) - 1;
      const float s2 = __shfl_sync(kFull, sc, src);
      if (lane < nbuf && s2 > ex_s) ++ex_rank;  // tokens arrive after every existing entry
    }
  }
  int* od = p.old_dest + (hb + ri) * kMaxB;
  if (lane < nbuf) od[lane] = ex_rank;
  // selected tokens
  for (int base = s0; base < s1; base += 32) {
    const int i = base + lane;
    const bool sel = i < s1 && tdest[i] >= 0;
    const float mine = sel ? tscore[i] : 0.f;
    int rank = 0;
    for (int c = 0; c < nbuf; ++c) {
      const float sc = __shfl_sync(kFull, ex_s, c);
      if (sc >= mine) ++rank;  // existing entries win ties
    }
    if (sel) {
      for (int i2 = s0; i2 < s1; ++i2) {
        if (tdest[i2] >= 0) {
          const float s2 = tscore[i2];
          if (s2 > mine || (s2 == mine && i2 < i)) ++rank;
        }
      }
    }
    __syncwarp();
    if (sel) tdest[i] = rank;
  }
  if (lane == 0) {
    const int n_cand = nbuf + n_sel;
    const int newcnt = min(p.B, n_cand);
    const int full = (n_sel > 0 && newcnt == p.B) ? 1 : 0;
    int4 info;
    info.x = newcnt - nbuf;
    info.y = max(0, n_cand - p.B);
    info.z = full | ((full && npiv < p.P) ? 2 : 0) | (nbuf << 4);
    info.w = n_sel;
    p.row_info[hb + ri] = info;
  }
}

// The same for short rows, one thread per row; rows with more than 32 tokens are queued for the
// warp-per-row kernel.
__global__ void __launch_bounds__(256) rows_rank_kernel(const MergeParams p) {
  grid_dep_wait();   // launched with programmatic serialization behind the previous kernel of the call
  const int h = blockIdx.y;
  const int ri = blockIdx.x * blockDim.x + threadIdx.x;
  if (p.plan[kPlanAnyValid] == 0) return;
  if (ri >= p.n_rows[h]) return;
  const long long hb = static_cast<long long>(h) * p.ncap;
  const int vx = p.row_vx[hb + ri];
  const int* rst = p.row_start + static_cast<long long>(h) * (p.ncap + 1);
  const int s0 = rst[ri], s1 = rst[ri + 1];
  if (s1 - s0 > 32) {
    p.defer_list[list_push(&p.plan[kPlanDeferCount])] = make_int2(h, ri);
    return;
  }
  const long long r = static_cast<long long>(h) * p.voxel_cap + vx;
  const int npiv = p.piv_row_cnt[r];
  const int nbuf = p.buf_row_cnt[r];
  const float* tscore = p.tok_score + hb;
  int* tdest = p.tok_dest + hb;
  unsigned sel_mask = 0u;      // bit j: token s0 + j goes to the buffer
  if (npiv > 0) {
    const float gate = row_gate(p, r, npiv);
    for (int i = s0; i < s1; ++i)
      if ((p.tok_sim[hb + i] < p.replace_thresh) && (fmaxf(tscore[i], 1e-6f) > gate)) sel_mask |= 1u << (i - s0);
  } else {
    sel_mask = (s1 - s0) == 32 ? 0xffffffffu : ((1u << (s1 - s0)) - 1u);
  }
  float ex[kMaxB];
#pragma unroll
  for (int c = 0; c < kMaxB; ++c) ex[c] = (c < nbuf) ? p.buf_S[p.buf_row_seg[r * p.B + c]] : 0.f;
  const int n_sel = __popc(sel_mask);
  int* od = p.old_dest + (hb + ri) * kMaxB;
#pragma unroll
  for (int c = 0; c < kMaxB; ++c) {
    if (c < nbuf) {
      int rank = c;  // buffered tokens are stored in rank order
      for (unsigned mm = sel_mask; mm; mm &= mm - 1) rank += (tscore[s0 + __ffs(mm) - 1] > ex[c]) ? 1 : 0;
      od[c] = rank;
    }
  }
  for (int i = s0; i < s1; ++i) {
    if (!((sel_mask >> (i - s0)) & 1u)) {
      tdest[i] = -1;
      continue;
    }
    const float mine = tscore[i];
    int rank = 0;
#pragma unroll
    for (int c = 0; c < kMaxB; ++c) rank += (c < nbuf && ex[c] >= mine) ? 1 : 0;
    for (unsigned mm = sel_mask; mm; mm &= mm - 1) {
      const int i2 = s0 + __ffs(mm) - 1;
      const float s2 = tscore[i2];
      rank += (s2 > mine || (s2 == mine && i2 < i)) ? 1 : 0;
    }
    tdest[i] = rank;
  }
  const int n_cand = nbuf + n_sel;
  const int newcnt = min(p.B, n_cand);
  const int full = (n_sel > 0 && newcnt == p.B) ? 1 : 0;
  int4 info;
  info.x = newcnt - nbuf;
  info.y = max(0, n_cand - p.B);
  info.z = full | ((full && npiv < p.P) ? 2 : 0) | (nbuf << 4);
  info.w = n_sel;
  p.row_info[hb + ri] = info;
}

__global__ void __launch_bounds__(256) rows_rank_long_kernel(const MergeParams p) {
  grid_dep_wait();   // launched with programmatic serialization behind the previous kernel of the call
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const int n = p.plan[kPlanDeferCount];
  for (int w = blockIdx.x * warps_per_block + (threadIdx.x >> 5); w < n; w += gridDim.x * warps_per_block) {
    const int2 hr = p.defer_list[w];
    rank_row_warp(p, hr.x, hr.y, lane);
  }
}

// ------------------------------------------------------------------------------------ scans
// pass 0 always runs; pass 1 only when pass 0 found the pools too small and rows were trimmed
__global__ void __launch_bounds__(1024, 1) scan_heads_kernel(const MergeParams p, const int pass) {
  grid_dep_wait();   // launched with programmatic serialization behind the previous kernel of the call
  __shared__ int warp_sums[32];
  __shared__ int sh_total;
  __shared__ int carry[4];
  if (pass == 1 && p.plan[kPlanShort] == 0) return;
  const int h = blockIdx.x;
  const long long hb = static_cast<long long>(h) * p.ncap;
  const int n = p.plan[kPlanAnyValid] ? p.n_rows[h] : 0;
  if (threadIdx.x < 4) carry[threadIdx.x] = 0;
  __syncthreads();
  for (int base = 0; base < n; base += 1024) {
    const int i = base + threadIdx.x;
    int4 info = make_int4(0, 0, 0, 0);
    if (i < n) info = p.row_info[hb + i];
    int4 pref;
    const int v0 = info.x, v1 = info.y, v2 = info.z & 1, v3 = (info.z >> 1) & 1;
    pref.x = carry[0] + block_scan(v0, warp_sums, &sh_total);
    const int t0 = sh_total;
    pref.y = carry[1] + block_scan(v1, warp_sums, &sh_total);
    const int t1 = sh_total;
    pref.z = carry[2] + block_scan(v2, warp_sums, &sh_total);
    const int t2 = sh_total;
    pref.w = carry[3] + block_scan(v3, warp_sums, &sh_total);
    const int t3 = sh_total;
    if (i < n) p.row_pref[hb + i] = pref;
    __syncthreads();
    if (threadIdx.x == 0) {
      carry[0] += t0; carry[1] += t1; carry[2] += t2; carry[3] += t3;
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) p.head_tot[h] = make_int4(carry[0], carry[1], carry[2], carry[3]);
}

__global__ void __launch_bounds__(1024, 1) scan_plan_kernel(const MergeParams p, const int pass) {
  grid_dep_wait();   // launched with programmatic serialization behind the previous kernel of the call
  __shared__ int warp_sums[32];
  __shared__ int sh_total;
  __shared__ int carry[4];
  if (pass == 1 && p.plan[kPlanShort] == 0) return;
  if (threadIdx.x < 4) carry[threadIdx.x] = 0;
  __syncthreads();
  for (int base = 0; base < p.heads; base += 1024) {
    const int h = base + threadIdx.x;
    int4 t = make_int4(0, 0, 0, 0);
    if (h < p.heads) t = p.head_tot[h];
    int4 b;
    b.x = carry[0] + block_scan(t.x, warp_sums, &sh_total);
    const int t0 = sh_total;
    b.y = carry[1] + block_scan(t.y, warp_sums, &sh_total);
    const int t1 = sh_total;
    b.z = carry[2] + block_scan(t.z, warp_sums, &sh_total);
    const int t2 = sh_total;
    b.w = carry[3] + block_scan(t.w, warp_sums, &sh_total);
    const int t3 = sh_total;
    if (h < p.heads) {
      p.head_base[h] = b;
      p.over_start_out[h] = b.y;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      carry[0] += t0; carry[1] += t1; carry[2] += t2; carry[3] += t3;
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    if (pass == 0 && p.voxel_count != nullptr) p.meta[STAC_META_VOXELS] = max(p.meta[STAC_META_VOXELS], *p.voxel_count);
    const int any = p.plan[kPlanAnyValid];
    const int total_add = carry[0], total_over = carry[1], total_full = carry[2], total_piv = carry[3];
    const int free_len = p.meta[STAC_META_BUF_FREE_LEN];
    const int buf_top = p.meta[STAC_META_BUF_TOP];
    const int piv_top = p.meta[STAC_META_PIV_TOP];
    const int k = min(total_add, free_len);
    p.plan[kPlanK] = k;
    p.plan[kPlanFreeLen] = free_len;
    p.plan[kPlanBufTop] = buf_top;
    p.plan[kPlanPivTop] = piv_top;
    p.plan[kPlanTotalAdd] = total_add;
    p.plan[kPlanTotalFull] = total_full;
    p.plan[kPlanTotalOver] = total_over;
    int abort = 0;
    if (any) {
      const int avail_buf = free_len + (p.buf_cap - buf_top);
      const int avail_piv = p.piv_cap - piv_top;
      if (pass == 0 && (total_add > avail_buf || total_piv > avail_piv)) {
        // The pools are bounded and this call does not fit: rows are trimmed in (head, voxel)
        // order by trim_rows_kernel and the plan is recomputed by pass 1.
        p.plan[kPlanShort] = 1;
        p.plan[kPlanAvailBuf] = avail_buf;
        p.plan[kPlanAvailPiv] = avail_piv;
        return;
      }
      if (buf_top + (total_add - k) > p.buf_cap || piv_top + total_piv > p.piv_cap || total_over > p.over_cap ||
          free_len - k + total_full * p.B > p.buf_cap)
        abort = 1;
    }
    p.plan[kPlanAbort] = abort;
    if (abort) report_error(p.err, DEV_POOL_CAPACITY);
    if (any && !abort) {
      p.over_start_out[p.heads] = total_over;
      p.meta[STAC_META_BUF_TOP] = buf_top + (total_add - k);
      p.meta[STAC_META_PIV_TOP] = piv_top + total_piv;
      p.meta[STAC_META_OVER_COUNT] = total_over;
      p.meta[STAC_META_BUF_FREE_LEN] = free_len - k + total_full * p.B;
      p.meta[STAC_META_BUF_USED] += total_add - total_full * p.B;
      p.meta[STAC_META_PIV_USED] += total_piv;
    }
  }
}

// ------------------------------------------------------------------------------------ phase B
// Bounded pools: a row that would open new buffer columns, or need a new pivot segment, beyond
// what is left is skipped as a whole (its selected tokens are dropped, the row stays as it
// was).  The cut follows the allocation order, i.e. (head, voxel) ascending, so it is
// deterministic; merges into existing pivots done in phase A stay.
__global__ void __launch_bounds__(256) trim_rows_kernel(const MergeParams p) {
  grid_dep_wait();   // launched with programmatic serialization behind the previous kernel of the call
  const int h = blockIdx.y;
  const int ri = blockIdx.x * blockDim.x + threadIdx.x;
  if (p.plan[kPlanAnyValid] == 0 || p.plan[kPlanShort] == 0) return;
  if (ri >= p.n_rows[h]) return;
  const long long hb = static_cast<long long>(h) * p.ncap;
  const int4 info = p.row_info[hb + ri];
  if (info.w == 0) return;
  const int4 pref = p.row_pref[hb + ri];
  const int4 hbase = p.head_base[h];
  const bool no_buf = info.x > 0 && hbase.x + pref.x + info.x > p.plan[kPlanAvailBuf];
  const bool no_piv = (info.z & 2) && hbase.w + pref.w + 1 > p.plan[kPlanAvailPiv];
  if (!no_buf && !no_piv) return;
  const int* rst = p.row_start + static_cast<long long>(h) * (p.ncap + 1);
  int dropped = 0;
  for (int i = rst[ri]; i < rst[ri + 1]; ++i) {
    if (p.tok_dest[hb + i] >= 0) {
      p.tok_dest[hb + i] = -1;
      ++dropped;
    }
  }
  p.row_info[hb + ri] = make_int4(0, 0, info.z & ~3, 0);
  atomicAdd(&p.meta[STAC_META_DROPPED], dropped);
}

// Phase B, step 1 (one thread per row): hand out the segment ids of the new columns in
// (row, column) order from the allocation plan, publish the new occupancy, and queue the rows
// whose buffered tokens change column or whose buffer filled up.
__global__ void __launch_bounds__(256) rows_phase_b1a_kernel(const MergeParams p) {
  grid_dep_wait();   // launched with programmatic serialization behind the previous kernel of the call
  const int h = blockIdx.y;
  const int ri = blockIdx.x * blockDim.x + threadIdx.x;
  if (p.plan[kPlanAnyValid] == 0 || p.plan[kPlanAbort] != 0) return;
  if (ri >= p.n_rows[h]) return;
  const long long hb = static_cast<long long>(h) * p.ncap;
  const int4 info = p.row_info[hb + ri];
  if (info.w == 0) return;  // nothing selected: the buffer is untouched
  const int vx = p.row_vx[hb + ri];
  const long long r = static_cast<long long>(h) * p.voxel_cap + vx;
  const int add_off = p.head_base[h].x + p.row_pref[hb + ri].x;
  const int nbuf = info.z >> 4;
  const int newcnt = nbuf + info.x;
  const int k_take = p.plan[kPlanK], free_len = p.plan[kPlanFreeLen], buf_top = p.plan[kPlanBufTop];
  for (int col = nbuf; col < newcnt; ++col) {
    const int q = add_off + (col - nbuf);
    p.buf_row_seg[r * p.B + col] = q < k_take ? p.buf_free[free_len - k_take + q] : buf_top + (q - k_take);
  }
  const int* od = p.old_dest + (hb + ri) * kMaxB;
  bool moves = false;
  for (int c = 0; c < nbuf; ++c) moves = moves || (od[c] != c);
  if (moves) p.move_list[list_push(&p.plan[kPlanMoveCount])] = make_int2(h, ri);
  if (info.z & 1) p.full_list[list_push(&p.plan[kPlanFullCount])] = make_int2(h, ri);
  else p.buf_row_cnt[r] = newcnt;
}

// Phase B, step 2 (one warp per queued row): buffered tokens only ever move to a higher column
// (new tokens push them down the ranking), so walking them from the last column to the first
// moves each one into a slot whose old content has already left.
template <typename T, int EPL>
__global__ void __launch_bounds__(256) rows_phase_b1m_kernel(const MergeParams p) {
  grid_dep_wait();   // launched with programmatic serialization behind the previous kernel of the call
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  if (p.plan[kPlanAnyValid] == 0 || p.plan[kPlanAbort] != 0) return;
  const int n_move = p.plan[kPlanMoveCount];
  const int B = p.B, D = p.D;
  T* bK = static_cast<T*>(p.buf_K);
  T* bV = static_cast<T*>(p.buf_V);
  T* oK = static_cast<T*>(p.over_K_out);
  T* oV = static_cast<T*>(p.over_V_out);
  for (int wi = blockIdx.x * warps_per_block + (threadIdx.x >> 5); wi < n_move; wi += gridDim.x * warps_per_block) {
    const int2 hr = p.move_list[wi];
    const int h = hr.x, ri = hr.y;
    const long long hb = static_cast<long long>(h) * p.ncap;
    const int4 info = p.row_info[hb + ri];
    const int vx = p.row_vx[hb + ri];
    const long long r = static_cast<long long>(h) * p.voxel_cap + vx;
    const int over_off = p.head_base[h].y + p.row_pref[hb + ri].y;
    const int nbuf = info.z >> 4;
    const int newcnt = nbuf + info.x;
    const int* od = p.old_dest + (hb + ri) * kMaxB;
    int my_seg = -1, ex_dest = -1;
    if (lane < newcnt) my_seg = p.buf_row_seg[r * B + lane];
    if (lane < nbuf) ex_dest = od[lane];
    for (int c = nbuf - 1; c >= 0; --c) {
      const int d = __shfl_sync(kFull, ex_dest, c);
      if (d == c) continue;
      const int sg = __shfl_sync(kFull, my_seg, c);
      float k[EPL], v[EPL];
#pragma unroll
      for (int e = 0; e < EPL; ++e) {
        k[e] = Elem<T>::load(bK + static_cast<long long>(sg) * D + lane * EPL + e);
        v[e] = Elem<T>::load(bV + static_cast<long long>(sg) * D + lane * EPL + e);
      }
      const float sc = p.buf_S[sg];
      __syncwarp();
      if (d < B) {
        const int dg = __shfl_sync(kFull, my_seg, d);
#pragma unroll
        for (int e = 0; e < EPL; ++e) {
          Elem<T>::store(bK + static_cast<long long>(dg) * D + lane * EPL + e, k[e]);
          Elem<T>::store(bV + static_cast<long long>(dg) * D + lane * EPL + e, v[e]);
        }
        if (lane == 0) p.buf_S[dg] = sc;
      } else {
        const long long o = over_off + (d - B);
#pragma unroll
        for (int e = 0; e < EPL; ++e) {
          Elem<T>::store(oK + o * D + lane * EPL + e, k[e]);
          Elem<T>::store(oV + o * D + lane * EPL + e, v[e]);
        }
        if (lane == 0) {
          p.over_S_out[o] = sc;
          p.over_hv_out[2 * o] = h;
          p.over_hv_out[2 * o + 1] = vx;
        }
      }
      __syncwarp();
    }
  }
}

// Phase B, step 3 (token-parallel): every selected token is copied to its column's segment or
// to its overflow slot; eight lanes per token, each moving 16 (bf16) or 32 (fp32) bytes of K and
// of V, all four loads in flight before the stores.
template <typename T>
__global__ void __launch_bounds__(256) tokens_place_kernel(const MergeParams p) {
  grid_dep_wait();   // launched with programmatic serialization behind the previous kernel of the call
  constexpr int kVec = static_cast<int>(sizeof(T)) * 8 / 16;   // 16-byte vectors per lane and row
  const int h = blockIdx.y;
  const int sub = threadIdx.x & 7;
  const int i = static_cast<int>((static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 3);
  if (p.plan[kPlanAnyValid] == 0 || p.plan[kPlanAbort] != 0) return;
  if (i >= p.n_tok[h]) return;
  const long long hb = static_cast<long long>(h) * p.ncap;
  // independent loads first (the sorted key is the voxel id), then the branch
  const int d = p.tok_dest[hb + i];
  const int ri = p.tok_row[hb + i];
  const int code = (((p.passes & 1) ? p.vals_b : p.vals_a) + hb)[i];
  const int vx = static_cast<int>((((p.passes & 1) ? p.keys_b : p.keys_a) + hb)[i]);
  if (d < 0) return;
  const uint4* src_k = reinterpret_cast<const uint4*>(token_row_ptr<T>(p, h, code, false)) + sub * kVec;
  const uint4* src_v = reinterpret_cast<const uint4*>(token_row_ptr<T>(p, h, code, true)) + sub * kVec;
  uint4 kv[kVec], vv[kVec];
#pragma unroll
  for (int j = 0; j < kVec; ++j) {
    kv[j] = src_k[j];
    vv[j] = src_v[j];
  }
  const float sc = p.tok_score[hb + i];
  T* dst_k;
  T* dst_v;
  if (d < p.B) {
    const long long r = static_cast<long long>(h) * p.voxel_cap + vx;
    const int sg = p.buf_row_seg[r * p.B + d];
    dst_k = static_cast<T*>(p.buf_K) + static_cast<long long>(sg) * p.D;
    dst_v = static_cast<T*>(p.buf_V) + static_cast<long long>(sg) * p.D;
    if (sub == 0) p.buf_S[sg] = sc;
  } else {
    const long long o = p.head_base[h].y + p.row_pref[hb + ri].y + (d - p.B);
    dst_k = static_cast<T*>(p.over_K_out) + o * p.D;
    dst_v = static_cast<T*>(p.over_V_out) + o * p.D;
    if (sub == 0) {
      p.over_S_out[o] = sc;
      p.over_hv_out[2 * o] = h;
      p.over_hv_out[2 * o + 1] = vx;
    }
  }
#pragma unroll
  for (int j = 0; j < kVec; ++j) {
    reinterpret_cast<uint4*>(dst_k)[sub * kVec + j] = kv[j];
    reinterpret_cast<uint4*>(dst_v)[sub * kVec + j] = vv[j];
  }
}

// Full buffers -> one pivot each, inserted into the row's pivot slots; the buffer row is released.
// Eight lanes per row, each holding eight of the 64 values of a token (16-byte loads), so a warp
// works on four rows at once.  Tokens are streamed (keys twice: once for the weights, once for
// the weighted mean; the second read hits the cache) so that few registers are live and many
// rows are in flight per SM.
template <typename T>
// (holding all eight key rows of a row in registers, at four CTAs per SM, measured 15 % slower for
// the whole merge than streaming them at eight CTAs per SM: these per-row kernels want threads)
__global__ void __launch_bounds__(128, 8) rows_phase_b2_kernel(const MergeParams p) {
  grid_dep_wait();   // launched with programmatic serialization behind the previous kernel of the call
  const int lane = threadIdx.x & 31, sub = threadIdx.x & 7;
  const int gbase = lane & 24;                       // first lane of this group
  const unsigned gmask = 0xffu << gbase;
  if (p.plan[kPlanAnyValid] == 0 || p.plan[kPlanAbort] != 0) return;
  const int n_full = p.plan[kPlanFullCount];
  const int groups = (gridDim.x * blockDim.x) >> 3;
  for (int wi = (blockIdx.x * blockDim.x + threadIdx.x) >> 3; wi < n_full; wi += groups) {
    const int2 hr = p.full_list[wi];
    const int h = hr.x, ri = hr.y;
    const long long hb = static_cast<long long>(h) * p.ncap;
    const int vx = p.row_vx[hb + ri];
    const long long r = static_cast<long long>(h) * p.voxel_cap + vx;
    const int4 pref = p.row_pref[hb + ri];
    const int4 hbase = p.head_base[h];
    const int full_off = hbase.z + pref.z, piv_off = hbase.w + pref.w;
    const int B = p.B, D = p.D;
    const T* bK = static_cast<const T*>(p.buf_K);
    const T* bV = static_cast<const T*>(p.buf_V);
    int my_seg = -1;
    if (sub < B) my_seg = p.buf_row_seg[r * B + sub];
    // ---- the buffer is full: B tokens -> one pivot (stac/merger.py:408-461)
    float ts = 0.f;
    if (sub < B) ts = fmaxf(p.buf_S[my_seg], 1e-6f);
    int seed = 0;
    float seed_s = -INFINITY, sumS = 0.f;
    for (int c = 0; c < B; ++c) {
      const float sc = __shfl_sync(gmask, ts, gbase + c);
      if (sc > seed_s) {
        seed_s = sc;
        seed = c;
      }
      sumS = __fadd_rn(sumS, sc);
    }
    float kn_seed[8];
    {
      const int sg = __shfl_sync(gmask, my_seg, gbase + seed);
      float k[8];
      Row8<T>::load(bK + static_cast<long long>(sg) * D, sub, k);
      float ss = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += k[e] * k[e];
      const float den = fmaxf(sqrtf(group8_sum(ss, gmask)), 1e-6f);
#pragma unroll
      for (int e = 0; e < 8; ++e) kn_seed[e] = __fdiv_rn(k[e], den);
    }
    // pass 1 over the keys: w_c = exp(cos(k_c, seed))
    float w[kMaxB];
    float Wsum = 0.f;
#pragma unroll
    for (int c = 0; c < kMaxB; ++c) {
      w[c] = 0.f;
      if (c < B) {
        const int sg = __shfl_sync(gmask, my_seg, gbase + c);
        float k[8];
        Row8<T>::load(bK + static_cast<long long>(sg) * D, sub, k);
        float ss = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) ss += k[e] * k[e];
        const float den = fmaxf(sqrtf(group8_sum(ss, gmask)), 1e-6f);
        float d = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) d += __fdiv_rn(k[e], den) * kn_seed[e];
        d = fminf(1.f, fmaxf(-1.f, group8_sum(d, gmask)));
        w[c] = expf(d);
        Wsum = __fadd_rn(Wsum, w[c]);
      }
    }
    // pass 2: the weighted means of keys and values
    float nk[8], nv[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) nk[e] = nv[e] = 0.f;
    const float wden = __fadd_rn(Wsum, 1e-8f);
#pragma unroll
    for (int c = 0; c < kMaxB; ++c) {
      if (c < B) {
        const float cn = __fdiv_rn(w[c], wden);
        const int sg = __shfl_sync(gmask, my_seg, gbase + c);
        float tk[8], tv[8];
        Row8<T>::load(bK + static_cast<long long>(sg) * D, sub, tk);
        Row8<T>::load(bV + static_cast<long long>(sg) * D, sub, tv);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          nk[e] = __fadd_rn(nk[e], __fmul_rn(cn, tk[e]));
          nv[e] = __fadd_rn(nv[e], __fmul_rn(cn, tv[e]));
        }
      }
    }
    // ---- insert the pivot (stac/merger.py:462-582)
    T* pK = static_cast<T*>(p.piv_K);
    T* pV = static_cast<T*>(p.piv_V);
    const int npiv = p.piv_row_cnt[r];
    int pseg;
    if (npiv < p.P) {
      pseg = p.plan[kPlanPivTop] + piv_off;
      if (sub == 0) {
        p.piv_row_seg[r * p.P + npiv] = pseg;
        p.piv_row_cnt[r] = npiv + 1;
      }
    } else {
      // saturated: fold the lowest-weight pivot into its most similar neighbour, reuse its slot
      int ps_l = -1;                  // lane q < P holds segment and weight of pivot q
      float pw_l = INFINITY;
      if (sub < p.P) {
        ps_l = p.piv_row_seg[r * p.P + sub];
        pw_l = p.piv_W[ps_l];
      }
      int victim = 0;
      float wmin = INFINITY;
      for (int q = 0; q < p.P; ++q) {
        const float wq = __shfl_sync(gmask, pw_l, gbase + q);
        if (wq < wmin) {
          wmin = wq;
          victim = q;
        }
      }
      // keys normalised in the pool dtype, as the reference does here (stac/merger.py:493-495)
      auto load_normalised = [&](int seg, float (&out)[8]) {
        float pk[8];
        Row8<T>::load(pK + static_cast<long long>(seg) * D, sub, pk);
        float ss = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) ss += pk[e] * pk[e];
        float nrm = Elem<T>::round(sqrtf(group8_sum(ss, gmask)));
        nrm = fmaxf(nrm, Elem<T>::round(1e-6f));
#pragma unroll
        for (int e = 0; e < 8; ++e) out[e] = Elem<T>::round(__fdiv_rn(pk[e], nrm));
      };
      const int vseg = __shfl_sync(gmask, ps_l, gbase + victim);
      const float Wv = __shfl_sync(gmask, pw_l, gbase + victim);
      float vn[8];
      load_normalised(vseg, vn);
      int nb = 0;
      float best = -INFINITY;
      for (int q = 0; q < p.P; ++q) {
        if (q == victim) continue;
        const int qseg = __shfl_sync(gmask, ps_l, gbase + q);
        float pkn[8];
        load_normalised(qseg, pkn);
        float d = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) d += pkn[e] * vn[e];
        d = Elem<T>::round(group8_sum(d, gmask));
        if (d > best) {
          best = d;
          nb = q;
        }
      }
      if (p.P == 1) nb = victim;   // no neighbour to fold into: the victim is simply replaced
      float scale;
      if (Elem<T>::kIsBf16) scale = Elem<T>::round(expf(Elem<T>::round(best - 1.0f)));
      else scale = expf(best - 1.0f);
      const int nseg = __shfl_sync(gmask, ps_l, gbase + nb);
      const float Wn = __shfl_sync(gmask, pw_l, gbase + nb);
      if (p.P > 1) {
        const float Wj = __fmul_rn(Wv, scale);
        const float denom = fmaxf(__fadd_rn(Wj, Wn), 1e-8f);
        const float fj = __fdiv_rn(Wj, denom), fk = __fdiv_rn(Wn, denom);
        float a[8], b[8];
        Row8<T>::load(pK + static_cast<long long>(vseg) * D, sub, a);
        Row8<T>::load(pK + static_cast<long long>(nseg) * D, sub, b);
#pragma unroll
        for (int e = 0; e < 8; ++e) b[e] = __fadd_rn(__fmul_rn(fj, a[e]), __fmul_rn(fk, b[e]));
        Row8<T>::store(pK + static_cast<long long>(nseg) * D, sub, b);
        Row8<T>::load(pV + static_cast<long long>(vseg) * D, sub, a);
        Row8<T>::load(pV + static_cast<long long>(nseg) * D, sub, b);
#pragma unroll
        for (int e = 0; e < 8; ++e) b[e] = __fadd_rn(__fmul_rn(fj, a[e]), __fmul_rn(fk, b[e]));
        Row8<T>::store(pV + static_cast<long long>(nseg) * D, sub, b);
        if (sub == 0) {
          p.piv_W[nseg] = denom;
          p.piv_S[nseg] = __fadd_rn(p.piv_S[vseg], p.piv_S[nseg]);
          p.piv_C[nseg] = __fadd_rn(p.piv_C[vseg], p.piv_C[nseg]);
        }
      }
      pseg = vseg;
    }
    Row8<T>::store(pK + static_cast<long long>(pseg) * D, sub, nk);
    Row8<T>::store(pV + static_cast<long long>(pseg) * D, sub, nv);
    if (sub == 0) {
      p.piv_W[pseg] = Wsum;
      p.piv_S[pseg] = sumS;
      p.piv_C[pseg] = static_cast<float>(B);
    }
    // ---- release the buffer row: segment ids go to the staging area in column order
    if (sub < B) {
      p.free_stage[full_off * B + sub] = my_seg;
      p.buf_row_seg[r * B + sub] = -1;
    }
    if (sub == 0) p.buf_row_cnt[r] = 0;
  }
}

// Freed ids are appended after the part of the free list that was not handed out.
__global__ void finalize_kernel(const MergeParams p) {
  grid_dep_wait();   // launched with programmatic serialization behind the previous kernel of the call
  if (p.plan[kPlanAnyValid] == 0 || p.plan[kPlanAbort] != 0) return;
  const int n_freed = p.plan[kPlanTotalFull] * p.B;
  const int base = p.plan[kPlanFreeLen] - p.plan[kPlanK];
  const int stride = gridDim.x * blockDim.x;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n_freed; i += stride) p.buf_free[base + i] = p.free_stage[i];
}

// No valid evicted token in the whole call: the reference returns before touching the
// carried overflow (stac/merger.py:1203-1208), so the list is carried over unchanged.
template <typename T>
__global__ void carry_overflow_kernel(const MergeParams p) {
  grid_dep_wait();   // launched with programmatic serialization behind the previous kernel of the call
  if (p.plan[kPlanAnyValid] != 0 && p.plan[kPlanAbort] == 0) return;
  const int n = p.over_start_in[p.heads];
  const long long total = static_cast<long long>(n) * p.D;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    static_cast<T*>(p.over_K_out)[i] = static_cast<const T*>(p.over_K_in)[i];
    static_cast<T*>(p.over_V_out)[i] = static_cast<const T*>(p.over_V_in)[i];
  }
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    p.over_S_out[i] = p.over_S_in[i];
    p.over_hv_out[2 * i] = p.over_hv_in[2 * i];
    p.over_hv_out[2 * i + 1] = p.over_hv_in[2 * i + 1];
  }
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i <= p.heads; i += stride)
    p.over_start_out[i] = p.over_start_in[i];
}

size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

struct ScratchLayout {
  size_t keys_a, keys_b, vals_a, vals_b, n_tok, n_rows, row_vx, row_start, row_info, row_pref, old_dest, tok_dest,
      tok_sim, tok_score, head_tot, head_base, plan, free_stage, defer_list, full_list, move_list, tok_row, tok_best, row_flag, merge_list, total;
};

ScratchLayout scratch_layout(int heads, int ncap, int buf_cap) {
  ScratchLayout L;
  size_t off = 0;
  const size_t hn = static_cast<size_t>(heads) * ncap;
  auto take = [&](size_t bytes) {
    const size_t o = off;
    off = align_up(off + bytes, 256);
    return o;
  };
  L.keys_a = take(hn * 4); L.keys_b = take(hn * 4); L.vals_a = take(hn * 4); L.vals_b = take(hn * 4);
  L.n_tok = take(static_cast<size_t>(heads) * 4); L.n_rows = take(static_cast<size_t>(heads) * 4);
  L.row_vx = take(hn * 4); L.row_start = take(static_cast<size_t>(heads) * (ncap + 1) * 4);
  L.row_info = take(hn * 16); L.row_pref = take(hn * 16); L.old_dest = take(hn * kMaxB * 4);
  L.tok_dest = take(hn * 4); L.tok_sim = take(hn * 4); L.tok_score = take(hn * 4);
  L.head_tot = take(static_cast<size_t>(heads) * 16); L.head_base = take(static_cast<size_t>(heads) * 16);
  L.plan = take(kPlanSize * 4); L.free_stage = take(static_cast<size_t>(buf_cap) * 4);
  L.defer_list = take(hn * 8); L.full_list = take(hn * 8);
  L.move_list = take(hn * 8); L.tok_row = take(hn * 4);
  L.tok_best = take(hn * 4); L.row_flag = take(hn * 4); L.merge_list = take(hn * 8);
  L.total = off;
  return L;
}

template <typename T>
int launch_merge(MergeParams& mp, cudaStream_t st) {
  if (cudaMemsetAsync(mp.plan, 0, kPlanSize * 4, st) != cudaSuccess) return STAC_ERR_CUDA;
  if (cudaMemsetAsync(mp.row_flag, 0, static_cast<size_t>(mp.heads) * mp.ncap * 4, st) != cudaSuccess) return STAC_ERR_CUDA;
  if (launch_behind(sort_tokens_kernel, dim3(mp.heads), dim3(1024), 0, st, mp) != cudaSuccess) return STAC_ERR_CUDA;
  const int warps = 8;
  dim3 grid_rows((mp.ncap + warps - 1) / warps, mp.heads);
  dim3 grid_a1((mp.ncap + 255) / 256, mp.heads);
  dim3 grid_sim(static_cast<unsigned>((static_cast<long long>(mp.ncap) * 8 + 255) / 256), mp.heads);
  if (launch_behind(tokens_sim_kernel<T>, dim3(grid_sim), dim3(256), 0, st, mp) != cudaSuccess) return STAC_ERR_CUDA;
  if (launch_behind(rows_merge_kernel<T, 2>, dim3(148 * 4), dim3(256), 0, st, mp) != cudaSuccess) return STAC_ERR_CUDA;
  if (launch_behind(rows_rank_kernel, dim3(grid_a1), dim3(256), 0, st, mp) != cudaSuccess) return STAC_ERR_CUDA;
  if (launch_behind(rows_rank_long_kernel, dim3(148 * 4), dim3(256), 0, st, mp) != cudaSuccess) return STAC_ERR_CUDA;
  if (launch_behind(scan_heads_kernel, dim3(mp.heads), dim3(1024), 0, st, mp, 0) != cudaSuccess) return STAC_ERR_CUDA;
  if (launch_behind(scan_plan_kernel, dim3(1), dim3(1024), 0, st, mp, 0) != cudaSuccess) return STAC_ERR_CUDA;
  if (launch_behind(trim_rows_kernel, dim3(grid_a1), dim3(256), 0, st, mp) != cudaSuccess) return STAC_ERR_CUDA;
  if (launch_behind(scan_heads_kernel, dim3(mp.heads), dim3(1024), 0, st, mp, 1) != cudaSuccess) return STAC_ERR_CUDA;
  if (launch_behind(scan_plan_kernel, dim3(1), dim3(1024), 0, st, mp, 1) != cudaSuccess) return STAC_ERR_CUDA;
  if (launch_behind(rows_phase_b1a_kernel, dim3(grid_a1), dim3(256), 0, st, mp) != cudaSuccess) return STAC_ERR_CUDA;
  if (launch_behind(rows_phase_b1m_kernel<T, 2>, dim3(148 * 6), dim3(256), 0, st, mp) != cudaSuccess) return STAC_ERR_CUDA;
  if (launch_behind(tokens_place_kernel<T>, dim3(grid_sim), dim3(256), 0, st, mp) != cudaSuccess) return STAC_ERR_CUDA;
  if (launch_behind(rows_phase_b2_kernel<T>, dim3(148 * 16), dim3(128), 0, st, mp) != cudaSuccess) return STAC_ERR_CUDA;
  if (launch_behind(finalize_kernel, dim3(148 * 4), dim3(256), 0, st, mp) != cudaSuccess) return STAC_ERR_CUDA;   // grid-stride over the freed ids (known on the device only)
  if (launch_behind(carry_overflow_kernel<T>, dim3(148), dim3(256), 0, st, mp) != cudaSuccess) return STAC_ERR_CUDA;
  return cudaGetLastError() == cudaSuccess ? STAC_OK : STAC_ERR_CUDA;
}

}  // namespace
}  // namespace stac

extern "C" {

size_t stac_merge_scratch_bytes(int heads, int tokens_per_head, int buf_cap) {
  if (heads <= 0 || tokens_per_head <= 0 || buf_cap < 0) return 0;
  return stac::scratch_layout(heads, tokens_per_head, buf_cap).total;
}

int stac_merge_insert(const stac_pool* pool, const stac_evicted* ev, void* scratch, size_t scratch_bytes,
                      int list_cap_per_head, int* dev_status, stac_stream_t stream) {
  if (pool == nullptr || ev == nullptr || scratch == nullptr) return STAC_ERR_BAD_ARG;
  if (pool->head_dim != 64 || (pool->elem_bytes != 2 && pool->elem_bytes != 4)) return STAC_ERR_BAD_ARG;
  if (pool->pivot_cap < 1 || pool->pivot_cap > stac::kMaxP || pool->budget_cap < 1 ||
      pool->budget_cap > stac::kMaxB)
    return STAC_ERR_BAD_ARG;
  if (pool->heads <= 0 || pool->voxel_cap <= 0 || pool->voxel_used < 0 || pool->voxel_used > pool->voxel_cap)
    return STAC_ERR_BAD_ARG;
  if (ev->tokens_per_head <= 0 || list_cap_per_head < ev->tokens_per_head || list_cap_per_head > STAC_MERGE_MAX_LIST)
    return STAC_ERR_BAD_ARG;
  const stac::ScratchLayout L = stac::scratch_layout(pool->heads, list_cap_per_head, pool->buf_cap);
  if (scratch_bytes < L.total) return STAC_ERR_CAPACITY;
  stac::MergeParams mp;
  mp.heads = pool->heads; mp.D = pool->head_dim; mp.P = pool->pivot_cap; mp.B = pool->budget_cap;
  mp.voxel_cap = pool->voxel_cap; mp.voxel_used = pool->voxel_used;
  mp.sim_thresh = pool->sim_thresh; mp.replace_thresh = pool->replace_thresh; mp.score_thresh = pool->score_thresh;
  mp.k_src = ev->k; mp.v_src = ev->v; mp.s_src = ev->scores; mp.vx_src = ev->voxel_ids; mp.idx = ev->positions;
  mp.src_head_stride = ev->kv_head_stride; mp.src_row_stride = ev->kv_row_stride;
  mp.meta_head_stride = ev->meta_head_stride; mp.n_new = ev->tokens_per_head;
  mp.buf_K = pool->buf_K; mp.buf_V = pool->buf_V; mp.buf_S = pool->buf_S;
  mp.buf_row_seg = pool->buf_row_seg; mp.buf_row_cnt = pool->buf_row_cnt; mp.buf_free = pool->buf_free;
  mp.buf_cap = pool->buf_cap;
  mp.piv_K = pool->piv_K; mp.piv_V = pool->piv_V; mp.piv_W = pool->piv_W; mp.piv_S = pool->piv_S;
  mp.piv_C = pool->piv_C; mp.piv_row_seg = pool->piv_row_seg; mp.piv_row_cnt = pool->piv_row_cnt;
  mp.piv_cap = pool->piv_cap;
  mp.over_K_in = pool->over_K_in; mp.over_V_in = pool->over_V_in; mp.over_S_in = pool->over_S_in;
  mp.over_hv_in = pool->over_hv_in; mp.over_start_in = pool->over_start_in;
  mp.over_K_out = pool->over_K_out; mp.over_V_out = pool->over_V_out; mp.over_S_out = pool->over_S_out;
  mp.over_hv_out = pool->over_hv_out; mp.over_start_out = pool->over_start_out; mp.over_cap = pool->over_cap;
  mp.meta = pool->meta;
  mp.voxel_count = pool->voxel_count;
  mp.ncap = list_cap_per_head;
  char* base = static_cast<char*>(scratch);
  mp.keys_a = reinterpret_cast<unsigned int*>(base + L.keys_a);
  mp.keys_b = reinterpret_cast<unsigned int*>(base + L.keys_b);
  mp.vals_a = reinterpret_cast<int*>(base + L.vals_a);
  mp.vals_b = reinterpret_cast<int*>(base + L.vals_b);
  mp.n_tok = reinterpret_cast<int*>(base + L.n_tok);
  mp.n_rows = reinterpret_cast<int*>(base + L.n_rows);
  mp.row_vx = reinterpret_cast<int*>(base + L.row_vx);
  mp.row_start = reinterpret_cast<int*>(base + L.row_start);
  mp.row_info = reinterpret_cast<int4*>(base + L.row_info);
  mp.row_pref = reinterpret_cast<int4*>(base + L.row_pref);
  mp.old_dest = reinterpret_cast<int*>(base + L.old_dest);
  mp.tok_dest = reinterpret_cast<int*>(base + L.tok_dest);
  mp.tok_sim = reinterpret_cast<float*>(base + L.tok_sim);
  mp.tok_score = reinterpret_cast<float*>(base + L.tok_score);
  mp.head_tot = reinterpret_cast<int4*>(base + L.head_tot);
  mp.head_base = reinterpret_cast<int4*>(base + L.head_base);
  mp.plan = reinterpret_cast<int*>(base + L.plan);
  mp.free_stage = reinterpret_cast<int*>(base + L.free_stage);
  mp.defer_list = reinterpret_cast<int2*>(base + L.defer_list);
  mp.full_list = reinterpret_cast<int2*>(base + L.full_list);
  mp.move_list = reinterpret_cast<int2*>(base + L.move_list);
  mp.tok_row = reinterpret_cast<int*>(base + L.tok_row);
  mp.tok_best = reinterpret_cast<int*>(base + L.tok_best);
  mp.row_flag = reinterpret_cast<int*>(base + L.row_flag);
  mp.merge_list = reinterpret_cast<int2*>(base + L.merge_list);
  int bits = 1;
  while ((1ll << bits) < pool->voxel_used) ++bits;
  mp.passes = (bits + 7) / 8;
  mp.err = dev_status;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (pool->elem_bytes == 2) return stac::launch_merge<__nv_bfloat16>(mp, st);
  return stac::launch_merge<float>(mp, st);
}

}  // extern "C"
