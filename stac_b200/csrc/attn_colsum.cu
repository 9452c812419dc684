// Window + pivot attention with per-key softmax column sums (H2O scores), head_dim 64, bf16.
//
// Replaces the reference's attn_cuda.flash_attn_bias_colsum (attn-cuda/csrc/launch.cu:87-158,
// kernels fwd_kernel.h:78-485 and colsum_kernel.h:22-325) and its Triton twin
// (stac/flash_attn_triton.py:900-1006).  Semantics: S = q k^T * scale + bias[n], softmax over
// the keys, O = P v, lse = logsumexp, colsum[n] = sum over (optionally strided) query rows of
// exp(S - lse) times M / M_sub.  Keys come from two segments that are never concatenated in
// memory: the hot cache rows [0, T_hot) of a head and the retrieved pivots [0, T_ret) with a
// per-key bias (log C, or -inf for padding).
//
// Two kernels, both tcgen05 + TMA:
//   attn_fwd_kernel     one CTA per (128 query rows, head): S = Q K^T into TMEM, online softmax
//                       by two warpgroups that take alternate key tiles (each with its own
//                       running max/sum/accumulator, merged at the end), P staged in shared
//                       memory as bf16, O_tile = P V into TMEM and folded into registers.
//   attn_colsum_kernel  one CTA per (128 keys, head): S^T = K Q^T into TMEM so that each thread
//                       owns one key (TMEM lane) and sums exp2(S^T - lse[m]) over the query
//                       columns in registers: no shuffles, no atomics, deterministic.
#include "common.cuh"
#include "stac_internal.h"

namespace stac {

namespace {

constexpr int kD = 64;
constexpr int kBM = 128;
constexpr int kBN = 128;
constexpr int kTileBytes = 128 * 128;  // 128 rows x 64 bf16
constexpr int kFwdStages = 4;
constexpr int kFwdThreads = 384;       // warpgroup 0: warp 0 TMA, warp 1 MMA (2, 3 idle); warpgroups 1, 2: softmax
static_assert(128 * 40 + 256 * 232 <= kFwdThreads * ((65536 / kFwdThreads) / 8 * 8),
              "exact forward kernel: setmaxnreg targets exceed the CTA's register allocation");
constexpr int kColGroup = 3;           // key tiles per item = exponent warpgroups of the column-sum kernel
constexpr int kColStages = kColGroup == 4 ? 3 : 4;
constexpr int kColThreads = 128 + kColGroup * 128;   // warpgroup 0 control (warp 0 TMA, warp 1 MMA issue), then exponent
#ifndef STAC_COL_PAIR_MASK
#define STAC_COL_PAIR_MASK 0x88
#endif
constexpr unsigned kColPairMask = STAC_COL_PAIR_MASK;   // which of 8 consecutive PAIRS of exponentials of the column-sum kernel run on the FMA pipes
#ifndef STAC_COL_FOLD_LSE
#define STAC_COL_FOLD_LSE 1
#endif
// 1: the row term -lse2[m] of the exponent is added to the score tile by the tensor core (a fifth
// K = 16 step whose operands are a tile of ones and the row values split into three bf16), so the
// exponent warps read nothing from shared memory; 0: they read it per score (LDS.128 per four).
constexpr bool kColFoldLse = STAC_COL_FOLD_LSE != 0;
constexpr int kColXBytes = 128 * 32;   // 128 rows x 16 bf16, no swizzle: [16 row groups][2 K chunks][8 rows][16 B]
constexpr int kColCtlRegs = 56;
constexpr int kColExpRegs = kColGroup == 4 ? 104 : 152;
// setmaxnreg only moves registers inside the CTA's allocation, which is fixed at launch to
// (registers per thread the launch bound allows, a multiple of 8) x threads.  A request beyond
// what the control warpgroup released would wait forever.
constexpr int kColLaunchRegs = (65536 / kColThreads) / 8 * 8;
static_assert(128 * kColCtlRegs + (kColThreads - 128) * kColExpRegs <= kColThreads * kColLaunchRegs,
              "column-sum kernel: setmaxnreg targets exceed the CTA's register allocation");
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

struct FwdSmem {
  uint8_t q[kTileBytes];
  uint8_t k[kFwdStages][kTileBytes];
  uint8_t v[kFwdStages][kTileBytes];
  uint8_t p[2][2 * kTileBytes];  // per warpgroup: 128 rows x 128 keys bf16 as two 64-key atoms
  float bias2[2][kBN];
  float xm[kBM];
  float xl[kBM];
  uint64_t bar_q;
  uint64_t kv_full[kFwdStages];
  uint64_t kv_empty[kFwdStages];
  uint64_t s_full[3];  // S tiles rotate over three TMEM buffers (tile j -> buffer j % 3)
  uint64_t s_free[3];
  uint64_t p_full[2];
  uint64_t o_full[2];
  uint64_t o_free[2];
  uint32_t tmem_base;
};

struct FwdParams {
  int M, H;
  int T_hot, T_ret;
  int n_hot_tiles, n_ret_tiles;
  float scale_log2;
  const float* bias_ret;
  long long bias_head_stride;
  __nv_bfloat16* out;
  long long out_row_stride;  // elements between query rows
  float* lse;                // [H, M] natural log or nullptr
  float* lse2;               // [H, lse2_stride] log2 domain
  long long lse2_stride;
  int* fallback;             // device flag: set by the fast kernel when a row needs the exact kernel
  int* err;
  // fast kernel only: items = (head, 128-row query tile), head-major
  int n_q_tiles, n_items;
  int split;                 // 1: the (item, key tile) units are cut evenly over the grid
  float* part;               // split == 1: two partial-result slots per CTA
  int* part_count;           // split == 1: one arrival counter per cut between CTA c and c + 1, zero on entry
  // column sums that the column-sum kernel will accumulate with atomic adds: cleared here
  float* zero_colsum;        // [H, zero_stride], entries [0, zero_width) of every head; or nullptr
  long long zero_stride;
  int zero_width;
};

__device__ __forceinline__ uint8_t* align1024(uint8_t* p) {
  return reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(p) + 1023) & ~static_cast<uintptr_t>(1023));
}

#ifdef STAC_TIMESTAMPS
// Debug build only: first start and last end of each kernel on the GPU's nanosecond timer.
__device__ unsigned long long g_ts[8] = {~0ull, 0ull, ~0ull, 0ull, ~0ull, 0ull, ~0ull, 0ull};
__device__ __forceinline__ void ts_mark(int k, bool end) {
  if (threadIdx.x == 0) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    if (end) atomicMax(&g_ts[2 * k + 1], t);
    else atomicMin(&g_ts[2 * k], t);
  }
}
#define STAC_TS(k, end) ts_mark(k, end)
#else
#define STAC_TS(k, end)
#endif

__global__ void __launch_bounds__(kFwdThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k_hot,
                const __grid_constant__ CUtensorMap tm_v_hot, const __grid_constant__ CUtensorMap tm_k_ret,
                const __grid_constant__ CUtensorMap tm_v_ret, const FwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  FwdSmem& sm = *reinterpret_cast<FwdSmem*>(align1024(smem_raw));
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m_tile = blockIdx.x;
  const int h = blockIdx.y;
  const int n_hot = p.n_hot_tiles;
  const int n_tiles = p.n_hot_tiles + p.n_ret_tiles;
  // This kernel is the exact (running-maximum) path.  When it is launched behind the fast
  // kernel it only runs if that one flagged a row whose scores outgrew its fixed reference.
  STAC_TS(1, false);
  grid_dep_wait();   // launched behind the fast kernel with programmatic serialization: its flag and outputs are final now
  if (p.fallback != nullptr && *reinterpret_cast<volatile int*>(p.fallback) == 0) {
    STAC_TS(1, true);
    return;
  }

  if (threadIdx.x == 0) {
    mbar_init(&sm.bar_q, 1);
    for (int s = 0; s < kFwdStages; ++s) {
      mbar_init(&sm.kv_full[s], 1);
      mbar_init(&sm.kv_empty[s], 1);
    }
    for (int b = 0; b < 3; ++b) {
      mbar_init(&sm.s_full[b], 1);
      mbar_init(&sm.s_free[b], 128);
    }
    for (int g = 0; g < 2; ++g) {
      mbar_init(&sm.p_full[g], 128);
      mbar_init(&sm.o_full[g], 1);
      mbar_init(&sm.o_free[g], 128);
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&sm.tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;

  if (warp < 4) {
  setmaxnreg_dec<40>();   // control warpgroup hands its registers to the softmax warps
  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k_hot);
      tma_prefetch_desc(&tm_v_hot);
      mbar_arrive_expect_tx(&sm.bar_q, kTileBytes);
      tma_load_3d(sm.q, &tm_q, &sm.bar_q, 0, h, m_tile * kBM);
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j % kFwdStages;
        const int round = j / kFwdStages;
        if (round > 0) mbar_wait(&sm.kv_empty[s], (round - 1) & 1, p.err, DEV_TIMEOUT_CONSUMER);
        mbar_arrive_expect_tx(&sm.kv_full[s], 2 * kTileBytes);
        if (j < n_hot) {
          tma_load_3d(sm.k[s], &tm_k_hot, &sm.kv_full[s], 0, j * kBN, h);
          tma_load_3d(sm.v[s], &tm_v_hot, &sm.kv_full[s], 0, j * kBN, h);
        } else {
          tma_load_3d(sm.k[s], &tm_k_ret, &sm.kv_full[s], 0, (j - n_hot) * kBN, h);
          tma_load_3d(sm.v[s], &tm_v_ret, &sm.kv_full[s], 0, (j - n_hot) * kBN, h);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(kBM, kBN, 0);
      constexpr uint32_t idesc_o = umma_idesc_bf16(kBM, kD, 1);
      mbar_wait(&sm.bar_q, 0, p.err, DEV_TIMEOUT_TMA);
      const uint64_t q_desc = smem_desc_sw128(smem_u32(sm.q));
      auto issue_s = [&](int j) {
        const int b = j % 3, round = j / 3, s = j % kFwdStages;
        mbar_wait(&sm.kv_full[s], (j / kFwdStages) & 1, p.err, DEV_TIMEOUT_TMA);
        if (round > 0) mbar_wait(&sm.s_free[b], (round - 1) & 1, p.err, DEV_TIMEOUT_CONSUMER);
        tc_fence_after();
        const uint64_t k_desc = smem_desc_sw128(smem_u32(sm.k[s]));
#pragma unroll
        for (int kk = 0; kk < kD / 16; ++kk)
          umma_ss(tmem + b * kBN, q_desc + 2 * kk, k_desc + 2 * kk, idesc_s, kk > 0);
        umma_commit(&sm.s_full[b]);
      };
      auto issue_pv = [&](int j) {
        const int g = j & 1, it = j >> 1, s = j % kFwdStages;
        mbar_wait(&sm.p_full[g], it & 1, p.err, DEV_TIMEOUT_CONSUMER);
        if (it > 0) mbar_wait(&sm.o_free[g], (it - 1) & 1, p.err, DEV_TIMEOUT_CONSUMER);
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < kBN / 16; ++kk) {
          const uint64_t a = smem_desc_sw128(smem_u32(sm.p[g]) + (kk >> 2) * kTileBytes) + 2 * (kk & 3);
          const uint64_t b = smem_desc_sw128(smem_u32(sm.v[s]) + kk * 2048);
          umma_ss(tmem + 3 * kBN + g * kD, a, b, idesc_o, kk > 0);
        }
        umma_commit(&sm.o_full[g]);
        umma_commit(&sm.kv_empty[s]);
      };
      // S tiles run up to three ahead of the softmax; P V of tile j follows its softmax:
      // S0 S1 S2 PV0 S3 PV1 S4 ...
#pragma unroll 1
      for (int step = 0; step < n_tiles + 3; ++step) {
        if (step >= 3) issue_pv(step - 3);
        if (step < n_tiles) issue_s(step);
      }
    }
  }
  } else {
    // ------------------------------------------------------------------ softmax warpgroups
    setmaxnreg_inc<232>();
    const int g = (warp - 4) >> 2;
    const int wq = warp & 3;                 // TMEM lane quarter this warp may touch
    const int row = wq * 32 + lane;          // query row inside the tile
    const int t = row;
    const uint32_t lane_base = static_cast<uint32_t>(wq * 32) << 16;
    const float c2 = p.scale_log2;
    float m_run = -INFINITY, l_run = 0.f, alpha_prev = 1.f;
    float acc[kD];
#pragma unroll
    for (int i = 0; i < kD; ++i) acc[i] = 0.f;
    uint32_t ra[32], rb[32];
    int it = 0;
    for (int j = g; j < n_tiles; j += 2, ++it) {
      const bool is_ret = j >= n_hot;
      const int n0 = (is_ret ? j - n_hot : j) * kBN;
      const int valid = min(kBN, (is_ret ? p.T_ret : p.T_hot) - n0);
      const bool need_bias = is_ret || valid < kBN;
      if (need_bias) {
        named_bar_sync(1 + g, 128);
        float b = -INFINITY;
        if (t < valid) b = is_ret ? p.bias_ret[h * p.bias_head_stride + n0 + t] * kLog2e : 0.f;
        sm.bias2[g][t] = b;
        named_bar_sync(1 + g, 128);
      }
      const int sb = j % 3;
      mbar_wait(&sm.s_full[sb], (j / 3) & 1, p.err, DEV_TIMEOUT_MMA);
      tc_fence_after();
      // TMEM loads are double-buffered (ra / rb): the next 32 columns are in flight while the
      // current ones are processed, and the chain runs through all three phases of a tile.
      const uint32_t s_addr = tmem + lane_base + sb * kBN;
      const uint32_t o_addr = tmem + lane_base + 3 * kBN + g * kD;
      tmem_ld32(s_addr, ra);
      tmem_ld_wait();
      // pass 1 over the S tile: row maximum in the log2 domain
      float mx = -INFINITY, mx_raw = -INFINITY, mx_r1 = -INFINITY, mx_r2 = -INFINITY, mx_r3 = -INFINITY;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t(&cur)[32] = (c & 1) ? rb : ra;
        uint32_t(&nxt)[32] = (c & 1) ? ra : rb;
        if (c < 3) {
          tmem_ld32(s_addr + (c + 1) * 32, nxt);
        } else if (it > 0) {
          mbar_wait(&sm.o_full[g], (it - 1) & 1, p.err, DEV_TIMEOUT_MMA);
          tc_fence_after();
          tmem_ld32(o_addr, nxt);       // first half of the previous P V tile
        } else {
          tmem_ld32(s_addr, nxt);       // first columns again, for pass 2
        }
        if (need_bias) {
#pragma unroll
          for (int i = 0; i < 32; ++i) mx = fmaxf(mx, fmaf(__uint_as_float(cur[i]), c2, sm.bias2[g][c * 32 + i]));
        } else {
          // raw maximum (the scale is positive, applied once after the loop)
#pragma unroll
          for (int i = 0; i < 32; i += 8) {   // four independent chains
            mx_raw = fmax3(mx_raw, __uint_as_float(cur[i]), __uint_as_float(cur[i + 1]));
            mx_r1 = fmax3(mx_r1, __uint_as_float(cur[i + 2]), __uint_as_float(cur[i + 3]));
            mx_r2 = fmax3(mx_r2, __uint_as_float(cur[i + 4]), __uint_as_float(cur[i + 5]));
            mx_r3 = fmax3(mx_r3, __uint_as_float(cur[i + 6]), __uint_as_float(cur[i + 7]));
          }
        }
        tmem_ld_wait();
      }
      if (!need_bias) mx = fmaxf(fmaxf(mx_raw, mx_r1), fmaxf(mx_r2, mx_r3)) * c2;
      const float m_new = fmaxf(m_run, mx);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = fast_exp2(m_run - m_use);
      // fold the previous P V tile of this warpgroup into the register accumulator
      if (it > 0) {
        tmem_ld32(o_addr + 32, rb);
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[i] = fmaf(acc[i], alpha_prev, __uint_as_float(ra[i]));
        tmem_ld_wait();
        tmem_ld32(s_addr, ra);
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[32 + i] = fmaf(acc[32 + i], alpha_prev, __uint_as_float(rb[i]));
        tmem_ld_wait();
        tc_fence_before();
        mbar_arrive(&sm.o_free[g]);
      }
      // pass 2: probabilities relative to the new maximum, bf16 into shared memory
      float rs = 0.f, rs2 = 0.f;
      uint8_t* prow = sm.p[g] + row * 128;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t(&cur)[32] = (c & 1) ? rb : ra;
        uint32_t(&nxt)[32] = (c & 1) ? ra : rb;
        if (c < 3) tmem_ld32(s_addr + (c + 1) * 32, nxt);
        // keys c*32 .. c*32+31 -> atom c/2, 16-byte chunks (c&1)*4 .. +3 of this row
        uint8_t* atom = prow + (c >> 1) * kTileBytes;
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          float pv[8];
          if (need_bias) {
#pragma unroll
            for (int i = 0; i < 8; ++i)
              pv[i] = fast_exp2(fmaf(__uint_as_float(cur[q4 * 8 + i]), c2, sm.bias2[g][c * 32 + q4 * 8 + i]) - m_use);
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) pv[i] = fast_exp2(fmaf(__uint_as_float(cur[q4 * 8 + i]), c2, -m_use));
          }
          rs += (pv[0] + pv[1]) + (pv[2] + pv[3]);
          rs2 += (pv[4] + pv[5]) + (pv[6] + pv[7]);
          const int chunk = (c & 1) * 4 + q4;
          uint4 val;
          val.x = pack_bf16x2(pv[0], pv[1]);
          val.y = pack_bf16x2(pv[2], pv[3]);
          val.z = pack_bf16x2(pv[4], pv[5]);
          val.w = pack_bf16x2(pv[6], pv[7]);
          *reinterpret_cast<uint4*>(atom + ((chunk ^ (row & 7)) << 4)) = val;
        }
        if (c < 3) tmem_ld_wait();
      }
      tc_fence_before();
      mbar_arrive(&sm.s_free[sb]);
      l_run = fmaf(l_run, alpha, rs + rs2);
      m_run = m_new;
      alpha_prev = alpha;
      fence_proxy_async_smem();
      mbar_arrive(&sm.p_full[g]);
    }
    if (it > 0) {
      mbar_wait(&sm.o_full[g], (it - 1) & 1, p.err, DEV_TIMEOUT_MMA);
      tc_fence_after();
      tmem_ld32(tmem + lane_base + 3 * kBN + g * kD, ra);
      tmem_ld32(tmem + lane_base + 3 * kBN + g * kD + 32, rb);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; ++i) acc[i] = fmaf(acc[i], alpha_prev, __uint_as_float(ra[i]));
#pragma unroll
      for (int i = 0; i < 32; ++i) acc[32 + i] = fmaf(acc[32 + i], alpha_prev, __uint_as_float(rb[i]));
      tc_fence_before();
    }
    // merge the two warpgroups' partial softmax states (warpgroup 1 -> shared -> warpgroup 0)
    float* xacc = reinterpret_cast<float*>(sm.p[1]);  // [64][128] floats = 32 KB, P[1] is idle now
    if (g == 1) {
#pragma unroll
      for (int i = 0; i < kD; ++i) xacc[i * kBM + row] = acc[i];
      sm.xm[row] = m_run;
      sm.xl[row] = l_run;
    }
    named_bar_sync(3, 256);
    if (g == 0) {
      const float m1 = sm.xm[row], l1 = sm.xl[row];
      const float m = fmaxf(m_run, m1);
      const float m_use = (m == -INFINITY) ? 0.f : m;
      const float e0 = fast_exp2(m_run - m_use), e1 = fast_exp2(m1 - m_use);
      const float l = l_run * e0 + l1 * e1;
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const int mrow = m_tile * kBM + row;
      if (mrow < p.M) {
        __nv_bfloat16* dst = p.out + static_cast<long long>(mrow) * p.out_row_stride + h * kD;
#pragma unroll
        for (int q8 = 0; q8 < kD / 8; ++q8) {
          float o[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] = (acc[q8 * 8 + i] * e0 + xacc[(q8 * 8 + i) * kBM + row] * e1) * inv;
          uint4 val;
          val.x = pack_bf16x2(o[0], o[1]);
          val.y = pack_bf16x2(o[2], o[3]);
          val.z = pack_bf16x2(o[4], o[5]);
          val.w = pack_bf16x2(o[6], o[7]);
          *reinterpret_cast<uint4*>(dst + q8 * 8) = val;
        }
        const float l2 = m_use + log2f(l);
        if (p.lse != nullptr) p.lse[static_cast<long long>(h) * p.M + mrow] = l2 * kLn2;
        p.lse2[static_cast<long long>(h) * p.lse2_stride + mrow] = l2;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
  STAC_TS(1, true);
}

// ---------------------------------------------------------------------------------------
// Fast forward kernel.  Softmax is invariant to the reference subtracted before the exponent,
// so instead of a running maximum every row uses ONE reference: the exact maximum of its
// first key tile.  Nothing is ever rescaled: P V accumulates in TMEM across all key tiles of
// the row block, the softmax warpgroups (four) take key tiles round-robin and keep only a partial
// row sum each.  The scheme is exact as long as no later score exceeds the reference by more
// than 2^60 (probabilities then stay far inside the bf16 / fp32 range); a row whose sum of
// probabilities leaves that range raises `fallback` and the exact kernel, launched right
// behind this one, recomputes the call.
//
// Shared memory carries only the operands TMA brings in.  Key tiles are 112 keys wide so that
// FOUR score buffers fit beside the output accumulator in the 512 TMEM columns (4 x 112 + 64):
// with four softmax warpgroups each has a buffer of its own and the other three keep the
// exponential unit busy while one waits for its buffer to go through P V and the next Q K^T
// (with three, the fourth buffer is scored ahead, so a warpgroup finds its next tile ready;
// measured 3.4 % slower at 4164 x 17697 keys than four).  The probabilities go back into
// the columns their scores came from (bf16, two per column) and feed the P V MMA as its A
// operand straight from tensor memory.  The tensor pipe has a floor of about 48 clocks per
// MMA instruction whatever its width and idles while its issuing thread does anything else,
// so scores use one wide instruction per K step, the two MMA streams (scores, P V) have a
// warp each, and the instructions of a group are issued back to back with operands prepared
// beforehand.
//
// Work = items (head, 128-row query tile) x key tiles.  With enough items the kernel runs one
// CTA per SM and cuts that unit sequence into equal contiguous ranges (no partly filled last
// wave); a CTA walks its range segment by segment, a segment being a run of key tiles of one
// item.  An item on a cut is computed in two parts by two CTAs, each with its own row
// references; the parts (unnormalised accumulator, row sums, references) go to a workspace, each
// CTA counts its arrival at the cut and the one that arrives second joins the two parts (plain
// split-softmax algebra, operands in a fixed order: same bits whichever CTA does it).  With at
// most half as many items as SMs every item is cut in exactly two halves instead.  Barrier
// phases, the score ring and the K/V rings run on across segments; the query tile, the row references and the partial row sums are double
// buffered by segment parity, and so are the barriers that several warpgroups arrive on per
// segment: a warpgroup without a tile in a short first or last segment runs one segment ahead,
// never two (a CTA's middle segments are whole items of at least kFastMinSplitTiles tiles, far
// longer than the few tiles the score ring lets the warpgroups be apart).
// ---------------------------------------------------------------------------------------
#ifndef STAC_FAST_WGS
#define STAC_FAST_WGS 4
#endif
constexpr int kFastWgs = STAC_FAST_WGS;            // softmax warpgroups (3 or 4); key tile c goes to warpgroup c % kFastWgs
static_assert(kFastWgs == 3 || kFastWgs == 4, "three or four softmax warpgroups");
// With three warpgroups a thread double-buffers its tensor-memory loads (64 score registers) and
// prefetches its next tile; with four the launch leaves 96 registers per thread, so loads are
// single-buffered and the fourth warp per scheduler hides their latency instead.  The hand-over
// rules between segments hold for both: a warpgroup's last tile of a middle segment (at least
// kFastMinSplitTiles >= 2 * kFastWgs tiles) lies kFastRing or more tiles into it, so its score
// buffer is a reused one and cannot be scored before the previous segment's accumulator has
// been read out.
constexpr bool kFastDouble = kFastWgs == 3;
constexpr int kFastThreads = 128 + 128 * kFastWgs;   // warpgroup 0 control (warps 0, 3 TMA, warps 1-2 MMA issue), then softmax
#ifndef STAC_FAST_STAGES
#define STAC_FAST_STAGES 5
#endif
constexpr int kFastKStages = STAC_FAST_STAGES;
constexpr int kFastVStages = STAC_FAST_STAGES;
#ifndef STAC_FAST_KEYS
#define STAC_FAST_KEYS 112
#endif
constexpr int kFT = STAC_FAST_KEYS;             // keys per tile: 112 (four score buffers); 80 (five buffers, one scored ahead) measured 2 % slower
static_assert(kFT % 32 == 16 && kFT <= kBN, "a tile is a number of 32-key chunks and one of 16");
static_assert(kFT == 112 || !kFastDouble, "the double-buffered path is written for 112-key tiles");
constexpr int kFastTileBytes = kFT * 128;       // kFT rows x 64 bf16
constexpr int kFastRing = (512 - kD) / kFT;     // score buffers beside the 64 accumulator columns
constexpr float kFastRowSumLimit = 1.152921504606846976e18f;  // 2^60
constexpr int kPartFloats = kBM * kD + 2 * kBM; // one partial result: O[128][64], row sums, row references
constexpr int kFastMaxCtas = 160;               // partial-result slots are provided for this many CTAs
// shorter key ranges run one CTA per item; every warpgroup has a tile at least kFastRing tiles into a
// middle segment, i.e. one whose score buffer was last used inside the same segment
constexpr int kFastMinSplitTiles = kFastRing + kFastWgs;
static_assert(kFastMinSplitTiles >= 2 * kFastWgs, "segment hand-over rule");
#ifndef STAC_FAST_PAIR_MASK
#define STAC_FAST_PAIR_MASK 0x8080u
#endif
constexpr unsigned kFastPairMask = STAC_FAST_PAIR_MASK;   // which of 16 consecutive PAIRS of exponentials run on the FMA pipes
// setmaxnreg targets; must fit the launch allocation
constexpr int kFastCtlRegs = kFastWgs == 3 ? 56 : 40, kFastSoftmaxRegs = kFastWgs == 3 ? 152 : 104;
static_assert(128 * kFastCtlRegs + 128 * kFastWgs * kFastSoftmaxRegs <= kFastThreads * ((65536 / kFastThreads) / 8 * 8),
              "fast forward kernel: setmaxnreg targets exceed the CTA's register allocation");

struct FastSmem {
  uint8_t q[2][kTileBytes];                     // query tile of the segment (parity)
  uint8_t k[kFastKStages][kFastTileBytes];
  uint8_t v[kFastVStages][kFastTileBytes];
  float bias2[kFastWgs][kBN];
  float m_ref[2][kBM];                          // row references of the segment (parity)
  float lpart[2][kFastWgs - 1][kBM];            // row sums of warpgroups 1.. (segment parity)
  int live[2][kFastWgs - 1];                    // did warpgroup 1.. see a key that is not masked (segment parity)
  uint64_t q_full[2];
  uint64_t q_empty[2];
  uint64_t k_full[kFastKStages];
  uint64_t k_empty[kFastKStages];
  uint64_t v_full[kFastVStages];
  uint64_t v_empty[kFastVStages];
  uint64_t s_full[kFastRing];    // scores of a tile are in TMEM
  uint64_t p_full[kFastRing];    // its probabilities are in TMEM
  uint64_t buf_free[kFastRing];  // the P V MMAs that read them are done
  uint64_t ref_ready[2];
  uint64_t l_ready[2];           // warpgroups 1.. have published their row sums of the segment (parity)
  uint64_t o_done;               // all P V MMAs of the segment are complete
  uint64_t o_free;               // the segment's accumulator has been read out of TMEM
  uint32_t tmem_base;
  int join_flag;                 // arrival count seen at a cut (1: the other part is complete)
};

// The (item, key tile) units of one CTA, walked segment by segment: a segment is a run of key
// tiles [t0, t1) of one item.  With `split` the units of the whole launch are cut into equal
// contiguous ranges, one per CTA (an item on a cut is then finished by two CTAs); without it
// CTA i owns item i.  Every role of the CTA walks the same sequence.
struct FwdWalk {
  long long u, u_end;
  int nt;
  __device__ FwdWalk(const FwdParams& p, int n_tiles) {
    nt = n_tiles;
    if (p.split) {
      const long long total = static_cast<long long>(p.n_items) * nt;
      u = total * blockIdx.x / gridDim.x;
      u_end = total * (blockIdx.x + 1) / gridDim.x;
    } else {
      u = static_cast<long long>(blockIdx.x) * nt;
      u_end = u + nt;
    }
  }
  __device__ bool next(int& item, int& t0, int& t1) {
    if (u >= u_end) return false;
    item = static_cast<int>(u / nt);
    t0 = static_cast<int>(u - static_cast<long long>(item) * nt);
    const long long e = static_cast<long long>(item + 1) * nt;
    t1 = static_cast<int>((e < u_end ? e : u_end) - static_cast<long long>(item) * nt);
    u = static_cast<long long>(item) * nt + t1;
    return true;
  }
};

// kN scores -> kN probabilities relative to the row reference, packed as bf16 pairs.  Scores
// are handled two at a time with the packed fp32 instructions (scale-and-subtract, row sums).
// The pairs whose bit is set in kFastPairMask take their exponentials on the FMA pipes (cubic,
// 8.6e-5 relative, far below the bf16 rounding of P) to relieve the exponential unit.
template <int kJ>
__device__ __forceinline__ uint64_t fast_exp_pair(uint64_t x2) {
  if ((kFastPairMask >> (kJ & 15)) & 1u) return poly_exp2_x2(x2);
  float x0, x1;
  unpack_f32x2(x2, x0, x1);
  return pack_f32x2(fast_exp2(x0), fast_exp2(x1));
}
template <bool kBias, int kN, int kI = 0>
__device__ __forceinline__ void fast_exp_chunk(const uint32_t (&s)[32], uint32_t (&pk)[16], const float* bias2,
                                               uint64_t c2c2, uint64_t negm2, uint64_t& l0, uint64_t& l1) {
  if constexpr (kI < kN) {
    uint64_t x0 = pack_f32x2(__uint_as_float(s[kI + 0]), __uint_as_float(s[kI + 1]));
    uint64_t x1 = pack_f32x2(__uint_as_float(s[kI + 2]), __uint_as_float(s[kI + 3]));
    if (kBias) {
      const float4 b = *reinterpret_cast<const float4*>(bias2 + kI);
      x0 = add_f32x2(fma_f32x2(x0, c2c2, pack_f32x2(b.x, b.y)), negm2);
      x1 = add_f32x2(fma_f32x2(x1, c2c2, pack_f32x2(b.z, b.w)), negm2);
    } else {
      x0 = fma_f32x2(x0, c2c2, negm2);
      x1 = fma_f32x2(x1, c2c2, negm2);
    }
    const uint64_t e0 = fast_exp_pair<kI / 2>(x0), e1 = fast_exp_pair<kI / 2 + 1>(x1);
    l0 = add_f32x2(l0, e0);
    l1 = add_f32x2(l1, e1);
    float a0, a1, a2, a3;
    unpack_f32x2(e0, a0, a1);
    unpack_f32x2(e1, a2, a3);
    pk[kI / 2] = pack_bf16x2(a0, a1);
    pk[kI / 2 + 1] = pack_bf16x2(a2, a3);
    fast_exp_chunk<kBias, kN, kI + 4>(s, pk, bias2, c2c2, negm2, l0, l1);
  }
}

template <int kN>
__device__ __forceinline__ float fast_max_chunk(const uint32_t (&s)[32], const float* bias2, bool need_bias, float c2,
                                                float mx) {
  if (need_bias) {
#pragma unroll
    for (int i = 0; i < kN; ++i) mx = fmaxf(mx, fmaf(__uint_as_float(s[i]), c2, bias2[i]));
  } else {
#pragma unroll
    for (int i = 0; i < kN; i += 2) mx = fmax3(mx, __uint_as_float(s[i]) * c2, __uint_as_float(s[i + 1]) * c2);
  }
  return mx;
}

__global__ void __launch_bounds__(kFastThreads, 1)
attn_fwd_fast_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k_hot,
                     const __grid_constant__ CUtensorMap tm_v_hot, const __grid_constant__ CUtensorMap tm_k_ret,
                     const __grid_constant__ CUtensorMap tm_v_ret, const FwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  FastSmem& sm = *reinterpret_cast<FastSmem*>(align1024(smem_raw));
  STAC_TS(0, false);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_hot = (p.T_hot + kFT - 1) / kFT;
  const int n_tiles = n_hot + (p.T_ret + kFT - 1) / kFT;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sm.q_full[i], 1);
      mbar_init(&sm.q_empty[i], 1);
      mbar_init(&sm.ref_ready[i], 128);
      mbar_init(&sm.l_ready[i], 128 * (kFastWgs - 1));
    }
    for (int s = 0; s < kFastKStages; ++s) {
      mbar_init(&sm.k_full[s], 1);
      mbar_init(&sm.k_empty[s], 1);
    }
    for (int s = 0; s < kFastVStages; ++s) {
      mbar_init(&sm.v_full[s], 1);
      mbar_init(&sm.v_empty[s], 1);
    }
    for (int b = 0; b < kFastRing; ++b) {
      mbar_init(&sm.s_full[b], 1);
      mbar_init(&sm.p_full[b], 128);
      mbar_init(&sm.buf_free[b], 1);
    }
    mbar_init(&sm.o_done, 1);
    mbar_init(&sm.o_free, 128);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&sm.tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;
  const uint32_t o_tmem = tmem + kFastRing * kFT;   // 64 columns behind the score buffers
  // The exact kernel behind this one may be scheduled as soon as an SM has room for it (that is,
  // when this CTA has left); it waits for this grid's completion before it reads the flag.
  grid_dep_launch();

  if (p.zero_colsum != nullptr) {
    // a slice of the column-sum output per CTA (the next kernel adds partial sums onto zeros)
    const long long total = static_cast<long long>(p.H) * p.zero_width;
    const long long lo = total * blockIdx.x / gridDim.x, hi = total * (blockIdx.x + 1) / gridDim.x;
    for (long long e = lo + threadIdx.x; e < hi; e += kFastThreads) {
      const long long hh = e / p.zero_width;
      p.zero_colsum[hh * p.zero_stride + (e - hh * p.zero_width)] = 0.f;
    }
  }

  if (warp < 4) {
    setmaxnreg_dec<kFastCtlRegs>();
    if (warp == 0 && lane == 0) {
      // ---------------------------------------------------------------- TMA producer: Q and K
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k_hot);
      FwdWalk walk(p, n_tiles);
      int seg = 0, item, t0, t1;
      int ks = 0, kr = 0;   // stage and round of the K ring
      for (; walk.next(item, t0, t1); ++seg) {
        const int h = item / p.n_q_tiles, m_tile = item - h * p.n_q_tiles;
        const int qb = seg & 1;
        if (seg >= 2) mbar_wait(&sm.q_empty[qb], ((seg >> 1) - 1) & 1, p.err, DEV_TIMEOUT_CONSUMER);
        mbar_arrive_expect_tx(&sm.q_full[qb], kTileBytes);
        tma_load_3d(sm.q[qb], &tm_q, &sm.q_full[qb], 0, h, m_tile * kBM);
        for (int j = t0; j < t1; ++j) {
          const bool hot = j < n_hot;
          const int n0 = (hot ? j : j - n_hot) * kFT;
          if (kr > 0) mbar_wait(&sm.k_empty[ks], (kr - 1) & 1, p.err, DEV_TIMEOUT_CONSUMER);
          mbar_arrive_expect_tx(&sm.k_full[ks], kFastTileBytes);
          tma_load_3d(sm.k[ks], hot ? &tm_k_hot : &tm_k_ret, &sm.k_full[ks], 0, n0, h);
          if (++ks == kFastKStages) { ks = 0; ++kr; }
        }
      }
    } else if (warp == 3 && lane == 0) {
      // ---------------------------------------------------------------- TMA producer: V
      // (its own thread: V tiles are released several tiles later than K tiles, and one
      // thread serving both rings in order would hold K back whenever the V ring is full)
      tma_prefetch_desc(&tm_v_hot);
      FwdWalk walk(p, n_tiles);
      int item, t0, t1;
      int vs = 0, vr = 0;
      while (walk.next(item, t0, t1)) {
        const int h = item / p.n_q_tiles;
        for (int j = t0; j < t1; ++j) {
          const bool hot = j < n_hot;
          const int n0 = (hot ? j : j - n_hot) * kFT;
          if (vr > 0) mbar_wait(&sm.v_empty[vs], (vr - 1) & 1, p.err, DEV_TIMEOUT_CONSUMER);
          mbar_arrive_expect_tx(&sm.v_full[vs], kFastTileBytes);
          tma_load_3d(sm.v[vs], hot ? &tm_v_hot : &tm_v_ret, &sm.v_full[vs], 0, n0, h);
          if (++vs == kFastVStages) { vs = 0; ++vr; }
        }
      }
    } else if (warp == 1) {
      // ---------------------------------------------------------------- MMA issuer: S = Q K^T
      // (all lanes run the loop, one elected lane issues)
      constexpr uint32_t idesc_s = umma_idesc_bf16(kBM, kFT, 0);
      const uint64_t q_desc0 = smem_desc_sw128(smem_u32(sm.q[0]));
      const uint64_t k_desc0 = smem_desc_sw128(smem_u32(sm.k[0]));
      FwdWalk walk(p, n_tiles);
      int seg = 0, item, t0, t1;
      int b = 0, round = 0, ks = 0, kr = 0;
      for (; walk.next(item, t0, t1); ++seg) {
        const int qb = seg & 1;
        const uint64_t q_desc = q_desc0 + static_cast<uint64_t>(qb * (kTileBytes >> 4));
        mbar_wait(&sm.q_full[qb], (seg >> 1) & 1, p.err, DEV_TIMEOUT_TMA);
#pragma unroll 1
        for (int j = t0; j < t1; ++j) {
          const uint64_t k_desc = k_desc0 + static_cast<uint64_t>(ks * (kFastTileBytes >> 4));
          const uint32_t d = tmem + b * kFT;
          mbar_wait(&sm.k_full[ks], kr & 1, p.err, DEV_TIMEOUT_TMA);
          if (round > 0) mbar_wait(&sm.buf_free[b], (round - 1) & 1, p.err, DEV_TIMEOUT_CONSUMER);
          tc_fence_after();
          if (elect_one()) {
            umma_ss(d, q_desc, k_desc, idesc_s, 0u);
            umma_ss(d, q_desc + 2, k_desc + 2, idesc_s, 1u);
            umma_ss(d, q_desc + 4, k_desc + 4, idesc_s, 1u);
            umma_ss(d, q_desc + 6, k_desc + 6, idesc_s, 1u);
            umma_commit(&sm.s_full[b]);
            umma_commit(&sm.k_empty[ks]);
            if (j == t1 - 1) umma_commit(&sm.q_empty[qb]);
          }
          __syncwarp();
          if (++ks == kFastKStages) { ks = 0; ++kr; }
          if (++b == kFastRing) { b = 0; ++round; }
        }
      }
    } else if (warp == 2) {
      // ---------------------------------------------------------------- MMA issuer: O += P V
      constexpr uint32_t idesc_o = umma_idesc_bf16(kBM, kD, 1);
      const uint64_t v_desc0 = smem_desc_sw128(smem_u32(sm.v[0]));
      FwdWalk walk(p, n_tiles);
      int seg = 0, item, t0, t1;
      int b = 0, round = 0, vs = 0, vr = 0;
      for (; walk.next(item, t0, t1); ++seg) {
#pragma unroll 1
        for (int j = t0; j < t1; ++j) {
          // A: 16 keys = 8 columns of packed probabilities; B: V advances 16 rows = 2048 bytes
          const uint32_t pa = tmem + b * kFT;
          const uint64_t vb = v_desc0 + static_cast<uint64_t>(vs * (kFastTileBytes >> 4));
          const uint32_t acc0 = j > t0 ? 1u : 0u;
          mbar_wait(&sm.v_full[vs], vr & 1, p.err, DEV_TIMEOUT_TMA);
          mbar_wait(&sm.p_full[b], round & 1, p.err, DEV_TIMEOUT_CONSUMER);
          // a new segment overwrites the accumulator: the previous one must have been read out
          if (j == t0 && seg > 0) mbar_wait(&sm.o_free, (seg - 1) & 1, p.err, DEV_TIMEOUT_CONSUMER);
          tc_fence_after();
          if (elect_one()) {
            umma_ts(o_tmem, pa, vb, idesc_o, acc0);
#pragma unroll
            for (int kk = 1; kk < kFT / 16; ++kk)
              umma_ts(o_tmem, pa + kk * 8, vb + static_cast<uint64_t>(kk * (2048 >> 4)), idesc_o, 1u);
            umma_commit(&sm.buf_free[b]);
            umma_commit(&sm.v_empty[vs]);
            if (j == t1 - 1) umma_commit(&sm.o_done);
          }
          __syncwarp();
          if (++vs == kFastVStages) { vs = 0; ++vr; }
          if (++b == kFastRing) { b = 0; ++round; }
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax warpgroups
    setmaxnreg_inc<kFastSoftmaxRegs>();
    const int g = (warp - 4) >> 2;
    const int wq = warp & 3;
    const int row = wq * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(wq * 32) << 16;
    const float c2 = p.scale_log2;
    const uint64_t c2c2 = pack_f32x2(c2, c2);
    const float* bias2 = sm.bias2[g];
    uint32_t ra[32], rb[32], pk[16];   // rb: second score buffer (three warpgroups) and the read-out of O
    bool overflow = false;
    FwdWalk walk(p, n_tiles);
    int seg = 0, item, t0, t1;
    int c_base = 0;   // key tiles of earlier segments: tile c of the CTA uses ring buffer c % kFastRing, warpgroup c % kFastWgs
    for (; walk.next(item, t0, t1); ++seg) {
      const int h = item / p.n_q_tiles, m_tile = item - h * p.n_q_tiles;
      const int len = t1 - t0;
      const int sb = seg & 1;
      float m_ref = 0.f;
      uint64_t l0 = 0ull, l1 = 0ull;    // four partial row sums, two per register pair
      uint64_t negm2 = 0ull;            // (-m_ref, -m_ref)
      bool have_ref = false;
      bool any_live = false;  // some key tile of this warpgroup in this segment had a key that is not masked
      bool fetching = false;  // the first 32 scores of the next tile are already on their way into ra
      for (int x = (g + kFastWgs - c_base % kFastWgs) % kFastWgs; x < len; x += kFastWgs) {
        const int c = c_base + x;
        const int b = c % kFastRing, round = c / kFastRing;
        const int j = t0 + x;
        const bool is_ret = j >= n_hot;
        const int n0 = (is_ret ? j - n_hot : j) * kFT;
        const int valid = min(kFT, (is_ret ? p.T_ret : p.T_hot) - n0);
        const bool need_bias = is_ret || valid < kFT;
        bool tile_live = true;   // false: every key of the tile is masked (padding behind the valid pivots)
        if (need_bias) {
          named_bar_sync(1 + g, 128);
          bool live = false;
          if (row < kFT) {
            float bv = -INFINITY;
            if (row < valid) bv = is_ret ? p.bias_ret[h * p.bias_head_stride + n0 + row] * kLog2e : 0.f;
            sm.bias2[g][row] = bv;
            live = bv != -INFINITY;
          }
          tile_live = named_bar_or(1 + g, 128, live);
        }
        any_live = any_live || tile_live;
        const uint32_t s_addr = tmem + lane_base + b * kFT;
        if (!fetching) {
          mbar_wait(&sm.s_full[b], round & 1, p.err, DEV_TIMEOUT_MMA);
          tc_fence_after();
          if (tile_live || !have_ref) tmem_ld32(s_addr, ra);
        }
        if (!tile_live && have_ref) {
          // nothing to exponentiate: all probabilities of this tile are zero
          if (fetching) tmem_ld_wait();      // the prefetched scores are not needed
#pragma unroll
          for (int i = 0; i < 16; ++i) pk[i] = 0u;
#pragma unroll
          for (int ch = 0; ch < kFT / 32; ++ch) tmem_st16(s_addr + 16 * ch, pk);
          tmem_st8(s_addr + (kFT - 16) / 2, pk);
          const int b2n = (c + kFastWgs) % kFastRing, round2n = (c + kFastWgs) / kFastRing;
          fetching = false;
          if (kFastDouble && x + kFastWgs < len &&
              __all_sync(0xffffffffu, mbar_test(&sm.s_full[b2n], round2n & 1))) {
            tc_fence_after();
            tmem_ld32(tmem + lane_base + b2n * kFT, ra);
            fetching = true;
          }
          tmem_st_wait();
          tc_fence_before();
          mbar_arrive(&sm.p_full[b]);
          continue;
        }
        if (!have_ref) {
          have_ref = true;
          if (x == 0) {
            // exact row maximum of the segment's first tile = the row's reference for the segment
            float mx = -INFINITY;
#pragma unroll
            for (int ch = 0; ch < kFT / 32; ++ch) {
              tmem_ld_wait();
              mx = fast_max_chunk<32>(ra, bias2 + 32 * ch, need_bias, c2, mx);
              if (ch + 1 < kFT / 32) tmem_ld32(s_addr + 32 * (ch + 1), ra);
              else tmem_ld16(s_addr + 32 * (ch + 1), ra);
            }
            tmem_ld_wait();
            mx = fast_max_chunk<16>(ra, bias2 + kFT - 16, need_bias, c2, mx);
            m_ref = (mx == -INFINITY) ? 0.f : mx;
            sm.m_ref[sb][row] = m_ref;
            mbar_arrive(&sm.ref_ready[sb]);
            tmem_ld32(s_addr, ra);
          } else {
            mbar_wait(&sm.ref_ready[sb], (seg >> 1) & 1, p.err, DEV_TIMEOUT_CONSUMER);
            m_ref = sm.m_ref[sb][row];
          }
          negm2 = pack_f32x2(-m_ref, -m_ref);
        }
        // keys 0..31 are on their way into ra
        if constexpr (kFastDouble) {
          tmem_ld_wait();
          tmem_ld32(s_addr + 32, rb);
          if (need_bias) fast_exp_chunk<true, 32>(ra, pk, bias2, c2c2, negm2, l0, l1);
          else fast_exp_chunk<false, 32>(ra, pk, bias2, c2c2, negm2, l0, l1);
          tmem_st16(s_addr, pk);
          tmem_ld_wait();
          tmem_ld32(s_addr + 64, ra);
          if (need_bias) fast_exp_chunk<true, 32>(rb, pk, bias2 + 32, c2c2, negm2, l0, l1);
          else fast_exp_chunk<false, 32>(rb, pk, bias2 + 32, c2c2, negm2, l0, l1);
          tmem_st16(s_addr + 16, pk);
          tmem_ld_wait();
          tmem_ld16(s_addr + 96, rb);
          if (need_bias) fast_exp_chunk<true, 32>(ra, pk, bias2 + 64, c2c2, negm2, l0, l1);
          else fast_exp_chunk<false, 32>(ra, pk, bias2 + 64, c2c2, negm2, l0, l1);
          tmem_st16(s_addr + 32, pk);
          tmem_ld_wait();
          // this warpgroup's next tile of the segment is normally scored by now: start fetching it
          // (never wait for it here: its buffer is released by another warpgroup's P V, which may
          // be behind this one)
          const int b2 = (c + kFastWgs) % kFastRing, round2 = (c + kFastWgs) / kFastRing;
          const bool more = x + kFastWgs < len;
          fetching = false;
          if (more && __all_sync(0xffffffffu, mbar_test(&sm.s_full[b2], round2 & 1))) {
            tc_fence_after();
            tmem_ld32(tmem + lane_base + b2 * kFT, ra);
            fetching = true;
          }
          if (need_bias) fast_exp_chunk<true, 16>(rb, pk, bias2 + 96, c2c2, negm2, l0, l1);
          else fast_exp_chunk<false, 16>(rb, pk, bias2 + 96, c2c2, negm2, l0, l1);
          tmem_st8(s_addr + 48, pk);
          if (more && !fetching && __all_sync(0xffffffffu, mbar_test(&sm.s_full[b2], round2 & 1))) {
            tc_fence_after();                  // second chance, a chunk later
            tmem_ld32(tmem + lane_base + b2 * kFT, ra);
            fetching = true;
          }
        } else {
          // one score buffer per thread: load, wait, convert, store, chunk by chunk
#pragma unroll
          for (int ch = 0; ch < kFT / 32; ++ch) {
            tmem_ld_wait();
            if (need_bias) fast_exp_chunk<true, 32>(ra, pk, bias2 + 32 * ch, c2c2, negm2, l0, l1);
            else fast_exp_chunk<false, 32>(ra, pk, bias2 + 32 * ch, c2c2, negm2, l0, l1);
            if (ch + 1 < kFT / 32) tmem_ld32(s_addr + 32 * (ch + 1), ra);
            else tmem_ld16(s_addr + 32 * (ch + 1), ra);
            tmem_st16(s_addr + 16 * ch, pk);
          }
          tmem_ld_wait();
          if (need_bias) fast_exp_chunk<true, 16>(ra, pk, bias2 + kFT - 16, c2c2, negm2, l0, l1);
          else fast_exp_chunk<false, 16>(ra, pk, bias2 + kFT - 16, c2c2, negm2, l0, l1);
          tmem_st8(s_addr + (kFT - 16) / 2, pk);
          fetching = false;
        }
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(&sm.p_full[b]);
      }
      // ---- end of the segment
      float la, lb, lc, ld;
      unpack_f32x2(l0, la, lb);
      unpack_f32x2(l1, lc, ld);
      const float lsum = (la + lb) + (lc + ld);
      overflow = overflow || !(lsum <= kFastRowSumLimit);   // also true for NaN
      if (g != 0) {
        sm.lpart[sb][g - 1][row] = lsum;
        if (row == 0) sm.live[sb][g - 1] = any_live ? 1 : 0;
        mbar_arrive(&sm.l_ready[sb]);
      } else {
        if (!have_ref) {
          mbar_wait(&sm.ref_ready[sb], (seg >> 1) & 1, p.err, DEV_TIMEOUT_CONSUMER);
          m_ref = sm.m_ref[sb][row];
        }
        mbar_wait(&sm.l_ready[sb], (seg >> 1) & 1, p.err, DEV_TIMEOUT_CONSUMER);
        float l = (lsum + sm.lpart[sb][0][row]) + sm.lpart[sb][1][row];
        if constexpr (kFastWgs == 4) l += sm.lpart[sb][2][row];
        // A segment whose keys are all masked has no reference (m_ref is a placeholder): it must not
        // take part in a join.  A segment with live keys whose probabilities all underflowed (its
        // first tile was masked, so the placeholder was used, and the live scores lie far below
        // it) cannot be represented: the exact kernel redoes the call.
        bool seg_live = any_live || sm.live[sb][0] != 0 || sm.live[sb][1] != 0;
        if constexpr (kFastWgs == 4) seg_live = seg_live || sm.live[sb][2] != 0;
        if (seg_live && !(l > 0.f)) overflow = true;
        mbar_wait(&sm.o_done, seg & 1, p.err, DEV_TIMEOUT_MMA);
        tc_fence_after();
        tmem_ld32(o_tmem + lane_base, ra);
        tmem_ld32(o_tmem + lane_base + 32, rb);
        tmem_ld_wait();
        tc_fence_before();
        mbar_arrive(&sm.o_free);
        const int mrow = m_tile * kBM + row;
        if (t0 == 0 && t1 == n_tiles) {
          // the whole item was done here: normalise and write the output rows
          const float inv = l > 0.f ? 1.f / l : 0.f;
          if (mrow < p.M) {
            __nv_bfloat16* dst = p.out + static_cast<long long>(mrow) * p.out_row_stride + h * kD;
#pragma unroll
            for (int q8 = 0; q8 < 4; ++q8) {
              uint4 val;
              val.x = pack_bf16x2(__uint_as_float(ra[q8 * 8 + 0]) * inv, __uint_as_float(ra[q8 * 8 + 1]) * inv);
              val.y = pack_bf16x2(__uint_as_float(ra[q8 * 8 + 2]) * inv, __uint_as_float(ra[q8 * 8 + 3]) * inv);
              val.z = pack_bf16x2(__uint_as_float(ra[q8 * 8 + 4]) * inv, __uint_as_float(ra[q8 * 8 + 5]) * inv);
              val.w = pack_bf16x2(__uint_as_float(ra[q8 * 8 + 6]) * inv, __uint_as_float(ra[q8 * 8 + 7]) * inv);
              *reinterpret_cast<uint4*>(dst + q8 * 8) = val;
            }
#pragma unroll
            for (int q8 = 0; q8 < 4; ++q8) {
              uint4 val;
              val.x = pack_bf16x2(__uint_as_float(rb[q8 * 8 + 0]) * inv, __uint_as_float(rb[q8 * 8 + 1]) * inv);
              val.y = pack_bf16x2(__uint_as_float(rb[q8 * 8 + 2]) * inv, __uint_as_float(rb[q8 * 8 + 3]) * inv);
              val.z = pack_bf16x2(__uint_as_float(rb[q8 * 8 + 4]) * inv, __uint_as_float(rb[q8 * 8 + 5]) * inv);
              val.w = pack_bf16x2(__uint_as_float(rb[q8 * 8 + 6]) * inv, __uint_as_float(rb[q8 * 8 + 7]) * inv);
              *reinterpret_cast<uint4*>(dst + 32 + q8 * 8) = val;
            }
            const float l2 = m_ref + log2f(l);
            if (p.lse != nullptr) p.lse[static_cast<long long>(h) * p.M + mrow] = l2 * kLn2;
            p.lse2[static_cast<long long>(h) * p.lse2_stride + mrow] = l2;
          }
        } else {
          // part of an item: unnormalised accumulator, row sum and row reference go to this
          // CTA's slot (slot 1: the item starts here and ends in the next CTA; slot 0: it began
          // in the previous CTA).  Whichever of the two CTAs gets there second joins the parts.
          const bool first_part = t0 == 0;
          const int cut = first_part ? blockIdx.x : blockIdx.x - 1;   // between CTA cut and cut + 1
          float* slot = p.part + static_cast<size_t>(2 * blockIdx.x + (first_part ? 1 : 0)) * kPartFloats;
          float4* orow = reinterpret_cast<float4*>(slot + row * kD);
#pragma unroll
          for (int q4 = 0; q4 < 8; ++q4)
            orow[q4] = make_float4(__uint_as_float(ra[q4 * 4 + 0]), __uint_as_float(ra[q4 * 4 + 1]),
                                   __uint_as_float(ra[q4 * 4 + 2]), __uint_as_float(ra[q4 * 4 + 3]));
#pragma unroll
          for (int q4 = 0; q4 < 8; ++q4)
            orow[8 + q4] = make_float4(__uint_as_float(rb[q4 * 4 + 0]), __uint_as_float(rb[q4 * 4 + 1]),
                                       __uint_as_float(rb[q4 * 4 + 2]), __uint_as_float(rb[q4 * 4 + 3]));
          slot[kBM * kD + row] = l;
          const float m_pub = seg_live ? m_ref : -INFINITY;
          slot[kBM * kD + kBM + row] = m_pub;
          __threadfence();                       // this thread's part is visible device-wide ...
          named_bar_sync(6, 128);                // ... and so is every other row's
          if (row == 0) sm.join_flag = atomicAdd(p.part_count + cut, 1);
          named_bar_sync(6, 128);
          if (sm.join_flag == 1) {
            // the other CTA's part was complete before its counter increment, which came first
            __threadfence();
            const float* other = p.part + static_cast<size_t>(first_part ? 2 * (cut + 1) : 2 * cut + 1) * kPartFloats;
            const float lo_ = __ldcg(other + kBM * kD + row), mo_ = __ldcg(other + kBM * kD + kBM + row);
            // a = the part with the item's first tiles, b = the part with its last ones
            const float la = first_part ? l : lo_, ma = first_part ? m_pub : mo_;
            const float lb = first_part ? lo_ : l, mb = first_part ? mo_ : m_pub;
            const float mm = fmaxf(ma, mb);
            const float m = (mm == -INFINITY) ? 0.f : mm;     // both parts fully masked: zeros, lse = -inf
            const float wa = exp2f(ma - m), wb = exp2f(mb - m);   // a masked part (-inf) weighs nothing
            // explicit operation order: the same bits whichever of the two CTAs computes the join
            const float lsum2 = __fmaf_rn(la, wa, __fmul_rn(lb, wb));
            const float inv = lsum2 > 0.f ? 1.f / lsum2 : 0.f;
            if (mrow < p.M) {
              const float4* orow_o = reinterpret_cast<const float4*>(other + row * kD);
              __nv_bfloat16* dst = p.out + static_cast<long long>(mrow) * p.out_row_stride + h * kD;
              auto join = [&](uint32_t own, float oth) {
                const float x = __uint_as_float(own);
                const float va = first_part ? x : oth, vb = first_part ? oth : x;
                return __fmul_rn(__fmaf_rn(va, wa, __fmul_rn(vb, wb)), inv);
              };
#pragma unroll
              for (int q8 = 0; q8 < 8; ++q8) {
                const float4 o0 = __ldcg(orow_o + 2 * q8), o1 = __ldcg(orow_o + 2 * q8 + 1);
                const uint32_t* r8 = q8 < 4 ? &ra[q8 * 8] : &rb[(q8 - 4) * 8];
                uint4 val;
                val.x = pack_bf16x2(join(r8[0], o0.x), join(r8[1], o0.y));
                val.y = pack_bf16x2(join(r8[2], o0.z), join(r8[3], o0.w));
                val.z = pack_bf16x2(join(r8[4], o1.x), join(r8[5], o1.y));
                val.w = pack_bf16x2(join(r8[6], o1.z), join(r8[7], o1.w));
                *reinterpret_cast<uint4*>(dst + q8 * 8) = val;
              }
              const float l2 = m + log2f(lsum2);
              if (p.lse != nullptr) p.lse[static_cast<long long>(h) * p.M + mrow] = l2 * kLn2;
              p.lse2[static_cast<long long>(h) * p.lse2_stride + mrow] = l2;
            }
          }
        }
      }
      c_base += len;
    }
    if (__any_sync(0xffffffffu, overflow) && lane == 0) atomicOr(p.fallback, 1);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
  STAC_TS(0, true);
}

// ---------------------------------------------------------------------------------------
// Column sums.  An item = (head, group of kColGroup 128-key tiles), head-major; its units are the
// 128-row query tiles.  All units of the launch form one sequence that is cut into equal
// contiguous ranges, one per persistent CTA, so every SM gets the same amount of work; an item
// that straddles a cut is finished by two CTAs, each adding its partial sums to the zeroed
// output with one atomic add per key (two addends onto zero give the same bits in either
// order).  A query tile is scored in two halves of 64 rows: for each half the MMA warp
// computes S^T = K Q^T for the key tiles of the group against the same query rows in shared memory
// (N = 64, two 64-column TMEM buffers per key tile); warpgroup w owns key tile w, one key
// (TMEM lane) per thread, so a thread's column sum never leaves its registers.  Three exponent
// warps per scheduler keep the exp2 unit busier than two did (85 % against 75 % of the active
// cycles); a fourth (kColGroup = 4, 104 registers per thread) measured the same as three.
// lse2 holds the row log-sum-exp in the log2 domain; rows past M_sub read as +inf so that
// padded query columns contribute exp2(-inf) = 0.
// ---------------------------------------------------------------------------------------
constexpr int kColExpThreads = kColGroup * 128;
constexpr int kColHalf = 64;           // query rows per score buffer

struct ColSmem {
  uint8_t k[2][kColGroup][kTileBytes];  // [item parity][key tile of the group]
  uint8_t q[kColStages][kTileBytes];
  uint64_t k_full[2];
  uint64_t k_empty[2];
  uint64_t q_full[kColStages];
  uint64_t q_empty[kColStages];
  uint64_t s_full[2];
  uint64_t s_free[2];
  uint64_t x_full[kColStages];            // the row-term operand of a query stage is written
  uint32_t tmem_base;
  int join_flag;                          // arrival count seen at a shared item
  alignas(16) uint8_t ax[kColXBytes];     // ones in K columns 0..2, same for every key
  alignas(16) uint8_t bx[kColStages][kColXBytes];   // per query row: -lse2 / c2 as hi, mid, lo bf16
  alignas(16) float lse2[4];  // (without the fold) flexible: n_q_tiles * 128 floats follow (negated, one head)
};

struct ColParams {
  int M_sub, H;
  int row_stride;  // query row sub-sampling stride
  int T_hot, T_ret;
  int n_hot_tiles, n_tiles;
  int n_groups, n_items;
  int n_q_tiles;
  int split;       // 1: units are cut evenly over the grid (items may be shared by two CTAs)
  float scale_log2;
  float correction;
  const float* bias_ret;
  long long bias_head_stride;
  const float* lse2;
  long long lse2_stride;
  float* colsum;  // [H, colsum_stride], hot keys first then retrieved
  long long colsum_stride;
  // Fewer items than CTAs: an item may be shared by three or more CTAs.  Each writes its partial
  // sums to a slot of its own (two per CTA: [0] an item that began in an earlier CTA, [1] an
  // item that goes on in the next one), counts its arrival at the item, and the CTA that arrives
  // last adds the parts in CTA order and stores the result: same bits whoever does it.  nullptr:
  // an item has at most two parts, added onto the zeroed output with one atomic each.
  float* parts;       // [2 * gridDim.x][kColGroup * kBN]
  int* part_count;    // [n_items], zero on entry, left zero
  int* err;
};

// The range of units of one CTA, walked item by item (same sequence in every role).
struct ColWalk {
  long long u, u_end;
  int nq;
  __device__ ColWalk(const ColParams& p) {
    nq = p.n_q_tiles;
    if (p.split) {
      const long long total = static_cast<long long>(p.n_items) * nq;
      u = total * blockIdx.x / gridDim.x;
      u_end = total * (blockIdx.x + 1) / gridDim.x;
    } else {
      u = static_cast<long long>(blockIdx.x) * nq;
      u_end = u + nq;
    }
  }
  __device__ bool next(int& item, int& i0, int& i1) {
    if (u >= u_end) return false;
    item = static_cast<int>(u / nq);
    i0 = static_cast<int>(u - static_cast<long long>(item) * nq);
    const long long e = static_cast<long long>(item + 1) * nq;
    i1 = static_cast<int>((e < u_end ? e : u_end) - static_cast<long long>(item) * nq);
    u = static_cast<long long>(item) * nq + i1;
    return true;
  }
};

// 16 scores of one key against 16 query rows: sum of exp2(score * c2 - lse2[row]), two rows at
// a time with the packed fp32 instructions.  The pairs whose bit is set in kColPairMask take
// their exponentials on the FMA pipes (cubic, 8.6e-5 relative): the exponential unit is the
// bottleneck of this kernel.
template <int kJ>
__device__ __forceinline__ uint64_t col_exp_pair(uint64_t s2, uint64_t c2c2, float n0, float n1) {
  const uint64_t x2 = kColFoldLse ? mul_f32x2(s2, c2c2) : fma_f32x2(s2, c2c2, pack_f32x2(n0, n1));
  if ((kColPairMask >> kJ) & 1u) return poly_exp2_x2(x2);
  float x0, x1;
  unpack_f32x2(x2, x0, x1);
  return pack_f32x2(fast_exp2(x0), fast_exp2(x1));
}
__device__ __forceinline__ void col_exp_chunk16(const uint32_t (&s)[32], const float4* nl4, uint64_t c2c2, uint64_t& a01,
                                                uint64_t& a23) {
  float4 n0, n1, n2, n3;
  if (kColFoldLse) {
    n0 = n1 = n2 = n3 = make_float4(0.f, 0.f, 0.f, 0.f);
  } else {
    n0 = nl4[0]; n1 = nl4[1]; n2 = nl4[2]; n3 = nl4[3];
  }
  auto sp = [&](int i) { return pack_f32x2(__uint_as_float(s[i]), __uint_as_float(s[i + 1])); };
  a01 = add_f32x2(a01, col_exp_pair<0>(sp(0), c2c2, n0.x, n0.y));
  a23 = add_f32x2(a23, col_exp_pair<1>(sp(2), c2c2, n0.z, n0.w));
  a01 = add_f32x2(a01, col_exp_pair<2>(sp(4), c2c2, n1.x, n1.y));
  a23 = add_f32x2(a23, col_exp_pair<3>(sp(6), c2c2, n1.z, n1.w));
  a01 = add_f32x2(a01, col_exp_pair<4>(sp(8), c2c2, n2.x, n2.y));
  a23 = add_f32x2(a23, col_exp_pair<5>(sp(10), c2c2, n2.z, n2.w));
  a01 = add_f32x2(a01, col_exp_pair<6>(sp(12), c2c2, n3.x, n3.y));
  a23 = add_f32x2(a23, col_exp_pair<7>(sp(14), c2c2, n3.z, n3.w));
}

// All half tiles of one item for one key (thread): returns the sum over the item's query rows.
// kFast: the key's bias was taken out of the exponent (every lane of the warp agrees).
// A 64-row half is read from TMEM in four pieces of 16 rows, the next piece always in flight
// (the first piece of the next half included: its buffer does not depend on this warpgroup
// finishing the current one).
template <bool kFast>
__device__ __forceinline__ float col_item_sum(ColSmem& sm, const ColParams& p, uint32_t t_base, const float* nl_item,
                                              int n_half, int& ui, float c2, float b2_in) {
  uint32_t ra[32], rb[32];   // 16 registers of each are used
  float a0 = 0.f;
  uint64_t a01 = 0ull, a23 = 0ull;
  const uint64_t c2c2 = pack_f32x2(c2, c2);
  auto consume = [&](const uint32_t (&r)[32], const float* nl) {
    if (kFast) {
      col_exp_chunk16(r, reinterpret_cast<const float4*>(nl), c2c2, a01, a23);
    } else {
#pragma unroll
      for (int q = 0; q < 16; ++q) a0 += fast_exp2(fmaf(__uint_as_float(r[q]), c2, kColFoldLse ? b2_in : b2_in + nl[q]));
    }
  };
  // first half tile of the item: nothing is in flight yet
  {
    const int g = ui & 1, it = ui >> 1;
    mbar_wait(&sm.s_full[g], it & 1, p.err, DEV_TIMEOUT_MMA);
    tc_fence_after();
    tmem_ld16(t_base + g * kColHalf, ra);
  }
  for (int hu = 0; hu < n_half; ++hu, ++ui) {
    const int g = ui & 1;
    const uint32_t s_addr = t_base + g * kColHalf;
    const float* nl = nl_item + hu * kColHalf;
    tmem_ld_wait();
    tmem_ld16(s_addr + 16, rb);
    consume(ra, nl);
    tmem_ld_wait();
    tmem_ld16(s_addr + 32, ra);
    consume(rb, nl + 16);
    tmem_ld_wait();
    tmem_ld16(s_addr + 48, rb);
    consume(ra, nl + 32);
    tmem_ld_wait();
    if (hu + 1 < n_half) {
      const int g2 = (ui + 1) & 1, it2 = (ui + 1) >> 1;
      mbar_wait(&sm.s_full[g2], it2 & 1, p.err, DEV_TIMEOUT_MMA);
      tc_fence_after();
      tmem_ld16(t_base + g2 * kColHalf, ra);
    }
    consume(rb, nl + 48);
    tc_fence_before();
    mbar_arrive(&sm.s_free[g]);
  }
  float b0, b1, b2, b3;
  unpack_f32x2(a01, b0, b1);
  unpack_f32x2(a23, b2, b3);
  return a0 + ((b0 + b1) + (b2 + b3));
}

__global__ void __launch_bounds__(kColThreads, 1)
attn_colsum_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k_hot,
                   const __grid_constant__ CUtensorMap tm_k_ret, const ColParams p) {
  extern __shared__ uint8_t smem_raw[];
  ColSmem& sm = *reinterpret_cast<ColSmem*>(align1024(smem_raw));
  STAC_TS(2, false);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int nq = p.n_q_tiles;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sm.k_full[i], 1);
      mbar_init(&sm.k_empty[i], 1);
      mbar_init(&sm.s_full[i], 1);
      mbar_init(&sm.s_free[i], kColExpThreads);
    }
    for (int s = 0; s < kColStages; ++s) {
      mbar_init(&sm.q_full[s], 1);
      mbar_init(&sm.q_empty[s], 1);
      mbar_init(&sm.x_full[s], 1);
    }
    mbar_fence_init();
  }
  if (kColFoldLse && threadIdx.x >= 128 && threadIdx.x < 256) {
    // the constant operand: row r = (1, 1, 1, 0, ..., 0) in bf16
    const int r = threadIdx.x - 128;
    uint8_t* dst = sm.ax + (r >> 3) * 256 + (r & 7) * 16;
    *reinterpret_cast<uint4*>(dst) = make_uint4(0x3F803F80u, 0x00003F80u, 0u, 0u);
    *reinterpret_cast<uint4*>(dst + 128) = make_uint4(0u, 0u, 0u, 0u);
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    tmem_alloc(&sm.tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;
  // Launched with programmatic serialization behind the forward kernels: barriers and tensor
  // memory are set up while they drain; the row log-sum-exps and the zeroed output are read
  // and written only after this point.
  grid_dep_wait();

  if (warp < 4) {
    setmaxnreg_dec<kColCtlRegs>();
    if (warp == 0 && lane == 0) {
      // ------------------------------------------------------------------ TMA producer
      tma_prefetch_desc(&tm_q);
      ColWalk walk(p);
      int n = 0, item, i0, i1;
      int s = 0, s_round = 0;   // stage and round of the query ring
      for (; walk.next(item, i0, i1); ++n) {
        const int h = item / p.n_groups, grp = item - h * p.n_groups;   // head-major item order
        const int kb = n & 1;
        if (n >= 2) mbar_wait(&sm.k_empty[kb], ((n >> 1) - 1) & 1, p.err, DEV_TIMEOUT_CONSUMER);
        mbar_arrive_expect_tx(&sm.k_full[kb], kColGroup * kTileBytes);
#pragma unroll
        for (int t = 0; t < kColGroup; ++t) {
          const int j = min(kColGroup * grp + t, p.n_tiles - 1);
          if (j < p.n_hot_tiles) tma_load_3d(sm.k[kb][t], &tm_k_hot, &sm.k_full[kb], 0, j * kBN, h);
          else tma_load_3d(sm.k[kb][t], &tm_k_ret, &sm.k_full[kb], 0, (j - p.n_hot_tiles) * kBN, h);
        }
        for (int i = i0; i < i1; ++i) {
          if (s_round > 0) mbar_wait(&sm.q_empty[s], (s_round - 1) & 1, p.err, DEV_TIMEOUT_CONSUMER);
          mbar_arrive_expect_tx(&sm.q_full[s], kTileBytes);
          tma_load_3d(sm.q[s], &tm_q, &sm.q_full[s], 0, h, i * kBM);
          if (++s == kColStages) { s = 0; ++s_round; }
        }
      }
    } else if (kColFoldLse && warp == 2) {
      // ------------------------------------------------------------------ row-term producer
      // For every query tile: x[m] = -lse2[m] / c2 split into three bf16 (24 bits together), so
      // that ones . (hi, mid, lo) added to the scores by the tensor core makes
      // (s + x) * c2 = s * c2 - lse2.  Rows past M_sub get a huge negative term: their
      // exponentials are exactly zero.
      ColWalk walk(p);
      const float inv_c2 = 1.f / p.scale_log2;
      int item, i0, i1;
      int s = 0, s_round = 0;
      while (walk.next(item, i0, i1)) {
        const int h = item / p.n_groups;
        for (int i = i0; i < i1; ++i) {
          if (s_round > 0) mbar_wait(&sm.q_empty[s], (s_round - 1) & 1, p.err, DEV_TIMEOUT_CONSUMER);
#pragma unroll
          for (int rr = 0; rr < 4; ++rr) {
            const int row = lane * 4 + rr;
            const int m = i * kBM + row;
            float x = -1e30f;
            if (m < p.M_sub)
              x = -p.lse2[static_cast<long long>(h) * p.lse2_stride + static_cast<long long>(m) * p.row_stride] * inv_c2;
            if (!(fabsf(x) < 1e30f)) x = -1e30f;   // lse2 = -inf (a row without live keys) or NaN: contributes nothing
            const __nv_bfloat16 hi = __float2bfloat16_rn(x);
            const float r1 = x - __bfloat162float(hi);
            const __nv_bfloat16 mid = __float2bfloat16_rn(r1);
            const __nv_bfloat16 lo = __float2bfloat16_rn(r1 - __bfloat162float(mid));
            uint8_t* dst = sm.bx[s] + (row >> 3) * 256 + (row & 7) * 16;
            const uint32_t w0 = static_cast<uint32_t>(__bfloat16_as_ushort(hi)) |
                                (static_cast<uint32_t>(__bfloat16_as_ushort(mid)) << 16);
            *reinterpret_cast<uint4*>(dst) = make_uint4(w0, static_cast<uint32_t>(__bfloat16_as_ushort(lo)), 0u, 0u);
            *reinterpret_cast<uint4*>(dst + 128) = make_uint4(0u, 0u, 0u, 0u);
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(&sm.x_full[s]);
          if (++s == kColStages) { s = 0; ++s_round; }
        }
      }
    } else if (warp == 1) {
      // ------------------------------------------------------------------ MMA issuer
      // (all lanes run the loop so that descriptors are warp-uniform; one elected lane issues)
      constexpr uint32_t idesc = umma_idesc_bf16(kBN, kColHalf, 0);
      const uint64_t ax_desc = smem_desc_nosw(smem_u32(sm.ax), 128, 256);
      const uint64_t bx_desc0 = smem_desc_nosw(smem_u32(sm.bx[0]), 128, 256);
      ColWalk walk(p);
      const uint64_t k_desc0 = smem_desc_sw128(smem_u32(sm.k[0][0]));
      const uint64_t q_desc0 = smem_desc_sw128(smem_u32(sm.q[0]));
      int ui = 0, n = 0, item, i0, i1;   // ui: running count of half tiles
      int s = 0, s_round = 0;
      for (; walk.next(item, i0, i1); ++n) {
        const int kb = n & 1;
        mbar_wait(&sm.k_full[kb], (n >> 1) & 1, p.err, DEV_TIMEOUT_TMA);
        const uint64_t k_desc = k_desc0 + static_cast<uint64_t>(kb * kColGroup * (kTileBytes >> 4));
        for (int i = i0; i < i1; ++i) {
          mbar_wait(&sm.q_full[s], s_round & 1, p.err, DEV_TIMEOUT_TMA);
          if (kColFoldLse) mbar_wait(&sm.x_full[s], s_round & 1, p.err, DEV_TIMEOUT_CONSUMER);
#pragma unroll
          for (int half = 0; half < 2; ++half, ++ui) {
            const int g = ui & 1, it = ui >> 1;
            // query rows 64*half.. of the tile: 8192 bytes further in the K-major tile
            const uint64_t q_desc = q_desc0 + static_cast<uint64_t>(s * (kTileBytes >> 4) + half * (8192 >> 4));
            const uint32_t d = tmem + g * kColHalf;
            if (it > 0) mbar_wait(&sm.s_free[g], (it - 1) & 1, p.err, DEV_TIMEOUT_CONSUMER);
            tc_fence_after();
            if (elect_one()) {
#pragma unroll
              for (int t = 0; t < kColGroup; ++t) {
                const uint64_t kd = k_desc + static_cast<uint64_t>(t * (kTileBytes >> 4));
                umma_ss(d + t * 128, kd, q_desc, idesc, 0u);
                umma_ss(d + t * 128, kd + 2, q_desc + 2, idesc, 1u);
                umma_ss(d + t * 128, kd + 4, q_desc + 4, idesc, 1u);
                umma_ss(d + t * 128, kd + 6, q_desc + 6, idesc, 1u);
                // the 64 rows of this half: eight row groups of 256 bytes further in the operand
                if (kColFoldLse)
                  umma_ss(d + t * 128, ax_desc, bx_desc0 + static_cast<uint64_t>((s * kColXBytes + half * 2048) >> 4),
                          idesc, 1u);
              }
              umma_commit(&sm.s_full[g]);
              if (half == 1) {
                umma_commit(&sm.q_empty[s]);
                if (i == i1 - 1) umma_commit(&sm.k_empty[kb]);
              }
            }
            __syncwarp();
          }
          if (++s == kColStages) { s = 0; ++s_round; }
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ exponent warpgroups
    setmaxnreg_inc<kColExpRegs>();
    const int w = (warp - 4) >> 2;   // which key tile of the group
    const int wq = warp & 3;
    const int key = wq * 32 + lane;  // key inside the tile = TMEM lane
    const int tid = threadIdx.x - 128;  // 0..383
    const uint32_t t_base = tmem + (static_cast<uint32_t>(wq * 32) << 16) + w * 128;
    const float c2 = p.scale_log2;
    ColWalk walk(p);
    int ui = 0, n = 0, item, i0, i1;
    int cur_h = -1;
    for (; walk.next(item, i0, i1); ++n) {
      const int h = item / p.n_groups, grp = item - h * p.n_groups;   // head-major item order
      // negated row log-sum-exps of the head's query rows, reloaded only when the head changes
      // (a CTA's items are consecutive, so that is once or twice per launch)
      float* nl_s = sm.lse2;
      if (!kColFoldLse && h != cur_h) {
        cur_h = h;
        named_bar_sync(1, kColExpThreads);   // everyone is done with the previous head's values
        for (int r = tid; r < nq * kBM; r += kColExpThreads) {
          float v = -INFINITY;
          if (r < p.M_sub)
            v = -p.lse2[static_cast<long long>(h) * p.lse2_stride + static_cast<long long>(r) * p.row_stride];
          nl_s[r] = v;
        }
        named_bar_sync(1, kColExpThreads);
      }
      const int j = kColGroup * grp + w;
      const bool exists = j < p.n_tiles;
      const bool is_ret = j >= p.n_hot_tiles;
      const int n0 = (is_ret ? j - p.n_hot_tiles : j) * kBN;
      const int valid = exists ? min(kBN, (is_ret ? p.T_ret : p.T_hot) - n0) : 0;
      // the key's bias multiplies its whole column: exp2(s c2 + b2 - lse2) = 2^b2 exp2(s c2 - lse2);
      // taken out of the exponent while it is small, else kept inside (rare, slower path)
      float b2 = 0.f;
      if (key < valid && is_ret) b2 = p.bias_ret[h * p.bias_head_stride + n0 + key] * kLog2e;
      // a bias of -inf (padding behind the valid pivots) masks the key: its column sum is 0
      const bool masked = b2 == -INFINITY;
      if (masked) b2 = 0.f;
      const bool b2_small = fabsf(b2) <= 32.f;
      const float b2_in = b2_small ? 0.f : b2;
      const bool warp_fast = __all_sync(0xffffffffu, b2_small);
      const int n_half = 2 * (i1 - i0);
      const float* nl_item = nl_s + i0 * kBM;
      // (warps whose 32 keys are all masked still run the sums: letting them only follow the
      // score buffers was measured slower in the stream, their polling disturbs the others)
      float sum = warp_fast ? col_item_sum<true>(sm, p, t_base, nl_item, n_half, ui, c2, 0.f)
                            : col_item_sum<false>(sm, p, t_base, nl_item, n_half, ui, c2, b2_in);
      if (key < valid) {
        sum *= p.correction;
        if (b2_small) sum *= exp2f(b2);
        if (masked) sum = 0.f;
      }
      float* dst = p.colsum + static_cast<long long>(h) * p.colsum_stride + (is_ret ? p.T_hot : 0) + n0 + key;
      if (i0 == 0 && i1 == nq) {
        if (key < valid) *dst = sum;
      } else if (p.parts == nullptr) {
        if (key < valid) atomicAdd(dst, sum);
      } else {
        constexpr int kSlot = kColGroup * kBN;
        float* slot = p.parts + static_cast<size_t>(2 * blockIdx.x + (i0 > 0 ? 0 : 1)) * kSlot;
        slot[w * kBN + key] = key < valid ? sum : 0.f;
        __threadfence();                          // this thread's part is visible device-wide ...
        named_bar_sync(1, kColExpThreads);        // ... and so is every other key's
        if (tid == 0) sm.join_flag = atomicAdd(p.part_count + item, 1);
        named_bar_sync(1, kColExpThreads);
        // CTA c owns the units [total * c / G, total * (c + 1) / G): owner(u) = ((u + 1) * G - 1) / total
        const long long total = static_cast<long long>(p.n_items) * nq, G = gridDim.x;
        const int c_first = static_cast<int>(((static_cast<long long>(item) * nq + 1) * G - 1) / total);
        const int c_last = static_cast<int>(((static_cast<long long>(item + 1) * nq) * G - 1) / total);
        if (sm.join_flag == c_last - c_first) {
          // every other part was complete before its counter increment, which came earlier
          __threadfence();
          if (key < valid) {
            float acc = 0.f;
            for (int c = c_first; c <= c_last; ++c)
              acc = __fadd_rn(acc, __ldcg(p.parts + static_cast<size_t>(2 * c + (c == c_first ? 1 : 0)) * kSlot + w * kBN + key));
            *dst = acc;
          }
          if (tid == 0) p.part_count[item] = 0;
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
  STAC_TS(2, true);
}

// ---------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// bf16 tensor seen as [d2][d1][64]; box = 64 x box1 x box2 elements, 128-byte swizzle.
int make_map(CUtensorMap* map, const void* base, uint64_t d1, uint64_t d2, uint64_t stride1_bytes,
             uint64_t stride2_bytes, uint32_t box1, uint32_t box2) {
  EncodeTiledFn enc = get_encode_fn();
  if (enc == nullptr) return STAC_ERR_CUDA;
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(kD), d1, d2};
  cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
  cuuint32_t box[3] = {static_cast<cuuint32_t>(kD), box1, box2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? STAC_OK : STAC_ERR_CUDA;
}

}  // namespace

void attn_subsample_plan(int M, float ratio, int* m_sub, int* stride, float* correction) {
  // attn-cuda/csrc/bindings.cpp:63-83
  if (ratio >= 0.999999f) {
    *m_sub = M; *stride = 1; *correction = 1.f;
    return;
  }
  int ms = static_cast<int>(M * ratio);
  if (ms < 128) ms = 128;
  ms = (ms / 128) * 128;
  if (ms >= M) {
    *m_sub = M; *stride = 1; *correction = 1.f;
  } else {
    *m_sub = ms;
    *stride = M / ms < 1 ? 1 : M / ms;
    *correction = static_cast<float>(M) / static_cast<float>(ms);
  }
}

// row log-sum-exps [H, M] followed by the fallback flag (64 floats of padding keep it aligned)
// fallback flag and the arrival counters of the split forward kernel follow the [H, M] values
size_t attn_lse2_elems(int M, int H) { return static_cast<size_t>(H) * static_cast<size_t>(M) + 64; }
size_t attn_lse2_elems_split(int M, int H) { return static_cast<size_t>(H) * static_cast<size_t>(M) + 512; }

// partial results of the split forward kernel (two slots per CTA), then the partial column sums of
// a column-sum launch with fewer items than CTAs (two slots per CTA)
constexpr size_t kFwdPartElems = static_cast<size_t>(2) * kFastMaxCtas * kPartFloats;
constexpr size_t kColPartElems = static_cast<size_t>(2) * kFastMaxCtas * kColGroup * kBN;
size_t attn_part_elems() { return kFwdPartElems + kColPartElems; }

int attn_colsum_launch(const AttnArgs& a, float* lse2, float* part, int* err, cudaStream_t stream) {
  if (a.D != kD) return STAC_ERR_BAD_ARG;
  if (a.M <= 0 || a.H <= 0 || a.T_hot < 0 || a.T_ret < 0 || a.T_hot + a.T_ret <= 0) return STAC_ERR_BAD_ARG;
  if (a.T_ret > 0 && (a.k_ret == nullptr || a.v_ret == nullptr || a.bias_ret == nullptr)) return STAC_ERR_BAD_ARG;
  if (a.T_hot > 0 && (a.k_hot == nullptr || a.v_hot == nullptr)) return STAC_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(a.q) | reinterpret_cast<uintptr_t>(a.k_hot) | reinterpret_cast<uintptr_t>(a.v_hot) |
       reinterpret_cast<uintptr_t>(a.k_ret) | reinterpret_cast<uintptr_t>(a.v_ret) |
       reinterpret_cast<uintptr_t>(a.out)) & 15)
    return STAC_ERR_BAD_ARG;

  int dev = 0;
  if (current_device(&dev) != STAC_OK) return STAC_ERR_CUDA;
  static PerDeviceFlag attr_done;   // the shared-memory opt-in is made once per device
  const int fwd_smem = static_cast<int>(sizeof(FwdSmem)) + 1024;
  int m_sub, stride;
  float corr;
  attn_subsample_plan(a.M, a.subsample_ratio, &m_sub, &stride, &corr);
  const int nq = (m_sub + kBM - 1) / kBM;
  const int col_smem = static_cast<int>(sizeof(ColSmem)) + (kColFoldLse ? 0 : nq * kBM * 4) + 1024;
  if (col_smem > 227 * 1024) return STAC_ERR_BAD_ARG;
  const int fast_smem = static_cast<int>(sizeof(FastSmem)) + 1024;
  if (attr_done.needs_setup(dev)) {
    if (cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, fwd_smem) != cudaSuccess)
      return STAC_ERR_CUDA;
    if (cudaFuncSetAttribute(attn_fwd_fast_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, fast_smem) !=
        cudaSuccess)
      return STAC_ERR_CUDA;
    if (cudaFuncSetAttribute(attn_colsum_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) !=
        cudaSuccess)
      return STAC_ERR_CUDA;
    attr_done.mark(dev);
  }

  const uint64_t eb = 2;  // bytes per element
  CUtensorMap tm_q, tm_qs, tm_kh, tm_vh, tm_kr, tm_vr;
  CUtensorMap tf_kh, tf_vh, tf_kr, tf_vr;   // the same tensors in 112-key boxes (fast kernel)
  int rc;
  // q[m, h, :]: dims {64, H, M}
  rc = make_map(&tm_q, a.q, a.H, a.M, kD * eb, a.q_row_stride * eb, 1, kBM);
  if (rc) return rc;
  rc = make_map(&tm_qs, a.q, a.H, m_sub, kD * eb, a.q_row_stride * eb * stride, 1, kBM);
  if (rc) return rc;
  // placeholders keep the maps valid when a segment is empty
  const void* kh = a.T_hot > 0 ? a.k_hot : a.k_ret;
  const void* vh = a.T_hot > 0 ? a.v_hot : a.v_ret;
  const int th = a.T_hot > 0 ? a.T_hot : a.T_ret;
  const long long sh = a.T_hot > 0 ? a.hot_head_stride : a.ret_head_stride;
  const long long rh = a.T_hot > 0 ? a.hot_row_stride : a.ret_row_stride;
  const void* kr = a.T_ret > 0 ? a.k_ret : a.k_hot;
  const void* vr = a.T_ret > 0 ? a.v_ret : a.v_hot;
  const int tr = a.T_ret > 0 ? a.T_ret : a.T_hot;
  const long long sr = a.T_ret > 0 ? a.ret_head_stride : a.hot_head_stride;
  const long long rr = a.T_ret > 0 ? a.ret_row_stride : a.hot_row_stride;
  rc = make_map(&tm_kh, kh, th, a.H, rh * eb, sh * eb, kBN, 1);
  if (rc) return rc;
  rc = make_map(&tm_vh, vh, th, a.H, rh * eb, sh * eb, kBN, 1);
  if (rc) return rc;
  rc = make_map(&tm_kr, kr, tr, a.H, rr * eb, sr * eb, kBN, 1);
  if (rc) return rc;
  rc = make_map(&tm_vr, vr, tr, a.H, rr * eb, sr * eb, kBN, 1);
  if (rc) return rc;
  rc = make_map(&tf_kh, kh, th, a.H, rh * eb, sh * eb, kFT, 1);
  if (rc) return rc;
  rc = make_map(&tf_vh, vh, th, a.H, rh * eb, sh * eb, kFT, 1);
  if (rc) return rc;
  rc = make_map(&tf_kr, kr, tr, a.H, rr * eb, sr * eb, kFT, 1);
  if (rc) return rc;
  rc = make_map(&tf_vr, vr, tr, a.H, rr * eb, sr * eb, kFT, 1);
  if (rc) return rc;

  const float scale_log2 = a.scale * kLog2e;
  FwdParams fp;
  fp.M = a.M; fp.H = a.H; fp.T_hot = a.T_hot; fp.T_ret = a.T_ret;
  fp.n_hot_tiles = (a.T_hot + kBN - 1) / kBN;
  fp.n_ret_tiles = (a.T_ret + kBN - 1) / kBN;
  fp.scale_log2 = scale_log2;
  fp.bias_ret = a.bias_ret; fp.bias_head_stride = a.bias_head_stride;
  fp.out = static_cast<__nv_bfloat16*>(a.out); fp.out_row_stride = a.out_row_stride;
  fp.lse = a.lse; fp.lse2 = lse2; fp.lse2_stride = a.M;
  fp.err = err;
  fp.fallback = reinterpret_cast<int*>(lse2 + static_cast<size_t>(a.H) * a.M);
  dim3 grid_f((a.M + kBM - 1) / kBM, a.H);
  int n_sm = 0;
  if (device_sm_count(dev, &n_sm) != STAC_OK) return STAC_ERR_CUDA;
  // fast kernel (fixed per-row reference) first; the exact kernel behind it returns at once
  // unless the fast one raised the flag.  With at least one item per SM (and a workspace for
  // the parts) the units are cut evenly over one CTA per SM; with at most half as many items as
  // SMs (few heads, e.g. a head-sharded stream) every item is cut in two halves, one CTA each;
  // else every CTA takes one item.  Either way an item is shared by at most two CTAs.
  fp.n_q_tiles = static_cast<int>(grid_f.x);
  fp.n_items = fp.n_q_tiles * a.H;
  const int n_tiles_f = (a.T_hot + kFT - 1) / kFT + (a.T_ret + kFT - 1) / kFT;
  int grid_split = 0;
  if (part != nullptr && n_sm <= kFastMaxCtas && n_tiles_f >= kFastMinSplitTiles) {
    if (fp.n_items >= n_sm) grid_split = n_sm;
    else if (2 * fp.n_items <= n_sm && n_tiles_f >= 2 * kFastMinSplitTiles) grid_split = 2 * fp.n_items;
  }
  fp.split = grid_split > 0 ? 1 : 0;
  fp.part = part;
  fp.part_count = fp.fallback + 1;      // only used (and only present in the workspace) when split
  const int grid_fast = fp.split ? grid_split : fp.n_items;
  // Column sums: with at least one item per SM the units are cut evenly over one CTA per SM and an
  // item on a cut gets one atomic add per key from each of its two CTAs (the forward kernel clears
  // the output for that).  With fewer items (few heads, short key ranges) and a workspace, the
  // units are still cut evenly; an item may then have three or more parts, which go through the
  // workspace and are added in CTA order by the CTA that finishes last.
  const int col_items = ((fp.n_hot_tiles + fp.n_ret_tiles + kColGroup - 1) / kColGroup) * a.H;
  const bool col_split = a.colsum != nullptr && col_items >= n_sm;
  // (worth it from about six units per CTA: below that the extra key-tile loads and the join of a
  // CTA that touches two items cost more than the even cut gains; measured at M = 1041, N = 2082)
  const bool col_parts = a.colsum != nullptr && !col_split && part != nullptr && n_sm <= kFastMaxCtas &&
                         static_cast<long long>(col_items) * ((m_sub + kBM - 1) / kBM) >= 6ll * n_sm;
  // flag, arrival counters of the forward cuts, arrival counters of the shared column-sum items
  if (cudaMemsetAsync(fp.fallback, 0, sizeof(int) * (col_parts ? 1 + 2 * kFastMaxCtas : fp.split ? 1 + kFastMaxCtas : 1),
                      stream) != cudaSuccess)
    return STAC_ERR_CUDA;
  fp.zero_colsum = col_split ? a.colsum : nullptr;
  fp.zero_stride = a.colsum_head_stride;
  fp.zero_width = a.T_hot + a.T_ret;
  attn_fwd_fast_kernel<<<grid_fast, kFastThreads, fast_smem, stream>>>(tm_q, tf_kh, tf_vh, tf_kr, tf_vr, fp);
  if (cudaGetLastError() != cudaSuccess) return STAC_ERR_CUDA;
  if (launch_behind(attn_fwd_kernel, grid_f, dim3(kFwdThreads), fwd_smem, stream, tm_q, tm_kh, tm_vh, tm_kr, tm_vr,
                    fp) != cudaSuccess)
    return STAC_ERR_CUDA;

  if (a.colsum != nullptr) {
    ColParams cp;
    cp.M_sub = m_sub; cp.H = a.H; cp.row_stride = stride;
    cp.T_hot = a.T_hot; cp.T_ret = a.T_ret;
    cp.n_hot_tiles = fp.n_hot_tiles; cp.n_q_tiles = nq;
    cp.n_tiles = fp.n_hot_tiles + fp.n_ret_tiles;
    cp.n_groups = (cp.n_tiles + kColGroup - 1) / kColGroup;
    cp.n_items = cp.n_groups * a.H;
    cp.scale_log2 = scale_log2; cp.correction = corr;
    cp.bias_ret = a.bias_ret; cp.bias_head_stride = a.bias_head_stride;
    cp.lse2 = lse2; cp.lse2_stride = a.M;
    cp.colsum = a.colsum; cp.colsum_stride = a.colsum_head_stride;
    cp.err = err;
    // enough items: cut the units evenly over one CTA per SM (an item is then shared by at most
    // two CTAs, which add their partial sums onto zeros); else one item per CTA
    cp.split = (col_split || col_parts) ? 1 : 0;      // col_split: the forward kernel has cleared a.colsum
    cp.parts = col_parts ? part + kFwdPartElems : nullptr;
    cp.part_count = fp.fallback + 1 + kFastMaxCtas;
    const int grid_c = cp.split ? n_sm : cp.n_items;
    if (launch_behind(attn_colsum_kernel, dim3(grid_c), dim3(kColThreads), col_smem, stream, tm_qs, tm_kh, tm_kr,
                      cp) != cudaSuccess)
      return STAC_ERR_CUDA;
  }
  return STAC_OK;
}

}  // namespace stac

// ---------------------------------------------------------------------------------------
// Allocation-free variant: the row log-sum-exp scratch lives in a fixed array inside the
// loaded module instead of a caller-provided workspace.
// ---------------------------------------------------------------------------------------
namespace stac {
namespace {

// One float per (head, query row).  Every GPU that loads the library carries these 512 KB
// until the process exits.
static __device__ __align__(256) float g_static_lse2[STAC_ATTN_STATIC_MAX_ROWS + 64];  // + fallback flag

float* g_static_lse2_ptr[kMaxDevices] = {nullptr};

// The array's name is only a host-side handle; the kernels need its device address, which
// differs per GPU.  Resolved once per device, with that device current.
int static_scratch_for_current_device(float** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return STAC_ERR_CUDA;
  if (g_static_lse2_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_static_lse2) != cudaSuccess || ptr == nullptr) return STAC_ERR_CUDA;
    g_static_lse2_ptr[dev] = static_cast<float*>(ptr);
  }
  *out = g_static_lse2_ptr[dev];
  return STAC_OK;
}

}  // namespace
}  // namespace stac

extern "C" int stac_attn_colsum_noalloc(const void* q, int64_t q_row_stride, const void* k_hot, const void* v_hot,
                                        int64_t hot_row_stride, int64_t hot_head_stride, int T_hot,
                                        const void* k_ret, const void* v_ret, int64_t ret_row_stride,
                                        int64_t ret_head_stride, int T_ret, const float* bias_ret,
                                        int64_t bias_head_stride, void* out, int64_t out_row_stride, float* lse,
                                        float* colsum, int64_t colsum_head_stride, int M, int H, int D, float scale,
                                        float subsample_ratio, int* dev_status, stac_stream_t stream) {
  if (q == nullptr || out == nullptr) return STAC_ERR_BAD_ARG;
  if (!(subsample_ratio > 0.f && subsample_ratio <= 1.f)) return STAC_ERR_BAD_ARG;
  if (M <= 0 || H <= 0) return STAC_ERR_BAD_ARG;
  // the fixed scratch holds H * M floats at most
  if (static_cast<long long>(M) * H > STAC_ATTN_STATIC_MAX_ROWS) return STAC_ERR_CAPACITY;
  if ((q_row_stride % 8) || (out_row_stride % 8) || (hot_head_stride % 8) || (ret_head_stride % 8) ||
      (hot_row_stride % 8) || (ret_row_stride % 8))
    return STAC_ERR_BAD_ARG;
  float* scratch = nullptr;
  const int rc = stac::static_scratch_for_current_device(&scratch);
  if (rc != STAC_OK) return rc;
  stac::AttnArgs a;
  a.q = q; a.q_row_stride = q_row_stride;
  a.k_hot = k_hot; a.v_hot = v_hot; a.hot_row_stride = hot_row_stride; a.hot_head_stride = hot_head_stride;
  a.T_hot = T_hot;
  a.k_ret = k_ret; a.v_ret = v_ret; a.ret_row_stride = ret_row_stride; a.ret_head_stride = ret_head_stride;
  a.T_ret = T_ret;
  a.bias_ret = bias_ret; a.bias_head_stride = bias_head_stride;
  a.out = out; a.out_row_stride = out_row_stride;
  a.lse = lse; a.colsum = colsum; a.colsum_head_stride = colsum_head_stride;
  a.M = M; a.H = H; a.D = D; a.scale = scale; a.subsample_ratio = subsample_ratio;
  // Every entry of the scratch that the column-sum pass reads (rows < M of each head) is
  // written by the forward pass of this same call, so nothing has to be cleared first.
  return stac::attn_colsum_launch(a, scratch, nullptr, dev_status, reinterpret_cast<cudaStream_t>(stream));
}

#ifdef STAC_TIMESTAMPS
extern "C" int stac_debug_stamps(unsigned long long* out, int reset) {
  if (out != nullptr && cudaMemcpyFromSymbol(out, stac::g_ts, sizeof(unsigned long long) * 8) != cudaSuccess) return 1;
  if (reset) {
    const unsigned long long init[8] = {~0ull, 0ull, ~0ull, 0ull, ~0ull, 0ull, ~0ull, 0ull};
    if (cudaMemcpyToSymbol(stac::g_ts, init, sizeof(init)) != cudaSuccess) return 1;
  }
  return 0;
}
#endif
