// Point -> voxel id table on the GPU: quantise, pack, upsert with the reference's deterministic
// id assignment, and the Chebyshev-cube neighbour query.
//
// Replaces stac/stac_voxel.py:339-347 (quantise + upsert call), stac/voxel.py:60-71 (key
// packing), stac/voxel.py:195-324 (BinaryVoxel.upsert: sorted-cache searchsorted, unique of
// the new keys, whole-table re-sort) and stac/voxel.py:371-521 + stac/stac_voxel.py:294-323
// (neighbour enumeration through a [Q,125] distance matrix and topk).
//
// Membership is an open-addressing hash table (64-bit packed key -> id).  Ids stay those of
// the reference: keys unseen so far are sorted among themselves and get n_old + rank
// (stac/voxel.py:277-278, 315-316), which one CTA computes with a bitonic sort in shared
// memory; the table itself is never re-sorted.
#include "common.cuh"
#include "stac_internal.h"

namespace stac {
namespace {

constexpr unsigned long long kEmpty = ~0ull;
constexpr int kSortCap = STAC_VOXEL_MAX_POINTS;  // points (hence new keys) per call
constexpr int kSortSmemKeys = 16384;              // new keys that the sort holds in shared memory

__device__ __forceinline__ unsigned long long hash64(unsigned long long x) {
  x ^= x >> 33;
  x *= 0xff51afd7ed558ccdull;
  x ^= x >> 33;
  x *= 0xc4ceb9fe1a85ec53ull;
  x ^= x >> 33;
  return x;
}

__device__ __forceinline__ int hash_lookup(const unsigned long long* hk, const int* hv, int cap, long long key) {
  const unsigned long long k = static_cast<unsigned long long>(key);
  unsigned int slot = static_cast<unsigned int>(hash64(k)) & (cap - 1);
  for (int probe = 0; probe < cap; ++probe) {
    const unsigned long long cur = hk[slot];
    if (cur == k) return hv[slot];
    if (cur == kEmpty) return -1;
    slot = (slot + 1) & (cap - 1);
  }
  return -1;
}

// key = (i + 2^20) + (j + 2^20) * 2^21 + (k + 2^20) * 2^42   (stac/voxel.py:60-71)
__device__ __forceinline__ long long pack_key(int i, int j, int k) {
  const long long off = 1ll << 20;
  return (static_cast<long long>(i) + off) + (static_cast<long long>(j) + off) * (1ll << 21) +
         (static_cast<long long>(k) + off) * (1ll << 42);
}

// One thread per point: ijk = floor(p / voxel_size) with an IEEE division (not a multiply by
// the reciprocal, which differs by one cell at boundaries), lookup, and collection of the
// keys that are not in the table yet.
__global__ void quantize_lookup_kernel(const float* __restrict__ pts, const int* __restrict__ ijk,
                                       const unsigned char* __restrict__ mask, int n,
                                       float vs, const unsigned long long* __restrict__ hk,
                                       const int* __restrict__ hv, int hcap, long long* __restrict__ pt_keys,
                                       int* __restrict__ ids, long long* __restrict__ new_keys,
                                       int* __restrict__ new_cnt) {
  grid_dep_wait();   // launched with programmatic serialization behind the previous kernel in the stream
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  if (mask != nullptr && mask[i] == 0) {
    ids[i] = -1;
    pt_keys[i] = -1;
    return;
  }
  int a, b, c;
  if (ijk != nullptr) {
    a = ijk[3 * i + 0];
    b = ijk[3 * i + 1];
    c = ijk[3 * i + 2];
  } else {
    a = static_cast<int>(floorf(__fdiv_rn(pts[3 * i + 0], vs)));
    b = static_cast<int>(floorf(__fdiv_rn(pts[3 * i + 1], vs)));
    c = static_cast<int>(floorf(__fdiv_rn(pts[3 * i + 2], vs)));
  }
  const long long key = pack_key(a, b, c);
  pt_keys[i] = key;
  const int id = hash_lookup(hk, hv, hcap, key);
  if (id >= 0) {
    ids[i] = id;
  } else {
    ids[i] = -2;  // resolved after the insert
    const int pos = atomicAdd(new_cnt, 1);
    new_keys[pos] = key;
  }
}

// Single CTA: sort the pending keys, drop duplicates, give the survivors ids n_old + rank in
// ascending key order, append them to the id -> key table and insert them in the hash table.
// Up to kSortSmemKeys keys are sorted in shared memory; a call with more new keys than that
// (chunks of sixteen frames and more, all on unseen ground) sorts them where they lie, in the
// scratch list, which has room for the padding up to the next power of two.
__global__ void __launch_bounds__(1024, 1)
insert_new_kernel(long long* new_keys, const int* __restrict__ new_cnt,
                  long long* __restrict__ table_keys, int table_cap, unsigned long long* __restrict__ hk,
                  int* __restrict__ hv, int hcap, int* __restrict__ n_voxels, int* err) {
  grid_dep_wait();   // launched with programmatic serialization behind the previous kernel in the stream
  extern __shared__ unsigned long long smem_keys[];
  __shared__ int warp_sums[32];
  __shared__ int carry;
  const int n = *new_cnt;
  if (n == 0) return;
  int np2 = 1;
  while (np2 < n) np2 <<= 1;
  unsigned long long* skeys = smem_keys;
  if (np2 <= kSortSmemKeys) {
    for (int i = threadIdx.x; i < np2; i += blockDim.x)
      skeys[i] = i < n ? static_cast<unsigned long long>(new_keys[i]) : kEmpty;
  } else {
    skeys = reinterpret_cast<unsigned long long*>(new_keys);
    for (int i = n + threadIdx.x; i < np2; i += blockDim.x) skeys[i] = kEmpty;
  }
  __syncthreads();
  for (int k = 2; k <= np2; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int i = threadIdx.x; i < np2; i += blockDim.x) {
        const int ixj = i ^ j;
        if (ixj > i) {
          const unsigned long long a = skeys[i], b = skeys[ixj];
          const bool up = (i & k) == 0;
          if ((a > b) == up) {
            skeys[i] = b;
            skeys[ixj] = a;
          }
        }
      }
      __syncthreads();
    }
  }
  const int n_old = *n_voxels;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int base = 0; base < n; base += blockDim.x) {
    const int i = base + threadIdx.x;
    int head = 0;
    unsigned long long key = 0;
    if (i < n) {
      key = skeys[i];
      head = (i == 0 || skeys[i - 1] != key) ? 1 : 0;
    }
    int incl = head;
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
    const int rank = carry + (warp > 0 ? warp_sums[warp - 1] : 0) + incl - head;
    if (head) {
      const int id = n_old + rank;
      if (id < table_cap) {
        table_keys[id] = static_cast<long long>(key);
        unsigned int slot = static_cast<unsigned int>(hash64(key)) & (hcap - 1);
        bool placed = false;
        for (int probe = 0; probe < hcap; ++probe) {
          const unsigned long long prev = atomicCAS(&hk[slot], kEmpty, key);
          if (prev == kEmpty) {
            hv[slot] = id;
            placed = true;
            break;
          }
          slot = (slot + 1) & (hcap - 1);
        }
        if (!placed) report_error(err, DEV_POOL_CAPACITY);
      } else {
        report_error(err, DEV_POOL_CAPACITY);
      }
    }
    __syncthreads();
    if (threadIdx.x == blockDim.x - 1) carry = carry + warp_sums[31];
    __syncthreads();
  }
  if (threadIdx.x == 0) *n_voxels = min(n_old + carry, table_cap);
}

__global__ void resolve_pending_kernel(const long long* __restrict__ pt_keys, int n,
                                       const unsigned long long* __restrict__ hk, const int* __restrict__ hv,
                                       int hcap, int* __restrict__ ids) {
  grid_dep_wait();   // launched with programmatic serialization behind the previous kernel in the stream
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  if (ids[i] == -2) ids[i] = hash_lookup(hk, hv, hcap, pt_keys[i]);
}

// One thread per (recent token, cube offset): flag the voxel at key + offset if it exists.
__global__ void neighbor_flag_kernel(const int* __restrict__ token_vx, int n_tokens, int R,
                                     const long long* __restrict__ table_keys, const int* __restrict__ n_voxels,
                                     const unsigned long long* __restrict__ hk, const int* __restrict__ hv, int hcap,
                                     unsigned char* __restrict__ flags) {
  grid_dep_wait();   // launched with programmatic serialization behind the previous kernel in the stream
  const int side = 2 * R + 1;
  const int cube = side * side * side;
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<long long>(n_tokens) * cube) return;
  const int t = static_cast<int>(idx / cube);
  const int o = static_cast<int>(idx % cube);
  const int id = token_vx[t];
  if (id < 0 || id >= *n_voxels) return;
  const long long dx = o / (side * side) - R;
  const long long dy = (o / side) % side - R;
  const long long dz = o % side - R;
  const long long key = table_keys[id] + dx + dy * (1ll << 21) + dz * (1ll << 42);
  const int nb = hash_lookup(hk, hv, hcap, key);
  if (nb >= 0) flags[nb] = 1;
}

// Single CTA: ascending list of flagged ids (or of all ids), flags cleared on the way.  Every
// thread takes 16 consecutive flags per round (one 16-byte load; the flag array is as long as the
// table capacity, a multiple of 16), so a table of 200 k voxels takes 13 rounds.
__global__ void __launch_bounds__(1024, 1)
compact_flags_kernel(unsigned char* __restrict__ flags, const int* __restrict__ n_voxels, int all_ids,
                     int* __restrict__ out_ids, int* __restrict__ out_count) {
  grid_dep_wait();   // launched with programmatic serialization behind the previous kernel in the stream
  __shared__ int warp_sums[32];
  __shared__ int carry;
  const int n = *n_voxels;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  constexpr int kPer = 16;
  for (int base = 0; base < n; base += blockDim.x * kPer) {
    const int i0 = base + threadIdx.x * kPer;
    unsigned int w[4] = {0u, 0u, 0u, 0u};
    if (i0 < n) {
      if (all_ids) {
        w[0] = w[1] = w[2] = w[3] = 0x01010101u;
      } else {
        const uint4 v = *reinterpret_cast<const uint4*>(flags + i0);
        w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
        if (v.x | v.y | v.z | v.w) *reinterpret_cast<uint4*>(flags + i0) = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    int f = 0;   // flagged ids among this thread's 16 (ids >= n are never flagged, but all_ids fills them)
#pragma unroll
    for (int k = 0; k < kPer; ++k)
      if (((w[k >> 2] >> ((k & 3) * 8)) & 0xffu) != 0u && i0 + k < n) ++f;
    int incl = f;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      int ws = warp_sums[lane];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, ws, o);
        if (lane >= o) ws += t;
      }
      warp_sums[lane] = ws;
    }
    __syncthreads();
    int pos = carry + (warp > 0 ? warp_sums[warp - 1] : 0) + incl - f;
#pragma unroll
    for (int k = 0; k < kPer; ++k)
      if (((w[k >> 2] >> ((k & 3) * 8)) & 0xffu) != 0u && i0 + k < n) out_ids[pos++] = i0 + k;
    __syncthreads();
    if (threadIdx.x == blockDim.x - 1) carry = carry + warp_sums[31];
    __syncthreads();
  }
  if (threadIdx.x == 0) *out_count = carry;
}

__global__ void fill_u64_kernel(unsigned long long* p, long long n, unsigned long long v) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) p[i] = v;
}

// Re-insert ids [0, n_voxels) into a (larger, cleared) hash table.
__global__ void rehash_kernel(const long long* __restrict__ table_keys, const int* __restrict__ n_voxels,
                              unsigned long long* __restrict__ hk, int* __restrict__ hv, int hcap) {
  const int id = blockIdx.x * blockDim.x + threadIdx.x;
  if (id >= *n_voxels) return;
  const unsigned long long key = static_cast<unsigned long long>(table_keys[id]);
  unsigned int slot = static_cast<unsigned int>(hash64(key)) & (hcap - 1);
  for (int probe = 0; probe < hcap; ++probe) {
    if (atomicCAS(&hk[slot], kEmpty, key) == kEmpty) {
      hv[slot] = id;
      return;
    }
    slot = (slot + 1) & (hcap - 1);
  }
}

bool is_pow2(long long x) { return x > 0 && (x & (x - 1)) == 0; }
size_t pow2_at_least(int n) {
  size_t p = 1;
  while (p < static_cast<size_t>(n)) p <<= 1;
  return p;
}


// One thread per output token: frame s, token t (the first `special` tokens of a frame are zero
// points with mask 0, the others patch centres in row-major order).
__global__ void pointmap_kernel(const float* __restrict__ wp, const float* __restrict__ conf, int S, int H, int W,
                                int oh, int ow, int special, float conf_threshold, float* __restrict__ pts,
                                uint8_t* __restrict__ mask) {
  const int n_tok = special + oh * ow;
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<long long>(S) * n_tok) return;
  const int s = static_cast<int>(idx / n_tok), t = static_cast<int>(idx - static_cast<long long>(s) * n_tok);
  float* o = pts + idx * 3;
  if (t < special) {
    o[0] = 0.f; o[1] = 0.f; o[2] = 0.f;
    mask[idx] = 0;
    return;
  }
  const int py = (t - special) / ow, px = (t - special) - py * ow;
  // source index and weights along one axis: src = max(scale * (d + 0.5) - 0.5, 0), every step rounded
  auto plan = [](int n_in, int n_out, int d, int& i0, int& i1, float& l0, float& l1) {
    const float scale = __fdiv_rn(static_cast<float>(n_in), static_cast<float>(n_out));
    float src = __fsub_rn(__fmul_rn(scale, __fadd_rn(static_cast<float>(d), 0.5f)), 0.5f);
    src = fmaxf(src, 0.f);
    i0 = min(static_cast<int>(src), n_in - 1);
    i1 = i0 + (i0 < n_in - 1 ? 1 : 0);
    l1 = fminf(fmaxf(__fsub_rn(src, static_cast<float>(i0)), 0.f), 1.f);
    l0 = __fsub_rn(1.f, l1);
  };
  int h0, h1, w0, w1;
  float a0, a1, b0, b1;
  plan(H, oh, py, h0, h1, a0, a1);
  plan(W, ow, px, w0, w1, b0, b1);
  const float w00 = __fmul_rn(a0, b0), w01 = __fmul_rn(a0, b1), w10 = __fmul_rn(a1, b0), w11 = __fmul_rn(a1, b1);
  const long long frame = static_cast<long long>(s) * H * W;
  const long long p00 = frame + static_cast<long long>(h0) * W + w0, p01 = frame + static_cast<long long>(h0) * W + w1;
  const long long p10 = frame + static_cast<long long>(h1) * W + w0, p11 = frame + static_cast<long long>(h1) * W + w1;
  auto tap4 = [&](float v00, float v01, float v10, float v11) {
    float r = __fmul_rn(w00, v00);
    r = __fadd_rn(r, __fmul_rn(w01, v01));
    r = __fadd_rn(r, __fmul_rn(w10, v10));
    return __fadd_rn(r, __fmul_rn(w11, v11));
  };
#pragma unroll
  for (int c = 0; c < 3; ++c) o[c] = tap4(wp[p00 * 3 + c], wp[p01 * 3 + c], wp[p10 * 3 + c], wp[p11 * 3 + c]);
  mask[idx] = tap4(conf[p00], conf[p01], conf[p10], conf[p11]) > conf_threshold ? 1 : 0;
}

}  // namespace
}  // namespace stac

extern "C" {

size_t stac_voxel_scratch_bytes(int n_points) {
  if (n_points <= 0) return 0;
  // per-point packed keys + pending key list (with room for the sort's padding to a power of
  // two) + pending counter (16-byte padded)
  return (static_cast<size_t>(n_points) + stac::pow2_at_least(n_points)) * 8 + 16;
}

int stac_voxel_hash_clear(void* hash_keys, int64_t hash_cap, stac_stream_t stream) {
  if (hash_keys == nullptr || !stac::is_pow2(hash_cap)) return STAC_ERR_BAD_ARG;
  const int threads = 256;
  const long long blocks = (hash_cap + threads - 1) / threads;
  stac::fill_u64_kernel<<<static_cast<unsigned>(blocks), threads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<unsigned long long*>(hash_keys), hash_cap, stac::kEmpty);
  return cudaGetLastError() == cudaSuccess ? STAC_OK : STAC_ERR_CUDA;
}

int stac_voxel_rehash(const int64_t* table_keys, const int* n_voxels, int table_cap, void* hash_keys, int* hash_vals,
                      int64_t hash_cap, stac_stream_t stream) {
  if (table_keys == nullptr || n_voxels == nullptr || hash_keys == nullptr || hash_vals == nullptr ||
      !stac::is_pow2(hash_cap) || hash_cap > (1ll << 30))
    return STAC_ERR_BAD_ARG;
  int rc = stac_voxel_hash_clear(hash_keys, hash_cap, stream);
  if (rc != STAC_OK) return rc;
  const int threads = 256;
  const int blocks = (table_cap + threads - 1) / threads;
  if (blocks > 0)
    stac::rehash_kernel<<<blocks, threads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const long long*>(table_keys), n_voxels, static_cast<unsigned long long*>(hash_keys),
        hash_vals, static_cast<int>(hash_cap));
  return cudaGetLastError() == cudaSuccess ? STAC_OK : STAC_ERR_CUDA;
}

int stac_voxel_upsert(const float* points, const int32_t* ijk, const uint8_t* mask, int n_points, float voxel_size,
                      int64_t* table_keys,
                      int table_cap, void* hash_keys, int* hash_vals, int64_t hash_cap, int* n_voxels, int* ids_out,
                      void* scratch, size_t scratch_bytes, int* dev_status, stac_stream_t stream) {
  if (n_points == 0) return STAC_OK;
  if ((points == nullptr) == (ijk == nullptr) || table_keys == nullptr || hash_keys == nullptr || hash_vals == nullptr ||
      n_voxels == nullptr || ids_out == nullptr || scratch == nullptr || (points != nullptr && !(voxel_size > 0.f)))
    return STAC_ERR_BAD_ARG;
  if (n_points < 0 || n_points > stac::kSortCap) return STAC_ERR_BAD_ARG;
  if (!stac::is_pow2(hash_cap) || hash_cap > (1ll << 30)) return STAC_ERR_BAD_ARG;
  if (scratch_bytes < stac_voxel_scratch_bytes(n_points)) return STAC_ERR_CAPACITY;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  long long* pt_keys = static_cast<long long*>(scratch);
  long long* new_keys = pt_keys + n_points;
  int* new_cnt = reinterpret_cast<int*>(new_keys + stac::pow2_at_least(n_points));
  if (cudaMemsetAsync(new_cnt, 0, sizeof(int), st) != cudaSuccess) return STAC_ERR_CUDA;
  const int threads = 256;
  const int blocks = (n_points + threads - 1) / threads;
  if (stac::launch_behind(stac::quantize_lookup_kernel, dim3(blocks), dim3(threads), 0, st, points, ijk, mask, n_points,
                          voxel_size, static_cast<const unsigned long long*>(hash_keys), hash_vals,
                          static_cast<int>(hash_cap), pt_keys, ids_out, new_keys, new_cnt) != cudaSuccess)
    return STAC_ERR_CUDA;
  int dev = 0;
  if (stac::current_device(&dev) != STAC_OK) return STAC_ERR_CUDA;
  static stac::PerDeviceFlag attr_done;   // the shared-memory opt-in is made once per device
  const int smem = stac::kSortSmemKeys * 8;
  if (attr_done.needs_setup(dev)) {
    if (cudaFuncSetAttribute(stac::insert_new_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) !=
        cudaSuccess)
      return STAC_ERR_CUDA;
    attr_done.mark(dev);
  }
  if (stac::launch_behind(stac::insert_new_kernel, dim3(1), dim3(1024), smem, st, new_keys, new_cnt,
                          reinterpret_cast<long long*>(table_keys), table_cap,
                          static_cast<unsigned long long*>(hash_keys), hash_vals, static_cast<int>(hash_cap), n_voxels,
                          dev_status) != cudaSuccess)
    return STAC_ERR_CUDA;
  if (stac::launch_behind(stac::resolve_pending_kernel, dim3(blocks), dim3(threads), 0, st, pt_keys, n_points,
                          static_cast<const unsigned long long*>(hash_keys), hash_vals, static_cast<int>(hash_cap),
                          ids_out) != cudaSuccess)
    return STAC_ERR_CUDA;
  return cudaGetLastError() == cudaSuccess ? STAC_OK : STAC_ERR_CUDA;
}

int stac_voxel_neighbors(const int* token_voxel_ids, int n_tokens, int radius_cells, int all_ids,
                         const int64_t* table_keys, const int* n_voxels, int table_cap, const void* hash_keys,
                         const int* hash_vals, int64_t hash_cap, uint8_t* flags, int* out_ids, int* out_count,
                         stac_stream_t stream) {
  if (table_keys == nullptr || n_voxels == nullptr || hash_keys == nullptr || hash_vals == nullptr ||
      flags == nullptr || out_ids == nullptr || out_count == nullptr || radius_cells < 0 || radius_cells > 8 ||
      table_cap <= 0)
    return STAC_ERR_BAD_ARG;
  // the flags are read 16 at a time
  if ((table_cap % 16) != 0 || (reinterpret_cast<uintptr_t>(flags) % 16) != 0) return STAC_ERR_BAD_ARG;
  if (!stac::is_pow2(hash_cap) || hash_cap > (1ll << 30)) return STAC_ERR_BAD_ARG;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (!all_ids && n_tokens > 0) {
    if (token_voxel_ids == nullptr) return STAC_ERR_BAD_ARG;
    const int side = 2 * radius_cells + 1;
    const long long total = static_cast<long long>(n_tokens) * side * side * side;
    const int threads = 256;
    const long long blocks = (total + threads - 1) / threads;
    if (stac::launch_behind(stac::neighbor_flag_kernel, dim3(static_cast<unsigned>(blocks)), dim3(threads), 0, st,
                            token_voxel_ids, n_tokens, radius_cells, reinterpret_cast<const long long*>(table_keys),
                            n_voxels, static_cast<const unsigned long long*>(hash_keys), hash_vals,
                            static_cast<int>(hash_cap), flags) != cudaSuccess)
      return STAC_ERR_CUDA;
  }
  if (stac::launch_behind(stac::compact_flags_kernel, dim3(1), dim3(1024), 0, st, flags, n_voxels, all_ids, out_ids,
                          out_count) != cudaSuccess)
    return STAC_ERR_CUDA;
  return cudaGetLastError() == cudaSuccess ? STAC_OK : STAC_ERR_CUDA;
}

int stac_pointmap_to_positions(const float* world_points, const float* conf, int S, int H, int W, int patch,
                               int special, float conf_threshold, float* points_out, uint8_t* mask_out,
                               stac_stream_t stream) {
  if (world_points == nullptr || conf == nullptr || points_out == nullptr || mask_out == nullptr)
    return STAC_ERR_BAD_ARG;
  if (S <= 0 || H <= 0 || W <= 0 || patch <= 0 || special < 0) return STAC_ERR_BAD_ARG;
  const int oh = H / patch > 1 ? H / patch : 1, ow = W / patch > 1 ? W / patch : 1;
  const long long n = static_cast<long long>(S) * (special + static_cast<long long>(oh) * ow);
  const int threads = 128;
  const long long blocks = (n + threads - 1) / threads;
  if (blocks > 0x7fffffffLL) return STAC_ERR_BAD_ARG;
  stac::pointmap_kernel<<<static_cast<unsigned>(blocks), threads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      world_points, conf, S, H, W, oh, ow, special, conf_threshold, points_out, mask_out);
  return cudaGetLastError() == cudaSuccess ? STAC_OK : STAC_ERR_CUDA;
}

}  // extern "C"
