/*
 * libstac_b200 -- C ABI of the B200 (sm_100a) implementation of STAC's KV-cache compression
 * hot path.  Every entry point takes raw device pointers, explicit sizes/strides in elements,
 * a CUDA stream, and returns an int status (STAC_OK = 0).  No entry point allocates device
 * memory, synchronises the stream or throws; scratch space is passed in by the caller.
 * `dev_status`, where present, points to one int32 in device memory that a kernel sets to a
 * non-zero stac_device_error code if one of its bounded waits or capacity checks fails (the
 * first error wins; the caller clears it).  It may be NULL.
 *
 * Citations name the reference interface each function stands in for, by path inside the
 * Rainzor/STAC tree.
 */
#ifndef STAC_B200_H_
#define STAC_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* stac_stream_t; /* a cudaStream_t */

enum stac_status {
  STAC_OK = 0,
  STAC_ERR_BAD_ARG = 1,   /* unsupported size, null or misaligned pointer */
  STAC_ERR_CUDA = 2,      /* a CUDA runtime/driver call failed */
  STAC_ERR_CAPACITY = 3,  /* caller-provided capacity (scratch, pool, table) is too small */
};

enum stac_device_error {
  STAC_DEV_OK = 0,
  STAC_DEV_TIMEOUT_TMA = 1,
  STAC_DEV_TIMEOUT_MMA = 2,
  STAC_DEV_TIMEOUT_CONSUMER = 3,
  STAC_DEV_SORT_CAPACITY = 4,
  STAC_DEV_POOL_CAPACITY = 5,
  STAC_DEV_TEST_TIMEOUT = 6,
};

/* Human-readable name of a stac_status value. */
const char* stac_status_string(int status);

/* Library/ABI version, bumped when a signature changes. */
int stac_abi_version(void);

/* ---------------------------------------------------------------------------------------
 * Window + pivot attention with per-key softmax column sums.
 *
 * Stands in for attn_cuda.flash_attn_bias_colsum(q, k, v, bias, softmax_scale,
 * return_colsum, subsample_ratio) (attn-cuda/attn_cuda/__init__.py:6-43,
 * attn-cuda/csrc/bindings.cpp:31-124) as called from stac/h2o.py:163-165 and
 * stac/stac_voxel.py:248-250, with the concatenation of hot and retrieved keys
 * (stac/stac_voxel.py:233-243) and the bias vector (stac/stac_voxel.py:270-282) folded in.
 *
 *   q, out     bf16 [M, H, 64]; consecutive rows q_row_stride / out_row_stride elements apart
 *   k_hot/v_hot bf16, key n of head h at n * hot_row_stride + h * hot_head_stride elements
 *              (64 contiguous values each), n < T_hot; bias 0.  [H,T,64] and [T,H,64] both fit.
 *   k_ret/v_ret bf16, same addressing with ret_row_stride / ret_head_stride, n < T_ret; may be
 *              NULL if T_ret == 0
 *   bias_ret   f32 [H, >=T_ret], heads bias_head_stride apart: log C per pivot, -inf for padding
 *   lse        f32 [H, M] natural-log row log-sum-exp, or NULL
 *   colsum     f32 [H, colsum_head_stride]: entries [0,T_hot) hot keys, [T_hot, T_hot+T_ret)
 *              retrieved keys; or NULL to skip the column-sum pass
 *   workspace  scratch of at least stac_attn_workspace_bytes(M, H) bytes, 256-byte aligned, contents
 *              need no initialisation: the per-row log-sum-exps passed from the forward to the
 *              column-sum pass, a few flags and counters (cleared by the call), then ~11 MB for the
 *              partial results of query tiles whose keys are shared by two CTAs when the forward
 *              pass is cut evenly over the SMs
 *   subsample_ratio in (0,1]: the column sums use rows 0, s, 2s, ... as in
 *              attn-cuda/csrc/bindings.cpp:63-83 (exact at 1.0)
 * All pointers 16-byte aligned; D must be 64.
 * ------------------------------------------------------------------------------------- */
size_t stac_attn_workspace_bytes(int M, int H);

int stac_attn_colsum(const void* q, int64_t q_row_stride,
                     const void* k_hot, const void* v_hot, int64_t hot_row_stride, int64_t hot_head_stride, int T_hot,
                     const void* k_ret, const void* v_ret, int64_t ret_row_stride, int64_t ret_head_stride, int T_ret,
                     const float* bias_ret, int64_t bias_head_stride,
                     void* out, int64_t out_row_stride,
                     float* lse, float* colsum, int64_t colsum_head_stride,
                     int M, int H, int D, float scale, float subsample_ratio,
                     void* workspace, size_t workspace_bytes,
                     int* dev_status, stac_stream_t stream);

/* ---------------------------------------------------------------------------------------
 * Voxel table: packed 63-bit key -> stable voxel id (append-only; id = insertion rank).
 *
 * Stands in for BinaryVoxel.upsert / neighbors (stac/voxel.py:195-324, :371-521) as called by
 * STACVoxelKV.append_positions and _search_recent_neighbors (stac/stac_voxel.py:326-365,
 * :294-323).  The caller owns all arrays:
 *   table_keys  i64 [table_cap]   packed key of voxel id i
 *   hash_keys   u64 [hash_cap], hash_vals i32 [hash_cap]: open-addressing table, hash_cap a
 *               power of two, kept at most half full by the caller (stac_voxel_rehash to grow)
 *   n_voxels    i32 device scalar, number of voxels in the table
 * ------------------------------------------------------------------------------------- */
#define STAC_VOXEL_MAX_POINTS 131072 /* points per stac_voxel_upsert call (125 frames of 1041 tokens) */

size_t stac_voxel_scratch_bytes(int n_points);

/* Mark every slot of the hash table empty. */
int stac_voxel_hash_clear(void* hash_keys, int64_t hash_cap, stac_stream_t stream);

/* Clear a (new, larger) hash table and re-insert ids [0, *n_voxels). */
int stac_voxel_rehash(const int64_t* table_keys, const int* n_voxels, int table_cap, void* hash_keys,
                      int* hash_vals, int64_t hash_cap, stac_stream_t stream);

/* ijk = floor(points / voxel_size) (fp32, true division), key = (i+2^20) + (j+2^20)*2^21 +
 * (k+2^20)*2^42; known keys keep their id, keys new in this call get *n_voxels + rank among
 * the sorted new unique keys.  points f32 [n,3], or ijk i32 [n,3] already quantised (exactly
 * one of the two non-NULL); mask u8 [n] or NULL (0 -> id -1); ids_out i32 [n].  *n_voxels is
 * updated on the device; no host synchronisation.  n_points <= STAC_VOXEL_MAX_POINTS; up to
 * 16384 new keys of a call are sorted in shared memory, more (a chunk of sixteen frames or
 * more on unseen ground) in the scratch, which stac_voxel_scratch_bytes sizes for it. */
int stac_voxel_upsert(const float* points, const int32_t* ijk, const uint8_t* mask, int n_points, float voxel_size,
                      int64_t* table_keys, int table_cap, void* hash_keys, int* hash_vals, int64_t hash_cap,
                      int* n_voxels, int* ids_out, void* scratch, size_t scratch_bytes,
                      int* dev_status, stac_stream_t stream);

/* StreamSession.get_pointmap (stream_session.py:213-256) for the "pointmap" prediction mode,
 * without the permutes and interpolate calls: world points f32 [S,H,W,3] and their confidence
 * f32 [S,H,W] are reduced to one point per patch by bilinear interpolation (align_corners =
 * False; output size H' = max(1, H/patch), W' = max(1, W/patch)); every frame gets `special`
 * zero points with mask 0 in front.  points_out f32 [S * (special + H'W'), 3], mask_out u8
 * [S * (special + H'W')] = (interpolated confidence > conf_threshold): the arguments of
 * STACVoxelKV.append_positions / stac_voxel_upsert.  fp32 arithmetic in the order of torch's
 * CPU kernel for this (channels-last) layout: the axis weights are multiplied first and the
 * four taps added left to right, nothing fused. */
int stac_pointmap_to_positions(const float* world_points, const float* conf, int S, int H, int W, int patch,
                               int special, float conf_threshold, float* points_out, uint8_t* mask_out,
                               stac_stream_t stream);

/* Ascending unique ids of the existing voxels inside the Chebyshev cube of `radius_cells`
 * around the voxels of `token_voxel_ids` (negative entries ignored); with all_ids != 0 every id
 * in the table instead.  flags u8 [table_cap] (16-byte aligned, table_cap a multiple of 16) must
 * be zero on entry and is zero on exit;
 * out_ids i32 [table_cap], *out_count i32 on the device. */
int stac_voxel_neighbors(const int* token_voxel_ids, int n_tokens, int radius_cells, int all_ids,
                         const int64_t* table_keys, const int* n_voxels, int table_cap,
                         const void* hash_keys, const int* hash_vals, int64_t hash_cap,
                         uint8_t* flags, int* out_ids, int* out_count, stac_stream_t stream);

/* ---------------------------------------------------------------------------------------
 * H2O bookkeeping on the hot cache (rows = managed layers x heads).
 * ------------------------------------------------------------------------------------- */

/* KVManager.append_kv (stac/kv_manager.py:227-309) for one layer: new keys/values, token t of
 * head h at k + h*k_head_stride + t*k_row_stride elements (64 contiguous values), go to
 * positions [old_T, old_T + T_new) of the cache [H][cache_head_stride]; their global token
 * ids first_token_id + t are written to token_idx i64 [H][idx_head_stride]. */
int stac_append_kv(const void* k, const void* v, int64_t k_head_stride, int64_t k_row_stride,
                   int64_t v_head_stride, int64_t v_row_stride, void* k_cache, void* v_cache,
                   int64_t cache_head_stride, int64_t* token_idx, int64_t idx_head_stride, int H, int T_new,
                   int old_T, int64_t first_token_id, int head_dim, int elem_bytes, stac_stream_t stream);

/* The epilogue of SparseAttention's QKV projection fused with append_kv
 * (causalvggt/layers/attention.py:119-128 and :141; LayerNorm = q_norm / k_norm over the head
 * dimension, causalvggt/layers/rope.py:148-188 for the 2-D rotary embedding).  qkv is the bf16
 * projection output [T_new][3][H][64] (tokens qkv_token_stride elements apart).  q and k get
 * LayerNorm in fp32 (weights / biases f32 [64]; pass NULL, NULL to skip) and the rotary embedding
 * from the caller's tables cos_table / sin_table f32 [n_pos][16] (the reference's frequency
 * cache for feature dimension 32: angle = position * 100^(-j/16); NULL to skip) at the integer
 * positions pos i64 [T_new][2] = (y, x); results are rounded to bf16.  q goes to q_out
 * [T_new][H][64] (rows q_out_row_stride apart), k and v to positions [old_T, old_T + T_new) of the
 * cache [H][cache_head_stride] and the token ids first_token_id + t to token_idx, as
 * stac_append_kv does.  head_dim is 64. */
int stac_qkv_epilogue_append(const void* qkv, int64_t qkv_token_stride, const float* q_norm_w, const float* q_norm_b,
                             const float* k_norm_w, const float* k_norm_b, float eps, const int64_t* pos,
                             const float* cos_table, const float* sin_table, int n_pos, void* q_out,
                             int64_t q_out_row_stride, void* k_cache, void* v_cache, int64_t cache_head_stride,
                             int64_t* token_idx, int64_t idx_head_stride, int H, int T_new, int old_T,
                             int64_t first_token_id, stac_stream_t stream);

/* HeavyHittersKV._update_scores (stac/h2o.py:177-216) for one layer: s = colsum * T_live / Tq;
 * positions >= old_T take s, older ones score * temperature + s; counts += 1. */
int stac_scores_update(const float* colsum, int64_t colsum_head_stride, float* scores, float* counts,
                       int64_t row_stride, int H, int T_live, int old_T, int Tq, float temperature,
                       stac_stream_t stream);

/* Keep set of HeavyHittersKV._parallel_prune_kv (stac/h2o.py:244-354): per row, positions with
 * is_base[t] != 0 (pinned and recent tokens) plus the highest-scoring others, n_keep in total
 * (ties at the cut: lower position first).  keep_idx i32 [n_rows, n_keep] and drop_idx i32
 * [n_rows, T - n_keep], both ascending. */
int stac_h2o_select(const float* scores, int64_t row_stride, int n_rows, const uint8_t* is_base, int T,
                    int n_keep, int* keep_idx, int* drop_idx, stac_stream_t stream);

/* Gather-compaction of the cache into a second set of buffers
 * (stac/h2o.py:356-436, stac/stac_voxel.py:409-419): dst[row, j] = src[row, keep[row, j]] for
 * K, V [n_rows, T_buf, head_dim], token ids i64, scores, counts f32 and voxel ids i32
 * [n_rows, T_buf]; tails [n_keep, T_buf) of the small arrays are reset (-1 / 0).
 * vx_src / vx_dst may both be NULL. */
int stac_compact(const int* keep_idx, int n_rows, int n_keep, int T_buf, int head_dim, int elem_bytes,
                 const void* k_src, const void* v_src, void* k_dst, void* v_dst,
                 const int64_t* ti_src, int64_t* ti_dst, const float* s_src, float* s_dst,
                 const float* c_src, float* c_dst, const int* vx_src, int* vx_dst, stac_stream_t stream);

/* ---------------------------------------------------------------------------------------
 * Voxel memory: per (pool head, voxel) row up to budget_cap buffered tokens and pivot_cap
 * pivots, one token per pool segment.  Same observable state as the reference's
 * SegmentedSlabPool with seg_size = 1 (stac/allocator.py:2036-2506): row_seg[row][column] is
 * the segment id, row_cnt[row] the occupied columns, a LIFO free list plus a bump counter.
 * Rows are laid out [heads][voxel_cap].  The caller owns and grows every array.  If a call
 * does not fit buf_cap / piv_cap, rows are skipped in (head, voxel) order (their selected tokens
 * are dropped and counted in STAC_META_DROPPED): a caller that stops growing gets a bounded pool.
 * ------------------------------------------------------------------------------------- */
enum stac_meta_index {       /* int32 counters in device memory, pool->meta[STAC_META_SIZE] */
  STAC_META_BUF_TOP = 0,     /* fresh buffer segment ids handed out so far */
  STAC_META_BUF_FREE_LEN = 1,/* entries in the buffer free list */
  STAC_META_PIV_TOP = 2,     /* pivot segment ids handed out so far */
  STAC_META_OVER_COUNT = 3,  /* tokens in the carried overflow list */
  STAC_META_BUF_USED = 4,    /* tokens currently buffered */
  STAC_META_PIV_USED = 5,    /* pivots currently stored */
  STAC_META_DROPPED = 6,     /* tokens dropped because a bounded pool was full (cumulative) */
  STAC_META_VOXELS = 7,      /* voxels in the table at the last insert (when pool->voxel_count is given) */
  STAC_META_SIZE = 8
};

typedef struct stac_pool {
  int heads, head_dim, elem_bytes;   /* elem_bytes: 2 = bf16, 4 = f32 storage of K and V */
  int pivot_cap, budget_cap;         /* P <= 4, B <= 8 */
  int voxel_cap, voxel_used;         /* row stride per head; voxels known at the last insert */
  float sim_thresh, replace_thresh, score_thresh;
  void* buf_K; void* buf_V; float* buf_S;       /* [buf_cap][head_dim], [buf_cap] */
  int* buf_row_seg; int* buf_row_cnt; int* buf_free; int buf_cap;
  void* piv_K; void* piv_V; float* piv_W; float* piv_S; float* piv_C;
  int* piv_row_seg; int* piv_row_cnt; int piv_cap;
  /* carried overflow tokens: list read by this call and list written by it (the caller swaps) */
  const void* over_K_in; const void* over_V_in; const float* over_S_in;
  const int* over_hv_in;      /* [n][2] (head, voxel) */
  const int* over_start_in;   /* [heads + 1] first list entry of each head */
  void* over_K_out; void* over_V_out; float* over_S_out; int* over_hv_out; int* over_start_out;
  int over_cap;
  int* meta;
  /* optional device scalar with the current number of voxels: an insert copies it to
   * meta[STAC_META_VOXELS], so that a host which passes only an upper bound as voxel_used (to
   * avoid reading the count back before the call) still learns the exact figure later */
  const int* voxel_count;
} stac_pool;

typedef struct stac_evicted {
  const void* k; const void* v;      /* token at position t of head h: k + h*kv_head_stride + t*kv_row_stride */
  int64_t kv_head_stride, kv_row_stride;
  const float* scores; const int* voxel_ids; /* [heads][meta_head_stride] indexed by position */
  int64_t meta_head_stride;
  const int* positions;              /* [heads][tokens_per_head] ascending positions, or NULL = 0..n-1 */
  int tokens_per_head;
} stac_evicted;

#define STAC_MERGE_MAX_LIST (1 << 22) /* (evicted + carried overflow) tokens of one pool head per call */

size_t stac_merge_scratch_bytes(int heads, int list_cap_per_head, int buf_cap);

/* One VoxelKVMerger.insert_and_merge call (stac/merger.py:1157-1255 and :765-918) with the
 * evicted tokens read in place.  list_cap_per_head bounds (evicted + carried overflow) tokens
 * of one head (<= STAC_MERGE_MAX_LIST; the scratch grows with heads * list_cap_per_head, about
 * 150 bytes each).  Counters in pool->meta are updated on the device. */
int stac_merge_insert(const stac_pool* pool, const stac_evicted* ev, void* scratch, size_t scratch_bytes,
                      int list_cap_per_head, int* dev_status, stac_stream_t stream);

/* VoxelKVMerger.retrieve with retrieve_size > 0 (stac/merger.py:1377-1482): per head the
 * pivots of the queried voxels (ascending ids < voxel_used) by W descending; out_K/out_V
 * [heads][R][head_dim], out_mask u8, out_bias f32 = log(max(C,1e-9)) or -inf, sel i32 scratch
 * [heads][R], out_idx i32 [heads][R][2] = (voxel, slot) or NULL.  R <= 8192. */
int stac_retrieve(const stac_pool* pool, const int* query_ids, const int* query_count, int retrieve_size,
                  int* sel, void* out_K, void* out_V, uint8_t* out_mask, float* out_bias, int* out_idx,
                  stac_stream_t stream);

/* Same computation and arguments as stac_attn_colsum, minus the workspace: the per-row
 * scratch sits in a fixed 512 KB array inside the library image on each GPU, so this call
 * never asks the driver for memory.  It has no counterpart in the reference.  It is meant
 * for hosts that cannot allocate at call time: a serving process that handed the whole GPU
 * to its own arena at start-up (a cudaMalloc would fail or fragment it), or a loop that cannot
 * tolerate the device-wide synchronisation an allocation implies.
 *   - M * H must not exceed STAC_ATTN_STATIC_MAX_ROWS, else STAC_ERR_CAPACITY.
 *   - The first call on a device looks up the array's device address (with that device
 *     current); make that first call outside any stream capture.
 *   - All calls on a device share the one array and it keeps the previous call's values;
 *     nothing needs clearing because each call writes every entry it later reads, but two
 *     calls that overlap on the GPU (different streams) race on it.  Serialise them. */
#define STAC_ATTN_STATIC_MAX_ROWS 131072 /* floats of fixed scratch = max M * H */

int stac_attn_colsum_noalloc(const void* q, int64_t q_row_stride,
                             const void* k_hot, const void* v_hot, int64_t hot_row_stride, int64_t hot_head_stride, int T_hot,
                             const void* k_ret, const void* v_ret, int64_t ret_row_stride, int64_t ret_head_stride, int T_ret,
                             const float* bias_ret, int64_t bias_head_stride,
                             void* out, int64_t out_row_stride,
                             float* lse, float* colsum, int64_t colsum_head_stride,
                             int M, int H, int D, float scale, float subsample_ratio,
                             int* dev_status, stac_stream_t stream);

/* Self-test of the bounded-wait mechanism: launches one CTA that waits on a barrier nothing
 * ever completes; the wait gives up after about `max_polls` polls, writes
 * STAC_DEV_TEST_TIMEOUT to *dev_status and the kernel exits normally. */
int stac_selftest_bounded_wait(int max_polls, int* dev_status, stac_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* STAC_B200_H_ */
