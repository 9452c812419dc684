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
 *   workspace  f32 scratch of at least stac_attn_workspace_bytes(M, H) bytes
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

/* Self-test of the bounded-wait mechanism: launches one CTA that waits on a barrier nothing
 * ever completes; the wait gives up after about `max_polls` polls, writes
 * STAC_DEV_TEST_TIMEOUT to *dev_status and the kernel exits normally. */
int stac_selftest_bounded_wait(int max_polls, int* dev_status, stac_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* STAC_B200_H_ */
