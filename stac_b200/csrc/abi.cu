// extern "C" entry points of libstac_b200.so: argument checks and dispatch only.
#include "common.cuh"
#include "stac_internal.h"

namespace stac {
namespace {

__global__ void bounded_wait_selftest_kernel(int max_polls, int* err) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_fence_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    // Nothing ever arrives on this barrier: the poll loop must run out and report.
    bool done = false;
    for (int it = 0; it < max_polls && !done; ++it) done = mbar_try_wait(&bar, 0);
    if (!done) report_error(err, DEV_TEST_TIMEOUT);
  }
}

}  // namespace

int current_device(int* dev) {
  int d = -1;
  if (cudaGetDevice(&d) != cudaSuccess || !device_index_ok(d)) return STAC_ERR_CUDA;
  *dev = d;
  return STAC_OK;
}

int device_sm_count(int dev, int* n_sm) {
  static PerDeviceValue<int> cache;
  int n = cache.get(dev);
  if (n == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return STAC_ERR_CUDA;
    cache.set(dev, n);
  }
  *n_sm = n;
  return STAC_OK;
}

}  // namespace stac

extern "C" {

const char* stac_status_string(int status) {
  switch (status) {
    case STAC_OK: return "ok";
    case STAC_ERR_BAD_ARG: return "bad argument";
    case STAC_ERR_CUDA: return "CUDA call failed";
    case STAC_ERR_CAPACITY: return "capacity too small";
    default: return "unknown status";
  }
}

int stac_abi_version(void) { return 2; }

size_t stac_attn_workspace_bytes(int M, int H) {
  if (M <= 0 || H <= 0) return 0;
  // row log-sum-exps (rounded up to 256 bytes), then the partial results of the split forward kernel
  const size_t lse_bytes = (stac::attn_lse2_elems_split(M, H) * sizeof(float) + 255) & ~static_cast<size_t>(255);
  return lse_bytes + stac::attn_part_elems() * sizeof(float);
}

int stac_attn_colsum(const void* q, int64_t q_row_stride, const void* k_hot, const void* v_hot,
                     int64_t hot_row_stride, int64_t hot_head_stride, int T_hot, const void* k_ret, const void* v_ret,
                     int64_t ret_row_stride, int64_t ret_head_stride, int T_ret, const float* bias_ret, int64_t bias_head_stride, void* out,
                     int64_t out_row_stride, float* lse, float* colsum, int64_t colsum_head_stride, int M, int H,
                     int D, float scale, float subsample_ratio, void* workspace, size_t workspace_bytes,
                     int* dev_status, stac_stream_t stream) {
  if (q == nullptr || out == nullptr || workspace == nullptr) return STAC_ERR_BAD_ARG;
  if (!(subsample_ratio > 0.f && subsample_ratio <= 1.f)) return STAC_ERR_BAD_ARG;
  if (workspace_bytes < stac_attn_workspace_bytes(M, H)) return STAC_ERR_CAPACITY;
  if (reinterpret_cast<uintptr_t>(workspace) & 255) return STAC_ERR_BAD_ARG;
  if ((q_row_stride % 8) || (out_row_stride % 8) || (hot_head_stride % 8) || (ret_head_stride % 8) ||
      (hot_row_stride % 8) || (ret_row_stride % 8))
    return STAC_ERR_BAD_ARG;
  stac::AttnArgs a;
  a.q = q; a.q_row_stride = q_row_stride;
  a.k_hot = k_hot; a.v_hot = v_hot; a.hot_row_stride = hot_row_stride; a.hot_head_stride = hot_head_stride; a.T_hot = T_hot;
  a.k_ret = k_ret; a.v_ret = v_ret; a.ret_row_stride = ret_row_stride; a.ret_head_stride = ret_head_stride; a.T_ret = T_ret;
  a.bias_ret = bias_ret; a.bias_head_stride = bias_head_stride;
  a.out = out; a.out_row_stride = out_row_stride;
  a.lse = lse; a.colsum = colsum; a.colsum_head_stride = colsum_head_stride;
  a.M = M; a.H = H; a.D = D; a.scale = scale; a.subsample_ratio = subsample_ratio;
  const size_t lse_bytes = (stac::attn_lse2_elems_split(M, H) * sizeof(float) + 255) & ~static_cast<size_t>(255);
  float* part = reinterpret_cast<float*>(static_cast<char*>(workspace) + lse_bytes);
  return stac::attn_colsum_launch(a, static_cast<float*>(workspace), part, dev_status,
                                  reinterpret_cast<cudaStream_t>(stream));
}

int stac_selftest_bounded_wait(int max_polls, int* dev_status, stac_stream_t stream) {
  if (max_polls <= 0 || dev_status == nullptr) return STAC_ERR_BAD_ARG;
  stac::bounded_wait_selftest_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(max_polls, dev_status);
  return cudaGetLastError() == cudaSuccess ? STAC_OK : STAC_ERR_CUDA;
}

}  // extern "C"
