// Internal declarations shared by the translation units of libstac_b200.so.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "../../include/stac_b200.h"
#include "per_device.h"

namespace stac {

struct AttnArgs {
  const void* q;            // bf16 [M, H, 64] with row stride q_row_stride elements
  long long q_row_stride;
  const void* k_hot;        // bf16; key n, head h at n*hot_row_stride + h*hot_head_stride
  const void* v_hot;
  long long hot_row_stride;
  long long hot_head_stride;
  int T_hot;
  const void* k_ret;        // bf16 [H, >=T_ret, 64]
  const void* v_ret;
  long long ret_row_stride;
  long long ret_head_stride;
  int T_ret;
  const float* bias_ret;    // [H, >=T_ret]
  long long bias_head_stride;
  void* out;                // bf16, same layout as q
  long long out_row_stride;
  float* lse;               // [H, M] or nullptr
  float* colsum;            // [H, colsum_head_stride] or nullptr
  long long colsum_head_stride;
  int M, H, D;
  float scale;
  float subsample_ratio;
};

// Ordinal of the current device (checked against kMaxDevices) / its SM count, cached per device.
int current_device(int* dev);
int device_sm_count(int dev, int* n_sm);

void attn_subsample_plan(int M, float ratio, int* m_sub, int* stride, float* correction);
size_t attn_lse2_elems(int M, int H);
size_t attn_lse2_elems_split(int M, int H);
size_t attn_part_elems();
// `part`: attn_part_elems() floats for the split forward kernel, or nullptr (one CTA per item then)
int attn_colsum_launch(const AttnArgs& a, float* lse2, float* part, int* err, cudaStream_t stream);

// Launch with programmatic stream serialization: the kernel may become resident while the
// kernel before it in the stream drains; it calls grid_dep_wait() before it touches anything
// that kernel wrote.  STAC_PDL=0 builds fall back to plain stream order.
#ifndef STAC_PDL
#define STAC_PDL 1
#endif
template <typename... KArgs, typename... Args>
cudaError_t launch_behind(void (*kernel)(KArgs...), dim3 grid, dim3 block, int smem, cudaStream_t stream,
                          const Args&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = static_cast<size_t>(smem);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = STAC_PDL;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}

}  // namespace stac
