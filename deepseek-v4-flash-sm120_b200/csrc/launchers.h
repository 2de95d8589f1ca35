// Host-side launch functions implemented by the kernel translation units.
#pragma once

#include <cuda_runtime.h>

#include "dsv4_b200.h"

namespace dsv4 {

struct AttnParams;

// CUDA-core cross-check kernels (simple_kernels.cu).
cudaError_t launch_simple_attn(const AttnParams& p, int kv_format, int d_qk, cudaStream_t st);
cudaError_t launch_combine(const Dsv4CombineArgs& a, cudaStream_t st);
int combine_max_splits();
cudaError_t launch_kv_store(const Dsv4StoreArgs& a, cudaStream_t st);
cudaError_t launch_gather_dequant(const void* kv, int64_t stride, int kv_format, int num_blocks,
                                  int page_block, const int32_t* indices, int n, void* rows,
                                  int method, cudaStream_t st);

// tcgen05 kernels (sparse_attn_sm100.cu).  `supported` reports whether the
// tensor-core kernel handles this (format, d_qk) pair.
bool sm100_attn_supported(int kv_format, int d_qk);
cudaError_t launch_sm100_attn(const AttnParams& p, int kv_format, int d_qk, cudaStream_t st);
cudaError_t read_attn_error(int* value, bool reset);
cudaError_t launch_umma_selftest(int mode, int n, int k, const void* a, const void* b, float* d,
                                 int32_t* status, cudaStream_t st);

}  // namespace dsv4
