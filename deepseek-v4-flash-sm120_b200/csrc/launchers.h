// Host-side launch functions implemented by the kernel translation units.
#pragma once

#include <cuda_runtime.h>

#include "dsv4_b200.h"

#include <cstdlib>

namespace dsv4 {

struct AttnParams;

// Programmatic dependent launch: with this attribute a kernel may be set up on the SMs
// while the kernel before it in the stream is still in its last phase; both kernels here
// execute griddepcontrol.wait before their first global access, so they still observe all
// of the predecessor's writes.  DSV4_NO_PDL=1 turns the attribute off.
// Returns the number of attributes written (0 or 1).
inline int add_overlap_attribute(cudaLaunchAttribute* attr) {
  static const bool off = [] {
    const char* e = std::getenv("DSV4_NO_PDL");
    return e != nullptr && e[0] != '\0' && e[0] != '0';
  }();
  if (off) return 0;
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  return 1;
}

// CUDA-core cross-check kernels (simple_kernels.cu).
cudaError_t launch_simple_attn(const AttnParams& p, int kv_format, int d_qk, cudaStream_t st);
cudaError_t launch_combine(const Dsv4CombineArgs& a, cudaStream_t st);
int combine_max_splits();
// `slots32` non-null: the slot mapping is int32 and a.slots is ignored.
cudaError_t launch_kv_store(const Dsv4StoreArgs& a, const int32_t* slots32, cudaStream_t st);
cudaError_t launch_gather_dequant(const void* kv, int64_t stride, int kv_format, int num_blocks,
                                  int page_block, const int32_t* indices, int n, void* rows,
                                  int method, cudaStream_t st);

// tcgen05 kernels (sparse_attn_sm100.cu).  `supported` reports whether the
// tensor-core kernel handles this (format, d_qk) pair.
bool sm100_attn_supported(int kv_format, int d_qk);
cudaError_t launch_sm100_attn(const AttnParams& p, int kv_format, int d_qk, cudaStream_t st);
cudaError_t read_attn_error(int* value, bool reset);
cudaError_t launch_gather_heads(const Dsv4GatherArgs& a, cudaStream_t st);
cudaError_t launch_umma_selftest(int mode, int n, int k, const void* a, const void* b, float* d,
                                 int32_t* status, cudaStream_t st);

}  // namespace dsv4
