// Sparse decode for callers that must not allocate.
//
// Who cannot allocate: code that runs while a CUDA graph is being captured or
// replayed with fixed buffers, code inside another framework's memory-pool
// callbacks or "no sync / no malloc" sections, and small embedders that link
// this library without torch and own no device allocator of their own.  For
// them every cudaMalloc (which also synchronises the device) is off limits, yet
// split-KV decode needs scratch for its partial results.
//
// This entry point therefore keeps the split-KV scratch in a fixed array that
// lives in the library's device image.  It is the same decode as
// dsv4_sparse_decode (same kernels, same arguments, same results); only where
// the partials go differs.
#include <mutex>

#include "dsv4_b200.h"

namespace {

// Partial outputs (fp32) followed by partial log-sum-exp values (fp32).  Held by
// every GPU that loads the library, from load until the process exits.
constexpr long long kMaxOFloats = DSV4_NOALLOC_MAX_O_FLOATS;
constexpr long long kMaxLseFloats = DSV4_NOALLOC_MAX_O_FLOATS / 512;
static __device__ __align__(256) float g_noalloc_scratch[kMaxOFloats + kMaxLseFloats];

constexpr int kMaxDevices = 64;
float* g_scratch_addr[kMaxDevices] = {};     // device address of the array, per device
std::mutex g_scratch_mu;

// `g_noalloc_scratch` in host code is only a handle for the runtime, not an
// address a kernel could use; the address valid on the current device has to be
// asked for, once per device, with that device current.
int scratch_for_current_device(float** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return DSV4_ERR_CUDA;
  std::lock_guard<std::mutex> lk(g_scratch_mu);
  if (g_scratch_addr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || p == nullptr)
      return DSV4_ERR_CUDA;
    g_scratch_addr[dev] = static_cast<float*>(p);
  }
  *out = g_scratch_addr[dev];
  return DSV4_OK;
}

}  // namespace

extern "C" int dsv4_sparse_decode_noalloc(const Dsv4DecodeArgs* args, void* cuda_stream) {
  if (!args) return DSV4_ERR_NULL;
  Dsv4DecodeArgs a = *args;
  a.o_accum = nullptr;
  a.lse_accum = nullptr;
  // Splits that are merged on chip leave no partials: only the sets that really reach the
  // scratch count against its size.
  const int sets = a.n_splits > 1 ? dsv4_decode_partial_sets(&a) : 1;
  if (sets > 1) {
    if (a.b < 0 || a.s_q < 1 || a.h_q < 1) return DSV4_ERR_SHAPE;
    const long long slots = static_cast<long long>(sets) * a.b * a.s_q * a.h_q;
    if (slots > kMaxLseFloats || slots * 512 > kMaxOFloats) return DSV4_ERR_SCRATCH_TOO_LARGE;
    float* base = nullptr;
    const int rc = scratch_for_current_device(&base);   // first call per device: one-time set-up
    if (rc != DSV4_OK) return rc;
    a.o_accum = base;
    a.lse_accum = base + kMaxOFloats;
  }
  // Nothing in the scratch has to start at zero: every slot the combine step reads is
  // written by this call's decode kernel first (empty ranges write -inf / 0 themselves).
  return dsv4_sparse_decode(&a, cuda_stream);
}
