// All-gather of per-head decode results over NVLink peer memory, for head-sharded
// (tensor-parallel) decode: one process per GPU, each GPU has computed h_q / world heads.
//
// One kernel per rank replaces the two library all-gathers (out, lse).  Every rank
//   1. copies its [rows, h_local, 512] BF16 shard and its lse shard into the gathered
//      buffers of every rank (its own included) with plain 16-byte stores to peer
//      pointers;
//   2. makes the stores visible system-wide, and its last CTA writes the step number
//      into this rank's slot of every rank's flag array;
//   3. that CTA then waits until every slot of the local flag array has reached the step
//      number: all shards have landed here.  The wait is bounded; when it runs out the
//      kernel writes a code to the caller's status word and returns.
// The ranks run on different GPUs, so the kernels that wait on one another really are
// concurrent.  The caller alternates between two sets of gathered buffers: a rank may
// overwrite set s only two steps later, and by then every peer has passed the flag
// exchange of the step in between, which it enters only after its own consumers of set
// s (earlier in its stream) are done.
// No multicast, no TMA: plain loads and stores over mapped peer memory.
#include <cuda_bf16.h>

#include "attn_params.cuh"
#include "launchers.h"

namespace dsv4 {
namespace {

constexpr int GATHER_THREADS = 256;
constexpr long long GATHER_SPINS = 1ll << 21;     // x >= 100 ns: a few hundred ms at most

__device__ __forceinline__ void st_release_sys(int32_t* p, int32_t v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int32_t ld_acquire_sys(const int32_t* p) {
  int32_t v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(GATHER_THREADS)
gather_heads_kernel(const Dsv4GatherArgs a) {
  grid_dependency_wait();          // the shard comes from the kernel just before in the stream
  const int world = a.world, rank = a.rank;
  const int h_q = a.h_local * world;
  // out: rows x h_local x 512 bf16 -> 64 chunks of 16 bytes per (row, head)
  const int64_t n_chunks = static_cast<int64_t>(a.b) * a.s_q * a.h_local * 64;
  const uint4* src = static_cast<const uint4*>(a.out_local);
  for (int64_t i = blockIdx.x * static_cast<int64_t>(GATHER_THREADS) + threadIdx.x; i < n_chunks;
       i += static_cast<int64_t>(gridDim.x) * GATHER_THREADS) {
    const int64_t rh = i >> 6;                      // row * h_local + head
    const int c = static_cast<int>(i & 63);
    const int64_t row = rh / a.h_local;
    const int h = static_cast<int>(rh - row * a.h_local);
    const uint4 v = src[i];
    const int64_t dst = (row * h_q + rank * a.h_local + h) * 64 + c;
    for (int p = 0; p < world; ++p) static_cast<uint4*>(a.peer_out[p])[dst] = v;
  }
  // lse: [b, h_local, s_q] -> [b, h_q, s_q]
  const int64_t n_lse = static_cast<int64_t>(a.b) * a.h_local * a.s_q;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(GATHER_THREADS) + threadIdx.x; i < n_lse;
       i += static_cast<int64_t>(gridDim.x) * GATHER_THREADS) {
    const int64_t bi = i / (static_cast<int64_t>(a.h_local) * a.s_q);
    const int64_t r = i - bi * a.h_local * a.s_q;
    const float v = a.lse_local[i];
    const int64_t dst = bi * h_q * a.s_q + static_cast<int64_t>(rank) * a.h_local * a.s_q + r;
    for (int p = 0; p < world; ++p) a.peer_lse[p][dst] = v;
  }
  __threadfence_system();
  __syncthreads();
  __shared__ int s_last;
  if (threadIdx.x == 0) {
    const unsigned int done = atomicAdd(reinterpret_cast<unsigned int*>(a.counter), 1u);
    s_last = (done + 1u) == gridDim.x;
    // The last CTA puts the counter back to zero, so the next call may use another grid
    // (the grid follows the batch size).  Calls that share a counter are ordered by the
    // stream, and no CTA of this launch touches the counter after its own increment.
    if (s_last) *reinterpret_cast<volatile unsigned int*>(a.counter) = 0u;
  }
  __syncthreads();
  if (!s_last) return;
  if (threadIdx.x < world) {
    __threadfence_system();
    st_release_sys(a.peer_flags[threadIdx.x] + rank, a.step);
    const int32_t* mine = a.peer_flags[rank] + threadIdx.x;
    long long spins = 0;
    while (ld_acquire_sys(mine) - a.step < 0) {     // wrap-safe comparison
      if (++spins > GATHER_SPINS) {
        atomicExch(a.status, 1 + static_cast<int>(threadIdx.x));
        break;
      }
      __nanosleep(100);
    }
  }
}

}  // namespace

cudaError_t launch_gather_heads(const Dsv4GatherArgs& a, cudaStream_t st) {
  const int64_t n_chunks = static_cast<int64_t>(a.b) * a.s_q * a.h_local * 64;
  int blocks = static_cast<int>((n_chunks + GATHER_THREADS - 1) / GATHER_THREADS);
  blocks = blocks < 1 ? 1 : blocks > 64 ? 64 : blocks;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(blocks);
  cfg.blockDim = dim3(GATHER_THREADS);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  cfg.attrs = attr;
  cfg.numAttrs = add_overlap_attribute(attr);
  return cudaLaunchKernelEx(&cfg, gather_heads_kernel, a);
}

}  // namespace dsv4
