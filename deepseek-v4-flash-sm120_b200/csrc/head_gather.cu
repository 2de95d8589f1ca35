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
constexpr unsigned long long GATHER_WAIT_NS = 300000000ull;    // bounded wait for the peers' flags

__device__ __forceinline__ void st_release_sys(int32_t* p, int32_t v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int32_t ld_acquire_sys(const int32_t* p) {
  int32_t v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// The flag exchange that ends a step, run by the last CTA of the grid: this rank's slot of
// every rank's flag array gets the step number (release, system scope), then the CTA waits,
// bounded, until every slot of the local array has reached it.
__device__ __forceinline__ void publish_and_wait(const Dsv4GatherArgs& a) {
  if (threadIdx.x < a.world) {
    st_release_sys(a.peer_flags[threadIdx.x] + a.rank, a.step);
    const int32_t* mine = a.peer_flags[a.rank] + threadIdx.x;
    // The flags live in this GPU's own memory, so polling them costs no NVLink traffic; no
    // pause between probes (a paused thread was measured to notice a change 0.5-0.9 us
    // late).  Bounded by wall-clock time: about 0.3 s.
    long long spins = 0;
    unsigned long long t0 = 0;
    while (ld_acquire_sys(mine) - a.step < 0) {     // wrap-safe comparison
      if ((++spins & 1023) == 0) {
        unsigned long long now;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
        if (t0 == 0) t0 = now;
        else if (now - t0 > GATHER_WAIT_NS) {
          atomicExch(a.status, 1 + static_cast<int>(threadIdx.x));
          break;
        }
      }
    }
  }
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
  // One system-scope fence per CTA, after the CTA's barrier: the barrier orders every thread's
  // peer stores before the fence, and the fence is cumulative.  (A fence per thread made each
  // of the grid's 32 K threads wait for a round trip over NVLink.)
  __syncthreads();
  __shared__ int s_last;
  if (threadIdx.x == 0) {
    __threadfence_system();
    const unsigned int done = atomicAdd(reinterpret_cast<unsigned int*>(a.counter), 1u);
    s_last = (done + 1u) == gridDim.x;
    // The last CTA puts the counter back to zero, so the next call may use another grid
    // (the grid follows the batch size).  Calls that share a counter are ordered by the
    // stream, and no CTA of this launch touches the counter after its own increment.
    if (s_last) {
      *reinterpret_cast<volatile unsigned int*>(a.counter) = 0u;
      __threadfence();                    // the other CTAs' increments happen before the flags
    }
  }
  __syncthreads();
  if (!s_last) return;
  publish_and_wait(a);
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
