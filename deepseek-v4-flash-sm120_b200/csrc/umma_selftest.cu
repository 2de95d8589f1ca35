// One 128 x n x k BF16 product through tcgen05.mma, with operands staged in
// shared memory exactly the way the attention kernel stages them.  It exists so
// the descriptor arithmetic (swizzle, K-major vs MN-major, k-step advance) can
// be verified on its own against a host matmul.
//
// mode 0 (the Q.K^T shape):   A [128, k] row-major, B [n, k] row-major,
//                             both K-major, 128-byte swizzle, 64-column blocks.
// mode 1 (the P.V shape):     A given as A^T [k, 128] row-major (M contiguous),
//                             B given as B^T [k, n]  row-major (N contiguous),
//                             both MN-major; A in 64-wide blocks with the
//                             128-byte swizzle, B with the swizzle its row
//                             width allows (n = 64/32/16 -> 128/64/32 B).
// D [128, n] fp32 row-major.  status: 0 ok, 1 = the MMA never signalled.
#include <cuda_bf16.h>

#include "launchers.h"
#include "sm100_ptx.cuh"

namespace dsv4 {
namespace {

using namespace ptx;

constexpr int ST_THREADS = 128;

__global__ void __launch_bounds__(ST_THREADS)
umma_selftest_kernel(int mode, int n, int k, const uint16_t* __restrict__ a,
                     const uint16_t* __restrict__ b, float* __restrict__ d, int32_t* status) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t s_bar;
  __shared__ uint32_t s_tmem;
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  // Operand A: k/64 (mode 0) or 2 (mode 1) blocks; operand B follows A.
  const uint32_t a_bytes = 128u * k * 2u;
  uint8_t* sa = sm;
  uint8_t* sb = sm + a_bytes;

  if (mode == 0) {
    // A block kb: [128 rows][64 cols]; element (r, c) at r*128 + ((c/8) ^ (r&7))*16 + (c%8)*2.
    for (int i = tid; i < 128 * k / 8; i += ST_THREADS) {       // 16-byte chunks
      int r = i / (k / 8), cc = i % (k / 8), kb = cc / 8, ch = cc % 8;
      uint4 v = *reinterpret_cast<const uint4*>(a + r * k + cc * 8);
      *reinterpret_cast<uint4*>(sa + kb * (128 * 128) + r * 128 + ((ch ^ (r & 7)) << 4)) = v;
    }
    for (int i = tid; i < n * k / 8; i += ST_THREADS) {
      int r = i / (k / 8), cc = i % (k / 8), kb = cc / 8, ch = cc % 8;
      uint4 v = *reinterpret_cast<const uint4*>(b + r * k + cc * 8);
      *reinterpret_cast<uint4*>(sb + kb * (n * 128) + r * 128 + ((ch ^ (r & 7)) << 4)) = v;
    }
  } else {
    // A^T [k rows][128]: M-block mb (64 wide) at mb * (k*128); row t at t*128, chunk ^ (t&7).
    for (int i = tid; i < k * 16; i += ST_THREADS) {
      int t = i / 16, cc = i % 16, mb = cc / 8, ch = cc % 8;
      uint4 v = *reinterpret_cast<const uint4*>(a + t * 128 + cc * 8);
      *reinterpret_cast<uint4*>(sa + mb * (k * 128) + t * 128 + ((ch ^ (t & 7)) << 4)) = v;
    }
    // B^T [k rows][n]: row width n*2 bytes = 128/64/32; chunk ^= f(row) per swizzle mode.
    const int row_bytes = n * 2, chunks = n / 8;
    for (int i = tid; i < k * chunks; i += ST_THREADS) {
      int t = i / chunks, ch = i % chunks;
      int x = (n == 64) ? (t & 7) : (n == 32) ? ((t >> 1) & 3) : ((t >> 2) & 1);
      uint4 v = *reinterpret_cast<const uint4*>(b + t * n + ch * 8);
      *reinterpret_cast<uint4*>(sb + t * row_bytes + ((ch ^ x) << 4)) = v;
    }
  }
  fence_async_smem();

  if (warp == 0) {
    tmem_alloc(smem_u32(&s_tmem), 64);
    tmem_relinquish();
  }
  if (tid == 0) {
    mbar_init(smem_u32(&s_bar), 1);
    mbar_init_fence();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = s_tmem;

  if (tid == 0) {
    const uint32_t a0 = smem_u32(sa), b0 = smem_u32(sb);
    if (mode == 0) {
      const uint32_t idesc = make_idesc_bf16(128, n, 0, 0);
      for (int ks = 0; ks < k / 16; ++ks) {
        const int kb = ks / 4, kin = ks % 4;
        uint64_t da = make_smem_desc(a0 + kb * (128 * 128) + kin * 32, 16, 1024, SWZ_128B);
        uint64_t db = make_smem_desc(b0 + kb * (n * 128) + kin * 32, 16, 1024, SWZ_128B);
        umma_bf16(tmem, da, db, idesc, ks > 0);
      }
    } else {
      const uint32_t idesc = make_idesc_bf16(128, n, 1, 1);
      const uint32_t swz = (n == 64) ? SWZ_128B : (n == 32) ? SWZ_64B : SWZ_32B;
      const uint32_t brow = n * 2;
      for (int ks = 0; ks < k / 16; ++ks) {
        uint64_t da = make_smem_desc(a0 + ks * 16 * 128, k * 128, 1024, SWZ_128B);
        uint64_t db = make_smem_desc(b0 + ks * 16 * brow, 8 * brow, 8 * brow, swz);
        umma_bf16(tmem, da, db, idesc, ks > 0);
      }
    }
    umma_commit(smem_u32(&s_bar));
  }
  const bool done = mbar_wait(smem_u32(&s_bar), 0);
  tc_fence_after_sync();
  if (done) {
    for (int c0 = 0; c0 < n; c0 += 16) {
      uint32_t r[16];
      tmem_ld16(tmem + (static_cast<uint32_t>(warp * 32) << 16) + c0, r);
      tmem_ld_wait();
      float* drow = d + (warp * 32 + lane) * n + c0;
#pragma unroll
      for (int i = 0; i < 16; ++i) drow[i] = __uint_as_float(r[i]);
    }
  }
  if (tid == 0) *status = done ? 0 : 1;
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 64);
}

}  // namespace

cudaError_t launch_umma_selftest(int mode, int n, int k, const void* a, const void* b, float* d,
                                 int32_t* status, cudaStream_t st) {
  const size_t smem = 128 * k * 2 + 64 * k * 2 + 1024;
  cudaError_t e = cudaFuncSetAttribute(umma_selftest_kernel,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(smem));
  if (e) return e;
  umma_selftest_kernel<<<1, ST_THREADS, smem, st>>>(mode, n, k, static_cast<const uint16_t*>(a),
                                                    static_cast<const uint16_t*>(b), d, status);
  return cudaGetLastError();
}

}  // namespace dsv4
