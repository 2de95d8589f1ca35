// Shared device/host helpers for the sparse-MLA kernels: KV layout traits,
// FP8(e4m3) x UE8M0 -> BF16 dequantisation, small math helpers.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "dsv4_b200.h"

namespace dsv4 {

constexpr int D_ROPE = 64;
constexpr int D_V = 512;

// Byte layout of one token (see Dsv4KvFormat).  ROW_BYTES is the FP8 latent
// followed by the BF16 RoPE values; scale bytes live in the page's second section.
template <int FMT> struct KvTraits;
template <> struct KvTraits<DSV4_KV_MODEL1> {
  static constexpr int D_NOPE = 448, TILE = 64, N_SCALE = 7, SLOTS = 8;
  static constexpr int ROW_BYTES = D_NOPE + 2 * D_ROPE, D_QK = D_NOPE + D_ROPE;
};
template <> struct KvTraits<DSV4_KV_V32> {
  static constexpr int D_NOPE = 512, TILE = 128, N_SCALE = 4, SLOTS = 4;
  static constexpr int ROW_BYTES = D_NOPE + 2 * D_ROPE, D_QK = D_NOPE + D_ROPE;
};

__host__ __device__ inline int kv_d_qk(int fmt_or_dqk_hint, int d_qk) {
  return fmt_or_dqk_hint == DSV4_KV_MODEL1 ? 512 : fmt_or_dqk_hint == DSV4_KV_V32 ? 576 : d_qk;
}

// ---------------------------------------------------------------------------
// Plain conversion: fp8 -> fp32, times 2^(s-127) in fp32, round to BF16.
// Byte 0 means 2^-127 (a fp32 subnormal), matching 2**(b-127) evaluated in fp32.
// ---------------------------------------------------------------------------
__device__ __forceinline__ float ue8m0_scale_f32(uint32_t s) {
  return s ? __uint_as_float(s << 23) : __uint_as_float(0x00400000u);
}

__device__ __forceinline__ float e4m3_to_f32(uint32_t byte) {
  __nv_fp8_e4m3 f;
  f.__x = static_cast<__nv_fp8_storage_t>(byte);
  return static_cast<float>(f);
}

__device__ __forceinline__ float dequant_plain(uint32_t byte, uint32_t s) {
  float v = __fmul_rn(e4m3_to_f32(byte), ue8m0_scale_f32(s));
  return __bfloat162float(__float2bfloat16_rn(v));
}

// ---------------------------------------------------------------------------
// Fast conversion used by the tensor-core kernels.  The e4m3 magnitude bits
// (eeee.mmm) dropped into a BF16 word at bit 4 read as value * 2^-120, for
// normals and subnormals alike, so ONE packed BF16 multiply by 2^(120+s-127)
// both rescales and applies the block scale; the product has at most four
// significant bits and is therefore exact.  Two e4m3 bytes -> one bf16x2 word.
// Valid for scale bytes 1..134 in one multiply; others take a second multiply.
// e4m3 NaN (0x7f/0xff) is not preserved (reads as +-480): a cache written by a
// saturating cast never holds it.
// ---------------------------------------------------------------------------
struct ScaleMul {
  uint32_t c1;   // bf16x2 multiplier applied first
  uint32_t c2;   // second multiplier, or 0 when one multiply is enough
};

__device__ __forceinline__ ScaleMul make_scale_mul(uint32_t s) {
  ScaleMul m;
  if (s >= 1 && s <= 134) {
    uint32_t c = (s + 120u) << 7;           // 2^(s-7)
    m.c1 = c | (c << 16);
    m.c2 = 0;
  } else {
    uint32_t c = 247u << 7;                 // 2^120
    uint32_t d = s ? (s << 7) : 0x0040u;    // 2^(s-127); byte 0 -> subnormal 2^-127
    m.c1 = c | (c << 16);
    m.c2 = d | (d << 16);
  }
  return m;
}

__device__ __forceinline__ uint32_t bf16x2_mul(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// w holds four e4m3 bytes; returns BF16 pairs (byte0, byte1) and (byte2, byte3).
__device__ __forceinline__ void dequant4_fast(uint32_t w, const ScaleMul& m, uint32_t& lo,
                                              uint32_t& hi) {
  uint32_t t0 = __byte_perm(w, 0u, 0x1404);     // [0, b0, 0, b1]
  uint32_t t1 = __byte_perm(w, 0u, 0x3424);     // [0, b2, 0, b3]
  uint32_t x0 = (t0 & 0x80008000u) | ((t0 >> 4) & 0x07F007F0u);
  uint32_t x1 = (t1 & 0x80008000u) | ((t1 >> 4) & 0x07F007F0u);
  x0 = bf16x2_mul(x0, m.c1);
  x1 = bf16x2_mul(x1, m.c1);
  if (m.c2) {
    x0 = bf16x2_mul(x0, m.c2);
    x1 = bf16x2_mul(x1, m.c2);
  }
  lo = x0;
  hi = x1;
}

// Hot-path variant for the common case of a single multiplier (ScaleMul::c2 == 0).
__device__ __forceinline__ void dequant4_one_mul(uint32_t w, uint32_t c1, uint32_t& lo,
                                                 uint32_t& hi) {
  const uint32_t t0 = __byte_perm(w, 0u, 0x1404);     // [0, b0, 0, b1]
  const uint32_t t1 = __byte_perm(w, 0u, 0x3424);     // [0, b2, 0, b3]
  lo = bf16x2_mul((t0 & 0x80008000u) | ((t0 >> 4) & 0x07F007F0u), c1);
  hi = bf16x2_mul((t1 & 0x80008000u) | ((t1 >> 4) & 0x07F007F0u), c1);
}

// The same through fp32 arithmetic (no dependence on packed-BF16 subnormal
// handling); kept as a cross-check of dequant4_fast.
__device__ __forceinline__ void dequant4_f32(uint32_t w, uint32_t s, uint32_t& lo, uint32_t& hi) {
  float sc = ue8m0_scale_f32(s);
  __nv_bfloat162 a = __floats2bfloat162_rn(__fmul_rn(e4m3_to_f32(w & 0xffu), sc),
                                           __fmul_rn(e4m3_to_f32((w >> 8) & 0xffu), sc));
  __nv_bfloat162 b = __floats2bfloat162_rn(__fmul_rn(e4m3_to_f32((w >> 16) & 0xffu), sc),
                                           __fmul_rn(e4m3_to_f32(w >> 24), sc));
  lo = *reinterpret_cast<uint32_t*>(&a);
  hi = *reinterpret_cast<uint32_t*>(&b);
}

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t h) { return __uint_as_float(h << 16); }

// Addresses of one token inside the paged cache.
template <int FMT>
__device__ __forceinline__ void token_ptrs(const uint8_t* kv, int64_t stride_block, int page_block,
                                           int idx, const uint8_t*& row, const uint8_t*& scales) {
  using T = KvTraits<FMT>;
  int page = idx / page_block;
  int r = idx - page * page_block;
  const uint8_t* base = kv + static_cast<int64_t>(page) * stride_block;
  row = base + static_cast<int64_t>(r) * T::ROW_BYTES;
  scales = base + static_cast<int64_t>(page_block) * T::ROW_BYTES + r * T::SLOTS;
}

}  // namespace dsv4
