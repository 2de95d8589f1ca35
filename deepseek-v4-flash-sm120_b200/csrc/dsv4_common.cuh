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
// FP8 e4m3 with a UE8M0 block scale -> BF16, two values per 32-bit word.
// e4m3 NaN (0x7f/0xff) is not preserved (reads as +-480): a cache written by a
// saturating cast never holds it.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t bf16x2_mul(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// e4m3 -> BF16 with the block scale.  The byte, sign-extended to 16 bits and shifted left by
// four, has the e4m3 magnitude bits where a BF16 word reads them as value * 2^-120 (normals
// and subnormals alike) and the sign in bit 15.  One packed multiply by c1 = 2^(s-7) then
// rescales and applies the UE8M0 scale 2^(s-127); it is exact (the value has at most four
// significant bits) unless the result leaves the BF16 range, where the single rounding is
// the same as that of an fp32 product rounded to BF16.  2^(s-7) is a finite BF16 number for
// scale bytes up to 134; beyond that c1 = 2^127 and a second multiply by c2 = 2^(s-134)
// follows (c2 = 1 otherwise).  `two` says whether the second multiply is applied: callers
// pass "c2 is not one", which the attention kernel evaluates once per tile and warp, so
// that the common case costs one multiply per two values.
// Branch-free and on the FMA pipe, which the attention kernel leaves idle; its integer pipe is the
// busy one.  (prmt through inline PTX: __byte_perm drops the selector bit that asks for the
// sign.)
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
  return d;
}
constexpr uint32_t MAX_ONE_MULTIPLY_SCALE = 134;     // largest scale byte with c2 == 1
constexpr uint32_t BF16X2_ONE = 0x3f803f80u;
struct ScalePair { uint32_t c1, c2; };               // packed BF16 factors
__device__ __forceinline__ ScalePair scale_pair(uint32_t s) {
  const uint32_t e1 = min(s + 120u, 254u);
  return ScalePair{e1 * 0x00800080u, (s + 247u - e1) * 0x00800080u};
}
// Does any of the four scale bytes in `w` need the second multiply?
__device__ __forceinline__ bool needs_second_multiply(uint32_t w) {
  return __vcmpgtu4(w, MAX_ONE_MULTIPLY_SCALE * 0x01010101u) != 0u;
}
__device__ __forceinline__ void dequant4(uint32_t w, const ScalePair& c, bool two, uint32_t& lo, uint32_t& hi) {
  const uint32_t t0 = prmt(w, 0u, 0x9180u);           // [b0, sign(b0), b1, sign(b1)]
  const uint32_t t1 = prmt(w, 0u, 0xB3A2u);           // [b2, sign(b2), b3, sign(b3)]
  lo = bf16x2_mul((t0 << 4) & 0x87F087F0u, c.c1);
  hi = bf16x2_mul((t1 << 4) & 0x87F087F0u, c.c1);
  if (two) {
    lo = bf16x2_mul(lo, c.c2);
    hi = bf16x2_mul(hi, c.c2);
  }
}

// The same through fp32 arithmetic (no dependence on packed-BF16 subnormal
// handling); kept as a cross-check of dequant4.
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
