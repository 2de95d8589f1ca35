// Sparse MLA attention on the 5th-generation tensor cores (tcgen05 + TMEM).
//
// One CTA handles one (request, block of <= 64 heads, split) and walks the
// request's index list in tiles of 128 entries.  Gathered KV rows are the M
// dimension of the MMAs ("tokens as M"), heads are N = 64:
//
//   S^T[128 tok, 64 heads]  = K[128 tok, d_qk]      . Q^T      (K-major A and B)
//   O^T[512 d_v, 64 heads] += V^T[512, 128 tok]     . P^T      (MN-major A and B)
//
// V is the first 512 columns of the same dequantised K tile, so ONE shared-
// memory tile serves both products: it is stored as d_qk/64 blocks of
// [128 tokens][64 values] with the 128-byte swizzle, which reads as K-major
// (contraction over d) for the first product and as MN-major (contraction over
// tokens) for the second.  With d_qk = 576 the tile (144 KB) and Q (72 KB) leave
// no room for a second tile or a staging ring, so gathered rows are staged in
// REGISTERS: each producer warp owns 16 rows of the tile, issues the 16-byte
// loads of the next tile while the current one is being multiplied, and writes
// them (dequantised to BF16) as soon as the P.V step that last read those 16
// rows has retired.  P^T (16 KB) reuses the RoPE block of the tile, which only
// Q.K^T reads, when d_qk = 576.
//
// Warp roles (13 warps): 0-3 softmax (one thread per tile row = TMEM lane),
// 4-11 producers (gather + dequantise + swizzled store), 12 MMA issue + TMEM.
// TMEM columns: [0,64) S^T, [64,320) the four 128-row slices of O^T.
//
// Softmax: running per-head reference max with lazy rescaling (O^T is touched
// only when a head's max grows by more than 2^8), denominators accumulated per
// thread and reduced across the 128 rows once, at the end.
//
// Every wait is bounded; a wait that gives up records a code in g_attn_error,
// and the CTA drains and returns without touching its outputs further.
#include "attn_params.cuh"
#include "launchers.h"
#include "sm100_ptx.cuh"

namespace dsv4 {

__device__ int g_attn_error = 0;

namespace {

using namespace ptx;

constexpr int TILE = 128;              // index entries per tile (= MMA M)
constexpr int HEADS = 64;              // heads per CTA (= MMA N)
constexpr int SOFTMAX_WARPS = 4, PRODUCER_WARPS = 8;
constexpr int MMA_WARP = SOFTMAX_WARPS + PRODUCER_WARPS;
constexpr int THREADS = (MMA_WARP + 1) * 32;          // 416
constexpr int KBLOCK_BYTES = TILE * 128;              // [128 tok][64 bf16]
constexpr int QBLOCK_BYTES = HEADS * 128;
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t COL_S = 0, COL_O = 64;
constexpr float LOG2E = 1.4426950408889634f, LN2 = 0.6931471805599453f;
constexpr float RESCALE_THRESHOLD = 8.0f;             // log2 units

enum ErrCode { ERR_KFULL = 1, ERR_PFULL = 2, ERR_SFULL = 3, ERR_KVFREE = 4, ERR_ODONE = 5 };

template <int FMT, int DQK> struct Cfg {
  static constexpr bool PAGED = FMT != DSV4_KV_BF16;
  static constexpr int NB = DQK / 64;                  // 64-wide blocks of the K tile
  static constexpr int NOPE_SEGS = PAGED ? (DQK - 64) / 64 : 0;   // 64-byte FP8 segments
  static constexpr bool P_ALIAS = (DQK == 576);        // P^T lives in the RoPE block
  static constexpr int K_BYTES = NB * KBLOCK_BYTES;
  static constexpr int Q_BYTES = NB * QBLOCK_BYTES;
  static constexpr int P_BYTES = P_ALIAS ? 0 : TILE * 128;
};

struct Ctrl {
  uint64_t k_full, s_full, p_full, o_done;
  uint64_t kv_free[PRODUCER_WARPS];
  uint32_t tmem;
  int resc[2];
  float wred[SOFTMAX_WARPS][HEADS];    // per-warp column partials (max, then sums)
  float mref[HEADS];                   // reference max, log2-scaled units
  float mtrue[HEADS];                  // true running max, log2-scaled units
  float alpha[HEADS];                  // rescale factor / final output factor
};

template <int FMT, int DQK>
constexpr size_t smem_bytes() {
  using C = Cfg<FMT, DQK>;
  return 1024 + C::K_BYTES + C::Q_BYTES + C::P_BYTES + sizeof(Ctrl);
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c,
                                             uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c),
               "r"(d) : "memory");
}

__device__ __forceinline__ uint4 ldg16(const uint8_t* p) {
  return __ldg(reinterpret_cast<const uint4*>(p));
}

// Column-wise reduction over the 32 lanes of a warp of a 32-column slice held
// one row per lane: afterwards v[0] of lane l is the reduction of column l.
template <bool IS_MAX>
__device__ __forceinline__ float warp_col_reduce32(float (&v)[32], int lane) {
#pragma unroll
  for (int w = 16; w >= 1; w >>= 1) {
    const bool up = (lane & w) != 0;
#pragma unroll
    for (int i = 0; i < w; ++i) {
      const float mine = up ? v[w + i] : v[i];
      const float other = up ? v[i] : v[w + i];
      const float got = __shfl_xor_sync(0xffffffffu, other, w);
      v[i] = IS_MAX ? fmaxf(mine, got) : mine + got;
    }
  }
  return v[0];
}

struct ListView {
  const int32_t* main_idx;
  const int32_t* extra_idx;
  int len, begin, end;
};

// Fetch list entry j (j < end): which cache it names and whether it is a row.
__device__ __forceinline__ bool list_entry(const AttnParams& p, const ListView& lv, int j,
                                           int& idx, bool& is_main) {
  is_main = j < lv.len;
  idx = is_main ? __ldg(lv.main_idx + j) : __ldg(lv.extra_idx + (j - lv.len));
  const int ntok = is_main ? p.n_tok : p.extra_n_tok;
  return idx >= 0 && idx < ntok;
}

// ---------------------------------------------------------------------------
// Producer: registers for one group of 8 rows (one row per 4 lanes).
// ---------------------------------------------------------------------------
template <int FMT, int DQK> struct RowRegs {
  using C = Cfg<FMT, DQK>;
  static constexpr int NVEC = C::PAGED ? C::NOPE_SEGS + 2 : C::NB * 2;
  uint4 v[NVEC];
  uint32_t sc[2];

  __device__ __forceinline__ void zero() {
#pragma unroll
    for (int i = 0; i < NVEC; ++i) v[i] = make_uint4(0, 0, 0, 0);
    sc[0] = sc[1] = 0x7f7f7f7fu;
  }

  // lane quarter qd (0..3) of the row's 4 lanes.
  __device__ __forceinline__ void load(const AttnParams& p, bool is_main, int idx, int qd) {
    const uint8_t* kv = is_main ? p.kv : p.extra_kv;
    const int64_t stride = is_main ? p.stride_kv : p.stride_extra_kv;
    if constexpr (C::PAGED) {
      const uint8_t *row, *scl;
      token_ptrs<FMT>(kv, stride, is_main ? p.page_block : p.extra_page_block, idx, row, scl);
#pragma unroll
      for (int i = 0; i < C::NOPE_SEGS; ++i) v[i] = ldg16(row + 64 * i + 16 * qd);
      v[C::NOPE_SEGS] = ldg16(row + 64 * C::NOPE_SEGS + 16 * qd);
      v[C::NOPE_SEGS + 1] = ldg16(row + 64 * C::NOPE_SEGS + 64 + 16 * qd);
      sc[0] = __ldg(reinterpret_cast<const uint32_t*>(scl));
      if constexpr (KvTraits<FMT>::SLOTS == 8) sc[1] = __ldg(reinterpret_cast<const uint32_t*>(scl) + 1);
    } else {
      const uint8_t* row = kv + static_cast<int64_t>(idx) * stride * 2;
#pragma unroll
      for (int i = 0; i < C::NB; ++i) {
        v[2 * i] = ldg16(row + 128 * i + 32 * qd);
        v[2 * i + 1] = ldg16(row + 128 * i + 32 * qd + 16);
      }
    }
  }

  // Write the row (tile row `row`, row & 7 == r) into the swizzled K tile.
  __device__ __forceinline__ void store(uint32_t k_base, int row, int r, int qd) const {
    const uint32_t rbase = k_base + row * 128;
    if constexpr (C::PAGED) {
      using T = KvTraits<FMT>;
#pragma unroll
      for (int i = 0; i < C::NOPE_SEGS; ++i) {
        const int tile_no = i * 64 / T::TILE;
        const uint32_t s = (sc[tile_no >> 2] >> (8 * (tile_no & 3))) & 0xffu;
        const ScaleMul mul = make_scale_mul(s);
        uint32_t o[8];
        dequant4_fast(v[i].x, mul, o[0], o[1]);
        dequant4_fast(v[i].y, mul, o[2], o[3]);
        dequant4_fast(v[i].z, mul, o[4], o[5]);
        dequant4_fast(v[i].w, mul, o[6], o[7]);
        const uint32_t a = rbase + i * KBLOCK_BYTES;
        st_shared_v4(a + (((2 * qd) ^ r) << 4), o[0], o[1], o[2], o[3]);
        st_shared_v4(a + (((2 * qd + 1) ^ r) << 4), o[4], o[5], o[6], o[7]);
      }
      const uint32_t a = rbase + C::NOPE_SEGS * KBLOCK_BYTES;          // RoPE block
      const uint4 x = v[C::NOPE_SEGS], y = v[C::NOPE_SEGS + 1];
      st_shared_v4(a + ((qd ^ r) << 4), x.x, x.y, x.z, x.w);
      st_shared_v4(a + (((4 + qd) ^ r) << 4), y.x, y.y, y.z, y.w);
    } else {
#pragma unroll
      for (int i = 0; i < C::NB; ++i) {
        const uint32_t a = rbase + i * KBLOCK_BYTES;
        st_shared_v4(a + (((2 * qd) ^ r) << 4), v[2 * i].x, v[2 * i].y, v[2 * i].z, v[2 * i].w);
        st_shared_v4(a + (((2 * qd + 1) ^ r) << 4), v[2 * i + 1].x, v[2 * i + 1].y, v[2 * i + 1].z,
                     v[2 * i + 1].w);
      }
    }
  }
};

template <int FMT, int DQK>
__device__ __forceinline__ void fetch_group(RowRegs<FMT, DQK>& regs, const AttnParams& p,
                                            const ListView& lv, int j, int qd) {
  int idx;
  bool is_main;
  if (j < lv.end && list_entry(p, lv, j, idx, is_main)) regs.load(p, is_main, idx, qd);
  else regs.zero();
}

// ---------------------------------------------------------------------------
// The kernel
// ---------------------------------------------------------------------------
template <int FMT, int DQK>
__global__ void __launch_bounds__(THREADS, 1)
sm100_attn_kernel(const AttnParams p) {
  using C = Cfg<FMT, DQK>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - raw);
  const uint32_t sK = base, sQ = base + C::K_BYTES;
  const uint32_t sP = C::P_ALIAS ? sK + (C::NB - 1) * KBLOCK_BYTES : sQ + C::Q_BYTES;
  Ctrl& ctrl = *reinterpret_cast<Ctrl*>(sm + C::K_BYTES + C::Q_BYTES + C::P_BYTES);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int req = blockIdx.x, hb = blockIdx.y, split = blockIdx.z;
  const int head0 = hb * HEADS;
  const int heads_here = min(HEADS, p.h_q - head0);
  const int bi = req / p.s_q, si = req % p.s_q;
  const bool decode = p.mode == MODE_DECODE;
  const bool mask_invalid = !decode || (p.flags & DSV4_FLAG_MASK_INVALID);
  const bool split_out = p.n_splits > 1;

  ListView lv;
  int xlen;
  request_lengths(p, req, lv.len, xlen);
  split_range(lv.len + xlen, p.n_splits, split, lv.begin, lv.end);
  lv.main_idx = idx_row(p.indices, p.stride_idx_b, p.stride_idx_s, req, p.s_q);
  lv.extra_idx = p.extra_kv ? idx_row(p.extra_indices, p.stride_xidx_b, p.stride_xidx_s, req, p.s_q)
                            : nullptr;
  const int n_tiles = (lv.end - lv.begin + TILE - 1) / TILE;

  const int64_t acc_slot0 = (static_cast<int64_t>(split) * p.n_req + req) * p.h_q + head0;
  __nv_bfloat16* out_base = p.out + bi * p.stride_o_b + si * p.stride_o_s + head0 * p.stride_o_h;

  if (n_tiles == 0) {
    // Nothing to attend to: write the empty result directly (uniform branch).
    const bool has_sink = p.sink != nullptr;
    if (tid < heads_here) {
      if (split_out) {
        p.lse_accum[acc_slot0 + tid] = -INFINITY;
      } else {
        float lse_v, ml_v;
        finalize_row(p.mode, -INFINITY, 0.f, has_sink, has_sink ? p.sink[head0 + tid] : 0.f,
                     lse_v, ml_v);
        p.lse[bi * p.stride_lse_b + si * p.stride_lse_s + (head0 + tid) * p.stride_lse_h] = lse_v;
        if (p.max_logits) p.max_logits[bi * p.stride_ml_b + head0 + tid] = ml_v;
      }
    }
    for (int i = tid; i < heads_here * (D_V / 8); i += THREADS) {
      const int h = i / (D_V / 8), c = i % (D_V / 8);
      if (split_out) {
        float4* d = reinterpret_cast<float4*>(p.o_accum + (acc_slot0 + h) * D_V + c * 8);
        d[0] = make_float4(0, 0, 0, 0);
        d[1] = make_float4(0, 0, 0, 0);
      } else {
        *reinterpret_cast<uint4*>(out_base + h * p.stride_o_h + c * 8) = make_uint4(0, 0, 0, 0);
      }
    }
    return;
  }

  // ---- set-up: barriers, TMEM, Q ---------------------------------------------------
  if (tid == 0) {
    mbar_init(smem_u32(&ctrl.k_full), PRODUCER_WARPS);
    mbar_init(smem_u32(&ctrl.s_full), 1);
    mbar_init(smem_u32(&ctrl.p_full), SOFTMAX_WARPS);
    mbar_init(smem_u32(&ctrl.o_done), 1);
    for (int i = 0; i < PRODUCER_WARPS; ++i) mbar_init(smem_u32(&ctrl.kv_free[i]), 1);
    ctrl.resc[0] = ctrl.resc[1] = 0;
    mbar_init_fence();
  }
  if (tid < HEADS) {
    ctrl.mref[tid] = -INFINITY;
    ctrl.mtrue[tid] = -INFINITY;
    ctrl.alpha[tid] = 1.f;
  }
  if (warp == MMA_WARP) {
    tmem_alloc(smem_u32(&ctrl.tmem), TMEM_COLS);
    tmem_relinquish();
  }
  {
    // Q[head][d] -> blocks [d/64][head][64], 128-byte swizzle; absent heads are zero.
    const __nv_bfloat16* qrow0 = p.q + bi * p.stride_q_b + si * p.stride_q_s + head0 * p.stride_q_h;
    for (int i = tid; i < HEADS * C::NB * 8; i += THREADS) {
      const int h = i / (C::NB * 8), cc = i % (C::NB * 8), kb = cc >> 3, ch = cc & 7;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (h < heads_here)
        v = __ldg(reinterpret_cast<const uint4*>(qrow0 + h * p.stride_q_h) + cc);
      st_shared_v4(sQ + kb * QBLOCK_BYTES + h * 128 + ((ch ^ (h & 7)) << 4), v.x, v.y, v.z, v.w);
    }
  }
  fence_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = ctrl.tmem;

  const uint32_t bar_k_full = smem_u32(&ctrl.k_full), bar_s_full = smem_u32(&ctrl.s_full);
  const uint32_t bar_p_full = smem_u32(&ctrl.p_full), bar_o_done = smem_u32(&ctrl.o_done);

  if (warp == MMA_WARP) {
    // =========================== MMA issue ==========================================
    if (lane == 0) {
      const uint32_t idesc_qk = make_idesc_bf16(TILE, HEADS, 0, 0);
      const uint32_t idesc_pv = make_idesc_bf16(128, HEADS, 1, 1);
      const uint64_t dK = make_smem_desc(sK, 16, 1024, SWZ_128B);            // K-major view
      const uint64_t dQ = make_smem_desc(sQ, 16, 1024, SWZ_128B);
      const uint64_t dV = make_smem_desc(sK, KBLOCK_BYTES, 1024, SWZ_128B);  // MN-major view
      const uint64_t dP = make_smem_desc(sP, 1024, 1024, SWZ_128B);
      bool ok = true;
      for (int t = 0; t < n_tiles && ok; ++t) {
        if (!mbar_wait(bar_k_full, t & 1)) { atomicExch(&g_attn_error, ERR_KFULL); ok = false; break; }
        tc_fence_after_sync();
#pragma unroll 1
        for (int kb = 0; kb < C::NB; ++kb) {
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            umma_bf16(tmem + COL_S, desc_advance(dK, kb * KBLOCK_BYTES + ks * 32),
                      desc_advance(dQ, kb * QBLOCK_BYTES + ks * 32), idesc_qk, (kb | ks) != 0);
        }
        umma_commit(bar_s_full);
        if (!mbar_wait(bar_p_full, t & 1)) { atomicExch(&g_attn_error, ERR_PFULL); ok = false; break; }
        tc_fence_after_sync();
#pragma unroll 1
        for (int j = 0; j < TILE / 16; ++j) {
#pragma unroll
          for (int m = 0; m < D_V / 128; ++m)
            umma_bf16(tmem + COL_O + m * HEADS,
                      desc_advance(dV, m * 2 * KBLOCK_BYTES + j * 2048),
                      desc_advance(dP, j * 2048), idesc_pv, (t | j) != 0);
          umma_commit(smem_u32(&ctrl.kv_free[j]));
        }
      }
      umma_commit(bar_o_done);
    }
    __syncwarp();
  } else if (warp >= SOFTMAX_WARPS) {
    // =========================== producers ==========================================
    const int pw = warp - SOFTMAX_WARPS, r = lane >> 2, qd = lane & 3;
    const int row0 = 16 * pw + r, row1 = row0 + 8;
    const uint32_t bar_free = smem_u32(&ctrl.kv_free[pw]);
    RowRegs<FMT, DQK> g0;
    fetch_group(g0, p, lv, lv.begin + row0, qd);
    if constexpr (C::PAGED) {
      RowRegs<FMT, DQK> g1;
      fetch_group(g1, p, lv, lv.begin + row1, qd);
      for (int t = 0; t < n_tiles; ++t) {
        if (t > 0 && !mbar_wait(bar_free, (t - 1) & 1)) { atomicExch(&g_attn_error, ERR_KVFREE); break; }
        g0.store(sK, row0, r, qd);
        g1.store(sK, row1, r, qd);
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_k_full);
        if (t + 1 < n_tiles) {
          const int j = lv.begin + (t + 1) * TILE;
          fetch_group(g0, p, lv, j + row0, qd);
          fetch_group(g1, p, lv, j + row1, qd);
        }
      }
    } else {
      // BF16 rows are twice as wide: one group of 8 rows is staged ahead, the
      // second is fetched once the tile rows are free.
      for (int t = 0; t < n_tiles; ++t) {
        if (t > 0 && !mbar_wait(bar_free, (t - 1) & 1)) { atomicExch(&g_attn_error, ERR_KVFREE); break; }
        const int j = lv.begin + t * TILE;
        g0.store(sK, row0, r, qd);
        fetch_group(g0, p, lv, j + row1, qd);
        g0.store(sK, row1, r, qd);
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_k_full);
        if (t + 1 < n_tiles) fetch_group(g0, p, lv, j + TILE + row0, qd);
      }
    }
  } else {
    // =========================== softmax + epilogue =================================
    const int row = tid;                                   // tile row == TMEM lane
    const uint32_t tlane = static_cast<uint32_t>(warp * 32) << 16;
    const float cs = p.sm_scale * LOG2E;
    float lsum[HEADS];
#pragma unroll
    for (int i = 0; i < HEADS; ++i) lsum[i] = 0.f;
    bool ok = true;

    for (int t = 0; t < n_tiles; ++t) {
      // Is this row masked (beyond the range, or an invalid index under masking rules)?
      bool masked = true;
      {
        const int j = lv.begin + t * TILE + row;
        if (j < lv.end) {
          int idx;
          bool is_main;
          const bool valid = list_entry(p, lv, j, idx, is_main);
          masked = !valid && mask_invalid;
        }
      }
      if (!mbar_wait(bar_s_full, t & 1)) { atomicExch(&g_attn_error, ERR_SFULL); ok = false; break; }
      tc_fence_after_sync();

      // pass 1: per-head max over the tile's rows
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        float v[32];
        uint32_t ra[16], rb[16];
        tmem_ld16(tmem + tlane + COL_S + half * 32, ra);
        tmem_ld16(tmem + tlane + COL_S + half * 32 + 16, rb);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          v[i] = masked ? -INFINITY : __uint_as_float(ra[i]);
          v[16 + i] = masked ? -INFINITY : __uint_as_float(rb[i]);
        }
        ctrl.wred[warp][half * 32 + lane] = warp_col_reduce32<true>(v, lane);
      }
      bar_sync(1, SOFTMAX_WARPS * 32);
      if (row < HEADS) {
        float tm = fmaxf(fmaxf(ctrl.wred[0][row], ctrl.wred[1][row]),
                         fmaxf(ctrl.wred[2][row], ctrl.wred[3][row])) * cs;
        ctrl.mtrue[row] = fmaxf(ctrl.mtrue[row], tm);
        const float mr = ctrl.mref[row];
        float alpha = 1.f;
        if (tm > mr + RESCALE_THRESHOLD) {                 // also the first finite max
          alpha = (mr == -INFINITY) ? 0.f : ex2(mr - tm);
          ctrl.mref[row] = tm;
          ctrl.resc[t & 1] = 1;
        }
        ctrl.alpha[row] = alpha;
      }
      if (row == 64) ctrl.resc[(t + 1) & 1] = 0;
      bar_sync(1, SOFTMAX_WARPS * 32);

      if (ctrl.resc[t & 1]) {
#pragma unroll
        for (int i = 0; i < HEADS; ++i) lsum[i] *= ctrl.alpha[i];
        if (t > 0) {
#pragma unroll 1
          for (int c = 0; c < (D_V / 128) * (HEADS / 16); ++c) {
            const int m = c / (HEADS / 16), c4 = c % (HEADS / 16);
            uint32_t o[16];
            const uint32_t addr = tmem + tlane + COL_O + m * HEADS + c4 * 16;
            tmem_ld16(addr, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i)
              o[i] = __float_as_uint(__uint_as_float(o[i]) * ctrl.alpha[c4 * 16 + i]);
            tmem_st16(addr, o);
          }
          tmem_st_wait();
        }
      }

      // pass 2: p = 2^(s*c - mref), denominators, P^T row to shared memory
#pragma unroll
      for (int c4 = 0; c4 < HEADS / 16; ++c4) {
        uint32_t s[16];
        tmem_ld16(tmem + tlane + COL_S + c4 * 16, s);
        tmem_ld_wait();
        uint32_t packed[8];
#pragma unroll
        for (int i = 0; i < 16; i += 2) {
          float m0 = ctrl.mref[c4 * 16 + i], m1 = ctrl.mref[c4 * 16 + i + 1];
          m0 = (m0 == -INFINITY) ? 0.f : m0;
          m1 = (m1 == -INFINITY) ? 0.f : m1;
          float p0 = masked ? 0.f : ex2(fmaf(__uint_as_float(s[i]), cs, -m0));
          float p1 = masked ? 0.f : ex2(fmaf(__uint_as_float(s[i + 1]), cs, -m1));
          __nv_bfloat162 pk = __floats2bfloat162_rn(p0, p1);
          // denominators use the rounded probabilities that P.V will see
          lsum[c4 * 16 + i] += __low2float(pk);
          lsum[c4 * 16 + i + 1] += __high2float(pk);
          packed[i >> 1] = *reinterpret_cast<uint32_t*>(&pk);
        }
        const uint32_t a = sP + row * 128;
        st_shared_v4(a + (((2 * c4) ^ (row & 7)) << 4), packed[0], packed[1], packed[2], packed[3]);
        st_shared_v4(a + (((2 * c4 + 1) ^ (row & 7)) << 4), packed[4], packed[5], packed[6], packed[7]);
      }
      fence_async_smem();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_p_full);
    }

    // ---- epilogue ------------------------------------------------------------------
    if (ok && !mbar_wait(bar_o_done, 0)) { atomicExch(&g_attn_error, ERR_ODONE); ok = false; }
    tc_fence_after_sync();
    if (ok) {
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = lsum[half * 32 + i];
        ctrl.wred[warp][half * 32 + lane] = warp_col_reduce32<false>(v, lane);
      }
      bar_sync(1, SOFTMAX_WARPS * 32);
      if (row < HEADS) {
        const float l = ctrl.wred[0][row] + ctrl.wred[1][row] + ctrl.wred[2][row] + ctrl.wred[3][row];
        const float mr = ctrl.mref[row];
        float f;
        if (split_out) {
          const bool empty = !(l > 0.f);
          f = empty ? 0.f : 1.f / l;
          if (row < heads_here) p.lse_accum[acc_slot0 + row] = empty ? -INFINITY : logf(l) + mr * LN2;
        } else {
          const bool has_sink = p.sink != nullptr;
          float lse_v, ml_v;
          f = finalize_row(p.mode, mr == -INFINITY ? -INFINITY : mr * LN2, l, has_sink,
                           (has_sink && row < heads_here) ? p.sink[head0 + row] : 0.f, lse_v, ml_v);
          if (row < heads_here) {
            p.lse[bi * p.stride_lse_b + si * p.stride_lse_s + (head0 + row) * p.stride_lse_h] = lse_v;
            if (p.max_logits)
              p.max_logits[bi * p.stride_ml_b + head0 + row] =
                  (ml_v == -INFINITY) ? -INFINITY : ctrl.mtrue[row] * LN2;
          }
        }
        ctrl.alpha[row] = f;
      }
      bar_sync(1, SOFTMAX_WARPS * 32);
      // O^T[d, head] -> out[head, d]: for a fixed head a warp writes 32 consecutive d.
#pragma unroll 1
      for (int c = 0; c < (D_V / 128) * (HEADS / 16); ++c) {
        const int m = c / (HEADS / 16), c4 = c % (HEADS / 16);
        uint32_t o[16];
        tmem_ld16(tmem + tlane + COL_O + m * HEADS + c4 * 16, o);
        tmem_ld_wait();
        const int d = m * 128 + row;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int h = c4 * 16 + i;
          if (h < heads_here) {
            const float val = __uint_as_float(o[i]) * ctrl.alpha[h];
            if (split_out) p.o_accum[(acc_slot0 + h) * D_V + d] = val;
            else out_base[h * p.stride_o_h + d] = __float2bfloat16_rn(val);
          }
        }
      }
    }
  }

  // ---- teardown --------------------------------------------------------------------
  tc_fence_before_sync();
  __syncthreads();
  if (warp == MMA_WARP) tmem_dealloc(tmem, TMEM_COLS);
}

template <int FMT, int DQK>
cudaError_t launch_one(const AttnParams& p, cudaStream_t st) {
  constexpr size_t smem = smem_bytes<FMT, DQK>();
  static bool configured = false;        // per process; the attribute is per function
  static int configured_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured || configured_dev != dev) {
    cudaError_t e = cudaFuncSetAttribute(sm100_attn_kernel<FMT, DQK>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem));
    if (e) return e;
    configured = true;
    configured_dev = dev;
  }
  dim3 grid(p.n_req, (p.h_q + HEADS - 1) / HEADS, p.n_splits);
  sm100_attn_kernel<FMT, DQK><<<grid, THREADS, smem, st>>>(p);
  return cudaGetLastError();
}

}  // namespace

bool sm100_attn_supported(int kv_format, int d_qk) {
  return (kv_format == DSV4_KV_MODEL1 && d_qk == 512) || (kv_format == DSV4_KV_V32 && d_qk == 576) ||
         (kv_format == DSV4_KV_BF16 && (d_qk == 512 || d_qk == 576));
}

cudaError_t launch_sm100_attn(const AttnParams& p, int kv_format, int d_qk, cudaStream_t st) {
  if (kv_format == DSV4_KV_MODEL1) return launch_one<DSV4_KV_MODEL1, 512>(p, st);
  if (kv_format == DSV4_KV_V32) return launch_one<DSV4_KV_V32, 576>(p, st);
  if (d_qk == 512) return launch_one<DSV4_KV_BF16, 512>(p, st);
  return launch_one<DSV4_KV_BF16, 576>(p, st);
}

cudaError_t read_attn_error(int* value, bool reset) {
  cudaError_t e = cudaMemcpyFromSymbol(value, g_attn_error, sizeof(int));
  if (e) return e;
  if (reset && *value) {
    const int zero = 0;
    e = cudaMemcpyToSymbol(g_attn_error, &zero, sizeof(int));
  }
  return e;
}

}  // namespace dsv4
