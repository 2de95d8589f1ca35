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
// REGISTERS: a tile is 8 "k-steps" of 16 rows; every warp owns four rows of two
// k-steps, issues their 16-byte loads a tile ahead, and converts and writes them
// (dequantised to BF16) as soon as the P.V MMA step that last read those rows has
// retired.  P^T (16 KB) reuses the RoPE block of the tile, which only Q.K^T
// reads, when d_qk = 576.
//
// All 16 warps are alike (512 threads x 128 registers = the whole register
// file) and move through the phases of a tile together: softmax of S^T (thread
// = one tile row = one TMEM lane, 16 of the 64 heads) -> refill the K tile behind
// the P.V product and reload the registers for the tile after.  The last warp
// also issues the MMAs (converged, one elected lane), which run asynchronously
// and report through mbarriers; it is blocked for the length of each product and
// therefore stages only the first tile, its rows being dealt to ten other warps
// afterwards.  Warp 0 owns TMEM.
// TMEM columns: [0,64) S^T, [64,320) the four 128-row slices of O^T.
//
// Softmax: running per-head reference max with lazy rescaling (O^T is touched
// only when a head's max grows by more than 2^8), denominators accumulated per
// thread and reduced across the 128 rows once, at the end.
//
// Two or four splits of a request are launched as one thread-block cluster and
// merged through distributed shared memory (cluster_merge); other split counts
// leave normalised partials for the combine kernel.
//
// Every mbarrier wait is bounded; a wait that gives up records a code in
// g_attn_error, and the CTA walks on without waiting again and drops its outputs.
#include "attn_params.cuh"
#include "launchers.h"
#include "sm100_ptx.cuh"

namespace dsv4 {

__device__ int g_attn_error = 0;

namespace {

using namespace ptx;

constexpr int TILE = 128;              // index entries per tile (= MMA M)
constexpr int HEADS = 64;              // heads per CTA (= MMA N)
constexpr int WARPS = 16;
constexpr int THREADS = WARPS * 32;    // 512 threads x 128 registers
constexpr int KSTEPS = TILE / 16;      // P.V contraction steps per tile
constexpr int COLS_PER_WARP = HEADS / (WARPS / 4);    // 16 head columns per softmax thread
constexpr int KBLOCK_BYTES = TILE * 128;              // [128 tok][64 bf16]
constexpr int QBLOCK_BYTES = HEADS * 128;
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t COL_S = 0, COL_O = 64;
constexpr float LOG2E = 1.4426950408889634f, LN2 = 0.6931471805599453f;
constexpr float RESCALE_THRESHOLD = 8.0f;             // log2 units
// The warp that issues the MMAs (its lane 0 stamps the debug timeline).
constexpr int ISSUE_TID = THREADS - 32;
constexpr int ISSUE_WARP = ISSUE_TID / 32;

enum ErrCode { ERR_KFULL = 1, ERR_PFULL = 2, ERR_SFULL = 3, ERR_KVFREE = 4, ERR_ODONE = 5 };

template <int FMT, int DQK> struct Cfg {
  static constexpr bool PAGED = FMT != DSV4_KV_BF16;
  static constexpr int NB = DQK / 64;                  // 64-wide blocks of the K tile
  static constexpr int NOPE_SEGS = PAGED ? (DQK - 64) / 64 : 0;   // 64-byte FP8 segments
  static constexpr bool P_ALIAS = (DQK == 576);        // P^T lives in the last block
  static constexpr int K_BYTES = NB * KBLOCK_BYTES;
  static constexpr int Q_BYTES = NB * QBLOCK_BYTES;
  static constexpr int P_BYTES = P_ALIAS ? 0 : TILE * 128;
  // words per tile row in the multiplier table: a (first, second) factor pair per scale
  // byte; V32 has 4 scale bytes, MODEL1 7 (padded to 8)
  static constexpr int MUL_PER_ROW = !PAGED ? 0 : (DQK == 576 ? 8 : 16);
  static constexpr int MUL_TAB_BYTES = 2 * TILE * MUL_PER_ROW * 4;      // double-buffered
};

struct Ctrl {
  uint64_t k_full, s_full, p_full, o_done;
  uint64_t kv_free[KSTEPS];            // one per P.V k-step (16 tile rows)
  uint32_t tmem;
  int resc[2];
  int fail;
  alignas(16) float wred[4][HEADS];    // per-lane-group column partials (max, then sums)
  alignas(16) float mref[HEADS];       // reference max, log2-scaled units (read as float4)
  float mtrue[HEADS];                  // true running max, log2-scaled units
  float alpha[HEADS];                  // rescale factor / final output factor
};

static_assert(sizeof(Ctrl) % 16 == 0, "the multiplier table behind Ctrl is read as uint4");

template <int FMT, int DQK>
constexpr size_t smem_bytes() {
  using C = Cfg<FMT, DQK>;
  return 1024 + C::K_BYTES + C::Q_BYTES + C::P_BYTES + sizeof(Ctrl) + C::MUL_TAB_BYTES;
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c,
                                             uint32_t d) {
  // volatile keeps it ordered against the barrier waits and fences (also volatile); no
  // memory clobber, so that independent conversions can be scheduled around it
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c),
               "r"(d));
}

// 16 bytes of a KV row.  The rows are read once, so they are not kept in L1 (its array is
// the one the tensor core reads its operands from).
__device__ __forceinline__ uint4 ldg16(const uint8_t* p) {
  uint4 v;
#ifdef DSV4_LDG_ALLOCATE
  v = __ldg(reinterpret_cast<const uint4*>(p));
#else
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
#endif
  return v;
}

__device__ __forceinline__ uint32_t ldg_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}

// Column-wise reduction, over the 32 lanes of a warp, of a 16-column slice held
// one row per lane: afterwards v[0] of lane l is the reduction of column l & 15.
template <bool IS_MAX>
__device__ __forceinline__ float warp_col_reduce16(float (&v)[16], int lane) {
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float got = __shfl_xor_sync(0xffffffffu, v[i], 16);
    v[i] = IS_MAX ? fmaxf(v[i], got) : v[i] + got;
  }
#pragma unroll
  for (int w = 8; w >= 1; w >>= 1) {
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

__device__ __forceinline__ uint32_t bf16x2_max(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("max.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// Column-wise maximum, over the 32 lanes of a warp, of 16 columns held one row per lane.
// Values are rounded to BF16 first (packed pairs halve the shuffles); the result only
// serves as the softmax reference point, which needs to be the same for every thread,
// not exact.  Lane l returns the maximum of column l & 15.
__device__ __forceinline__ float warp_col_max16_bf16(const float (&v)[16], int lane) {
  uint32_t pk[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    __nv_bfloat162 t = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    pk[i] = *reinterpret_cast<uint32_t*>(&t);
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) pk[i] = bf16x2_max(pk[i], __shfl_xor_sync(0xffffffffu, pk[i], 16));
#pragma unroll
  for (int w = 4; w >= 1; w >>= 1) {            // lanes 8, 4, 2 apart: halve the register set
    const bool up = (lane & (2 * w)) != 0;
#pragma unroll
    for (int i = 0; i < w; ++i) {
      const uint32_t mine = up ? pk[w + i] : pk[i];
      const uint32_t other = up ? pk[i] : pk[w + i];
      pk[i] = bf16x2_max(mine, __shfl_xor_sync(0xffffffffu, other, 2 * w));
    }
  }
  const uint32_t r = bf16x2_max(pk[0], __shfl_xor_sync(0xffffffffu, pk[0], 1));
  return __uint_as_float((lane & 1) ? (r & 0xffff0000u) : (r << 16));
}

// Debug timeline: SM cycle counter of CTA (0,0,0) into p.prof[slot] when a buffer is set.
// Compiled in only with -DDSV4_TIMELINE (the stamps cost instructions in the hot loop).
__device__ __forceinline__ void stamp(const AttnParams& p, int slot) {
#ifdef DSV4_TIMELINE
  if (p.prof != nullptr && (blockIdx.x | blockIdx.y | blockIdx.z) == 0) p.prof[slot] = clock64();
#else
  (void)p;
  (void)slot;
#endif
}
constexpr int PROF_TILE0 = 8, PROF_PER_TILE = 8, PROF_MAX_TILES = 15;
// Per-CTA wall-clock stamps (global timer, ns) at slots 256 + 4 * cta + k; the buffer holds
// 256 + 4 * CTAs values.
__device__ __forceinline__ void stamp_cta(const AttnParams& p, int k) {
#ifdef DSV4_TIMELINE
  if (p.prof != nullptr) {
    const int cta = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    p.prof[256 + 4 * cta + k] = static_cast<long long>(t);
  }
#else
  (void)p;
  (void)k;
#endif
}

struct ListView {
  const int32_t* main_idx;
  const int32_t* extra_idx;
  int len, begin, end;
};

// List entry j without branching: entries past the end of the range read as -1.
// EXTRA says whether a second (extra) list may follow the main one.
template <bool EXTRA>
__device__ __forceinline__ int list_index(const ListView& lv, int j) {
  const bool in_range = j < lv.end;
  const int32_t* src = lv.main_idx + j;
  if constexpr (EXTRA) {
    if (j >= lv.len) src = lv.extra_idx + (j - lv.len);
  }
  return in_range ? __ldg(src) : -1;
}

// ---------------------------------------------------------------------------
// Register staging of one tile.  A tile is 8 "k-steps" of 16 rows (the rows one
// P.V MMA step contracts over).  Warp w owns, in the two k-steps j = (w >> 2) and
// j = 4 + (w >> 2), the four rows 4 * (w & 3) .. +4: lane l holds, for each
// 128-byte line c of a row, one 16-byte chunk of row (l & 1) + 2 (l >> 4).  The eight
// lanes that a 128-bit shared-memory store handles together thus belong to two rows whose
// swizzle patterns differ in the lowest bit, and the chunk a lane takes within a line is
// chosen (differently for converted and for copied lines) so that those eight lanes hit
// eight different 16-byte bank groups: no store is replayed.
// A warp-wide load touches four cache lines, the line number is a
// compile-time constant of every load/convert/store (addresses reduce to a
// per-thread base plus an immediate), and a warp needs two list entries and two
// waits per tile.  When P.V retires k-step j the four warps owning it refill it;
// the owners of different k-steps sit on different schedulers.
//   paged layouts: a row is CH 16-byte chunks: FP8 chunks (16 values -> two BF16
//                  chunks of block chunk/4) then 8 RoPE chunks (copied to the last block);
//   flat BF16:     a row is d_qk/8 chunks copied as they are; rows are twice as wide,
//                  so the two k-steps are staged one after the other.
// Scale factors come from a per-tile table in shared memory (one load per row).
// ---------------------------------------------------------------------------
template <int FMT, int DQK> struct Stage {
  using C = Cfg<FMT, DQK>;
  static constexpr int CH = C::PAGED ? C::NOPE_SEGS * 4 + 8 : DQK / 8;   // 16-byte chunks per row
  static constexpr int FP8_CH = C::PAGED ? C::NOPE_SEGS * 4 : 0;
  static constexpr int LINES = (CH + 7) / 8;
  static constexpr int PHASES = C::PAGED ? 1 : 2;
  static constexpr int HALVES = 2 / PHASES;                // k-steps held in registers at once
  // Line c holds no FP8 chunk (it is copied, not converted).
  __host__ __device__ static constexpr bool copied_line(int c) { return 8 * c >= FP8_CH; }
  uint4 d[HALVES][LINES];
};

// Per-thread constants of the staging geometry.
struct Geo {
  int jsub;     // k-steps handled: jsub and 4 + jsub
  int rloc;     // row within a k-step: 4 * (w & 3) + (l & 1) + 2 * (l >> 4)
  int piece;    // 16-byte chunk within a converted (FP8) line; it is stored as two chunks
  int piece_cp; // 16-byte chunk within a line that is copied as it is
  __device__ __forceinline__ int row(int jhalf) const { return 16 * (4 * jhalf + jsub) + rloc; }
};

// Cache geometry of list entry j (main or extra cache).
struct CacheSel {
  const uint8_t* kv;
  int64_t stride;
  int ntok, pb, sh;
};
template <bool EXTRA>
__device__ __forceinline__ CacheSel cache_of(const AttnParams& p, const ListView& lv, int j) {
  CacheSel c{p.kv, p.stride_kv, p.n_tok, p.page_block, p.page_shift};
  if constexpr (EXTRA) {
    if (j >= lv.len)
      c = CacheSel{p.extra_kv, p.stride_extra_kv, p.extra_n_tok, p.extra_page_block, p.extra_page_shift};
  }
  return c;
}

// Row start of token idx, or null when idx names no row (negative or out of range);
// `scl` gets the address of its scale bytes (paged layouts).
template <int FMT>
__device__ __forceinline__ const uint8_t* row_ptr(const CacheSel& c, int idx, const uint8_t*& scl) {
  scl = nullptr;
  if (static_cast<unsigned>(idx) >= static_cast<unsigned>(c.ntok)) return nullptr;
  if constexpr (FMT == DSV4_KV_BF16) {
    return c.kv + static_cast<int64_t>(idx) * c.stride * 2;
  } else {
    using T = KvTraits<FMT>;
    const int page = c.sh >= 0 ? (idx >> c.sh) : (idx / c.pb);
    const int rr = idx - page * c.pb;
    const uint8_t* pbase = c.kv + static_cast<int64_t>(page) * c.stride;
    scl = pbase + c.pb * T::ROW_BYTES + rr * T::SLOTS;
    return pbase + rr * T::ROW_BYTES;
  }
}

// Issue the loads of this lane's row of k-step 4 * jhalf + jsub (list entry j, token
// idx) into one register set.
template <int FMT, int DQK, bool EXTRA>
__device__ __forceinline__ void load_half(uint4 (&d)[Stage<FMT, DQK>::LINES], const AttnParams& p,
                                          const ListView& lv, int j, int idx, const Geo& geo) {
  using S = Stage<FMT, DQK>;
  const uint8_t* scl;
  const uint8_t* row = row_ptr<FMT>(cache_of<EXTRA>(p, lv, j), idx, scl);
  if (row == nullptr) {                  // the entry names no row: a row of zeros
#pragma unroll
    for (int c = 0; c < S::LINES; ++c) d[c] = make_uint4(0, 0, 0, 0);
    return;
  }
#pragma unroll
  for (int c = 0; c < S::LINES; ++c) {
    const int piece = S::copied_line(c) ? geo.piece_cp : geo.piece;
    if constexpr (8 * (S::LINES - 1) + 7 < S::CH) {
      d[c] = ldg16(row + 16 * piece + 128 * c);       // every line is full
    } else {
      d[c] = make_uint4(0, 0, 0, 0);
      if (8 * c + 7 < S::CH || 8 * c + piece < S::CH) d[c] = ldg16(row + 16 * piece + 128 * c);
    }
  }
}

// One line of a row only (line number known at run time; warp-uniform).
template <int FMT, int DQK, bool EXTRA>
__device__ __forceinline__ void load_one_line(uint4& d, int line, const AttnParams& p,
                                              const ListView& lv, int j, int idx, const Geo& geo) {
  using S = Stage<FMT, DQK>;
  const uint8_t* scl;
  const uint8_t* row = row_ptr<FMT>(cache_of<EXTRA>(p, lv, j), idx, scl);
  const int piece = S::copied_line(line) ? geo.piece_cp : geo.piece;
  d = make_uint4(0, 0, 0, 0);
  if (row != nullptr && 8 * line + piece < S::CH) d = ldg16(row + 16 * piece + 128 * line);
}

// Convert and store line LINE of the staged row `v` (tile row `row`).  `mul_row` holds the
// row's entries of the multiplier table: per scale byte s a pair of packed-BF16 factors,
// (2^(s-7), 1) normally, (2^120, 2^(s-127)) for s = 0 or s > 134.  Both multiplies are always
// done (the second is exact either way): straight-line code beats a branch per line here.
template <int FMT, int DQK, int LINE>
__device__ __forceinline__ void store_line(const uint4& v, uint32_t sK, int row, const Geo& geo,
                                           const uint32_t (&mul_row)[Cfg<FMT, DQK>::MUL_PER_ROW + 2]) {
  using S = Stage<FMT, DQK>;
  using C = Cfg<FMT, DQK>;
  const int piece = S::copied_line(LINE) ? geo.piece_cp : geo.piece;
  const int x = row & 7;
  const uint32_t rbase = sK + row * 128;
  const int ci = 8 * LINE + piece;
  if constexpr (C::PAGED) {
    using T = KvTraits<FMT>;
    constexpr bool ALL_FP8 = 8 * LINE + 7 < S::FP8_CH, NO_FP8 = 8 * LINE >= S::FP8_CH;
    if (ALL_FP8 || (!NO_FP8 && ci < S::FP8_CH)) {
      uint32_t c1, c2;
      if constexpr (T::TILE == 128) {                           // 8 chunks per scale tile
        c1 = mul_row[2 * LINE];
        c2 = mul_row[2 * LINE + 1];
      } else {                                                  // 4 chunks per scale tile
        c1 = (piece & 4) ? mul_row[4 * LINE + 2] : mul_row[4 * LINE];
        c2 = (piece & 4) ? mul_row[4 * LINE + 3] : mul_row[4 * LINE + 1];
      }
      uint32_t o[8];
      dequant4_one_mul(v.x, c1, o[0], o[1]);
      dequant4_one_mul(v.y, c1, o[2], o[3]);
      dequant4_one_mul(v.z, c1, o[4], o[5]);
      dequant4_one_mul(v.w, c1, o[6], o[7]);
#pragma unroll
      for (int k = 0; k < 8; ++k) o[k] = bf16x2_mul(o[k], c2);  // 1.0 except for rare scale bytes
      const uint32_t a = rbase + (ci >> 2) * KBLOCK_BYTES + (((2 * (ci & 3)) ^ x) << 4);
      st_shared_v4(a, o[0], o[1], o[2], o[3]);
      st_shared_v4(a ^ 16, o[4], o[5], o[6], o[7]);             // the neighbouring chunk
    } else if (ci < S::CH) {
      const uint32_t a = rbase + (C::NB - 1) * KBLOCK_BYTES;
      st_shared_v4(a + (((ci - S::FP8_CH) ^ x) << 4), v.x, v.y, v.z, v.w);
    }
  } else {
    const uint32_t a = rbase + LINE * KBLOCK_BYTES;             // line == 64-column block
    st_shared_v4(a + ((piece ^ x) << 4), v.x, v.y, v.z, v.w);
  }
}

template <int FMT, int DQK, int LINE>
__device__ __forceinline__ void store_lines(const uint4 (&d)[Stage<FMT, DQK>::LINES], uint32_t sK,
                                            int row, const Geo& geo,
                                            const uint32_t (&mul_row)[Cfg<FMT, DQK>::MUL_PER_ROW + 2]) {
  if constexpr (LINE < Stage<FMT, DQK>::LINES) {
    store_line<FMT, DQK, LINE>(d[LINE], sK, row, geo, mul_row);
    store_lines<FMT, DQK, LINE + 1>(d, sK, row, geo, mul_row);
  }
}

// The same for one line whose number is known only at run time (warp-uniform).
template <int FMT, int DQK, int LINE = 0>
__device__ __forceinline__ void store_one_line(const uint4& d, int line, uint32_t sK, int row,
                                               const Geo& geo,
                                               const uint32_t (&mul_row)[Cfg<FMT, DQK>::MUL_PER_ROW + 2]) {
  if constexpr (LINE < Stage<FMT, DQK>::LINES) {
    if (line == LINE) store_line<FMT, DQK, LINE>(d, sK, row, geo, mul_row);
    else store_one_line<FMT, DQK, LINE + 1>(d, line, sK, row, geo, mul_row);
  }
}

// ---------------------------------------------------------------------------
// Merging the splits of one request inside a thread-block cluster.
// The `cs` CTAs of a cluster (consecutive splits, cluster dimension z) finish with
// un-normalised O^T in TMEM, denominators l[h] and reference maxima m[h].  Each CTA
//   1. copies its O^T, as it is, into its own shared memory as [head][d] fp32 (128 KB in
//      the K tile region, which its own last product has released) and publishes (l, m);
//   2. meets the others at a cluster barrier;
//   3. reads every CTA's (l, m) through distributed shared memory and derives, per head,
//      the weights 2^(m_s - M) / L of all sources (times the sink factor when this
//      cluster holds all splits of the request);
//   4. pulls slice r = its rank (d in [r, r+1) * 512 / cs) of every source with 16-byte
//      ld.shared::cluster loads, sums in rank order and writes either the final BF16
//      output or one normalised fp32 partial per cluster;
//   5. meets the others again, so that no CTA retires while its memory is still read.
// Partial traffic to L2 and the combine kernel's input shrink by the cluster size, and
// with n_splits == cs there is no combine launch at all.  An empty split (no tile) takes
// part with l = 0, m = -inf (weight 0; its memory is not read); a CTA whose bounded wait
// gave up still walks every barrier (its peers must not be left waiting) and only drops
// its own stores.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_rank(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ float ld_cluster_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
  return v;
}

// Everything the merge needs, by value (the kernel's parameter block must not have its
// address taken: that would move it to local memory for the whole kernel).
struct MergeOut {
  int cluster, n_splits, mode;
  const float* sink;
  float* lse;
  float* lse_accum;
  float* o_accum;
  __nv_bfloat16* out;
  int64_t stride_o_b, stride_o_s, stride_o_h, stride_lse_b, stride_lse_s, stride_lse_h;
  long long* prof;         // debug timeline (see stamp), or null
};
__device__ __forceinline__ MergeOut merge_out_of(const AttnParams& p) {
  return MergeOut{p.cluster, p.n_splits, p.mode, p.sink, p.lse, p.lse_accum, p.o_accum, p.out,
                  p.stride_o_b, p.stride_o_s, p.stride_o_h, p.stride_lse_b, p.stride_lse_s,
                  p.stride_lse_h, p.prof};
}
struct MergeCtx {
  uint32_t stage;          // shared address of the staging area (the K tile region)
  uint32_t tmem_o;         // TMEM address of this warp's lanes of O^T (column COL_O), or unused
  int heads_here, head0, bi, si;
  int64_t acc_slot0;       // (cluster index * n_req + req) * h_q + head0
  bool empty;              // this split had no tile: no TMEM, contributes zeros
};

__device__ __forceinline__ void stamp_merge(const MergeOut& p, int slot) {
#ifdef DSV4_TIMELINE
  if (p.prof != nullptr && (blockIdx.x | blockIdx.y | blockIdx.z) == 0 && threadIdx.x == 0)
    p.prof[slot] = clock64();
#else
  (void)p;
  (void)slot;
#endif
}

// Step (4) of the merge for a cluster of CS CTAs: thread = 4 consecutive d of one head; the
// loads of BATCH items from all CS sources go out before the first is used (a remote load
// takes on the order of a microsecond).
template <int CS, int BATCH>
__device__ __forceinline__ void pull_slices(const MergeOut& p, const Ctrl& ctrl, const MergeCtx& c,
                                            float* const (&wtab)[4], uint32_t rank, bool final_out) {
  constexpr int DL = D_V / CS, QUADS = DL / 4;
  const int tid = threadIdx.x;
  const int n_items = c.heads_here * QUADS;
  __nv_bfloat16* out_base = p.out + c.bi * p.stride_o_b + c.si * p.stride_o_s + c.head0 * p.stride_o_h;
  for (int item0 = tid; item0 < n_items; item0 += BATCH * THREADS) {
    float4 v[BATCH][CS];
#pragma unroll
    for (int k = 0; k < BATCH; ++k) {
      const int item = item0 + k * THREADS;
      const int h = item / QUADS, q = item - h * QUADS;
      const uint32_t a_loc = c.stage + (h * D_V + rank * DL + 4 * q) * 4;
#pragma unroll
      for (int r = 0; r < CS; ++r) {
        v[k][r] = make_float4(0.f, 0.f, 0.f, 0.f);
        // weight 0: an empty split, whose memory holds nothing
        if (item < n_items && wtab[r][h] != 0.f) {
          if (r == static_cast<int>(rank)) {             // this CTA's own copy: plain shared load
            asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                         : "=f"(v[k][r].x), "=f"(v[k][r].y), "=f"(v[k][r].z), "=f"(v[k][r].w) : "r"(a_loc));
          } else {
            const uint32_t a = map_to_rank(a_loc, r);
            asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                         : "=f"(v[k][r].x), "=f"(v[k][r].y), "=f"(v[k][r].z), "=f"(v[k][r].w) : "r"(a));
          }
        }
      }
    }
#pragma unroll
    for (int k = 0; k < BATCH; ++k) {
      const int item = item0 + k * THREADS;
      if (item >= n_items || ctrl.fail) continue;
      const int h = item / QUADS, q = item - h * QUADS;
      const int d0 = rank * DL + 4 * q;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int r = 0; r < CS; ++r) {                     // rank order: reproducible sums
        const float w = wtab[r][h];
        acc.x = fmaf(w, v[k][r].x, acc.x);
        acc.y = fmaf(w, v[k][r].y, acc.y);
        acc.z = fmaf(w, v[k][r].z, acc.z);
        acc.w = fmaf(w, v[k][r].w, acc.w);
      }
      if (final_out) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
        *reinterpret_cast<uint2*>(out_base + h * p.stride_o_h + d0) =
            make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
      } else {
        *reinterpret_cast<float4*>(p.o_accum + (c.acc_slot0 + h) * D_V + d0) = acc;
      }
    }
  }
}

__device__ __noinline__ void cluster_merge(const MergeOut p, Ctrl& ctrl, const MergeCtx c,
                                           float l_own, float m_own) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int cs = p.cluster;                              // 2 or 4
  const uint32_t rank = cluster_rank();
  const bool final_out = p.n_splits == cs;

  // (1) own O^T -> own shared memory [head][d]; thread = one d (TMEM lane), 16 heads per load
  if (tid < HEADS) {
    ctrl.wred[0][tid] = l_own;
    ctrl.wred[1][tid] = m_own;
  }
  if (!c.empty) {
    const int m = warp >> 2, lg = warp & 3;
    const int d = m * 128 + lg * 32 + lane;
#pragma unroll 1
    for (int c4 = 0; c4 < HEADS / 16; ++c4) {
      uint32_t o[16];
      tmem_ld16(c.tmem_o + m * HEADS + c4 * 16, o);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 16; ++i)
        asm volatile("st.shared.b32 [%0], %1;" ::"r"(c.stage + ((c4 * 16 + i) * D_V + d) * 4), "r"(o[i]) : "memory");
    }
  }
  stamp_merge(p, 240);
  cluster_sync_all();                                    // (2)
  stamp_merge(p, 241);

  // (3) weights of all sources for head tid.  The table (4 sources x 64 heads) reuses arrays
  // that are idle by now; wred[0] and wred[1] stay untouched, the peers are reading them.
  float* wtab[4] = {ctrl.alpha, ctrl.wred[2], ctrl.wred[3], ctrl.mtrue};
  if (tid < HEADS) {
    const uint32_t a_l = smem_u32(&ctrl.wred[0][tid]), a_m = smem_u32(&ctrl.wred[1][tid]);
    float ms[4], ls[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      ms[r] = -INFINITY;
      ls[r] = 0.f;
      if (r < cs) {
        ms[r] = ld_cluster_f32(map_to_rank(a_m, r));
        ls[r] = ld_cluster_f32(map_to_rank(a_l, r));
      }
    }
    const float big = fmaxf(fmaxf(ms[0], ms[1]), fmaxf(ms[2], ms[3]));
    float w[4], total = 0.f;
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      w[r] = (ms[r] == -INFINITY) ? 0.f : ex2(ms[r] - big);
      total += w[r] * ls[r];
    }
    float f;
    if (final_out) {
      const bool has_sink = p.sink != nullptr;
      float lse_v, ml_v;
      f = finalize_row(p.mode, big == -INFINITY ? -INFINITY : big * LN2, total, has_sink,
                       (has_sink && tid < c.heads_here) ? p.sink[c.head0 + tid] : 0.f, lse_v, ml_v);
      if (rank == 0 && tid < c.heads_here && !ctrl.fail)
        p.lse[c.bi * p.stride_lse_b + c.si * p.stride_lse_s + (c.head0 + tid) * p.stride_lse_h] = lse_v;
    } else {
      const bool none = !(total > 0.f);
      f = none ? 0.f : 1.f / total;
      if (rank == 0 && tid < c.heads_here && !ctrl.fail)
        p.lse_accum[c.acc_slot0 + tid] = none ? -INFINITY : logf(total) + big * LN2;
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) wtab[r][tid] = w[r] * f;
  }
  __syncthreads();
  stamp_merge(p, 242);

  // (4) pull this rank's slice of every source
  if (cs == 2) pull_slices<2, 8>(p, ctrl, c, wtab, rank, final_out);
  else pull_slices<4, 4>(p, ctrl, c, wtab, rank, final_out);
  stamp_merge(p, 243);
  cluster_sync_all();                                    // (5) peers are done reading this CTA
  stamp_merge(p, 244);
}

// ---------------------------------------------------------------------------
// The kernel
// ---------------------------------------------------------------------------
template <int FMT, int DQK, bool EXTRA>
__global__ void __launch_bounds__(THREADS, 1)
sm100_attn_kernel(const AttnParams p) {
  using C = Cfg<FMT, DQK>;
  using S = Stage<FMT, DQK>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - raw);
  const uint32_t sK = base, sQ = base + C::K_BYTES;
  const uint32_t sP = C::P_ALIAS ? sK + (C::NB - 1) * KBLOCK_BYTES : sQ + C::Q_BYTES;
  Ctrl& ctrl = *reinterpret_cast<Ctrl*>(sm + C::K_BYTES + C::Q_BYTES + C::P_BYTES);
  uint32_t* mul_tab = reinterpret_cast<uint32_t*>(sm + C::K_BYTES + C::Q_BYTES + C::P_BYTES + sizeof(Ctrl));

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  grid_dependency_wait();          // inputs may come from the kernel before this one in the stream
  if (tid == 0) stamp(p, 0);
  if (tid == 0) stamp_cta(p, 0);
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
  lv.extra_idx = (EXTRA && p.extra_kv) ? idx_row(p.extra_indices, p.stride_xidx_b, p.stride_xidx_s, req, p.s_q)
                            : nullptr;
  const int n_tiles = (lv.end - lv.begin + TILE - 1) / TILE;

  // Partials are indexed by cluster when the splits of a cluster are merged on chip.
  const int64_t acc_slot0 = (static_cast<int64_t>(split / p.cluster) * p.n_req + req) * p.h_q + head0;
  __nv_bfloat16* out_base = p.out + bi * p.stride_o_b + si * p.stride_o_s + head0 * p.stride_o_h;

  if (n_tiles == 0 && p.cluster > 1) {
    // Nothing to attend to, but the peers of the cluster count on this CTA at their barriers.
    if (tid == 0) ctrl.fail = 0;
    __syncthreads();
    MergeCtx mc{sK, 0u, heads_here, head0, bi, si, acc_slot0, true};
    cluster_merge(merge_out_of(p), ctrl, mc, 0.f, -INFINITY);
    return;
  }
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

  // Set-up.  Order matters for latency: the list entries are requested first, then Q (which
  // depends on nothing), then, as the entries arrive, the first tile's rows and their scale
  // bytes; Q and the multipliers are written to shared memory while the rows are in flight.
  S stage;
  const Geo geo{warp >> 2, 4 * (warp & 3) + (lane & 1) + 2 * (lane >> 4),
                ((lane >> 1) & 3) + 4 * ((lane >> 3) & 1), 2 * ((lane >> 1) & 3) + ((lane >> 3) & 1)};
  int tidx[2];       // list entries of this lane's staged rows (k-steps jsub and 4 + jsub)
  tidx[0] = list_index<EXTRA>(lv, lv.begin + geo.row(0));
  tidx[1] = list_index<EXTRA>(lv, lv.begin + geo.row(1));
  // Softmax geometry: TMEM lanes 32*lg.. (tile rows), head columns 16*cg..16*cg+15.
  const int lg = warp & 3, cg = warp >> 2;
  const int row = lg * 32 + lane;
  // The list entry of this thread's own tile row (masking; scale-table fill by tid < 128).
  int ridx = list_index<EXTRA>(lv, lv.begin + row);
  // List entries are fetched ahead so that no address ever waits on them: tidx / ridx
  // belong to the tile staged in registers, tidx_next / ridx_n1 to the one after,
  // ridx_n2 to the one after that.
  int tidx_next[2] = {-1, -1}, ridx_n1 = -1, ridx_n2 = -1;
  // The warp that issues the MMAs is blocked for the length of every product, so after the
  // first tile it stages nothing: the lines of its two row groups (k-steps 3 and 7) are
  // spread over warps 0 .. 2 LINES - 1, one line each, held in one more register set `xd`
  // (loaded a tile ahead like the others; xidx_next is the list entry it is loaded from).
  constexpr bool SPARE_ISSUER = S::HALVES == 2;
  const bool has_x = SPARE_ISSUER && warp < 2 * S::LINES;
  const int xline = warp % S::LINES;
  const int xk = warp < S::LINES ? ISSUE_WARP >> 2 : 4 + (ISSUE_WARP >> 2);
  const int xrow = 16 * xk + 4 * (ISSUE_WARP & 3) + (lane & 1) + 2 * (lane >> 4);
  int xidx_next = -1;
  uint4 xd = make_uint4(0, 0, 0, 0);
  if (n_tiles > 1) {
    tidx_next[0] = list_index<EXTRA>(lv, lv.begin + TILE + geo.row(0));
    tidx_next[1] = list_index<EXTRA>(lv, lv.begin + TILE + geo.row(1));
    ridx_n1 = ridx_n2 = list_index<EXTRA>(lv, lv.begin + TILE + row);
    if (has_x) xidx_next = list_index<EXTRA>(lv, lv.begin + TILE + xrow);
  }
  // Multipliers of tile row `tid` into the table of tile `slot` (threads 0..127): one load
  // of the row's scale bytes (issued early, `ScaleWords`), later a pair of packed factors
  // per byte into the table.
  struct ScaleWords { uint32_t w[C::PAGED ? KvTraits<C::PAGED ? FMT : DSV4_KV_V32>::SLOTS / 4 : 1]; };
  auto load_scales = [&](int j, int idx) {
    ScaleWords sw;
    if constexpr (C::PAGED) {
      using T = KvTraits<FMT>;
#pragma unroll
      for (int k = 0; k < T::SLOTS / 4; ++k) sw.w[k] = 0x7f7f7f7fu;
      if (tid < TILE) {
        const uint8_t* scl;
        const uint8_t* r = row_ptr<FMT>(cache_of<EXTRA>(p, lv, j), j < lv.end ? idx : -1, scl);
        if (r != nullptr) {
#pragma unroll
          for (int k = 0; k < T::SLOTS / 4; ++k) sw.w[k] = ldg_u32(reinterpret_cast<const uint32_t*>(scl) + k);
        }
      }
    } else {
      sw.w[0] = 0;
    }
    return sw;
  };
  // Ask the memory system to bring the row of list entry (j, idx) into L2 (threads 0..127, one
  // row each; a bulk prefetch ties up no register).  Used for the second tile only, whose
  // register loads cannot be issued before the first tile is converted: in the steady state
  // the same prefetch a tile ahead made things slower (b = 64: 60 -> 67 us).
  auto prefetch_row = [&](int j, int idx) {
    if (tid < TILE && j < lv.end) {
      const uint8_t* scl;
      const uint8_t* r = row_ptr<FMT>(cache_of<EXTRA>(p, lv, j), idx, scl);
      constexpr uint32_t ROW = C::PAGED ? KvTraits<C::PAGED ? FMT : DSV4_KV_V32>::ROW_BYTES : DQK * 2;
      if (r != nullptr)
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(r), "r"(ROW) : "memory");
    }
  };
  auto store_scales = [&](int slot, const ScaleWords& sw) {
    if constexpr (C::PAGED) {
      using T = KvTraits<FMT>;
      if (tid < TILE) {
        uint32_t* dst = mul_tab + (slot * TILE + tid) * C::MUL_PER_ROW;
#pragma unroll
        for (int k = 0; k < T::N_SCALE; ++k) {
          const ScaleMul m = make_scale_mul((sw.w[k >> 2] >> (8 * (k & 3))) & 0xffu);
          dst[2 * k] = m.c1;
          dst[2 * k + 1] = m.c2 ? m.c2 : 0x3F803F80u;           // packed BF16 1.0
        }
      }
    }
  };

  // ---- set-up: Q requests, barriers, TMEM, first tile -----------------------------------
  // Q[head][d] -> blocks [d/64][head][64], 128-byte swizzle; absent heads are zero.
  const __nv_bfloat16* qrow0 = p.q + bi * p.stride_q_b + si * p.stride_q_s + head0 * p.stride_q_h;
  constexpr int Q_CHUNKS = HEADS * C::NB * 8;
  constexpr int Q_BATCH = (Q_CHUNKS + THREADS - 1) / THREADS;     // all in flight at once
  uint4 qv[Q_BATCH];
#pragma unroll
  for (int it = 0; it < Q_BATCH; ++it) {
    const int i = tid + it * THREADS;
    const int h = i / (C::NB * 8), cc = i % (C::NB * 8);
    qv[it] = make_uint4(0, 0, 0, 0);
    if (i < Q_CHUNKS && h < heads_here)
      qv[it] = ldg16(reinterpret_cast<const uint8_t*>(qrow0 + h * p.stride_q_h) + 16 * cc);
  }
  if (tid == 0) {
    mbar_init(smem_u32(&ctrl.k_full), WARPS);
    mbar_init(smem_u32(&ctrl.s_full), 1);
    mbar_init(smem_u32(&ctrl.p_full), WARPS);
    mbar_init(smem_u32(&ctrl.o_done), 1);
    for (int i = 0; i < KSTEPS; ++i) mbar_init(smem_u32(&ctrl.kv_free[i]), 1);
    ctrl.resc[0] = ctrl.resc[1] = 0;
    ctrl.fail = 0;
    mbar_init_fence();
  }
  if (tid < HEADS) {
    ctrl.mref[tid] = -INFINITY;
    ctrl.mtrue[tid] = -INFINITY;
    ctrl.alpha[tid] = 1.f;
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(&ctrl.tmem), TMEM_COLS);
    tmem_relinquish();
  }
  // First use of the list entries: the first tile's rows and scale bytes go in flight.
#pragma unroll
  for (int hh = 0; hh < S::HALVES; ++hh)
    load_half<FMT, DQK, EXTRA>(stage.d[hh], p, lv, lv.begin + geo.row(hh), tidx[hh], geo);
  const ScaleWords sw0 = load_scales(lv.begin + row, ridx);
#pragma unroll
  for (int it = 0; it < Q_BATCH; ++it) {
    const int i = tid + it * THREADS;
    const int h = i / (C::NB * 8), cc = i % (C::NB * 8), kb = cc >> 3, ch = cc & 7;
    if (i < Q_CHUNKS)
      st_shared_v4(sQ + kb * QBLOCK_BYTES + h * 128 + ((ch ^ (h & 7)) << 4), qv[it].x, qv[it].y,
                   qv[it].z, qv[it].w);
  }
  store_scales(0, sw0);
  fence_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  // The first tile's rows have had HBM to themselves; now, while they are converted, the
  // second tile's rows are brought into L2.
  if (n_tiles > 1) prefetch_row(lv.begin + TILE + row, ridx_n1);
  const uint32_t tmem = ctrl.tmem;
  if (tid == 0) stamp(p, 1);
  if (tid == 0) stamp_cta(p, 1);
#define TSTAMP(t, k) do { if ((t) < PROF_MAX_TILES) stamp(p, PROF_TILE0 + (t) * PROF_PER_TILE + (k)); } while (0)

  const uint32_t bar_k_full = smem_u32(&ctrl.k_full), bar_s_full = smem_u32(&ctrl.s_full);
  const uint32_t bar_p_full = smem_u32(&ctrl.p_full), bar_o_done = smem_u32(&ctrl.o_done);
  const uint32_t bar_kv_free0 = smem_u32(&ctrl.kv_free[0]);
  bool ok = true;      // false once one of this thread's bounded waits has given up

  // ---- MMA issue (thread 0 only) -----------------------------------------------------
  const uint32_t idesc_qk = make_idesc_bf16(TILE, HEADS, 0, 0);
  const uint32_t idesc_pv = make_idesc_bf16(128, HEADS, 1, 1);
  const uint64_t dK = make_smem_desc(sK, 16, 1024, SWZ_128B);            // K-major view
  const uint64_t dQ = make_smem_desc(sQ, 16, 1024, SWZ_128B);
  const uint64_t dV = make_smem_desc(sK, KBLOCK_BYTES, 1024, SWZ_128B);  // MN-major view
  const uint64_t dP = make_smem_desc(sP, 1024, 1024, SWZ_128B);
  // Both issue routines are run by the whole issuing warp, converged; one elected lane
  // issues the MMAs and the commits (see umma_bf16_elect).
  const uint32_t elected = elect_one();
  const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem, 0);
  auto issue_qk = [&](int t, bool& ok) {
    if (ok && !mbar_wait_warp(bar_k_full, t & 1, lane)) { atomicExch(&g_attn_error, ERR_KFULL); ok = false; }
    tc_fence_after_sync();
    if (lane == 0) TSTAMP(t, 1);
#pragma unroll 1
    for (int kb = 0; kb < C::NB; ++kb) {     // four 16-wide steps of one 64-column block
#pragma unroll
      for (int k4 = 0; k4 < 4; ++k4)
        umma_bf16_elect(tmem_u + COL_S, dK + static_cast<uint64_t>((kb * KBLOCK_BYTES + k4 * 32) >> 4),
                        dQ + static_cast<uint64_t>((kb * QBLOCK_BYTES + k4 * 32) >> 4), idesc_qk,
                        (kb | k4) != 0, elected);
    }
    umma_commit_elect(bar_s_full, elected);
  };
  auto issue_pv = [&](int t, bool last, bool& ok) {
    if (ok && !mbar_wait_warp(bar_p_full, t & 1, lane)) { atomicExch(&g_attn_error, ERR_PFULL); ok = false; }
    tc_fence_after_sync();
    if (lane == 0) TSTAMP(t, 5);
#pragma unroll 1
    for (int j = 0; j < KSTEPS; ++j) {       // the four 128-row slices of O^T for one k-step
      const uint32_t acc = (t | j) != 0;
#pragma unroll
      for (int mb = 0; mb < 4; ++mb)
        umma_bf16_elect(tmem_u + COL_O + mb * HEADS,
                        dV + static_cast<uint64_t>((j * 2048 + mb * 2 * KBLOCK_BYTES) >> 4),
                        dP + static_cast<uint64_t>((j * 2048) >> 4), idesc_pv, acc, elected);
      umma_commit_elect(bar_kv_free0 + 8 * j, elected);
    }
    if (last) umma_commit_elect(bar_o_done, elected);
  };

  // ---- refill of the K tile from the staged registers -------------------------------
  // `wait_tile` >= 0: rows of k-step j may be overwritten only once the P.V step j of
  // that tile has retired.  After a wait has given up (`ok` false) no further wait is
  // attempted, but every thread keeps walking the same path so that the CTA-wide
  // barriers below stay matched; the outputs are then suppressed.
  // As soon as a register set has been stored it is reloaded with the same rows of the
  // next tile (list entries tidx_next; `has_next` false on the last tile), so the gather
  // is spread over the whole P.V phase instead of hitting memory in one burst.
  auto refill = [&](int j0, int wait_tile, int slot, bool has_next, bool& ok) {
    const bool first = wait_tile < 0;
    const bool spared = SPARE_ISSUER && warp == ISSUE_WARP;     // stages the first tile only
    const bool extra = has_x && !first;
    auto wait_free = [&](int j) {
      if (!first && ok && !mbar_wait_warp(bar_kv_free0 + 8 * j, wait_tile & 1, lane)) {
        atomicExch(&g_attn_error, ERR_KVFREE);
        ok = false;
      }
    };
    auto row_multipliers = [&](uint32_t (&mrow)[C::MUL_PER_ROW + 2], int trow) {
      if constexpr (C::PAGED) {                   // one vector load each 4
        const uint4* src = reinterpret_cast<const uint4*>(mul_tab + (slot * TILE + trow) * C::MUL_PER_ROW);
#pragma unroll
        for (int k = 0; k < C::MUL_PER_ROW / 4; ++k) {
          const uint4 m4 = src[k];
          mrow[4 * k] = m4.x; mrow[4 * k + 1] = m4.y; mrow[4 * k + 2] = m4.z; mrow[4 * k + 3] = m4.w;
        }
      }
      mrow[C::MUL_PER_ROW] = mrow[C::MUL_PER_ROW + 1] = 0;
    };
    auto store_set = [&](const uint4 (&d)[S::LINES], int trow) {
      uint32_t mrow[C::MUL_PER_ROW + 2];
      row_multipliers(mrow, trow);
      store_lines<FMT, DQK, 0>(d, sK, trow, geo, mrow);
    };
    auto publish = [&]() {                   // this warp's part of the tile is in shared memory
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_k_full);
    };
    if (spared && !first) {
      publish();
      return;
    }
    const bool reload = has_next && !spared;
    if constexpr (S::HALVES == 2) {
      // Both k-steps are staged.  Each register set is reloaded as soon as it has been stored:
      // that spreads the gather over the P.V phase (all SMs gather in step, and a burst holds
      // the issuing warps up for as long as HBM takes to serve it).
#pragma unroll
      for (int jhalf = 0; jhalf < 2; ++jhalf) {
        wait_free(4 * jhalf + geo.jsub);
        if (lane == 0 && wait_tile == 2) stamp(p, 150 + 32 * jhalf + warp);       // k-step free
        store_set(stage.d[jhalf], geo.row(jhalf));
        if (reload)                        // the same rows of the next tile
          load_half<FMT, DQK, EXTRA>(stage.d[jhalf], p, lv, j0 + TILE + geo.row(jhalf), tidx_next[jhalf], geo);
      }
      if (extra) {                         // this warp's line of the issuing warp's rows
        wait_free(xk);
        uint32_t mrow[C::MUL_PER_ROW + 2];
        row_multipliers(mrow, xrow);
        store_one_line<FMT, DQK>(xd, xline, sK, xrow, geo, mrow);
      }
      publish();
      if (lane == 0 && wait_tile == 2) stamp(p, 214 + warp);                     // arrived
      if (has_x && has_next)
        load_one_line<FMT, DQK, EXTRA>(xd, xline, p, lv, j0 + TILE + xrow, xidx_next, geo);
    } else {
      // One register set: the second k-step is loaded once the first is stored, then the
      // first k-step of the next tile.
#pragma unroll
      for (int jhalf = 0; jhalf < 2; ++jhalf) {
        wait_free(4 * jhalf + geo.jsub);
        store_set(stage.d[0], geo.row(jhalf));
        if (jhalf == 0) {
          load_half<FMT, DQK, EXTRA>(stage.d[0], p, lv, j0 + geo.row(1), tidx[1], geo);
        } else {
          publish();
          if (has_next)
            load_half<FMT, DQK, EXTRA>(stage.d[0], p, lv, j0 + TILE + geo.row(0), tidx_next[0], geo);
        }
      }
    }
  };

  const uint32_t tlane = static_cast<uint32_t>(lg * 32) << 16;
  const float cs = p.sm_scale * LOG2E;
  float lsum[COLS_PER_WARP];
#pragma unroll
  for (int i = 0; i < COLS_PER_WARP; ++i) lsum[i] = 0.f;


  ScaleWords sw_next = {};
  // Iteration t = -1 only fills the first tile; iteration t >= 0 runs tile t and, behind
  // its P.V product, fills tile t + 1.
#pragma unroll 1
  for (int t = -1; t < n_tiles; ++t) {
    const bool more = t + 1 < n_tiles;
    if (t >= 0) {
    if (warp == ISSUE_WARP) issue_qk(t, ok);
    if (t + 2 < n_tiles) {                       // list entries of the tile after next
      const int j2 = lv.begin + (t + 2) * TILE;
      tidx_next[0] = list_index<EXTRA>(lv, j2 + geo.row(0));
      tidx_next[1] = list_index<EXTRA>(lv, j2 + geo.row(1));
      ridx_n2 = list_index<EXTRA>(lv, j2 + row);
      if (has_x) xidx_next = list_index<EXTRA>(lv, j2 + xrow);
    }
    // Is this thread's row masked (beyond the range, or an invalid entry under masking rules)?
    bool masked = true;
    {
      const int j = lv.begin + t * TILE + row;
      if (j < lv.end) {
        const int ntok = (EXTRA && j >= lv.len) ? p.extra_n_tok : p.n_tok;
        masked = static_cast<unsigned>(ridx) >= static_cast<unsigned>(ntok) && mask_invalid;
      }
    }

    if (ok && !mbar_wait_warp(bar_s_full, t & 1, lane)) { atomicExch(&g_attn_error, ERR_SFULL); ok = false; }
    tc_fence_after_sync();
    // Scale bytes of the tile after next (its list entries arrived during Q.K^T); they
    // become multipliers at the end of this iteration.
    if (t + 2 < n_tiles) sw_next = load_scales(lv.begin + (t + 2) * TILE + row, ridx_n2);
    if (tid == 0) TSTAMP(t, 2);

    // pass 1: per-head max over the tile's rows
    {
      uint32_t ra[16];
      tmem_ld16(tmem + tlane + COL_S + cg * 16, ra);
      tmem_ld_wait();
      float v[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) v[i] = masked ? -INFINITY : __uint_as_float(ra[i]);
      const float cm = warp_col_max16_bf16(v, lane);
      if (lane < 16) ctrl.wred[lg][cg * 16 + lane] = cm;
    }
    __syncthreads();
    if (tid < HEADS) {
      float tm = fmaxf(fmaxf(ctrl.wred[0][tid], ctrl.wred[1][tid]),
                       fmaxf(ctrl.wred[2][tid], ctrl.wred[3][tid])) * cs;
      ctrl.mtrue[tid] = fmaxf(ctrl.mtrue[tid], tm);
      const float mr = ctrl.mref[tid];
      float alpha = 1.f;
      if (tm > mr + RESCALE_THRESHOLD) {                 // also the first finite max
        alpha = (mr == -INFINITY) ? 0.f : ex2(mr - tm);
        ctrl.mref[tid] = tm;
        ctrl.resc[t & 1] = 1;
      }
      ctrl.alpha[tid] = alpha;
    }
    if (tid == 64) ctrl.resc[(t + 1) & 1] = 0;
    __syncthreads();
    if (tid == 0) TSTAMP(t, 3);

    if (ctrl.resc[t & 1]) {
#pragma unroll
      for (int i = 0; i < COLS_PER_WARP; ++i) lsum[i] *= ctrl.alpha[cg * 16 + i];
      if (t > 0) {
        // this warp rescales slice cg of O^T for its 32 TMEM lanes
#pragma unroll 1
        for (int c4 = 0; c4 < HEADS / 16; ++c4) {
          uint32_t o[16];
          const uint32_t addr = tmem + tlane + COL_O + cg * HEADS + c4 * 16;
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

    // pass 2: p = 2^(s*c - mref), denominators, this thread's 32 bytes of the P^T row
    {
      uint32_t s[16];
      tmem_ld16(tmem + tlane + COL_S + cg * 16, s);   // warp-collective: all lanes take part
      tmem_ld_wait();
      if (__any_sync(0xffffffffu, masked)) {          // rare: ragged tile or masked entries
        const uint32_t ninf = __float_as_uint(-INFINITY);
#pragma unroll
        for (int i = 0; i < 16; ++i) s[i] = masked ? ninf : s[i];
      }
      uint32_t pk[8];
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        float4 mu = *reinterpret_cast<const float4*>(&ctrl.mref[cg * 16 + q4 * 4]);
        mu.x = (mu.x == -INFINITY) ? 0.f : mu.x;      // nothing seen yet: any finite offset will do
        mu.y = (mu.y == -INFINITY) ? 0.f : mu.y;
        mu.z = (mu.z == -INFINITY) ? 0.f : mu.z;
        mu.w = (mu.w == -INFINITY) ? 0.f : mu.w;
        const float p0 = ex2(fmaf(__uint_as_float(s[q4 * 4 + 0]), cs, -mu.x));
        const float p1 = ex2(fmaf(__uint_as_float(s[q4 * 4 + 1]), cs, -mu.y));
        const float p2 = ex2(fmaf(__uint_as_float(s[q4 * 4 + 2]), cs, -mu.z));
        const float p3 = ex2(fmaf(__uint_as_float(s[q4 * 4 + 3]), cs, -mu.w));
        lsum[q4 * 4 + 0] += p0;
        lsum[q4 * 4 + 1] += p1;
        lsum[q4 * 4 + 2] += p2;
        lsum[q4 * 4 + 3] += p3;
        __nv_bfloat162 a = __floats2bfloat162_rn(p0, p1), b = __floats2bfloat162_rn(p2, p3);
        pk[q4 * 2] = *reinterpret_cast<uint32_t*>(&a);
        pk[q4 * 2 + 1] = *reinterpret_cast<uint32_t*>(&b);
      }
      const uint32_t prow = sP + row * 128;
      const int x = row & 7;
      st_shared_v4(prow + (((2 * cg) ^ x) << 4), pk[0], pk[1], pk[2], pk[3]);
      st_shared_v4(prow + (((2 * cg + 1) ^ x) << 4), pk[4], pk[5], pk[6], pk[7]);
    }
    fence_async_smem();
    tc_fence_before_sync();
    __syncwarp();
    if (lane == 0) mbar_arrive(bar_p_full);
    if (tid == 0) TSTAMP(t, 4);
    if (warp == ISSUE_WARP) issue_pv(t, !more, ok);

    }  // t >= 0

    // fill tile t + 1 (behind the P.V product of tile t, if there is one)
    if (more) {
      refill(lv.begin + (t + 1) * TILE, t, (t + 1) & 1, t + 2 < n_tiles, ok);
      if (tid == 0) TSTAMP(t + 1, 0);
      if (tid == THREADS - 32) TSTAMP(t + 1, 7);
      if (lane == 0 && t == 2) stamp(p, 230 + warp);                             // refill returned
    }
    // The registers now hold (or are receiving) tile t + 2: publish its multipliers (read
    // after the two CTA barriers of the next iteration).
    tidx[0] = tidx_next[0];
    tidx[1] = tidx_next[1];
    if (t >= 0 && t + 2 < n_tiles) store_scales(t & 1, sw_next);
    if (t < 0 && n_tiles > 1) store_scales(1, load_scales(lv.begin + TILE + row, ridx_n2));
    if (t >= 0) {
      ridx = ridx_n1;
      ridx_n1 = ridx_n2;
    }
  }

  // The kernel after this one in the stream (the split combine, or the next layer) may be
  // set up on the SMs while the epilogue runs; it waits for this grid's end before it reads.
  grid_launch_dependents();

  // ---- final denominators and output factors ---------------------------------------
  if (ok && !mbar_wait_warp(bar_o_done, 0, lane)) { atomicExch(&g_attn_error, ERR_ODONE); ok = false; }
  tc_fence_after_sync();
  if (tid == 0) stamp(p, 3);
  if (tid == 0) stamp_cta(p, 2);
  if (!ok) ctrl.fail = 1;
  {
    float v[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = lsum[i];
    const float cm = warp_col_reduce16<false>(v, lane);
    if (lane < 16) ctrl.wred[lg][cg * 16 + lane] = cm;
  }
  __syncthreads();
  if (p.cluster > 1) {
    float l = 0.f, mr = -INFINITY;
    if (tid < HEADS) {
      l = ctrl.wred[0][tid] + ctrl.wred[1][tid] + ctrl.wred[2][tid] + ctrl.wred[3][tid];
      mr = ctrl.mref[tid];
    }
    MergeCtx mc{sK, tmem + tlane + COL_O, heads_here, head0, bi, si, acc_slot0, false};
    cluster_merge(merge_out_of(p), ctrl, mc, l, mr);
  } else {
  if (tid < HEADS && !ctrl.fail) {
    const float l = ctrl.wred[0][tid] + ctrl.wred[1][tid] + ctrl.wred[2][tid] + ctrl.wred[3][tid];
    const float mr = ctrl.mref[tid];
    float f;
    if (split_out) {
      const bool empty = !(l > 0.f);
      f = empty ? 0.f : 1.f / l;
      if (tid < heads_here) p.lse_accum[acc_slot0 + tid] = empty ? -INFINITY : logf(l) + mr * LN2;
    } else {
      const bool has_sink = p.sink != nullptr;
      float lse_v, ml_v;
      f = finalize_row(p.mode, mr == -INFINITY ? -INFINITY : mr * LN2, l, has_sink,
                       (has_sink && tid < heads_here) ? p.sink[head0 + tid] : 0.f, lse_v, ml_v);
      if (tid < heads_here) {
        p.lse[bi * p.stride_lse_b + si * p.stride_lse_s + (head0 + tid) * p.stride_lse_h] = lse_v;
        if (p.max_logits)
          p.max_logits[bi * p.stride_ml_b + head0 + tid] =
              (ml_v == -INFINITY) ? -INFINITY : ctrl.mtrue[tid] * LN2;
      }
    }
    ctrl.alpha[tid] = f;
  }
  __syncthreads();

  // ---- epilogue: warp w drains O^T slice w / 4 for TMEM lanes 32 * (w % 4).. --------
  if (!ctrl.fail) {
    const int m = warp >> 2;
    const int d = m * 128 + lg * 32 + lane;
#pragma unroll 1
    for (int c4 = 0; c4 < HEADS / 16; ++c4) {
      uint32_t o[16];
      tmem_ld16(tmem + tlane + COL_O + m * HEADS + c4 * 16, o);
      tmem_ld_wait();
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
  }  // not clustered

  // ---- teardown --------------------------------------------------------------------
  if (tid == 0) stamp(p, 4);
  tc_fence_before_sync();
  __syncthreads();
  if (tid == 0) stamp(p, 5);
  if (tid == 0) stamp_cta(p, 3);
  if (warp == 0) tmem_dealloc(tmem, TMEM_COLS);
}

template <int FMT, int DQK, bool EXTRA>
cudaError_t launch_one(const AttnParams& p, cudaStream_t st) {
  constexpr size_t smem = smem_bytes<FMT, DQK>();
  static bool configured = false;        // per process; the attribute is per function
  static int configured_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured || configured_dev != dev) {
    cudaError_t e = cudaFuncSetAttribute(sm100_attn_kernel<FMT, DQK, EXTRA>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem));
    if (e) return e;
    configured = true;
    configured_dev = dev;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.n_req, (p.h_q + HEADS - 1) / HEADS, p.n_splits);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  cfg.attrs = attr;
  cfg.numAttrs = add_overlap_attribute(attr);
  if (p.cluster > 1) {
    attr[cfg.numAttrs].id = cudaLaunchAttributeClusterDimension;
    attr[cfg.numAttrs].val.clusterDim.x = 1;
    attr[cfg.numAttrs].val.clusterDim.y = 1;
    attr[cfg.numAttrs].val.clusterDim.z = p.cluster;
    ++cfg.numAttrs;
  }
  return cudaLaunchKernelEx(&cfg, sm100_attn_kernel<FMT, DQK, EXTRA>, p);
}

}  // namespace

bool sm100_attn_supported(int kv_format, int d_qk) {
  return (kv_format == DSV4_KV_MODEL1 && d_qk == 512) || (kv_format == DSV4_KV_V32 && d_qk == 576) ||
         (kv_format == DSV4_KV_BF16 && (d_qk == 512 || d_qk == 576));
}

cudaError_t launch_sm100_attn(const AttnParams& p, int kv_format, int d_qk, cudaStream_t st) {
  const bool extra = p.extra_kv != nullptr;
  if (kv_format == DSV4_KV_MODEL1)
    return extra ? launch_one<DSV4_KV_MODEL1, 512, true>(p, st) : launch_one<DSV4_KV_MODEL1, 512, false>(p, st);
  if (kv_format == DSV4_KV_V32)
    return extra ? launch_one<DSV4_KV_V32, 576, true>(p, st) : launch_one<DSV4_KV_V32, 576, false>(p, st);
  if (d_qk == 512) return launch_one<DSV4_KV_BF16, 512, false>(p, st);
  return launch_one<DSV4_KV_BF16, 576, false>(p, st);
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
