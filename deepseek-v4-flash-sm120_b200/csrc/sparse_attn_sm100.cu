// Sparse MLA attention on the 5th-generation tensor cores (tcgen05 + TMEM).
//
// One CTA handles one (request, block of NH <= 64 heads, split) and walks the
// request's index list in tiles of 128 entries.  Gathered KV rows are the M
// dimension of the MMAs ("tokens as M"), heads are N = NH (16, 32 or 64):
//
//   S^T[128 tok, NH heads]  = K[128 tok, d_qk]      . Q^T      (K-major A and B)
//   O^T[512 d_v, NH heads] += V^T[512, 128 tok]     . P^T      (MN-major A and B)
//
// V is the first 512 columns of the same dequantised K tile, so ONE shared-
// memory tile serves both products: it is stored as d_qk/64 blocks of
// [128 tokens][64 values] with the 128-byte swizzle, which reads as K-major
// (contraction over d) for the first product and as MN-major (contraction over
// tokens) for the second.  With d_qk = 576 the tile (144 KB) and Q (72 KB) leave
// no room for a second tile, so the tile is recycled BLOCK BY BLOCK:
//
//   * P.V runs slice-major: the eight k-steps of output slice 0 (d 0..127, tile
//     blocks 0 and 1), then slice 1, ... each followed by a tcgen05.commit.  When
//     slice g retires, blocks 2g and 2g+1 are dead and the worker warps write the
//     same blocks of the NEXT tile over them (group g of the refill);
//   * Q.K^T of the next tile is issued block by block behind the refill, each
//     group of blocks waiting on its own mbarrier, so the tensor pipe goes from
//     P.V(t) straight into Q.K^T(t+1) and only idles while softmax(t+1) runs.
//
// Gathered FP8 rows are staged in REGISTERS a tile ahead (16 worker warps x 128-byte
// lines: 80 KB in flight per SM): a worker owns two rows of the tile; when a group
// is free it converts and stores the matching 128-byte line of its rows and at once
// re-issues the loads of the same line of the tile after.  Flat BF16 rows (prefill
// workspace) need no conversion and go from global to shared memory with cp.async.
//
// Warps: 16 workers (gather, convert, softmax, epilogue) and one warp that only issues
// MMAs (converged, one elected lane).  TMEM columns: [0, NH) S^T, [64 + 64 mb, +NH) the
// four 128-row slices of O^T.
//
// Softmax: per-head reference maximum with lazy rescaling.  A tile is first evaluated
// against the reference as it stands; only if some logit exceeds it by more than 2^8
// (always on the first tile) do the workers meet, raise the reference and rescale O^T.
// The common tile costs one named barrier (an OR over the workers) and no reduction;
// denominators are accumulated per thread and reduced across the 128 rows once, at the end.
//
// Two or four splits of a request are launched as one thread-block cluster and
// merged through distributed shared memory (cluster_merge); other split counts
// leave normalised partials for the combine kernel.
//
// Every mbarrier wait is bounded; a wait that gives up records a code in
// g_attn_error, and the CTA walks on without waiting again, drops its outputs and
// writes NaN into the log-sum-exp slots it owns so that the failure is visible
// downstream without a host synchronisation.
#include <mutex>
#include <type_traits>

#include "attn_params.cuh"
#include "launchers.h"
#include "sm100_ptx.cuh"

namespace dsv4 {

__device__ int g_attn_error = 0;

namespace {

using namespace ptx;

constexpr int TILE = 128;              // index entries per tile (= MMA M)
constexpr int MAX_HEADS = 64;          // most heads per CTA (= largest MMA N)
constexpr int WORKER_WARPS = 16;
constexpr int WORKERS = WORKER_WARPS * 32;
// A fifth warpgroup holds the warp that only issues MMAs (its other three warps idle at
// the CTA barriers).  It gives most of its registers back (setmaxnreg), which is what lets
// the 16 worker warps, four per scheduler, have 112 registers each: a 17th full-size warp
// would cap every thread at 96.
constexpr int THREADS = WORKERS + 128;
constexpr int ISSUE_WARP = WORKER_WARPS;
// Registers move between warpgroups inside the CTA's own allocation (640 threads x 96 at
// launch): 512 x 112 + 128 x 32 uses it up exactly.  Asking for more would block for ever.
constexpr int LAUNCH_REGS = 96, WORKER_REGS = 112, ISSUER_REGS = 32;
static_assert(WORKERS * WORKER_REGS + (THREADS - WORKERS) * ISSUER_REGS <= THREADS * LAUNCH_REGS,
              "setmaxnreg.inc can only take what setmaxnreg.dec gave back");
static_assert(THREADS * (LAUNCH_REGS + 8) > 65536, "LAUNCH_REGS is what the launch bound yields");
constexpr int KSTEPS = TILE / 16;      // P.V contraction steps per tile
constexpr int KBLOCK_BYTES = TILE * 128;              // [128 tok][64 bf16]
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t COL_S = 0, COL_O = 64, O_SLICE_COLS = 64;
constexpr float LOG2E = 1.4426950408889634f, LN2 = 0.6931471805599453f;
constexpr float RESCALE_THRESHOLD = 8.0f;             // log2 units
constexpr float NEG_HUGE = -3.0e38f;                  // "no reference maximum yet"
constexpr int WORKER_BARRIER = 1;                     // named barrier of the 512 workers

enum ErrCode { ERR_BLKFULL = 1, ERR_PFULL = 2, ERR_SFULL = 3, ERR_SLICEFREE = 4, ERR_ODONE = 5 };

template <int FMT, int DQK, int NH> struct Cfg {
  static_assert(NH == 16 || NH == 32 || NH == 64, "heads per CTA");
  static constexpr bool PAGED = FMT != DSV4_KV_BF16;
  static constexpr int NB = DQK / 64;                  // 64-wide blocks of the K tile
  static constexpr int NG = NB == 9 ? 5 : 4;           // refill groups: block pairs, then block 8
  static constexpr int NOPE_SEGS = PAGED ? (DQK - 64) / 64 : 0;   // 64-byte FP8 segments
  static constexpr bool P_ALIAS = (DQK == 576);        // P^T lives in the last block
  static constexpr int K_BYTES = NB * KBLOCK_BYTES;
  static constexpr int QBLOCK_BYTES = NH * 128;
  static constexpr int Q_BYTES = NB * QBLOCK_BYTES;
  static constexpr int P_ROW_BYTES = NH * 2;
  static constexpr int P_BYTES = P_ALIAS ? 0 : TILE * P_ROW_BYTES;
  static constexpr int CPW = NH / 4;                   // head columns per softmax thread
  static constexpr uint32_t P_SWIZZLE = NH == 64 ? SWZ_128B : NH == 32 ? SWZ_64B : SWZ_32B;
};

struct Ctrl {
  uint64_t blk_full[5];                // group g of the K tile is in shared memory
  uint64_t slice_free[4];              // P.V slice mb has retired (blocks 2mb, 2mb+1 are dead)
  uint64_t s_full, p_full, o_done;
  uint32_t tmem;
  int resc;
  int fail;
  int pad;
  alignas(16) float wred[4][MAX_HEADS];  // per-lane-group column partials (max, then sums)
  alignas(16) float mref[MAX_HEADS];     // reference max, log2-scaled units (read as float4)
  float alpha[MAX_HEADS];                // rescale factor / final output factor
  float aux[MAX_HEADS];                  // fourth weight table of the cluster merge
  float wmax[4][MAX_HEADS];              // per-lane-group column maxima of the raw scores (prefill)
  // Where the rows of the tiles being loaded live: one entry per tile row (row start or
  // null, scale bytes or null), written by one thread per row, read by the eight threads
  // that stage the row.  Two tiles, alternating.
  alignas(16) const uint8_t* rows[2][TILE][2];
};

template <int FMT, int DQK, int NH>
constexpr size_t smem_bytes() {
  using C = Cfg<FMT, DQK, NH>;
  return 1024 + C::K_BYTES + C::Q_BYTES + C::P_BYTES + sizeof(Ctrl);
}

template <int I, int N, class F>
__device__ __forceinline__ void static_for(F&& f) {
  if constexpr (I < N) {
    f(std::integral_constant<int, I>{});
    static_for<I + 1, N>(f);
  }
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
__device__ __forceinline__ void st_shared_v2(uint32_t addr, uint32_t a, uint32_t b) {
  asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(addr), "r"(a), "r"(b));
}

// 16 bytes of a KV row.  The rows are read once, so they are not kept in L1 (its array is
// the one the tensor core reads its operands from); L2 is asked for 256-byte granules, so that
// the neighbouring 128-byte line of the row, which another request of the same thread wants,
// comes along (measured against the other cache operators: 1-2 % per call; plain and .cg
// loads are 2-5 % slower).
__device__ __forceinline__ uint4 ldg16(const uint8_t* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.L2::256B.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

__device__ __forceinline__ uint32_t ldg_u32(const uint8_t* p) {
  uint32_t v;
  asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}

__device__ __forceinline__ uint32_t bf16x2_max(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("max.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&t);
}

// Column-wise maximum, over the 32 lanes of a warp, of N columns held one row per lane as
// N/2 packed BF16 pairs (column 2i in the low half of pk[i]).  Lane l returns the maximum
// of column l & (N - 1).  The array is used as scratch.
template <int N>
__device__ __forceinline__ float warp_col_max_packed(uint32_t (&pk)[N / 2], int lane) {
  constexpr int NP = N / 2;
#pragma unroll
  for (int d = 16; d >= 2 * NP; d >>= 1) {      // lanes further apart than the columns: plain max
#pragma unroll
    for (int i = 0; i < NP; ++i) pk[i] = bf16x2_max(pk[i], __shfl_xor_sync(0xffffffffu, pk[i], d));
  }
#pragma unroll
  for (int w = NP / 2; w >= 1; w >>= 1) {       // lanes 2w apart: halve the register set
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

// Column-wise sum, over the 32 lanes of a warp, of N columns held one row per lane:
// afterwards v[0] of lane l is the sum of column l & (N - 1).
template <int N>
__device__ __forceinline__ float warp_col_sum(float (&v)[N], int lane) {
#pragma unroll
  for (int d = 16; d >= N; d >>= 1) {
#pragma unroll
    for (int i = 0; i < N; ++i) v[i] += __shfl_xor_sync(0xffffffffu, v[i], d);
  }
#pragma unroll
  for (int w = N / 2; w >= 1; w >>= 1) {
    const bool up = (lane & w) != 0;
#pragma unroll
    for (int i = 0; i < w; ++i) {
      const float mine = up ? v[w + i] : v[i];
      const float other = up ? v[i] : v[w + i];
      v[i] = mine + __shfl_xor_sync(0xffffffffu, other, w);
    }
  }
  return v[0];
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
constexpr int PROF_TILE0 = 8, PROF_PER_TILE = 32, PROF_MAX_TILES = 30;
constexpr int PROF_CTA0 = 1024;
// Per-CTA wall-clock stamps (global timer, ns) at slots 1024 + 4 * cta + k; the buffer holds
// 1024 + 4 * CTAs values.
__device__ __forceinline__ void stamp_cta(const AttnParams& p, int k) {
#ifdef DSV4_TIMELINE
  if (p.prof != nullptr) {
    const int cta = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    p.prof[PROF_CTA0 + 4 * cta + k] = static_cast<long long>(t);
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
// Staging geometry.  A tile is 8 "k-steps" of 16 rows (the rows one P.V MMA step
// contracts over).  Worker warp w owns, in the k-steps j = (w >> 2) and 4 + (w >> 2),
// the four rows 4 * (w & 3) .. +4, i.e. a thread owns two rows 64 apart: lane l holds,
// for each 128-byte line c of a row, one 16-byte chunk of row (l & 1) + 2 (l >> 4).  The
// eight lanes that a 128-bit shared-memory store handles together thus belong to two
// rows whose swizzle patterns differ in the lowest bit, and the chunk a lane takes
// within a line is chosen (differently for converted and for copied lines) so that those
// eight lanes hit eight different 16-byte bank groups: no store is replayed.
//   paged layouts: a row is CH 16-byte chunks: FP8 chunks (16 values -> two BF16
//                  chunks of block chunk/4) then 8 RoPE chunks (copied to the last block);
//                  line c < 4 of the FP8 part is exactly the pair of blocks 2c, 2c+1;
//   flat BF16:     a row is d_qk/8 chunks copied as they are; line c is block c.
// ---------------------------------------------------------------------------
template <int FMT, int DQK> struct Stage {
  static constexpr bool PAGED = FMT != DSV4_KV_BF16;
  static constexpr int NOPE_SEGS = PAGED ? (DQK - 64) / 64 : 0;
  static constexpr int CH = PAGED ? NOPE_SEGS * 4 + 8 : DQK / 8;   // 16-byte chunks per row
  static constexpr int FP8_CH = PAGED ? NOPE_SEGS * 4 : 0;
  static constexpr int LINES = (CH + 7) / 8;
  static constexpr int REG_LINES = PAGED ? LINES : 1;              // BF16 rows are not staged
  // Line c holds no FP8 chunk (it is copied, not converted).
  __host__ __device__ static constexpr bool copied_line(int c) { return 8 * c >= FP8_CH; }
  // Lines of refill group g: [first, last].
  __host__ __device__ static constexpr int first_line(int g, int ng) {
    return PAGED ? g : 2 * g;
  }
  __host__ __device__ static constexpr int last_line(int g, int ng) {
    return PAGED ? (g == ng - 1 ? LINES - 1 : g) : (2 * g + 1 < LINES ? 2 * g + 1 : LINES - 1);
  }
  uint4 d[2][REG_LINES];
};

// Per-thread constants of the staging geometry.
struct Geo {
  int jsub;     // k-steps handled: jsub and 4 + jsub
  int rloc;     // row within a k-step: 4 * (w & 3) + (l & 1) + 2 * (l >> 4)
  int piece;    // 16-byte chunk within a converted (FP8) line; it is stored as two chunks
  int piece_cp; // 16-byte chunk within a line that is copied as it is
  __device__ __forceinline__ int row(int hh) const { return 16 * (4 * hh + jsub) + rloc; }
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
    scl = pbase + static_cast<int64_t>(c.pb) * T::ROW_BYTES + rr * T::SLOTS;
    return pbase + static_cast<int64_t>(rr) * T::ROW_BYTES;
  }
}

// The UE8M0 scale bytes of one row, as loaded (one or two 32-bit words).
template <int FMT> struct ScaleWords {
  static constexpr int N = FMT == DSV4_KV_MODEL1 ? 2 : 1;
  uint32_t w[N];
};
constexpr uint32_t NEUTRAL_SCALES = 0x7f7f7f7fu;       // 2^0 in every byte

// Scale words of a row from the address of its scale bytes (null: neutral scales).
template <int FMT>
__device__ __forceinline__ void load_scale_words(ScaleWords<FMT>& sw, const uint8_t* scl) {
#pragma unroll
  for (int k = 0; k < ScaleWords<FMT>::N; ++k) sw.w[k] = NEUTRAL_SCALES;
  if constexpr (FMT != DSV4_KV_BF16) {
    if (scl != nullptr) {
#pragma unroll
      for (int k = 0; k < ScaleWords<FMT>::N; ++k) sw.w[k] = ldg_u32(scl + 4 * k);
    }
  }
}

// Issue the load of this lane's chunk of line LINE of `row` (null: zeros).
template <int FMT, int DQK, int LINE>
__device__ __forceinline__ void load_line(uint4& d, const uint8_t* row, const Geo& geo) {
  using S = Stage<FMT, DQK>;
  const int piece = S::copied_line(LINE) ? geo.piece_cp : geo.piece;
  d = make_uint4(0, 0, 0, 0);
  if (row != nullptr && (8 * LINE + 7 < S::CH || 8 * LINE + piece < S::CH))
    d = ldg16(row + 16 * piece + 128 * LINE);
}

// Scale byte that applies to this lane's FP8 chunk of line LINE.
template <int FMT, int LINE>
__device__ __forceinline__ uint32_t scale_byte_of(const ScaleWords<FMT>& sw, int piece) {
  if constexpr (FMT == DSV4_KV_V32) {                 // one scale per 128 values = per line
    return (sw.w[0] >> ((8 * LINE) & 31)) & 0xffu;
  } else {                                            // one per 64 values = per half line
    return __byte_perm(sw.w[0], sw.w[1], 2 * LINE + (piece >> 2)) & 0xffu;
  }
}

// Convert and store line LINE of the staged row `v` (tile row `row`).
template <int FMT, int DQK, int LINE>
__device__ __forceinline__ void store_line(const uint4& v, uint32_t sK, int row, const Geo& geo,
                                           const ScaleWords<FMT>& sw, bool two) {
  using S = Stage<FMT, DQK>;
  constexpr int NB = DQK / 64;
  const int piece = S::copied_line(LINE) ? geo.piece_cp : geo.piece;
  const int x = row & 7;
  const uint32_t rbase = sK + row * 128;
  const int ci = 8 * LINE + piece;
  if constexpr (S::PAGED) {
    constexpr bool ALL_FP8 = 8 * LINE + 7 < S::FP8_CH, NO_FP8 = 8 * LINE >= S::FP8_CH;
    if (ALL_FP8 || (!NO_FP8 && ci < S::FP8_CH)) {
      const ScalePair c = scale_pair(scale_byte_of<FMT, LINE>(sw, piece));
      const uint32_t a = rbase + (ci >> 2) * KBLOCK_BYTES + (((2 * (ci & 3)) ^ x) << 4);
      uint32_t o[8];
      dequant4(v.x, c, false, o[0], o[1]);
      dequant4(v.y, c, false, o[2], o[3]);
      dequant4(v.z, c, false, o[4], o[5]);
      dequant4(v.w, c, false, o[6], o[7]);
      if (two) {                               // warp-uniform, and next to never taken
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = bf16x2_mul(o[i], c.c2);
      }
      st_shared_v4(a, o[0], o[1], o[2], o[3]);
      st_shared_v4(a ^ 16, o[4], o[5], o[6], o[7]);             // the neighbouring chunk
    } else if (ci < S::CH) {
      const uint32_t a = rbase + (NB - 1) * KBLOCK_BYTES;
      st_shared_v4(a + (((ci - S::FP8_CH) ^ x) << 4), v.x, v.y, v.z, v.w);
    }
  } else {
    (void)sw;
    const uint32_t a = rbase + LINE * KBLOCK_BYTES;             // line == 64-column block
    st_shared_v4(a + ((piece ^ x) << 4), v.x, v.y, v.z, v.w);
  }
}

// ---------------------------------------------------------------------------
// Merging the splits of one request inside a thread-block cluster.
// The `cs` CTAs of a cluster (consecutive splits, cluster dimension z) finish with
// un-normalised O^T in TMEM, denominators l[h] and reference maxima m[h].  CTA r owns
// slice r of the output (d in [r, r+1) * 512 / cs).  Each CTA
//   1. meets the others at a cluster barrier (it arrives as soon as its own last product has
//      retired and waits only here, after its local reductions): from here on every CTA's K
//      tile region and small tables may be written by its peers;
//   2. PUSHES: its (l, m) into every CTA's tables, and each 128-row slice of its O^T,
//      straight from TMEM, into the staging area of the CTA that owns those d
//      ([source][head][d] fp32 in the K tile region; st.shared::cluster, which does not
//      wait for an answer the way a remote load does);
//   3. meets the others again (release / acquire: the pushes are visible);
//   4. derives, per head, the weights 2^(m_s - M) / L of all sources (times the sink
//      factor when this cluster holds all splits of the request) from its own tables;
//   5. sums its slice over the sources, in rank order, out of its own shared memory and
//      writes either the final BF16 output or one normalised fp32 partial per cluster.
// After step 3 no CTA touches another's memory, so none has to outlive the others.
// Partial traffic to L2 and the combine kernel's input shrink by the cluster size, and
// with n_splits == cs there is no combine launch at all.  An empty split (no tile) takes
// part with l = 0, m = "none" (weight 0) and stages zeros; a CTA
// whose bounded wait gave up still walks every barrier (its peers must not be left
// waiting) and only drops its own stores.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_arrive() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  cluster_arrive();
  cluster_wait();
}
__device__ __forceinline__ uint32_t map_to_rank(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void st_cluster_b32(uint32_t addr, uint32_t v) {
  asm volatile("st.shared::cluster.b32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
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
  long long* prof;         // debug timeline buffer or null
};
__device__ __forceinline__ MergeOut merge_out_of(const AttnParams& p) {
  return MergeOut{p.cluster, p.n_splits, p.mode, p.sink, p.lse, p.lse_accum, p.o_accum, p.out,
                  p.stride_o_b, p.stride_o_s, p.stride_o_h, p.stride_lse_b, p.stride_lse_s,
                  p.stride_lse_h, p.prof};
}
constexpr int PROF_MERGE0 = 990;       // five stamps of the cluster merge (CTA (0,0,0), thread 0)
__device__ __forceinline__ void stamp_merge(const MergeOut& p, int k) {
#ifdef DSV4_TIMELINE
  if (p.prof != nullptr && threadIdx.x == 0 && (blockIdx.x | blockIdx.y | blockIdx.z) == 0)
    p.prof[PROF_MERGE0 + k] = clock64();
#else
  (void)p;
  (void)k;
#endif
}
struct MergeCtx {
  uint32_t stage;          // shared address of the staging area (the K tile region)
  uint32_t tmem_o;         // TMEM address of this warp's lanes of O^T (column COL_O), or unused
  int heads_here, head0, bi, si;
  int64_t acc_slot0;       // (cluster index * n_req + req) * h_q + head0
  bool empty;              // this split had no tile: no TMEM, contributes zeros
};

// Step 5 of the merge for a cluster of CS CTAs: an item is 8 consecutive d of one head
// (two 16-byte loads per source, one 16-byte store of BF16); staging area
// [source][NH heads][512 / CS] fp32 in this CTA's own memory.  Kept lean: the epilogue is
// bound by instruction issue (16 warps, every instruction counts 512 times).
template <int NH, int CS>
__device__ __forceinline__ void sum_slices(const MergeOut& p, const MergeCtx& c, const float* wtab,
                                           uint32_t rank, bool final_out) {
  constexpr int DL = D_V / CS, OCTS = DL / 8;
  const int tid = threadIdx.x;
  const int n_items = c.heads_here * OCTS;
  __nv_bfloat16* out_base = p.out + c.bi * p.stride_o_b + c.si * p.stride_o_s + c.head0 * p.stride_o_h;
#pragma unroll 2
  for (int item = tid < WORKERS ? tid : n_items; item < n_items; item += WORKERS) {
    const int h = item / OCTS, o = item - h * OCTS;
    float acc[8];
#pragma unroll
    for (int r = 0; r < CS; ++r) {                       // rank order: reproducible sums
      const uint32_t a = c.stage + ((r * NH + h) * DL + 8 * o) * 4;
      float v[8];
      asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                   : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]) : "r"(a));
      asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                   : "=f"(v[4]), "=f"(v[5]), "=f"(v[6]), "=f"(v[7]) : "r"(a + 16));
      const float w = wtab[r * MAX_HEADS + h];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = r == 0 ? w * v[i] : fmaf(w, v[i], acc[i]);
    }
    const int d0 = rank * DL + 8 * o;
    if (final_out) {
      uint32_t w4[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        __nv_bfloat162 t = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
        w4[i] = *reinterpret_cast<uint32_t*>(&t);
      }
      *reinterpret_cast<uint4*>(out_base + h * p.stride_o_h + d0) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
    } else {
      float4* dst = reinterpret_cast<float4*>(p.o_accum + (c.acc_slot0 + h) * D_V + d0);
      dst[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
      dst[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
    }
  }
}

// `m_own` is in log2-scaled units, NEG_HUGE or -inf when the split saw nothing.  Called by
// the 512 workers (the MMA warpgroup mirrors the barriers), or by the whole CTA when the
// split is empty.
template <int NH>
__device__ __noinline__ void cluster_merge(const MergeOut p, Ctrl& ctrl, const MergeCtx c,
                                           float l_own, float m_own) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int cs = p.cluster;                              // 2 or 4
  const int dl = D_V / cs;
  const uint32_t rank = cluster_rank();
  const bool final_out = p.n_splits == cs;

  cluster_wait();                                        // (1): the caller has arrived already
  stamp_merge(p, 0);

  // (2) tables: wred[source] = l, wmax[source] = m (both idle by now, in every CTA)
  if (tid < MAX_HEADS) {
    const uint32_t a_l = smem_u32(&ctrl.wred[rank][tid]), a_m = smem_u32(&ctrl.wmax[rank][tid]);
    const float mv = (m_own <= NEG_HUGE) ? -INFINITY : m_own;
    for (int r = 0; r < cs; ++r) {
      st_cluster_b32(map_to_rank(a_l, r), __float_as_uint(l_own));
      st_cluster_b32(map_to_rank(a_m, r), __float_as_uint(mv));
    }
  }
  // O^T: thread = one d (TMEM lane), 16 heads per load; a warp's 32 d go to one owner,
  // 128 contiguous bytes per store.  An empty split stages zeros (its weight is zero, and
  // zero times whatever the memory held before need not be zero).
  if (tid < WORKERS) {
    const int m = warp >> 2, lg = warp & 3;
    const int d = m * 128 + lg * 32 + lane;
    const uint32_t owner = static_cast<uint32_t>(d / dl);
    const uint32_t local = c.stage + ((rank * NH) * dl + (d - owner * dl)) * 4;
    const uint32_t dst = owner == rank ? local : map_to_rank(local, owner);
#pragma unroll 1
    for (int c4 = 0; c4 < NH / 16; ++c4) {
      uint32_t o[16];
      if (!c.empty) {
        tmem_ld16(c.tmem_o + m * O_SLICE_COLS + c4 * 16, o);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) o[i] = 0u;
      }
      if (owner == rank) {
#pragma unroll
        for (int i = 0; i < 16; ++i)
          asm volatile("st.shared.b32 [%0], %1;" ::"r"(dst + (c4 * 16 + i) * dl * 4), "r"(o[i]) : "memory");
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) st_cluster_b32(dst + (c4 * 16 + i) * dl * 4, o[i]);
      }
    }
  }
  stamp_merge(p, 1);
  cluster_sync_all();                                    // (3)
  stamp_merge(p, 2);

  // (4) weights of all sources for head tid; the table (4 sources x 64 heads) lives in the
  // row table of the tile loop, which is idle by now
  float* wtab = reinterpret_cast<float*>(&ctrl.rows[0][0][0]);
  if (tid < MAX_HEADS) {
    float ms[4], ls[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      ms[r] = r < cs ? ctrl.wmax[r][tid] : -INFINITY;
      ls[r] = r < cs ? ctrl.wred[r][tid] : 0.f;
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
    for (int r = 0; r < 4; ++r) wtab[r * MAX_HEADS + tid] = w[r] * f;
  }
  __syncthreads();
  stamp_merge(p, 3);

  // (5) this rank's slice, summed over the sources
  if (!ctrl.fail) {
    if (cs == 2) sum_slices<NH, 2>(p, c, wtab, rank, final_out);
    else sum_slices<NH, 4>(p, c, wtab, rank, final_out);
  }
  stamp_merge(p, 4);
  // A CTA whose wait gave up makes the request's result visibly invalid.
  if (ctrl.fail && tid < c.heads_here) {
    if (final_out) p.lse[c.bi * p.stride_lse_b + c.si * p.stride_lse_s + (c.head0 + tid) * p.stride_lse_h] = NAN;
    else p.lse_accum[c.acc_slot0 + tid] = NAN;
  }
}

// ---------------------------------------------------------------------------
// Raising the softmax references (all 512 workers; the first tile, and any tile in which
// some score exceeds its head's reference by more than the threshold).  Column maxima of
// S^T over the tile's rows (BF16-rounded: the reference only has to be the same for every
// thread, not exact), a new reference where the maximum has grown by more than the
// threshold (also the first finite one), and O^T in TMEM scaled down to it; the factors
// stay in ctrl.alpha (ctrl.resc says whether any differs from one) for the caller's
// denominators.  Out of line on purpose: it is rare, and the tile loop must stay small.
// `tmem_lanes` is the TMEM base address with this warp's lane offset applied.
// ---------------------------------------------------------------------------
template <int NH>
__device__ __noinline__ void raise_references(Ctrl& ctrl, uint32_t tmem_lanes, bool masked, float cs,
                                              bool rescale_o) {
  constexpr int CPW = NH / 4;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int lg = warp & 3, cg = warp >> 2;
  {
    uint32_t s[CPW];
    tmem_ld_cols<CPW>(tmem_lanes + COL_S + cg * CPW, s);
    tmem_ld_wait();
    uint32_t pk[CPW / 2];
#pragma unroll
    for (int i = 0; i < CPW / 2; ++i) {
      const float a = masked ? -INFINITY : __uint_as_float(s[2 * i]);
      const float b = masked ? -INFINITY : __uint_as_float(s[2 * i + 1]);
      pk[i] = pack_bf16x2(a, b);
    }
    const float cm = warp_col_max_packed<CPW>(pk, lane);
    if (lane < CPW) ctrl.wred[lg][cg * CPW + lane] = cm;
  }
  if (tid == 0) ctrl.resc = 0;
  bar_sync(WORKER_BARRIER, WORKERS);
  if (tid < NH) {
    const float tm = fmaxf(fmaxf(ctrl.wred[0][tid], ctrl.wred[1][tid]),
                           fmaxf(ctrl.wred[2][tid], ctrl.wred[3][tid])) * cs;
    const float mr = ctrl.mref[tid];
    float alpha = 1.f;
    if (tm > mr + RESCALE_THRESHOLD) {
      alpha = (mr <= NEG_HUGE) ? 0.f : ex2(mr - tm);
      ctrl.mref[tid] = tm;
      ctrl.resc = 1;
    }
    ctrl.alpha[tid] = alpha;
  }
  bar_sync(WORKER_BARRIER, WORKERS);
  if (ctrl.resc && rescale_o) {
    // this warp rescales slice cg of O^T for its 32 TMEM lanes
#pragma unroll 1
    for (int c4 = 0; c4 < NH / 16; ++c4) {
      uint32_t o[16];
      const uint32_t addr = tmem_lanes + COL_O + cg * O_SLICE_COLS + c4 * 16;
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

// ---------------------------------------------------------------------------
// The kernel
// ---------------------------------------------------------------------------
template <int FMT, int DQK, int NH, bool EXTRA>
__global__ void __launch_bounds__(THREADS, 1)
sm100_attn_kernel(const AttnParams p) {
  using C = Cfg<FMT, DQK, NH>;
  using S = Stage<FMT, DQK>;
  constexpr int CPW = C::CPW;
  constexpr int NG = C::NG;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - raw);
  const uint32_t sK = base, sQ = base + C::K_BYTES;
  const uint32_t sP = C::P_ALIAS ? sK + (C::NB - 1) * KBLOCK_BYTES : sQ + C::Q_BYTES;
  Ctrl& ctrl = *reinterpret_cast<Ctrl*>(sm + C::K_BYTES + C::Q_BYTES + C::P_BYTES);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool worker = warp < WORKER_WARPS;
  grid_dependency_wait();          // inputs may come from the kernel before this one in the stream
  if (tid == 0) stamp(p, 0);
  if (tid == 0) stamp_cta(p, 0);
  const bool decode = p.mode == MODE_DECODE;
  // Prefill walks its query rows last to first: with causal lists the late rows are the
  // long ones, and the grid should end on short rows, not on a wave of the longest.
  const int req = decode ? blockIdx.x : gridDim.x - 1 - blockIdx.x;
  const int hb = blockIdx.y, split = blockIdx.z;
  const int head0 = hb * NH;
  const int heads_here = min(NH, p.h_q - head0);
  const int bi = req / p.s_q, si = req % p.s_q;
  const bool mask_invalid = !decode || (p.flags & DSV4_FLAG_MASK_INVALID);
  const bool split_out = p.n_splits > 1;
  const bool want_ml = p.max_logits != nullptr;

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
    cluster_arrive();
    __syncthreads();
    MergeCtx mc{sK, 0u, heads_here, head0, bi, si, acc_slot0, true};
    cluster_merge<NH>(merge_out_of(p), ctrl, mc, 0.f, -INFINITY);
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

  const uint32_t bar_blk_full0 = smem_u32(&ctrl.blk_full[0]), bar_slice_free0 = smem_u32(&ctrl.slice_free[0]);
  const uint32_t bar_s_full = smem_u32(&ctrl.s_full), bar_p_full = smem_u32(&ctrl.p_full);
  const uint32_t bar_o_done = smem_u32(&ctrl.o_done);
  bool ok = true;      // false once one of this thread's bounded waits has given up
#define TSTAMP(t, k) do { if ((t) < PROF_MAX_TILES) stamp(p, PROF_TILE0 + (t) * PROF_PER_TILE + (k)); } while (0)

  if (!worker) {
    // ======================= the fifth warpgroup: MMA issue ===============================
    // It keeps 32 registers per thread and runs no code in common with the workers from here
    // on: only the CTA-wide (and cluster-wide) barriers, which it meets in the same order.
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(ISSUER_REGS));
    // Its part of the set-up, off the workers' critical path: the barriers and TMEM (the warp
    // next to the issuing one allocates and, at the end, frees it).
    if (tid == WORKERS) {
      // a group is published by the 16 worker warps, or (flat BF16 rows) by the completion of
      // every worker thread's asynchronous copies
      for (int i = 0; i < 5; ++i) mbar_init(bar_blk_full0 + 8 * i, C::PAGED ? WORKER_WARPS : WORKERS);
      for (int i = 0; i < 4; ++i) mbar_init(bar_slice_free0 + 8 * i, 1);
      mbar_init(bar_s_full, 1);
      mbar_init(bar_p_full, WORKER_WARPS);
      mbar_init(bar_o_done, 1);
      ctrl.resc = 0;
      ctrl.fail = 0;
      mbar_init_fence();
    }
    if (warp == ISSUE_WARP + 1) {
      tmem_alloc(smem_u32(&ctrl.tmem), TMEM_COLS);
      tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();                 // set-up done: barriers initialised, TMEM allocated, Q stored
    tc_fence_after_sync();
    if (warp == ISSUE_WARP) {
      // Run by the whole warp, converged; one elected lane issues the MMAs and the commits
      // (see umma_bf16_elect).
      const uint32_t tmem_u = ctrl.tmem;
      const uint32_t idesc_qk = make_idesc_bf16(TILE, NH, 0, 0);
      const uint32_t idesc_pv = make_idesc_bf16(128, NH, 1, 1);
      const uint64_t dK = make_smem_desc(sK, 16, 1024, SWZ_128B);            // K-major view
      const uint64_t dQ = make_smem_desc(sQ, 16, 1024, SWZ_128B);
      const uint64_t dV = make_smem_desc(sK, KBLOCK_BYTES, 1024, SWZ_128B);  // MN-major view
      const uint64_t dP = make_smem_desc(sP, 8 * C::P_ROW_BYTES, 8 * C::P_ROW_BYTES, C::P_SWIZZLE);
      const uint32_t elected = elect_one();
#pragma unroll 1
      for (int t = 0; t < n_tiles; ++t) {
        // Q.K^T of tile t, group by group as the blocks arrive.  The issue loops are fully
        // unrolled on purpose: issuing is what bounds the tensor pipe at N <= 64 (about 50 clk
        // per MMA unrolled, 75 rolled, against 30 clk of execution).
        static_for<0, NG>([&](auto gc) {
          constexpr int g = decltype(gc)::value;
          if (ok && !mbar_wait_warp(bar_blk_full0 + 8 * g, t & 1, lane)) {
            atomicExch(&g_attn_error, ERR_BLKFULL);
            ok = false;
          }
          tc_fence_after_sync();
          if (lane == 0 && g == 0) TSTAMP(t, 1);
#pragma unroll
          for (int kb = 2 * g; kb < 2 * g + 2 && kb < C::NB; ++kb) {
#pragma unroll
            for (int k4 = 0; k4 < 4; ++k4)
              umma_bf16_elect(tmem_u + COL_S, dK + static_cast<uint64_t>((kb * KBLOCK_BYTES + k4 * 32) >> 4),
                              dQ + static_cast<uint64_t>((kb * C::QBLOCK_BYTES + k4 * 32) >> 4), idesc_qk,
                              (kb | k4) != 0, elected);
          }
        });
        umma_commit_elect(bar_s_full, elected);
        if (lane == 0) TSTAMP(t, 2);
#ifdef DSV4_TIMELINE
        if (lane == 0) {                 // when does the commit really arrive? (pure spin)
          for (int i = 0; i < (1 << 20) && !mbar_test(bar_s_full, t & 1); ++i) {}
          TSTAMP(t, 18);
        }
        __syncwarp();
#endif
        // P.V of tile t, one 128-row slice of O^T after the other
        if (ok && !mbar_wait_warp(bar_p_full, t & 1, lane)) {
          atomicExch(&g_attn_error, ERR_PFULL);
          ok = false;
        }
        tc_fence_after_sync();
        if (lane == 0) TSTAMP(t, 5);
#pragma unroll 1
        for (int mb = 0; mb < 4; ++mb) {
#pragma unroll
          for (int j = 0; j < KSTEPS; ++j)
            umma_bf16_elect(tmem_u + COL_O + mb * O_SLICE_COLS,
                            dV + static_cast<uint64_t>((j * 2048 + mb * 2 * KBLOCK_BYTES) >> 4),
                            dP + static_cast<uint64_t>((j * 16 * C::P_ROW_BYTES) >> 4), idesc_pv,
                            (t | j) != 0, elected);
          umma_commit_elect(bar_slice_free0 + 8 * mb, elected);
        }
        if (t + 1 == n_tiles) umma_commit_elect(bar_o_done, elected);
        if (lane == 0) TSTAMP(t, 6);
#ifdef DSV4_TIMELINE
        if (lane == 0) {
          for (int mb = 0; mb < 4; ++mb) {
            for (int i = 0; i < (1 << 20) && !mbar_test(bar_slice_free0 + 8 * mb, t & 1); ++i) {}
            TSTAMP(t, 19 + mb);
          }
        }
        __syncwarp();
#endif
      }
      if (!ok) ctrl.fail = 1;
    }
    grid_launch_dependents();
    // the same CTA-wide and cluster-wide barriers as the workers' epilogue, in the same order
    __syncthreads();
    if (p.cluster > 1) {
      cluster_sync_all();
      cluster_sync_all();
      __syncthreads();
    } else {
      __syncthreads();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    if (warp == ISSUE_WARP + 1) tmem_dealloc(ctrl.tmem, TMEM_COLS);
    return;
  }

  // ======================= the worker warps ===============================================
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(WORKER_REGS));

  // ---- set-up ---------------------------------------------------------------------------
  // Order matters for latency: the list entries are requested first, then, as they arrive,
  // the first tile's rows and their scale bytes (DRAM: what the first product waits for),
  // then Q; Q is written to shared memory while the rows are in flight.
  S stage;
  const Geo geo{warp >> 2, 4 * (warp & 3) + (lane & 1) + 2 * (lane >> 4),
                ((lane >> 1) & 3) + 4 * ((lane >> 3) & 1), 2 * ((lane >> 1) & 3) + ((lane >> 3) & 1)};
  // Softmax geometry: TMEM lanes 32*lg.. (tile rows), head columns CPW*cg .. +CPW.
  const int lg = warp & 3, cg = warp >> 2;
  const int row = lg * 32 + lane;

  // Rows are requested from memory LOAD_AHEAD tiles before they are stored: FP8 rows a whole
  // tile ahead (register staging), BF16 rows when their blocks are free (cp.async).  Where
  // the rows of a tile live is worked out once per row, by thread `tid` < 128 for tile row
  // `tid`, and handed to the staging threads through ctrl.rows; the list entry it starts
  // from is fetched an iteration earlier (e_pref).
  constexpr int LOAD_AHEAD = S::PAGED ? 2 : 1;
  auto write_rows = [&](int tile, int entry) {           // threads 0..127
    const uint8_t* scl;
    const int j = lv.begin + tile * TILE + tid;
    const uint8_t* r = row_ptr<FMT>(cache_of<EXTRA>(p, lv, j), entry, scl);
    *reinterpret_cast<ulonglong2*>(&ctrl.rows[tile & 1][tid][0]) =
        make_ulonglong2(reinterpret_cast<unsigned long long>(r), reinterpret_cast<unsigned long long>(scl));
  };
  // (a) The list entries go first: the tile-0 rows of this thread, the row-table entry of
  // the first tile the loop requests and of the one after, the row that decides masking.
  // Everything below that does not need them is issued behind their latency.
  int e0[2] = {-1, -1};
  if constexpr (S::PAGED) {
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) e0[hh] = list_index<EXTRA>(lv, lv.begin + geo.row(hh));
  }
  constexpr int FIRST_TABLE_TILE = LOAD_AHEAD - 1;       // the tile the first fill requests
  int e_first = -1, e_pref = -1;
  if (tid < TILE) {
    if (FIRST_TABLE_TILE < n_tiles) e_first = list_index<EXTRA>(lv, lv.begin + FIRST_TABLE_TILE * TILE + tid);
    if (FIRST_TABLE_TILE + 1 < n_tiles)
      e_pref = list_index<EXTRA>(lv, lv.begin + (FIRST_TABLE_TILE + 1) * TILE + tid);
  }
  // this thread's own tile row: its list entry decides masking when invalid entries are masked
  int ridx = 0, ridx_next = 0;
  if (mask_invalid) ridx = list_index<EXTRA>(lv, lv.begin + row);
  if (tid == 0) stamp(p, 971);

  // (b) First use of the list entries: the first tile's rows and scale bytes go in flight,
  // ahead of Q: they come from DRAM and are what the first product waits for, and the SM
  // keeps only so many loads in flight.
  ScaleWords<FMT> sw_cur[2], sw_ld[2];
  const uint8_t* row_ld[2] = {nullptr, nullptr};
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    sw_cur[hh].w[0] = sw_ld[hh].w[0] = NEUTRAL_SCALES;
    if constexpr (ScaleWords<FMT>::N == 2) sw_cur[hh].w[1] = sw_ld[hh].w[1] = NEUTRAL_SCALES;
  }
  if constexpr (S::PAGED) {
    // tile 0 is requested at once, by the staging threads themselves
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      const int j = lv.begin + geo.row(hh);
      const uint8_t* scl;
      const uint8_t* r0 = row_ptr<FMT>(cache_of<EXTRA>(p, lv, j), e0[hh], scl);
      load_scale_words<FMT>(sw_cur[hh], scl);
      static_for<0, S::LINES>([&](auto lc) {
        load_line<FMT, DQK, decltype(lc)::value>(stage.d[hh][decltype(lc)::value], r0, geo);
      });
    }
  }
  if (tid == 0) stamp(p, 972);

  // (c) Q[head][d] -> blocks [d/64][head][64], 128-byte swizzle; absent heads are zero.
  const __nv_bfloat16* qrow0 = p.q + bi * p.stride_q_b + si * p.stride_q_s + head0 * p.stride_q_h;
  constexpr int Q_CHUNKS = NH * C::NB * 8;
  constexpr int Q_BATCH = (Q_CHUNKS + WORKERS - 1) / WORKERS;     // all in flight at once
  uint4 qv[Q_BATCH];
#pragma unroll
  for (int it = 0; it < Q_BATCH; ++it) {
    const int i = tid + it * WORKERS;
    const int h = i / (C::NB * 8), cc = i % (C::NB * 8);
    qv[it] = make_uint4(0, 0, 0, 0);
    if (i < Q_CHUNKS && h < heads_here)
      qv[it] = ldg16(reinterpret_cast<const uint8_t*>(qrow0 + h * p.stride_q_h) + 16 * cc);
  }
  if (tid == 0) stamp(p, 974);

  // (d) the row table of the first tile the loop requests; the softmax references
  if (tid < TILE && FIRST_TABLE_TILE < n_tiles) write_rows(FIRST_TABLE_TILE, e_first);
  if (tid < MAX_HEADS) {
    ctrl.mref[tid] = NEG_HUGE;
    ctrl.alpha[tid] = 1.f;
  }
  // (e) Q into shared memory (the barriers and the TMEM allocation are the fifth
  // warpgroup's part of the set-up)
#pragma unroll
  for (int it = 0; it < Q_BATCH; ++it) {
    const int i = tid + it * WORKERS;
    const int h = i / (C::NB * 8), cc = i % (C::NB * 8), kb = cc >> 3, ch = cc & 7;
    if (i < Q_CHUNKS)
      st_shared_v4(sQ + kb * C::QBLOCK_BYTES + h * 128 + ((ch ^ (h & 7)) << 4), qv[it].x, qv[it].y,
                   qv[it].z, qv[it].w);
  }
  if (tid == 0) stamp(p, 975);
  fence_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = ctrl.tmem;
  if (tid == 0) stamp(p, 1);
  if (tid == 0) stamp_cta(p, 1);

  {
    // ======================= the worker warps =============================================
    // Fill of the K tile with tile `st_tile` (st_tile = t + 1 behind the P.V product of tile
    // t, or 0 at the start), group by group.  `wait_tile` >= 0: group g may be overwritten
    // only once P.V slice min(g, 3) of that tile has retired (block 8 carries P^T, which
    // every slice reads).  After a wait has given up (`ok` false) no further wait is
    // attempted, but every thread keeps walking the same path so that the barriers stay
    // matched; the outputs are then suppressed.
    // Paged: the rows are in registers; each line is reloaded with the same line of tile
    // `ld_tile` as soon as it has been stored.  BF16: the rows of tile ld_tile == st_tile
    // are copied with cp.async, and group g publishes itself: each thread's arrival on the
    // group's barrier is tied to the completion of its copies, so no thread waits for them.
    auto publish = [&](int g) {              // this warp's part of group g is in shared memory
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_blk_full0 + 8 * g);
    };
    auto fill = [&](int wait_tile, bool load_next) {
      // Does any row this warp converts in this tile carry a scale byte beyond the reach of
      // one multiply?  (Warp-uniform, so the second multiply is a branch, not a predicate.)
      bool two = false;
      if constexpr (S::PAGED) {
        bool mine = false;
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
#pragma unroll
          for (int k = 0; k < ScaleWords<FMT>::N; ++k) mine |= needs_second_multiply(sw_cur[hh].w[k]);
        }
        two = __any_sync(0xffffffffu, mine);
      }
      static_for<0, NG>([&](auto gc) {
        constexpr int g = decltype(gc)::value;
        constexpr int FREED_BY = g < 3 ? g : 3;
        constexpr int L0 = S::first_line(g, NG), L1 = S::last_line(g, NG);
        if (wait_tile >= 0 && ok && !mbar_wait(bar_slice_free0 + 8 * FREED_BY, wait_tile & 1)) {
          atomicExch(&g_attn_error, ERR_SLICEFREE);
          ok = false;
        }
        if (tid == 0) TSTAMP(wait_tile + 1, 8 + 2 * g);
        if constexpr (S::PAGED) {
          static_for<L0, L1 + 1>([&](auto lc) {
            constexpr int line = decltype(lc)::value;
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
              store_line<FMT, DQK, line>(stage.d[hh][line], sK, geo.row(hh), geo, sw_cur[hh], two);
            }
          });
          // the requests for the same lines of the tile after next go out before the proxy
          // fence: issuing them takes as long as the stores above need to drain
          if (load_next) {
            static_for<L0, L1 + 1>([&](auto lc) {
              constexpr int line = decltype(lc)::value;
#pragma unroll
              for (int hh = 0; hh < 2; ++hh) load_line<FMT, DQK, line>(stage.d[hh][line], row_ld[hh], geo);
            });
          }
          publish(g);
          if (tid == 0) TSTAMP(wait_tile + 1, 9 + 2 * g);
        } else {
          static_for<L0, L1 + 1>([&](auto lc) {
            constexpr int line = decltype(lc)::value;
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
              const int r = geo.row(hh);
              const uint32_t dst = sK + line * KBLOCK_BYTES + r * 128 + ((geo.piece_cp ^ (r & 7)) << 4);
              const uint8_t* src = row_ld[hh] != nullptr ? row_ld[hh] + 128 * line + 16 * geo.piece_cp
                                                         : p.kv;
              cp_async16(dst, src, row_ld[hh] != nullptr ? 16u : 0u);
            }
          });
          // every worker thread arrives on the group's barrier when its own copies land
          cp_async_mbar_arrive(bar_blk_full0 + 8 * g);
        }
      });
    };
    // Where the rows of tile `ld_tile` live (ctrl.rows, written before the barrier this
    // thread last passed), and their scale bytes on the way.
    auto advance_loads = [&](int ld_tile) {
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        row_ld[hh] = nullptr;
        const uint8_t* scl = nullptr;
        if (ld_tile < n_tiles) {
          const ulonglong2 e = *reinterpret_cast<const ulonglong2*>(&ctrl.rows[ld_tile & 1][geo.row(hh)][0]);
          row_ld[hh] = reinterpret_cast<const uint8_t*>(e.x);
          scl = reinterpret_cast<const uint8_t*>(e.y);
        }
        load_scale_words<FMT>(sw_ld[hh], scl);
      }
    };

    const uint32_t tlane = static_cast<uint32_t>(lg * 32) << 16;
    const float cs = p.sm_scale * LOG2E;
    float lsum[CPW];
#pragma unroll
    for (int i = 0; i < CPW; ++i) lsum[i] = 0.f;
    uint32_t mlpk[CPW / 2];              // running maxima of the raw scores, packed BF16 (prefill)
#pragma unroll
    for (int i = 0; i < CPW / 2; ++i) mlpk[i] = 0xff80ff80u;     // -inf, -inf

    // Iteration t = -1 only fills tile 0; iteration t >= 0 runs the softmax of tile t and,
    // behind its P.V product, fills tile t + 1.
#pragma unroll 1
    for (int t = -1; t < n_tiles; ++t) {
      const bool more = t + 1 < n_tiles;
      const int ld_tile = t + LOAD_AHEAD;          // tile whose rows are requested in this iteration
      if (t >= 0) {
        // rows of the tile this iteration's fill requests (published by the barrier below)
        if (tid < TILE) {
          if (ld_tile < n_tiles) write_rows(ld_tile, e_pref);
          if (ld_tile + 1 < n_tiles) e_pref = list_index<EXTRA>(lv, lv.begin + (ld_tile + 1) * TILE + tid);
        }
        if (mask_invalid && more) ridx_next = list_index<EXTRA>(lv, lv.begin + (t + 1) * TILE + row);
        // Is this thread's row masked (beyond the range, or an invalid entry under masking rules)?
        bool masked = true;
        {
          const int j = lv.begin + t * TILE + row;
          if (j < lv.end) {
            const int ntok = (EXTRA && j >= lv.len) ? p.extra_n_tok : p.n_tok;
            masked = mask_invalid && static_cast<unsigned>(ridx) >= static_cast<unsigned>(ntok);
          }
        }
        const bool any_masked = __any_sync(0xffffffffu, masked);
        if (tid == 0) TSTAMP(t, 23);

        if (ok && !mbar_wait(bar_s_full, t & 1)) { atomicExch(&g_attn_error, ERR_SFULL); ok = false; }
        tc_fence_after_sync();
        if (tid == 0) TSTAMP(t, 3);

        float y[CPW];
        auto load_scores = [&](bool track_max) {
          uint32_t s[CPW];
          tmem_ld_cols<CPW>(tmem + tlane + COL_S + cg * CPW, s);     // warp-collective
          tmem_ld_wait();
          if (any_masked) {                       // rare: ragged tile or masked entries
            const uint32_t ninf = __float_as_uint(-INFINITY);
#pragma unroll
            for (int i = 0; i < CPW; ++i) s[i] = masked ? ninf : s[i];
          }
          if (track_max && want_ml) {
#pragma unroll
            for (int i = 0; i < CPW / 2; ++i)
              mlpk[i] = bf16x2_max(mlpk[i], pack_bf16x2(__uint_as_float(s[2 * i]), __uint_as_float(s[2 * i + 1])));
          }
          float ymax = -INFINITY;
#pragma unroll
          for (int q4 = 0; q4 < CPW / 4; ++q4) {
            const float4 mu = *reinterpret_cast<const float4*>(&ctrl.mref[cg * CPW + q4 * 4]);
            y[q4 * 4 + 0] = fmaf(__uint_as_float(s[q4 * 4 + 0]), cs, -mu.x);
            y[q4 * 4 + 1] = fmaf(__uint_as_float(s[q4 * 4 + 1]), cs, -mu.y);
            y[q4 * 4 + 2] = fmaf(__uint_as_float(s[q4 * 4 + 2]), cs, -mu.z);
            y[q4 * 4 + 3] = fmaf(__uint_as_float(s[q4 * 4 + 3]), cs, -mu.w);
            ymax = fmaxf(fmaxf(ymax, fmaxf(y[q4 * 4 + 0], y[q4 * 4 + 1])), fmaxf(y[q4 * 4 + 2], y[q4 * 4 + 3]));
          }
          return ymax;
        };
        const float ymax = load_scores(true);
        // Does any score of the tile exceed its reference by more than the threshold?
        if (bar_red_or(WORKER_BARRIER, WORKERS, ymax > RESCALE_THRESHOLD)) {
          raise_references<NH>(ctrl, tmem + tlane, masked, cs, t > 0);
          if (ctrl.resc) {
#pragma unroll
            for (int i = 0; i < CPW; ++i) lsum[i] *= ctrl.alpha[cg * CPW + i];
          }
          // (alpha / resc are rewritten only behind the next tile's barrier, which every
          // worker reaches after it has read them here)
          load_scores(false);
        }

        // p = 2^y, denominators, this thread's part of the P^T row
        {
          uint32_t pk[CPW / 2];
#pragma unroll
          for (int i = 0; i < CPW / 2; ++i) {
            const float p0 = ex2(y[2 * i]), p1 = ex2(y[2 * i + 1]);
            lsum[2 * i] += p0;
            lsum[2 * i + 1] += p1;
            pk[i] = pack_bf16x2(p0, p1);
          }
          if constexpr (NH == 64) {
            const uint32_t prow = sP + row * 128;
            const int x = row & 7;
            st_shared_v4(prow + (((2 * cg) ^ x) << 4), pk[0], pk[1], pk[2], pk[3]);
            st_shared_v4(prow + (((2 * cg + 1) ^ x) << 4), pk[4], pk[5], pk[6], pk[7]);
          } else if constexpr (NH == 32) {
            const uint32_t prow = sP + row * 64;
            st_shared_v4(prow + ((cg ^ ((row >> 1) & 3)) << 4), pk[0], pk[1], pk[2], pk[3]);
          } else {
            const uint32_t prow = sP + row * 32;
            st_shared_v2(prow + (((cg >> 1) ^ ((row >> 2) & 1)) << 4) + (cg & 1) * 8, pk[0], pk[1]);
          }
        }
        fence_async_smem();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_p_full);
        if (tid == 0) TSTAMP(t, 4);
        ridx = ridx_next;
      }  // t >= 0

      // fill tile t + 1 (behind the P.V product of tile t, if there is one)
      if (more) {
        advance_loads(ld_tile);
        if constexpr (S::PAGED) {
          // registers hold tile t + 1 (scales sw_cur); they are refilled with tile t + 2
          fill(t, ld_tile < n_tiles);
          if (tid == 0) TSTAMP(t + 1, 7);
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) sw_cur[hh] = sw_ld[hh];
        } else {
          fill(t, true);                                // rows of tile t + 1
        }
        if (tid == 0) TSTAMP(t + 1, 0);
      }
    }

    // ---- this warp's share of the final denominators (and of the logit maxima) ---------
    {
      float v[CPW];
#pragma unroll
      for (int i = 0; i < CPW; ++i) v[i] = lsum[i];
      const float cm = warp_col_sum<CPW>(v, lane);
      if (lane < CPW) ctrl.wred[lg][cg * CPW + lane] = cm;
    }
    if (want_ml) {
      const float mx = warp_col_max_packed<CPW>(mlpk, lane);
      if (lane < CPW) ctrl.wmax[lg][cg * CPW + lane] = mx;
    }
  }
#undef TSTAMP

  // The kernel after this one in the stream (the split combine, or the next layer) may be
  // set up on the SMs while the epilogue runs; it waits for this grid's end before it reads.
  grid_launch_dependents();

  // ---- final denominators and output factors ---------------------------------------
  if (ok && !mbar_wait(bar_o_done, 0)) { atomicExch(&g_attn_error, ERR_ODONE); ok = false; }
  tc_fence_after_sync();
  // This thread is done with the K tile: tell the cluster now, wait for it in the merge.
  if (p.cluster > 1) cluster_arrive();
  if (tid == 0) stamp(p, 3);
  if (tid == 0) stamp_cta(p, 2);
  if (!ok) ctrl.fail = 1;
  __syncthreads();
  const uint32_t tlane_o = static_cast<uint32_t>(lg * 32) << 16;
  if (p.cluster > 1) {
    float l = 0.f, mr = -INFINITY;
    if (tid < NH) {
      l = ctrl.wred[0][tid] + ctrl.wred[1][tid] + ctrl.wred[2][tid] + ctrl.wred[3][tid];
      mr = ctrl.mref[tid];
    }
    MergeCtx mc{sK, tmem + tlane_o + COL_O, heads_here, head0, bi, si, acc_slot0, false};
    cluster_merge<NH>(merge_out_of(p), ctrl, mc, l, mr);
  } else {
    if (tid < NH && !ctrl.fail) {
      const float l = ctrl.wred[0][tid] + ctrl.wred[1][tid] + ctrl.wred[2][tid] + ctrl.wred[3][tid];
      const float mr = ctrl.mref[tid];
      const float m_nat = (mr <= NEG_HUGE) ? -INFINITY : mr * LN2;
      float f;
      if (split_out) {
        const bool empty = !(l > 0.f) || m_nat == -INFINITY;
        f = empty ? 0.f : 1.f / l;
        if (tid < heads_here) p.lse_accum[acc_slot0 + tid] = empty ? -INFINITY : logf(l) + m_nat;
      } else {
        const bool has_sink = p.sink != nullptr;
        float lse_v, ml_v;
        f = finalize_row(p.mode, m_nat, l, has_sink,
                         (has_sink && tid < heads_here) ? p.sink[head0 + tid] : 0.f, lse_v, ml_v);
        if (tid < heads_here) {
          p.lse[bi * p.stride_lse_b + si * p.stride_lse_s + (head0 + tid) * p.stride_lse_h] = lse_v;
          if (want_ml) {
            const float mx = fmaxf(fmaxf(ctrl.wmax[0][tid], ctrl.wmax[1][tid]),
                                   fmaxf(ctrl.wmax[2][tid], ctrl.wmax[3][tid]));
            p.max_logits[bi * p.stride_ml_b + head0 + tid] =
                (ml_v == -INFINITY) ? -INFINITY : mx * p.sm_scale;
          }
        }
      }
      ctrl.alpha[tid] = f;
    }
    __syncthreads();

    // ---- epilogue: worker warp w drains O^T slice w / 4 for TMEM lanes 32 * (w % 4).. ----
    if (!ctrl.fail) {
      const int m = warp >> 2;
      const int d = m * 128 + lg * 32 + lane;
#pragma unroll 1
      for (int c4 = 0; c4 < NH / 16; ++c4) {
        uint32_t o[16];
        tmem_ld16(tmem + tlane_o + COL_O + m * O_SLICE_COLS + c4 * 16, o);
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
    // A CTA whose wait gave up wrote nothing; NaN in its log-sum-exp slots makes that
    // visible to whatever consumes the result (the combine step propagates it).
    if (ctrl.fail && tid < heads_here) {
      if (split_out) p.lse_accum[acc_slot0 + tid] = NAN;
      else p.lse[bi * p.stride_lse_b + si * p.stride_lse_s + (head0 + tid) * p.stride_lse_h] = NAN;
    }
  }  // not clustered

  // ---- teardown --------------------------------------------------------------------
  if (tid == 0) stamp(p, 4);
  tc_fence_before_sync();
  __syncthreads();
  if (tid == 0) stamp(p, 5);
  if (tid == 0) stamp_cta(p, 3);
}

// The dynamic shared-memory limit of a kernel is a per-device attribute: set once per
// (instantiation, device).
constexpr int MAX_DEVICES = 64;
std::mutex g_configure_mu;

template <int FMT, int DQK, int NH, bool EXTRA>
cudaError_t launch_one(const AttnParams& p, cudaStream_t st) {
  constexpr size_t smem = smem_bytes<FMT, DQK, NH>();
  static bool configured[MAX_DEVICES] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e) return e;
  if (dev < 0 || dev >= MAX_DEVICES) return cudaErrorInvalidDevice;
  {
    std::lock_guard<std::mutex> lk(g_configure_mu);
    if (!configured[dev]) {
      e = cudaFuncSetAttribute(sm100_attn_kernel<FMT, DQK, NH, EXTRA>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
      if (e) return e;
      configured[dev] = true;
    }
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.n_req, (p.h_q + NH - 1) / NH, p.n_splits);
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
  return cudaLaunchKernelEx(&cfg, sm100_attn_kernel<FMT, DQK, NH, EXTRA>, p);
}

// Heads per CTA (the MMA N): the smallest of 16 / 32 / 64 that holds all heads, so a
// tensor-parallel shard of 16 heads pays for N = 16 products and a 16-head Q, not for 64.
// DSV4_HEADS_PER_CTA=64 forces the widest shape (measurement hook).
int heads_per_cta(int h_q) {
  static const int forced = [] {
    const char* e = std::getenv("DSV4_HEADS_PER_CTA");
    return e ? std::atoi(e) : 0;
  }();
  if (forced == 16 || forced == 32 || forced == 64) return h_q <= forced ? forced : 64;
  return h_q <= 16 ? 16 : h_q <= 32 ? 32 : 64;
}

template <int FMT, int DQK>
cudaError_t launch_paged(const AttnParams& p, cudaStream_t st) {
  if (p.extra_kv != nullptr) return launch_one<FMT, DQK, 64, true>(p, st);
  switch (heads_per_cta(p.h_q)) {
    case 16: return launch_one<FMT, DQK, 16, false>(p, st);
    case 32: return launch_one<FMT, DQK, 32, false>(p, st);
    default: return launch_one<FMT, DQK, 64, false>(p, st);
  }
}

}  // namespace

bool sm100_attn_supported(int kv_format, int d_qk) {
  return (kv_format == DSV4_KV_MODEL1 && d_qk == 512) || (kv_format == DSV4_KV_V32 && d_qk == 576) ||
         (kv_format == DSV4_KV_BF16 && (d_qk == 512 || d_qk == 576));
}

int sm100_attn_heads_per_cta(int h_q, bool extra) { return extra ? 64 : heads_per_cta(h_q); }

cudaError_t launch_sm100_attn(const AttnParams& p, int kv_format, int d_qk, cudaStream_t st) {
  if (kv_format == DSV4_KV_MODEL1) return launch_paged<DSV4_KV_MODEL1, 512>(p, st);
  if (kv_format == DSV4_KV_V32) return launch_paged<DSV4_KV_V32, 576>(p, st);
  if (d_qk == 512) return launch_one<DSV4_KV_BF16, 512, 64, false>(p, st);
  return launch_one<DSV4_KV_BF16, 576, 64, false>(p, st);
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
