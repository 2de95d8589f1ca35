/*
 * dsv4_b200.h — C ABI of the B200 (sm_100a) sparse-MLA attention library.
 *
 * Every entry point takes plain device pointers, sizes and element strides; no
 * framework types cross this boundary.  Nothing here allocates, frees, retains
 * or synchronises unless a comment says so: the caller owns inputs, outputs and
 * scratch, and work is queued on the CUDA stream passed in.  Every function
 * returns DSV4_OK or a DSV4_ERR_* code (never aborts the process);
 * dsv4_strerror() turns a code into text.
 *
 * Citations name the interface of the reference project
 * (ambientlight/deepseek-v4-flash-sm120) that the entry point stands in for.
 */
#ifndef DSV4_B200_H_
#define DSV4_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DSV4_ABI_VERSION 1

enum Dsv4Status {
  DSV4_OK = 0,
  DSV4_ERR_NULL = 1,        /* a required pointer is null                      */
  DSV4_ERR_SHAPE = 2,       /* a size is out of the supported range            */
  DSV4_ERR_LAYOUT = 3,      /* d_qk / KV layout / page stride do not agree     */
  DSV4_ERR_ALIGN = 4,       /* a pointer or stride breaks an alignment rule    */
  DSV4_ERR_ARCH = 5,        /* the current device is not sm_100                */
  DSV4_ERR_CUDA = 6,        /* a CUDA runtime call failed (see dsv4_last_cuda_error) */
  DSV4_ERR_SCRATCH = 7,     /* partials leave the chip but scratch pointers are null */
  DSV4_ERR_UNSUPPORTED = 8, /* valid request that this build does not implement */
  DSV4_ERR_SCRATCH_TOO_LARGE = 9 /* dsv4_sparse_decode_noalloc: partials exceed the built-in scratch */
};

/* KV-cache token layouts.  A page of P tokens is two sections:
 *   [P x (d_nope FP8 e4m3 bytes + 64 BF16 RoPE values)] [P x scale_slots UE8M0 bytes]
 * MODEL1: d_nope 448, one scale per 64 values, 7 scales + 1 pad  -> 576 + 8 = 584 B/token
 *         (reference: tests/reference.py:7-14, csrc/sm120/decode/sparse_decode_kernel.cuh:27-39)
 * V32   : d_nope 512, one scale per 128 values, 4 scales         -> 640 + 4 = 644 B/token
 *         (reference: csrc/common/params.h:12-15 names it; the benchmark configs use it)
 * BF16  : flat rows of d_qk BF16 values, no paging (prefill workspace,
 *         reference: csrc/common/params.h:99-102)                                      */
enum Dsv4KvFormat { DSV4_KV_BF16 = 0, DSV4_KV_MODEL1 = 1, DSV4_KV_V32 = 2 };

enum Dsv4Flags {
  /* Decode only: treat an index < 0 or >= num_tokens as masked (-inf) the way
   * upstream FlashMLA does.  Default (flag clear) follows the reference oracle:
   * such an index gathers a zero row that still scores logit 0
   * (tests/reference.py:110-119).                                                      */
  DSV4_FLAG_MASK_INVALID = 1,
  /* Run the plain CUDA-core kernels instead of the tcgen05 ones (debug aid).           */
  DSV4_FLAG_IMPL_SIMPLE = 2,
  /* Decode with n_splits > 1: stop after writing the partials; the caller runs
   * dsv4_split_combine itself (lets a benchmark time the two kernels apart).           */
  DSV4_FLAG_NO_COMBINE = 4,
  /* Decode only: a topk_length below one means "attend to nothing" (out 0, lse = sink
   * or -inf), as the reference's CUDA kernel treats it
   * (csrc/sm120/decode/sparse_decode_kernel.cuh:373-375).  Default (flag clear)
   * follows the reference's torch oracle, which raises such a length to one
   * (tests/reference.py:108-109).                                                      */
  DSV4_FLAG_ZERO_LENGTH_EMPTY = 8
};

/* ---------------------------------------------------------------------------
 * Sparse decode: replaces dsv4_kernel::sparse_decode_fwd
 * (csrc/api/sparse_decode.cpp:27-220) and its parameter block
 * SparseAttnDecodeParams (csrc/common/params.h:34-97).
 *
 * For request r = (b_idx, s_idx) the kernel attends q[r] over the rows named by
 * indices[r, 0:len) of the paged cache (then extra_indices[r, 0:extra_len) of
 * the extra cache when given), V being the first 512 columns of the dequantised
 * row, and writes out[r] (BF16) and lse[r] (fp32, natural log, sink-merged).
 * len = clamp(topk_length[b_idx], 1, topk) when topk_length is given, else topk
 * (lower bound 0 with DSV4_FLAG_ZERO_LENGTH_EMPTY).
 * Strides are in elements of the tensor's own type, except stride_kv_block and
 * stride_extra_kv_block which are in BYTES.  All inner dimensions are dense.
 * q rows and KV pages must be 16-byte aligned.
 *
 * When n_splits > 1 each request's list is cut into n_splits ranges.  Groups of
 * consecutive ranges (4, 2 or 1 of them: a thread-block cluster) are merged on
 * chip; each group writes one locally normalised fp32 partial to o_accum
 * [n_splits, b*s_q, h_q, 512] / lse_accum [n_splits, b*s_q, h_q] (the first
 * dsv4_decode_partial_sets(args) slots are used), and the same call then runs
 * the combine step over those.  With a single group the result is final and
 * neither scratch nor a combine is touched.
 * ------------------------------------------------------------------------- */
typedef struct Dsv4DecodeArgs {
  int32_t b, s_q, h_q, d_qk, d_v, topk;
  int32_t kv_format;            /* DSV4_KV_MODEL1 or DSV4_KV_V32                 */
  int32_t num_blocks, page_block_size;
  int32_t extra_num_blocks, extra_page_block_size, extra_topk;
  int32_t n_splits;             /* >= 1; see dsv4_plan_splits                    */
  int32_t flags;                /* Dsv4Flags                                     */
  float sm_scale;
  int32_t _pad0;

  const void* q;                /* BF16 [b, s_q, h_q, d_qk]                      */
  const void* kv;               /* bytes [num_blocks, stride_kv_block]           */
  const int32_t* indices;       /* [b, s_q, topk]                                */
  const int32_t* topk_length;   /* [b] or null                                   */
  const float* attn_sink;       /* [h_q] or null                                 */
  const void* extra_kv;         /* or null                                       */
  const int32_t* extra_indices; /* [b, s_q, extra_topk] or null                  */
  const int32_t* extra_topk_length; /* [b] or null                               */

  void* out;                    /* BF16 [b, s_q, h_q, 512]                       */
  float* lse;                   /* fp32, addressed with the three lse strides    */
  float* o_accum;               /* scratch, dsv4_decode_partial_sets(args) > 1   */
  float* lse_accum;             /* scratch, dsv4_decode_partial_sets(args) > 1   */

  int64_t stride_q_b, stride_q_s, stride_q_h;
  int64_t stride_kv_block, stride_extra_kv_block;
  int64_t stride_indices_b, stride_indices_s;
  int64_t stride_extra_indices_b, stride_extra_indices_s;
  int64_t stride_o_b, stride_o_s, stride_o_h;
  int64_t stride_lse_b, stride_lse_s, stride_lse_h;
} Dsv4DecodeArgs;

int dsv4_sparse_decode(const Dsv4DecodeArgs* args, void* cuda_stream);

/* ---------------------------------------------------------------------------
 * Sparse decode without any allocation.  No counterpart in the reference (its
 * host code allocates the split-KV partials on every call,
 * csrc/api/sparse_decode.cpp:176-182).
 *
 * For callers that cannot obtain device memory at call time: code running under
 * CUDA-graph capture or replay, code inside another runtime's no-allocation /
 * no-synchronisation sections, embedders without an allocator.  Same arguments
 * and results as dsv4_sparse_decode, except that args->o_accum / lse_accum are
 * ignored: the split-KV partials go to a fixed array inside the library's device
 * image (DSV4_NOALLOC_MAX_O_FLOATS fp32 values of partial output plus one
 * log-sum-exp per 512 of them, about 16 MiB, held by every GPU that loads the
 * library until the process exits).  The call performs no cudaMalloc / cudaFree
 * and uses no allocating library routine.
 *
 *  - Limit: sets * b * s_q * h_q * 512 <= DSV4_NOALLOC_MAX_O_FLOATS, where sets =
 *    dsv4_decode_partial_sets(args) is the number of partial sets that really
 *    reach the scratch (splits merged on chip leave none, so n_splits of 2 or 4
 *    never hit the limit; batch 16 x 64 heads x 8 splits fits exactly); larger
 *    requests return DSV4_ERR_SCRATCH_TOO_LARGE and launch nothing.
 *  - The FIRST call on each device looks up the array's device address (a cheap,
 *    one-time query with that device current).  Make that first call before any
 *    stream capture begins.
 *  - All calls on a device share the one array and it keeps whatever the last
 *    call left in it.  Nothing needs clearing (each call writes every slot it
 *    later reads), but two calls whose kernels overlap on the GPU (different
 *    streams, or graph branches) race on it: serialise them.
 * ------------------------------------------------------------------------- */
#define DSV4_NOALLOC_MAX_O_FLOATS 4194304
int dsv4_sparse_decode_noalloc(const Dsv4DecodeArgs* args, void* cuda_stream);

/* Split count for a decode call: a pure function of shapes and the SM count, so
 * it is stable under CUDA-graph capture.  Stands in for the heuristic at
 * csrc/api/sparse_decode.cpp:147-171 (the policy differs: it is sized for one
 * CTA per SM that owns up to 64 heads and walks 128-row tiles).                  */
int dsv4_plan_splits(int b, int s_q, int h_q, int topk, int extra_topk, int num_sms);

/* Number of partial sets a decode call with these arguments leaves in o_accum /
 * lse_accum (n_splits divided by the on-chip merge width; 1 = none, the output is
 * final).  Callers that pass DSV4_FLAG_NO_COMBINE give this as n_splits to
 * dsv4_split_combine.  No reference counterpart.                                  */
int dsv4_decode_partial_sets(const Dsv4DecodeArgs* args);

/* ---------------------------------------------------------------------------
 * All-gather of head-sharded decode results over NVLink peer memory (tensor
 * parallel over heads: every GPU runs dsv4_sparse_decode on h_q / world heads of
 * the same requests).  Stands in for the two NCCL all-gathers a head-sharded
 * caller of the reference would issue after sparse_decode_fwd; the reference
 * itself has no multi-GPU code.
 *
 * peer_out[r] / peer_lse[r] / peer_flags[r] are rank r's gathered buffers
 * (BF16 [b, s_q, h_local*world, 512], fp32 [b, h_local*world, s_q], int32[world],
 * flags zero-initialised) as mapped into THIS process (peer-mapped device memory,
 * e.g. CUDA IPC or symmetric memory); entry `rank` is the local one.  `step` must
 * increase by one per call and the caller must alternate between two sets of
 * gathered buffers (the flag array is shared by both).  `counter` is a local
 * zero-initialised int32, `status` a local int32 that receives a non-zero code
 * when a peer's shard did not arrive within the bounded wait (~0.3 s).
 * All ranks must call it for the same step; the kernel returns once every shard
 * has landed locally.  No host synchronisation.
 * ------------------------------------------------------------------------- */
#define DSV4_MAX_PEERS 8
typedef struct Dsv4GatherArgs {
  int32_t world, rank, b, s_q, h_local, step;
  const void* out_local;        /* BF16 [b, s_q, h_local, 512], dense              */
  const float* lse_local;       /* fp32 [b, h_local, s_q], dense                   */
  void* peer_out[DSV4_MAX_PEERS];
  float* peer_lse[DSV4_MAX_PEERS];
  int32_t* peer_flags[DSV4_MAX_PEERS];
  int32_t* counter;
  int32_t* status;
} Dsv4GatherArgs;

int dsv4_gather_heads(const Dsv4GatherArgs* args, void* cuda_stream);

/* Head-sharded decode and its exchange in one call: decode this rank's h_q heads
 * (decode->h_q == gather->h_local) into decode->out / decode->lse, which must be dense, and
 * leave the result of ALL ranks' heads in every rank's gathered buffers.  The exchange
 * kernel of dsv4_gather_heads is queued behind the decode with programmatic dependent
 * launch, so it is resident on the GPU before the rows are final; it reads the rows once
 * and stores them to every rank with 16-byte peer stores (no multicast, no TMA).
 * gather->out_local / lse_local are ignored.  Same step / buffer-set rules as
 * dsv4_gather_heads.  No reference counterpart (the reference has no multi-GPU code).    */
int dsv4_sparse_decode_gather(const Dsv4DecodeArgs* decode, const Dsv4GatherArgs* gather,
                              void* cuda_stream);

/* ---------------------------------------------------------------------------
 * Split-KV combine alone: replaces dsv4_split_kv_combine
 * (csrc/sm120/decode/split_kv_combine.cuh:23-110).
 * o_accum fp32 [n_splits, n_rows, h_q, 512] and lse_accum fp32
 * [n_splits, n_rows, h_q], both dense; row r of the output lives at
 * out + (r / s_q) * stride_o_b + (r % s_q) * stride_o_s  (likewise lse).
 * ------------------------------------------------------------------------- */
typedef struct Dsv4CombineArgs {
  int32_t n_rows, s_q, h_q, n_splits;
  const float* o_accum;
  const float* lse_accum;
  const float* attn_sink;       /* [h_q] or null                                 */
  void* out;                    /* BF16                                          */
  float* lse;
  int64_t stride_o_b, stride_o_s, stride_o_h;
  int64_t stride_lse_b, stride_lse_s, stride_lse_h;
} Dsv4CombineArgs;

int dsv4_split_combine(const Dsv4CombineArgs* args, void* cuda_stream);

/* ---------------------------------------------------------------------------
 * Sparse prefill: replaces dsv4_kernel::sparse_prefill_fwd
 * (csrc/api/sparse_prefill.cpp:27-136, SparseAttnPrefillParams
 * csrc/common/params.h:103-135).  kv_format DSV4_KV_BF16 is the reference's
 * flat workspace kv[s_kv, d_qk]; MODEL1 / V32 read the FP8 paged cache directly
 * (s_kv = num_blocks * page_block_size).  An index < 0, >= s_kv, or at a
 * position >= topk_length[i] is masked.  Outputs: out BF16 [s_q, h_q, 512],
 * max_logits and lse fp32 [s_q, h_q] (natural log; lse excludes the sink; a row
 * with nothing to attend to gives out 0, max_logits -inf, lse +inf).
 * ------------------------------------------------------------------------- */
typedef struct Dsv4PrefillArgs {
  int32_t s_q, s_kv, h_q, d_qk, d_v, topk;
  int32_t kv_format;
  int32_t num_blocks, page_block_size;
  int32_t flags;
  float sm_scale;
  int32_t _pad0;

  const void* q;                /* BF16 [s_q, h_q, d_qk]                         */
  const void* kv;               /* BF16 [s_kv, d_qk] or paged bytes              */
  const int32_t* indices;       /* [s_q, topk]                                   */
  const float* attn_sink;       /* [h_q] or null                                 */
  const int32_t* topk_length;   /* [s_q] or null                                 */
  void* out;
  float* max_logits;
  float* lse;

  int64_t stride_q_s, stride_q_h;
  int64_t stride_kv_row;        /* elements (BF16) or bytes per page (paged)     */
  int64_t stride_indices_s;
  int64_t stride_o_s, stride_o_h;
  int64_t stride_ml_s, stride_lse_s;
} Dsv4PrefillArgs;

int dsv4_sparse_prefill(const Dsv4PrefillArgs* args, void* cuda_stream);

/* ---------------------------------------------------------------------------
 * KV store / quantise.  The reference has no such kernel: its cache is written
 * by the serving framework (tests/reference.py:48-49 names quant_k_cache_v4).
 * Per token i with slot s = slots[i] >= 0 (page s / P, row s % P): for each
 * tile of quant_tile latent values e = ceil(log2(max(amax, 1e-4) / 448)), scale
 * byte e + 127, fp8 = saturating round-to-nearest-even e4m3 of x * 2^-e; RoPE
 * copied as BF16; unused scale slots written as zero.
 * ------------------------------------------------------------------------- */
typedef struct Dsv4StoreArgs {
  int32_t n_tokens, kv_format, num_blocks, page_block_size;
  const void* k_nope;           /* BF16 [n_tokens, d_nope]                       */
  const void* k_rope;           /* BF16 [n_tokens, 64]                           */
  const int64_t* slots;         /* [n_tokens]; negative = skip                   */
  void* kv;                     /* paged cache bytes                             */
  int64_t stride_nope, stride_rope, stride_kv_block;   /* elements, elements, bytes */
} Dsv4StoreArgs;

int dsv4_kv_store(const Dsv4StoreArgs* args, void* cuda_stream);

/* The same store for the form the serving framework's cache writer has its operands in
 * (the step before the path: tests/reference.py:45-58 names quant_k_cache_v4 as the
 * producer of the bytes the kernels read): one BF16 row per token holding the latent
 * values followed by the 64 RoPE values, [n_tokens, d_qk] with any row stride that is a
 * multiple of 8 elements (a view of a wider projection output needs no copy), and the
 * framework's slot mapping as int32 or int64.  Same arithmetic and bytes as
 * dsv4_kv_store.  No reference counterpart.                                             */
typedef struct Dsv4StoreRowsArgs {
  int32_t n_tokens, kv_format, num_blocks, page_block_size;
  const void* k;                /* BF16 [n_tokens, d_qk], d_qk = 512 (MODEL1) / 576 (V32) */
  const void* loc;              /* [n_tokens] cache slots; negative = skip       */
  void* kv;                     /* paged cache bytes                             */
  int64_t stride_k, stride_kv_block;                   /* elements, bytes        */
  int32_t loc_is_int64;         /* 0: loc is int32, 1: loc is int64              */
  int32_t reserved;
} Dsv4StoreRowsArgs;

int dsv4_kv_store_rows(const Dsv4StoreRowsArgs* args, void* cuda_stream);

/* ===========================================================================
 * TEST HOOKS.  The three entries marked "test hook" below (dsv4_gather_dequant,
 * dsv4_debug_set_timeline, dsv4_umma_selftest) exist for the test-suite and for
 * profiling; a serving integration binds none of them.
 * ===========================================================================
 *
 * Test hook.  Gather + dequantise only: rows[i] = dequantised d_qk BF16 values of
 * token indices[i], or zeros for an index outside [0, num_blocks * page_block_size).
 * method == 0 converts with the device function the attention kernel converts with
 * (dequant4 in csrc/dsv4_common.cuh: two packed-BF16 multiplies), but stores the rows
 * linearly, so it pins the conversion and the page addressing, not the kernel's
 * shared-memory arrangement; the kernel's own path is pinned by decodes whose lists
 * hold a single entry (the output must equal the value row).  method == 1 converts
 * through fp32 instead (reference: load_kv_chunk,
 * csrc/sm120/decode/sparse_decode_kernel.cuh:101-167).                                 */
int dsv4_gather_dequant(const void* kv, int64_t stride_kv_block, int32_t kv_format,
                        int32_t num_blocks, int32_t page_block_size,
                        const int32_t* indices, int32_t n, void* rows_bf16,
                        int32_t method, void* cuda_stream);

/* Device facts, cached per device after the first call (reference: Arch,
 * csrc/common/params.h:138-156, which queries on every call).                         */
int dsv4_device_info(int device, int* major, int* minor, int* num_sms);

/* Device-side health word of the tensor-core attention kernels on the current
 * device: 0, or the code of the first bounded wait that gave up (the kernel then
 * returned early and its outputs are not valid).  Copies from the device, so it
 * SYNCHRONISES with work already queued; reset != 0 clears the word.  A serving
 * loop need not call it; the tests do after every launch.                             */
int dsv4_device_status(int32_t* status_out, int reset);

/* Test hook / debug aid: give the attention kernels a device buffer of at least
 * 1024 + 4 * (CTAs of the largest launch) int64.  CTA (0,0,0) of every later launch
 * writes SM cycle-counter stamps of its pipeline stages into the first 1024 slots and
 * every CTA four global-timer stamps (start, set-up done, last product done, end)
 * behind them (null switches it off).  Process-wide; not for production.  The stamps
 * exist only in a library built with -DDSV4_TIMELINE; otherwise this is a no-op.     */
int dsv4_debug_set_timeline(void* device_buffer);

/* Text for a status code; the last CUDA error string seen by this thread.             */
const char* dsv4_strerror(int status);
const char* dsv4_last_cuda_error(void);
int dsv4_abi_version(void);

/* Test hook.  Tensor-core self-test: one 128 x n x k BF16 product
 * through tcgen05.mma with the shared-memory operand arrangement the attention
 * kernel uses (mode 0: both operands K-major; mode 1: A and B MN-major).
 * a, b, d are device pointers (BF16, BF16, fp32 row-major [128, n]).                   */
int dsv4_umma_selftest(int mode, int n, int k, const void* a, const void* b, float* d,
                       int32_t* status, void* cuda_stream);

#ifdef __cplusplus
}
#endif
#endif /* DSV4_B200_H_ */
