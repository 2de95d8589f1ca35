// extern "C" entry points: argument validation, translation to the kernel-side
// parameter block, dispatch.  Allocates nothing and never synchronises.
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "attn_params.cuh"
#include "launchers.h"

namespace {

thread_local char g_cuda_err[256] = "";

int cuda_fail(cudaError_t e) {
  std::snprintf(g_cuda_err, sizeof(g_cuda_err), "%s: %s", cudaGetErrorName(e),
                cudaGetErrorString(e));
  return DSV4_ERR_CUDA;
}

struct DevInfo { int major = 0, minor = 0, sms = 0; bool ok = false; };
constexpr int MAX_DEVICES = 64;
DevInfo g_dev[MAX_DEVICES];
std::mutex g_dev_mu;

int device_info(int device, DevInfo& out) {
  if (device < 0 || device >= MAX_DEVICES) return DSV4_ERR_SHAPE;
  std::lock_guard<std::mutex> lk(g_dev_mu);
  DevInfo& d = g_dev[device];
  if (!d.ok) {
    cudaError_t e;
    if ((e = cudaDeviceGetAttribute(&d.major, cudaDevAttrComputeCapabilityMajor, device)) ||
        (e = cudaDeviceGetAttribute(&d.minor, cudaDevAttrComputeCapabilityMinor, device)) ||
        (e = cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, device)))
      return cuda_fail(e);
    d.ok = true;
  }
  out = d;
  return DSV4_OK;
}

int current_device_is_sm100() {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e) return cuda_fail(e);
  DevInfo d;
  int rc = device_info(dev, d);
  if (rc) return rc;
  if (d.major != 10 && std::getenv("DSV4_KERNEL_FORCE") == nullptr) return DSV4_ERR_ARCH;
  return DSV4_OK;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int check_paged(int kv_format, int d_qk, int page_block, int64_t stride_block, const void* kv) {
  int per_tok;
  if (kv_format == DSV4_KV_MODEL1) { per_tok = 584; if (d_qk != 512) return DSV4_ERR_LAYOUT; }
  else if (kv_format == DSV4_KV_V32) { per_tok = 644; if (d_qk != 576) return DSV4_ERR_LAYOUT; }
  else return DSV4_ERR_LAYOUT;
  if (page_block < 1) return DSV4_ERR_SHAPE;
  if (stride_block < static_cast<int64_t>(page_block) * per_tok) return DSV4_ERR_LAYOUT;
  if ((stride_block & 15) || !aligned16(kv)) return DSV4_ERR_ALIGN;
  return DSV4_OK;
}

long long* g_timeline = nullptr;

int log2_or_minus1(int v) {
  if (v <= 0 || (v & (v - 1))) return -1;
  int s = 0;
  while ((1 << s) < v) ++s;
  return s;
}

bool want_simple(int flags) {
  if (flags & DSV4_FLAG_IMPL_SIMPLE) return true;
  const char* e = std::getenv("DSV4_IMPL");
  return e && std::strcmp(e, "simple") == 0;
}

}  // namespace

extern "C" {

int dsv4_abi_version(void) { return DSV4_ABI_VERSION; }

const char* dsv4_last_cuda_error(void) { return g_cuda_err; }

const char* dsv4_strerror(int s) {
  switch (s) {
    case DSV4_OK: return "ok";
    case DSV4_ERR_NULL: return "a required pointer is null";
    case DSV4_ERR_SHAPE: return "a size is outside the supported range";
    case DSV4_ERR_LAYOUT: return "d_qk, KV format and page stride do not describe a supported cache layout";
    case DSV4_ERR_ALIGN: return "a pointer or stride is not 16-byte aligned";
    case DSV4_ERR_ARCH: return "the current device is not compute capability 10.x (set DSV4_KERNEL_FORCE to override)";
    case DSV4_ERR_CUDA: return "a CUDA runtime call failed";
    case DSV4_ERR_SCRATCH: return "this split count leaves partials: o_accum and lse_accum are needed";
    case DSV4_ERR_UNSUPPORTED: return "this request is valid but not implemented by this build";
    case DSV4_ERR_SCRATCH_TOO_LARGE: return "split-KV partials exceed the built-in scratch of dsv4_sparse_decode_noalloc (partial sets * b * s_q * h_q * 512 > DSV4_NOALLOC_MAX_O_FLOATS)";
    default: return "unknown status";
  }
}

int dsv4_device_info(int device, int* major, int* minor, int* num_sms) {
  DevInfo d;
  int rc = device_info(device, d);
  if (rc) return rc;
  if (major) *major = d.major;
  if (minor) *minor = d.minor;
  if (num_sms) *num_sms = d.sms;
  return DSV4_OK;
}

int dsv4_plan_splits(int b, int s_q, int h_q, int topk, int extra_topk, int num_sms) {
  if (b < 1 || s_q < 1 || h_q < 1 || topk < 1 || num_sms < 1) return 1;
  const int tile = 128;   // rows one CTA consumes per pipeline step
  const long base = static_cast<long>(b) * s_q * ((h_q + 63) / 64);
  const int tiles = (topk + std::max(extra_topk, 0) + tile - 1) / tile;
  if (base >= num_sms || tiles <= 1) return 1;
  // Cost of a plan in tile-times: waves of CTAs, each walking its tiles plus a
  // fixed prologue/epilogue; a split plan pays one more pass for the combine.
  const double fixed = 0.75, combine = 0.6;
  int best = 1;
  double best_cost = 1e30;
  const int max_s = std::min({tiles, dsv4::combine_max_splits(), 128});
  for (int s = 1; s <= max_s; ++s) {
    const int per = (tiles + s - 1) / s;
    if (s > 1 && (s - 1) * per >= tiles) continue;          // last split would be empty
    const long ctas = base * s;
    const long waves = (ctas + num_sms - 1) / num_sms;
    double cost = waves * (per + fixed) + (s > 1 ? combine + 0.02 * s : 0.0);
    if (cost < best_cost - 1e-9) { best_cost = cost; best = s; }
  }
  return best;
}

int dsv4_split_combine(const Dsv4CombineArgs* a, void* stream) {
  if (!a || !a->o_accum || !a->lse_accum || !a->out || !a->lse) return DSV4_ERR_NULL;
  if (a->n_rows < 0 || a->s_q < 1 || a->h_q < 1 || a->n_splits < 1 ||
      a->n_splits > dsv4::combine_max_splits())
    return DSV4_ERR_SHAPE;
  if (!aligned16(a->o_accum) || (reinterpret_cast<uintptr_t>(a->out) & 7u) ||
      (a->stride_o_b & 3) || (a->stride_o_s & 3) || (a->stride_o_h & 3))
    return DSV4_ERR_ALIGN;
  if (a->n_rows == 0) return DSV4_OK;
  cudaError_t e = dsv4::launch_combine(*a, static_cast<cudaStream_t>(stream));
  return e ? cuda_fail(e) : DSV4_OK;
}

// Splits merged on chip by one thread-block cluster of the tensor-core kernel.  The merge
// pays when it makes the output final (no partials through L2, no combine launch): measured
// on B200, two splits per request (b = 64) gain 8 % per call, whereas merging 8 splits in
// groups of 2 or 4 and still combining the groups loses 9-11 %.  So: the whole request in one
// cluster when n_splits is 2 or 4 (clusters of 4 CTAs with this kernel's shared-memory
// footprint still fill the GPU, clusters of 8 do not), otherwise no cluster.
// DSV4_CLUSTER=1 turns clusters off; DSV4_CLUSTER=group forces groups of 2 or 4 for any
// n_splits they divide (measurement hook).
static int cluster_size_for(int n_splits, bool simple_impl) {
  if (simple_impl || n_splits < 2) return 1;
  static const int mode = [] {
    const char* e = std::getenv("DSV4_CLUSTER");
    if (!e) return 0;
    if (!std::strcmp(e, "group")) return 2;
    return std::atoi(e) == 1 ? 1 : 0;
  }();
  if (mode == 1) return 1;
  if (mode == 2) return (n_splits % 4 == 0) ? 4 : (n_splits % 2 == 0) ? 2 : 1;
  return (n_splits == 2 || n_splits == 4) ? n_splits : 1;
}

int dsv4_decode_partial_sets(const Dsv4DecodeArgs* a) {
  if (!a || a->n_splits < 1) return 0;
  const bool simple = want_simple(a->flags) || !dsv4::sm100_attn_supported(a->kv_format, a->d_qk);
  return a->n_splits / cluster_size_for(a->n_splits, simple);
}

int dsv4_sparse_decode(const Dsv4DecodeArgs* a, void* stream) {
  if (!a || !a->q || !a->kv || !a->indices || !a->out || !a->lse) return DSV4_ERR_NULL;
  if (a->b < 0 || a->s_q < 1 || a->h_q < 1 || a->topk < 1 || a->num_blocks < 1 ||
      a->n_splits < 1 || a->n_splits > dsv4::combine_max_splits() || a->d_v != dsv4::D_V)
    return DSV4_ERR_SHAPE;
  int rc = check_paged(a->kv_format, a->d_qk, a->page_block_size, a->stride_kv_block, a->kv);
  if (rc) return rc;
  if (a->extra_kv) {
    if (!a->extra_indices) return DSV4_ERR_NULL;
    if (a->extra_topk < 1 || a->extra_num_blocks < 1) return DSV4_ERR_SHAPE;
    rc = check_paged(a->kv_format, a->d_qk, a->extra_page_block_size, a->stride_extra_kv_block,
                     a->extra_kv);
    if (rc) return rc;
  }
  if (!aligned16(a->q) || (a->stride_q_b & 7) || (a->stride_q_s & 7) || (a->stride_q_h & 7) ||
      !aligned16(a->out) || (a->stride_o_b & 7) || (a->stride_o_s & 7) || (a->stride_o_h & 7))
    return DSV4_ERR_ALIGN;
  // Scratch is needed only when partials really leave the chip (see dsv4_decode_partial_sets).
  if (dsv4_decode_partial_sets(a) > 1) {
    if (!a->o_accum || !a->lse_accum) return DSV4_ERR_SCRATCH;
    if (!aligned16(a->o_accum)) return DSV4_ERR_ALIGN;
  }
  if ((rc = current_device_is_sm100())) return rc;
  if (a->b == 0) return DSV4_OK;

  dsv4::AttnParams p{};
  p.n_req = a->b * a->s_q;
  p.s_q = a->s_q;
  p.h_q = a->h_q;
  p.topk = a->topk;
  p.extra_topk = a->extra_kv ? a->extra_topk : 0;
  p.n_splits = a->n_splits;
  const bool simple = want_simple(a->flags) || !dsv4::sm100_attn_supported(a->kv_format, a->d_qk);
  p.cluster = cluster_size_for(a->n_splits, simple);
  const int partial_sets = a->n_splits / p.cluster;
  p.flags = a->flags;
  p.mode = dsv4::MODE_DECODE;
  p.page_block = a->page_block_size;
  p.n_tok = a->num_blocks * a->page_block_size;
  p.extra_page_block = a->extra_kv ? a->extra_page_block_size : 1;
  p.extra_n_tok = a->extra_kv ? a->extra_num_blocks * a->extra_page_block_size : 0;
  p.page_shift = log2_or_minus1(p.page_block);
  p.extra_page_shift = log2_or_minus1(p.extra_page_block);
  p.sm_scale = a->sm_scale;
  p.q = static_cast<const __nv_bfloat16*>(a->q);
  p.kv = static_cast<const uint8_t*>(a->kv);
  p.extra_kv = static_cast<const uint8_t*>(a->extra_kv);
  p.indices = a->indices;
  p.extra_indices = a->extra_kv ? a->extra_indices : nullptr;
  p.topk_length = a->topk_length;
  p.extra_topk_length = a->extra_kv ? a->extra_topk_length : nullptr;
  p.sink = a->attn_sink;
  p.out = static_cast<__nv_bfloat16*>(a->out);
  p.lse = a->lse;
  p.max_logits = nullptr;
  p.o_accum = a->o_accum;
  p.lse_accum = a->lse_accum;
  p.stride_q_b = a->stride_q_b; p.stride_q_s = a->stride_q_s; p.stride_q_h = a->stride_q_h;
  p.stride_kv = a->stride_kv_block; p.stride_extra_kv = a->stride_extra_kv_block;
  p.stride_idx_b = a->stride_indices_b; p.stride_idx_s = a->stride_indices_s;
  p.stride_xidx_b = a->stride_extra_indices_b; p.stride_xidx_s = a->stride_extra_indices_s;
  p.stride_o_b = a->stride_o_b; p.stride_o_s = a->stride_o_s; p.stride_o_h = a->stride_o_h;
  p.stride_lse_b = a->stride_lse_b; p.stride_lse_s = a->stride_lse_s; p.stride_lse_h = a->stride_lse_h;
  p.prof = g_timeline;

  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e;
  if (simple)
    e = dsv4::launch_simple_attn(p, a->kv_format, a->d_qk, st);
  else
    e = dsv4::launch_sm100_attn(p, a->kv_format, a->d_qk, st);
  if (e) return cuda_fail(e);
  if (partial_sets > 1 && !(a->flags & DSV4_FLAG_NO_COMBINE)) {
    Dsv4CombineArgs c{};
    c.n_rows = p.n_req; c.s_q = a->s_q; c.h_q = a->h_q; c.n_splits = partial_sets;
    c.o_accum = a->o_accum; c.lse_accum = a->lse_accum; c.attn_sink = a->attn_sink;
    c.out = a->out; c.lse = a->lse;
    c.stride_o_b = a->stride_o_b; c.stride_o_s = a->stride_o_s; c.stride_o_h = a->stride_o_h;
    c.stride_lse_b = a->stride_lse_b; c.stride_lse_s = a->stride_lse_s; c.stride_lse_h = a->stride_lse_h;
    if ((e = dsv4::launch_combine(c, st))) return cuda_fail(e);
  }
  return DSV4_OK;
}

int dsv4_sparse_prefill(const Dsv4PrefillArgs* a, void* stream) {
  if (!a || !a->q || !a->kv || !a->indices || !a->out || !a->max_logits || !a->lse)
    return DSV4_ERR_NULL;
  if (a->s_q < 0 || a->s_kv < 0 || a->h_q < 1 || a->topk < 1 || a->d_v != dsv4::D_V)
    return DSV4_ERR_SHAPE;
  int rc;
  if (a->kv_format == DSV4_KV_BF16) {
    if (a->d_qk != 512 && a->d_qk != 576) return DSV4_ERR_LAYOUT;
    if (!aligned16(a->kv) || (a->stride_kv_row & 7)) return DSV4_ERR_ALIGN;
  } else {
    if ((rc = check_paged(a->kv_format, a->d_qk, a->page_block_size, a->stride_kv_row, a->kv)))
      return rc;
    if (a->num_blocks < 1) return DSV4_ERR_SHAPE;
  }
  if (!aligned16(a->q) || (a->stride_q_s & 7) || (a->stride_q_h & 7) || !aligned16(a->out) ||
      (a->stride_o_s & 7) || (a->stride_o_h & 7))
    return DSV4_ERR_ALIGN;
  if ((rc = current_device_is_sm100())) return rc;
  if (a->s_q == 0) return DSV4_OK;

  dsv4::AttnParams p{};
  p.n_req = a->s_q;
  p.s_q = 1;
  p.h_q = a->h_q;
  p.topk = a->topk;
  p.n_splits = 1;
  p.cluster = 1;
  p.flags = a->flags;
  p.mode = dsv4::MODE_PREFILL;
  p.page_block = a->kv_format == DSV4_KV_BF16 ? 1 : a->page_block_size;
  p.n_tok = a->kv_format == DSV4_KV_BF16 ? a->s_kv : a->num_blocks * a->page_block_size;
  p.extra_page_block = 1;
  p.page_shift = log2_or_minus1(p.page_block);
  p.extra_page_shift = 0;
  p.sm_scale = a->sm_scale;
  p.q = static_cast<const __nv_bfloat16*>(a->q);
  p.kv = static_cast<const uint8_t*>(a->kv);
  p.indices = a->indices;
  p.topk_length = a->topk_length;
  p.sink = a->attn_sink;
  p.out = static_cast<__nv_bfloat16*>(a->out);
  p.lse = a->lse;
  p.max_logits = a->max_logits;
  p.stride_q_b = a->stride_q_s; p.stride_q_h = a->stride_q_h;
  p.stride_kv = a->stride_kv_row;
  p.stride_idx_b = a->stride_indices_s;
  p.stride_o_b = a->stride_o_s; p.stride_o_h = a->stride_o_h;
  p.stride_lse_b = a->stride_lse_s; p.stride_lse_h = 1;
  p.stride_ml_b = a->stride_ml_s;
  p.prof = g_timeline;

  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e;
  if (want_simple(a->flags) || !dsv4::sm100_attn_supported(a->kv_format, a->d_qk))
    e = dsv4::launch_simple_attn(p, a->kv_format, a->d_qk, st);
  else
    e = dsv4::launch_sm100_attn(p, a->kv_format, a->d_qk, st);
  return e ? cuda_fail(e) : DSV4_OK;
}

int dsv4_kv_store(const Dsv4StoreArgs* a, void* stream) {
  if (!a || !a->k_nope || !a->k_rope || !a->slots || !a->kv) return DSV4_ERR_NULL;
  if (a->n_tokens < 0 || a->num_blocks < 1 || a->page_block_size < 1) return DSV4_ERR_SHAPE;
  const int d_qk = a->kv_format == DSV4_KV_MODEL1 ? 512 : 576;
  int rc = check_paged(a->kv_format, d_qk, a->page_block_size, a->stride_kv_block, a->kv);
  if (rc) return rc;
  if (!aligned16(a->k_nope) || !aligned16(a->k_rope) || (a->stride_nope & 7) || (a->stride_rope & 7))
    return DSV4_ERR_ALIGN;
  cudaError_t e = dsv4::launch_kv_store(*a, nullptr, static_cast<cudaStream_t>(stream));
  return e ? cuda_fail(e) : DSV4_OK;
}

int dsv4_kv_store_rows(const Dsv4StoreRowsArgs* r, void* stream) {
  if (!r || !r->k || !r->loc || !r->kv) return DSV4_ERR_NULL;
  if (r->n_tokens < 0 || r->num_blocks < 1 || r->page_block_size < 1) return DSV4_ERR_SHAPE;
  if (r->kv_format != DSV4_KV_MODEL1 && r->kv_format != DSV4_KV_V32) return DSV4_ERR_LAYOUT;
  const int d_qk = r->kv_format == DSV4_KV_MODEL1 ? 512 : 576;
  int rc = check_paged(r->kv_format, d_qk, r->page_block_size, r->stride_kv_block, r->kv);
  if (rc) return rc;
  // the RoPE values start d_qk - 64 elements into the row: 896 / 1024 bytes, a multiple of 16
  if (!aligned16(r->k) || (r->stride_k & 7) || r->stride_k < d_qk) return DSV4_ERR_ALIGN;
  Dsv4StoreArgs a{};
  a.n_tokens = r->n_tokens; a.kv_format = r->kv_format;
  a.num_blocks = r->num_blocks; a.page_block_size = r->page_block_size;
  a.k_nope = r->k;
  a.k_rope = static_cast<const uint16_t*>(r->k) + (d_qk - 64);
  a.stride_nope = a.stride_rope = r->stride_k;
  a.kv = r->kv; a.stride_kv_block = r->stride_kv_block;
  a.slots = r->loc_is_int64 ? static_cast<const int64_t*>(r->loc) : nullptr;
  const int32_t* loc32 = r->loc_is_int64 ? nullptr : static_cast<const int32_t*>(r->loc);
  cudaError_t e = dsv4::launch_kv_store(a, loc32, static_cast<cudaStream_t>(stream));
  return e ? cuda_fail(e) : DSV4_OK;
}

int dsv4_gather_dequant(const void* kv, int64_t stride_kv_block, int32_t kv_format,
                        int32_t num_blocks, int32_t page_block_size, const int32_t* indices,
                        int32_t n, void* rows_bf16, int32_t method, void* stream) {
  if (!kv || !indices || !rows_bf16) return DSV4_ERR_NULL;
  if (n < 0 || num_blocks < 1) return DSV4_ERR_SHAPE;
  const int d_qk = kv_format == DSV4_KV_MODEL1 ? 512 : 576;
  int rc = check_paged(kv_format, d_qk, page_block_size, stride_kv_block, kv);
  if (rc) return rc;
  if (!aligned16(rows_bf16)) return DSV4_ERR_ALIGN;
  cudaError_t e = dsv4::launch_gather_dequant(kv, stride_kv_block, kv_format, num_blocks,
                                              page_block_size, indices, n, rows_bf16, method,
                                              static_cast<cudaStream_t>(stream));
  return e ? cuda_fail(e) : DSV4_OK;
}

int dsv4_debug_set_timeline(void* device_buffer) {
  g_timeline = static_cast<long long*>(device_buffer);
  return DSV4_OK;
}

int dsv4_device_status(int32_t* status_out, int reset) {
  if (!status_out) return DSV4_ERR_NULL;
  int v = 0;
  cudaError_t e = dsv4::read_attn_error(&v, reset != 0);
  if (e) return cuda_fail(e);
  *status_out = v;
  return DSV4_OK;
}

int dsv4_gather_heads(const Dsv4GatherArgs* a, void* stream) {
  if (!a || !a->out_local || !a->lse_local || !a->counter || !a->status) return DSV4_ERR_NULL;
  if (a->world < 1 || a->world > DSV4_MAX_PEERS || a->rank < 0 || a->rank >= a->world || a->b < 0 ||
      a->s_q < 1 || a->h_local < 1)
    return DSV4_ERR_SHAPE;
  for (int r = 0; r < a->world; ++r) {
    if (!a->peer_out[r] || !a->peer_lse[r] || !a->peer_flags[r]) return DSV4_ERR_NULL;
    if (!aligned16(a->peer_out[r])) return DSV4_ERR_ALIGN;
  }
  if (!aligned16(a->out_local)) return DSV4_ERR_ALIGN;
  cudaError_t e = dsv4::launch_gather_heads(*a, static_cast<cudaStream_t>(stream));
  return e ? cuda_fail(e) : DSV4_OK;
}

int dsv4_sparse_decode_gather(const Dsv4DecodeArgs* d, const Dsv4GatherArgs* g, void* stream) {
  if (!d || !g || !g->counter || !g->status || !d->out || !d->lse) return DSV4_ERR_NULL;
  if (g->world < 1 || g->world > DSV4_MAX_PEERS || g->rank < 0 || g->rank >= g->world ||
      g->b != d->b || g->s_q != d->s_q || g->h_local != d->h_q)
    return DSV4_ERR_SHAPE;
  for (int r = 0; r < g->world; ++r) {
    if (!g->peer_out[r] || !g->peer_lse[r] || !g->peer_flags[r]) return DSV4_ERR_NULL;
    if (!aligned16(g->peer_out[r])) return DSV4_ERR_ALIGN;
  }
  // the local result must be dense: it is what the exchange kernel reads
  if (d->stride_o_h != 512 || d->stride_o_s != static_cast<int64_t>(d->h_q) * 512 ||
      d->stride_o_b != static_cast<int64_t>(d->s_q) * d->h_q * 512 || d->stride_lse_s != 1 ||
      d->stride_lse_h != d->s_q || d->stride_lse_b != static_cast<int64_t>(d->h_q) * d->s_q)
    return DSV4_ERR_LAYOUT;
  // Decode (with its split combine, when the plan has one) and the exchange kernel behind it
  // with programmatic dependent launch: the exchange kernel is resident before the rows are
  // final.  A combine step that stored straight into the peers' buffers was measured 1-2 us
  // slower per step than this pair (more CTAs fencing at system scope, narrower NVLink
  // stores), so it was taken out again.
  int rc = dsv4_sparse_decode(d, stream);
  if (rc) return rc;
  Dsv4GatherArgs ga = *g;
  ga.out_local = d->out;
  ga.lse_local = d->lse;
  return dsv4_gather_heads(&ga, stream);
}

int dsv4_umma_selftest(int mode, int n, int k, const void* a, const void* b, float* d,
                       int32_t* status, void* stream) {
  if (!a || !b || !d || !status) return DSV4_ERR_NULL;
  if (mode < 0 || mode > 1 || n < 16 || n > 64 || (n & 15) || k < 64 || k > 256 || (k & 63))
    return DSV4_ERR_SHAPE;
  int rc = current_device_is_sm100();
  if (rc) return rc;
  cudaError_t e = dsv4::launch_umma_selftest(mode, n, k, a, b, d, status,
                                             static_cast<cudaStream_t>(stream));
  return e ? cuda_fail(e) : DSV4_OK;
}

}  // extern "C"
