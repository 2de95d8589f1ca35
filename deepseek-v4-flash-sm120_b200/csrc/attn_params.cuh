// Kernel-side parameter block shared by the decode and prefill kernels, and
// the request/split bookkeeping both implementations must agree on.
#pragma once

#include "dsv4_common.cuh"

namespace dsv4 {

// Programmatic dependent launch (see add_overlap_attribute): block until the kernel before
// this one in the stream has completed and its writes are visible / allow the kernel after
// this one to be set up.  Both are no-ops when the launch carries no such dependency.
__device__ __forceinline__ void grid_dependency_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void grid_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

enum AttnMode : int { MODE_DECODE = 0, MODE_PREFILL = 1 };

constexpr int SPLIT_GRANULE = 16;    // split ranges are multiples of 16 list entries

struct AttnParams {
  int n_req;          // decode: b * s_q ; prefill: s_q
  int s_q;            // decode: query tokens per request ; prefill: 1
  int h_q, topk, extra_topk, n_splits, flags, mode;
  int cluster;        // splits merged on chip per thread-block cluster (1, 2 or 4; divides n_splits)
  int page_block, n_tok;              // main cache: tokens per page, total tokens (s_kv)
  int extra_page_block, extra_n_tok;
  int page_shift, extra_page_shift;   // log2 of the page size, or -1 when it is not a power of two
  float sm_scale;

  const __nv_bfloat16* q;
  const uint8_t* kv;                  // paged bytes, or BF16 rows for DSV4_KV_BF16
  const uint8_t* extra_kv;
  const int32_t* indices;
  const int32_t* extra_indices;
  const int32_t* topk_length;         // per batch entry (decode) / per query (prefill)
  const int32_t* extra_topk_length;
  const float* sink;

  __nv_bfloat16* out;
  float* lse;
  float* max_logits;                  // prefill only
  float* o_accum;                     // [n_splits, n_req, h_q, 512]
  float* lse_accum;                   // [n_splits, n_req, h_q]

  int64_t stride_q_b, stride_q_s, stride_q_h;
  int64_t stride_kv, stride_extra_kv;           // bytes per page, or elements per BF16 row
  int64_t stride_idx_b, stride_idx_s, stride_xidx_b, stride_xidx_s;
  int64_t stride_o_b, stride_o_s, stride_o_h;
  int64_t stride_lse_b, stride_lse_s, stride_lse_h;
  int64_t stride_ml_b;                          // max_logits row stride (prefill)
  long long* prof;                              // optional timeline buffer (debug), or null
};

// Effective list lengths of request `req`: `len` entries of the main list then
// `xlen` of the extra list.  Decode raises a length below one to one, as the
// reference oracle does (tests/reference.py:108-109), unless
// DSV4_FLAG_ZERO_LENGTH_EMPTY asks for the reference kernel's clamp at zero; prefill
// clamps at zero.
__device__ __forceinline__ void request_lengths(const AttnParams& p, int req, int& len, int& xlen) {
  int bi = req / p.s_q;
  len = p.topk;
  if (p.topk_length) len = min(len, p.topk_length[bi]);
  len = max(len, (p.mode == MODE_DECODE && !(p.flags & DSV4_FLAG_ZERO_LENGTH_EMPTY)) ? 1 : 0);
  xlen = 0;
  if (p.extra_kv) {
    xlen = p.extra_topk;
    if (p.extra_topk_length) xlen = min(xlen, p.extra_topk_length[bi]);
    xlen = max(xlen, 0);
  }
}

// Range [begin, end) of the concatenated list handled by `split`.
__device__ __forceinline__ void split_range(int total, int n_splits, int split, int& begin,
                                            int& end) {
  if (n_splits <= 1) { begin = 0; end = total; return; }
  int per = (total + n_splits - 1) / n_splits;
  per = (per + SPLIT_GRANULE - 1) / SPLIT_GRANULE * SPLIT_GRANULE;
  begin = min(split * per, total);
  end = min(begin + per, total);
}

__device__ __forceinline__ const int32_t* idx_row(const int32_t* base, int64_t sb, int64_t ss,
                                                  int req, int s_q) {
  return base + (req / s_q) * sb + (req % s_q) * ss;
}

// Final (o, lse) fix-up shared by the non-split epilogue and the combine step.
// l is the softmax denominator relative to m.  Returns the factor that turns the
// un-normalised accumulator into the output and sets lse_out (and ml_out).
__device__ __forceinline__ float finalize_row(int mode, float m, float l, bool has_sink,
                                              float sink, float& lse_out, float& ml_out) {
  if (l == 0.0f || m == -INFINITY) {
    if (mode == MODE_PREFILL) { lse_out = INFINITY; ml_out = -INFINITY; }
    else { lse_out = has_sink ? sink : -INFINITY; ml_out = -INFINITY; }
    return 0.0f;
  }
  float log_sum = logf(l) + m;
  ml_out = m;
  float f = 1.0f / l;
  if (has_sink) f *= 1.0f / (1.0f + expf(sink - log_sum));
  if (mode == MODE_PREFILL || !has_sink) {
    lse_out = log_sum;
  } else {
    float mm = fmaxf(log_sum, sink);
    lse_out = mm + logf(expf(log_sum - mm) + expf(sink - mm));
  }
  return f;
}

}  // namespace dsv4
