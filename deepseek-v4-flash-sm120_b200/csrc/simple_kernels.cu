// Plain CUDA-core kernels: a straightforward attention kernel used as an
// on-device cross-check of the tensor-core path (DSV4_FLAG_IMPL_SIMPLE), the
// split-KV combine, the FP8 KV store/quantise kernel and the gather+dequantise
// probe.  One CTA of the attention kernel handles one (request, head, split).
#include "attn_params.cuh"
#include "launchers.h"

namespace dsv4 {

namespace {

constexpr int SIMPLE_THREADS = 128;
constexpr int SIMPLE_CHUNK = 128;

template <int FMT> struct RowReader {
  using T = KvTraits<FMT>;
  static constexpr int D_QK = T::D_QK;
  const uint8_t* row;
  const uint8_t* scales;
  __device__ float at(int d) const {
    if (d < T::D_NOPE) return dequant_plain(row[d], scales[d / T::TILE]);
    uint16_t h = *reinterpret_cast<const uint16_t*>(row + T::D_NOPE + 2 * (d - T::D_NOPE));
    return bf16_bits_to_f32(h);
  }
  __device__ void locate(const uint8_t* kv, int64_t stride, int page_block, int idx) {
    token_ptrs<FMT>(kv, stride, page_block, idx, row, scales);
  }
};

template <int DQK> struct RowReaderBf16 {
  static constexpr int D_QK = DQK;
  const uint8_t* row;
  const uint8_t* scales;
  __device__ float at(int d) const {
    return bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(row)[d]);
  }
  __device__ void locate(const uint8_t* kv, int64_t stride, int, int idx) {
    row = kv + static_cast<int64_t>(idx) * stride * 2;
    scales = nullptr;
  }
};

__device__ __forceinline__ float block_reduce(float v, bool is_max, float* red) {
  for (int o = 16; o > 0; o >>= 1) {
    float w = __shfl_xor_sync(0xffffffffu, v, o);
    v = is_max ? fmaxf(v, w) : v + w;
  }
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = red[0];
  for (int i = 1; i < SIMPLE_THREADS / 32; ++i) r = is_max ? fmaxf(r, red[i]) : r + red[i];
  return r;
}

template <class Reader>
__global__ void __launch_bounds__(SIMPLE_THREADS)
simple_attn_kernel(AttnParams p) {
  constexpr int DQK = Reader::D_QK;
  __shared__ float s_q[DQK];
  __shared__ float s_p[SIMPLE_CHUNK];
  __shared__ const uint8_t* s_row[SIMPLE_CHUNK];
  __shared__ const uint8_t* s_scl[SIMPLE_CHUNK];
  __shared__ float s_red[SIMPLE_THREADS / 32];

  const int req = blockIdx.x, h = blockIdx.y, split = blockIdx.z, tid = threadIdx.x;
  const bool decode = p.mode == MODE_DECODE;
  const bool mask_invalid = !decode || (p.flags & DSV4_FLAG_MASK_INVALID);

  const __nv_bfloat16* qrow = p.q + (req / p.s_q) * p.stride_q_b + (req % p.s_q) * p.stride_q_s +
                              h * p.stride_q_h;
  for (int d = tid; d < DQK; d += SIMPLE_THREADS) s_q[d] = __bfloat162float(qrow[d]);

  int len, xlen;
  request_lengths(p, req, len, xlen);
  int begin, end;
  split_range(len + xlen, p.n_splits, split, begin, end);
  const int32_t* idx_main = idx_row(p.indices, p.stride_idx_b, p.stride_idx_s, req, p.s_q);
  const int32_t* idx_extra = p.extra_kv
      ? idx_row(p.extra_indices, p.stride_xidx_b, p.stride_xidx_s, req, p.s_q) : nullptr;

  float m_run = -INFINITY, l_run = 0.f;
  float acc[D_V / SIMPLE_THREADS] = {0.f, 0.f, 0.f, 0.f};
  __syncthreads();

  for (int c0 = begin; c0 < end; c0 += SIMPLE_CHUNK) {
    const int j = c0 + tid;
    float logit = -INFINITY;
    const uint8_t* row = nullptr;
    const uint8_t* scl = nullptr;
    if (j < end) {
      const bool main_list = j < len;
      const int idx = main_list ? idx_main[j] : idx_extra[j - len];
      const int ntok = main_list ? p.n_tok : p.extra_n_tok;
      if (idx >= 0 && idx < ntok) {
        Reader r;
        r.locate(main_list ? p.kv : p.extra_kv, main_list ? p.stride_kv : p.stride_extra_kv,
                 main_list ? p.page_block : p.extra_page_block, idx);
        float dot = 0.f;
        for (int d = 0; d < DQK; ++d) dot = fmaf(s_q[d], r.at(d), dot);
        logit = dot * p.sm_scale;
        row = r.row;
        scl = r.scales;
      } else if (!mask_invalid) {
        logit = 0.f;    // zero row: scores 0, contributes V = 0
      }
    }
    float m_new = fmaxf(m_run, block_reduce(logit, true, s_red));
    float pj = (logit == -INFINITY) ? 0.f : expf(logit - m_new);
    float corr = (m_run == -INFINITY) ? 0.f : expf(m_run - m_new);
    float l_chunk = block_reduce(pj, false, s_red);
    l_run = l_run * corr + l_chunk;
    m_run = m_new;
    __syncthreads();
    s_p[tid] = pj;
    s_row[tid] = row;
    s_scl[tid] = scl;
    __syncthreads();
#pragma unroll
    for (int i = 0; i < D_V / SIMPLE_THREADS; ++i) acc[i] *= corr;
    const int n = min(SIMPLE_CHUNK, end - c0);
    for (int t = 0; t < n; ++t) {
      if (s_row[t] == nullptr || s_p[t] == 0.f) continue;
      Reader r;
      r.row = s_row[t];
      r.scales = s_scl[t];
      const float pt = s_p[t];
#pragma unroll
      for (int i = 0; i < D_V / SIMPLE_THREADS; ++i)
        acc[i] = fmaf(pt, r.at(tid + i * SIMPLE_THREADS), acc[i]);
    }
  }

  if (p.n_splits > 1) {
    const int64_t slot = (static_cast<int64_t>(split) * p.n_req + req) * p.h_q + h;
    const bool empty = (l_run == 0.f);
    if (tid == 0) p.lse_accum[slot] = empty ? -INFINITY : logf(l_run) + m_run;
    const float inv = empty ? 0.f : 1.f / l_run;
#pragma unroll
    for (int i = 0; i < D_V / SIMPLE_THREADS; ++i)
      p.o_accum[slot * D_V + tid + i * SIMPLE_THREADS] = acc[i] * inv;
    return;
  }
  const bool has_sink = p.sink != nullptr;
  float lse_v, ml_v;
  const float f = finalize_row(p.mode, m_run, l_run, has_sink, has_sink ? p.sink[h] : 0.f, lse_v,
                               ml_v);
  const int bi = req / p.s_q, si = req % p.s_q;
  if (tid == 0) {
    p.lse[bi * p.stride_lse_b + si * p.stride_lse_s + h * p.stride_lse_h] = lse_v;
    if (p.max_logits) p.max_logits[bi * p.stride_ml_b + h] = ml_v;
  }
  __nv_bfloat16* orow = p.out + bi * p.stride_o_b + si * p.stride_o_s + h * p.stride_o_h;
#pragma unroll
  for (int i = 0; i < D_V / SIMPLE_THREADS; ++i)
    orow[tid + i * SIMPLE_THREADS] = __float2bfloat16_rn(acc[i] * f);
}

// ---------------------------------------------------------------------------
// Split-KV combine.  One CTA per (row, group of 8 heads); a warp owns one head:
// it reads the head's n_splits lse values once, forms the weights in registers
// (splits strided over lanes) and then streams the partial rows with 16-byte
// loads, each lane owning 16 output columns.
// ---------------------------------------------------------------------------
constexpr int COMBINE_WARPS = 8;
constexpr int COMBINE_MAX_SPLITS = 256;
constexpr int COMBINE_BATCH = 16;         // partial rows in flight per thread

// Warp (row, head, part) merges columns [part, part + 1) * 32 * VEC of the n_splits partial
// rows: every lane owns VEC consecutive floats per split and keeps COMBINE_BATCH loads in
// flight.  VEC = 4 (four warps per head) when there are many (row, head) pairs, VEC = 1
// (sixteen warps per head) when there are few, so that the grid still fills the GPU.
template <int VEC>
__global__ void __launch_bounds__(COMBINE_WARPS * 32)
combine_kernel(Dsv4CombineArgs a) {
  constexpr int PARTS = D_V / (32 * VEC);
  __shared__ float s_w[COMBINE_WARPS][COMBINE_MAX_SPLITS];
  grid_dependency_wait();                 // the partials come from the kernel just before
  const int row = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int unit = blockIdx.y * COMBINE_WARPS + warp;
  const int h = unit / PARTS, part = unit % PARTS;
  if (h >= a.h_q) return;
  const int64_t rows_h = static_cast<int64_t>(a.n_rows) * a.h_q;
  const int64_t slot0 = static_cast<int64_t>(row) * a.h_q + h;

  float m = -INFINITY;
  for (int s = lane; s < a.n_splits; s += 32) m = fmaxf(m, a.lse_accum[s * rows_h + slot0]);
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  float l = 0.f;
  for (int s = lane; s < a.n_splits; s += 32) {
    float v = a.lse_accum[s * rows_h + slot0];
    float w = (v == -INFINITY) ? 0.f : expf(v - m);
    s_w[warp][s] = w;
    l += w;
  }
  for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
  __syncwarp();

  const bool has_sink = a.attn_sink != nullptr;
  float lse_v, ml_v;
  const float f = finalize_row(MODE_DECODE, m, l, has_sink, has_sink ? a.attn_sink[h] : 0.f,
                               lse_v, ml_v);
  const int bi = row / a.s_q, si = row % a.s_q;
  if (lane == 0 && part == 0)
    a.lse[bi * a.stride_lse_b + si * a.stride_lse_s + h * a.stride_lse_h] = lse_v;

  float acc[VEC];
#pragma unroll
  for (int j = 0; j < VEC; ++j) acc[j] = 0.f;
  const int col = (part * 32 + lane) * VEC;
  const float* src = a.o_accum + slot0 * D_V + col;
  const int64_t split_stride = rows_h * D_V;
  for (int s0 = 0; s0 < a.n_splits; s0 += COMBINE_BATCH) {
    float v[COMBINE_BATCH][VEC];
    float w[COMBINE_BATCH];
#pragma unroll
    for (int k = 0; k < COMBINE_BATCH; ++k) {
      const int s = s0 + k;
      w[k] = s < a.n_splits ? s_w[warp][s] : 0.f;
#pragma unroll
      for (int j = 0; j < VEC; ++j) v[k][j] = 0.f;
      if (w[k] != 0.f) {
        if constexpr (VEC == 4) {
          const float4 t = __ldg(reinterpret_cast<const float4*>(src + s * split_stride));
          v[k][0] = t.x; v[k][1] = t.y; v[k][2] = t.z; v[k][3] = t.w;
        } else {
          v[k][0] = __ldg(src + s * split_stride);
        }
      }
    }
#pragma unroll
    for (int k = 0; k < COMBINE_BATCH; ++k) {       // fixed order: the result does not depend on timing
#pragma unroll
      for (int j = 0; j < VEC; ++j) acc[j] = fmaf(w[k], v[k][j], acc[j]);
    }
  }
  __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(a.out) + bi * a.stride_o_b +
                        si * a.stride_o_s + h * a.stride_o_h + col;
  if constexpr (VEC == 4) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(acc[0] * f, acc[1] * f);
    __nv_bfloat162 hi = __floats2bfloat162_rn(acc[2] * f, acc[3] * f);
    *reinterpret_cast<uint2*>(orow) =
        make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
  } else {
    *orow = __float2bfloat16_rn(acc[0] * f);
  }
}

// ---------------------------------------------------------------------------
// KV store / quantise.  HBM-bound: per token d_nope * 2 + 128 bytes in, 644 / 584 bytes out.
// A warp handles STORE_TOKENS tokens at a time: lane l owns 16 consecutive latent values of
// each, and all of the warp's loads (two 16-byte loads per lane and token, plus the RoPE
// rows) are in flight before the first value is looked at.  Tile amax by shuffles, e4m3 by
// the hardware saturating convert.
// ---------------------------------------------------------------------------
constexpr int STORE_TOKENS = 4;          // tokens in flight per warp
constexpr int STORE_WARPS = 8;

template <int FMT>
__global__ void __launch_bounds__(STORE_WARPS * 32)
kv_store_kernel(Dsv4StoreArgs a, const int32_t* slots32) {
  using T = KvTraits<FMT>;
  constexpr int PER_LANE = 16;                      // 32 lanes x 16 = 512 >= D_NOPE
  constexpr int LANES_PER_TILE = T::TILE / PER_LANE;
  grid_dependency_wait();                           // the rows may come from the kernel before
  const int lane = threadIdx.x & 31;
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int tok0 = warp * STORE_TOKENS;
  const bool active = lane * PER_LANE < T::D_NOPE;
  const int64_t n_slots = static_cast<int64_t>(a.num_blocks) * a.page_block_size;

  int64_t slot[STORE_TOKENS];
  uint4 v[STORE_TOKENS][2], rope[STORE_TOKENS];
#pragma unroll
  for (int k = 0; k < STORE_TOKENS; ++k) {
    const int tok = tok0 + k;
    slot[k] = tok >= a.n_tokens ? -1 : slots32 ? static_cast<int64_t>(slots32[tok]) : a.slots[tok];
    v[k][0] = v[k][1] = rope[k] = make_uint4(0, 0, 0, 0);
  }
#pragma unroll
  for (int k = 0; k < STORE_TOKENS; ++k) {
    if (slot[k] < 0 || slot[k] >= n_slots) continue;
    const int tok = tok0 + k;
    if (active) {
      const uint4* src = reinterpret_cast<const uint4*>(
          reinterpret_cast<const __nv_bfloat16*>(a.k_nope) + static_cast<int64_t>(tok) * a.stride_nope +
          lane * PER_LANE);
      v[k][0] = __ldg(src);
      v[k][1] = __ldg(src + 1);
    }
    if (lane < 8)   // RoPE: 64 BF16 = 128 B = 8 x 16 B
      rope[k] = __ldg(reinterpret_cast<const uint4*>(
                          reinterpret_cast<const __nv_bfloat16*>(a.k_rope) +
                          static_cast<int64_t>(tok) * a.stride_rope) + lane);
  }
#pragma unroll
  for (int k = 0; k < STORE_TOKENS; ++k) {
    if (slot[k] < 0 || slot[k] >= n_slots) continue;         // warp-uniform
    const int page = static_cast<int>(slot[k] / a.page_block_size);
    const int r = static_cast<int>(slot[k] - static_cast<int64_t>(page) * a.page_block_size);
    uint8_t* base = reinterpret_cast<uint8_t*>(a.kv) + static_cast<int64_t>(page) * a.stride_kv_block;
    uint8_t* row = base + static_cast<int64_t>(r) * T::ROW_BYTES;
    uint8_t* scl = base + static_cast<int64_t>(a.page_block_size) * T::ROW_BYTES + r * T::SLOTS;
    const uint32_t w[8] = {v[k][0].x, v[k][0].y, v[k][0].z, v[k][0].w,
                           v[k][1].x, v[k][1].y, v[k][1].z, v[k][1].w};
    float x[PER_LANE];
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      x[2 * i] = __uint_as_float(w[i] << 16);
      x[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
      amax = fmaxf(amax, fmaxf(fabsf(x[2 * i]), fabsf(x[2 * i + 1])));
    }
#pragma unroll
    for (int o = 1; o < LANES_PER_TILE; o <<= 1)
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    // e = ceil(log2(max(amax, 1e-4) / 448)) from the fp32 exponent field.
    const float rr = fmaxf(amax, 1e-4f) / 448.0f;
    const uint32_t rb = __float_as_uint(rr);
    const int e = static_cast<int>(rb >> 23) - 127 + ((rb & 0x7fffffu) ? 1 : 0);
    const float inv = __uint_as_float(static_cast<uint32_t>(127 - e) << 23);   // 2^-e, |e| small
    if (active) {
      uint32_t packed[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint16_t a01 = __nv_cvt_float2_to_fp8x2(make_float2(x[4 * i] * inv, x[4 * i + 1] * inv),
                                                      __NV_SATFINITE, __NV_E4M3);
        const uint16_t a23 = __nv_cvt_float2_to_fp8x2(make_float2(x[4 * i + 2] * inv, x[4 * i + 3] * inv),
                                                      __NV_SATFINITE, __NV_E4M3);
        packed[i] = static_cast<uint32_t>(a01) | (static_cast<uint32_t>(a23) << 16);
      }
      *reinterpret_cast<uint4*>(row + lane * PER_LANE) =
          make_uint4(packed[0], packed[1], packed[2], packed[3]);
      if (lane % LANES_PER_TILE == 0) scl[lane / LANES_PER_TILE] = static_cast<uint8_t>(e + 127);
    }
    if (lane >= 32 - (T::SLOTS - T::N_SCALE) && T::SLOTS > T::N_SCALE)
      scl[T::N_SCALE + (31 - lane)] = 0;
    if (lane < 8) *reinterpret_cast<uint4*>(row + T::D_NOPE + lane * 16) = rope[k];
  }
}

// ---------------------------------------------------------------------------
// Gather + dequantise probe: one warp per index, 16 FP8 bytes per lane through
// the same routines the tensor-core kernel uses.
// ---------------------------------------------------------------------------
template <int FMT>
__global__ void __launch_bounds__(256)
gather_dequant_kernel(const uint8_t* kv, int64_t stride, int page_block, int n_tok,
                      const int32_t* indices, int n, __nv_bfloat16* rows, int method) {
  using T = KvTraits<FMT>;
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= n) return;
  const int idx = indices[warp];
  uint4* dst = reinterpret_cast<uint4*>(rows + static_cast<int64_t>(warp) * T::D_QK);
  if (idx < 0 || idx >= n_tok) {
    for (int c = lane; c < T::D_QK / 8; c += 32) dst[c] = make_uint4(0, 0, 0, 0);
    return;
  }
  const uint8_t *row, *scl;
  token_ptrs<FMT>(kv, stride, page_block, idx, row, scl);
  if (lane * 16 < T::D_NOPE) {
    const uint4 raw = *reinterpret_cast<const uint4*>(row + lane * 16);
    const uint32_t s = scl[lane * 16 / T::TILE];
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    uint32_t o[8];
    const ScalePair mul = scale_pair(s);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (method == 0) dequant4(w[i], mul, mul.c2 != BF16X2_ONE, o[2 * i], o[2 * i + 1]);
      else dequant4_f32(w[i], s, o[2 * i], o[2 * i + 1]);
    }
    dst[lane * 2] = make_uint4(o[0], o[1], o[2], o[3]);
    dst[lane * 2 + 1] = make_uint4(o[4], o[5], o[6], o[7]);
  }
  if (lane < 8) dst[T::D_NOPE / 8 + lane] = *reinterpret_cast<const uint4*>(row + T::D_NOPE + lane * 16);
}

}  // namespace

cudaError_t launch_simple_attn(const AttnParams& p, int kv_format, int d_qk, cudaStream_t st) {
  dim3 grid(p.n_req, p.h_q, p.n_splits), block(SIMPLE_THREADS);
  if (kv_format == DSV4_KV_MODEL1)
    simple_attn_kernel<RowReader<DSV4_KV_MODEL1>><<<grid, block, 0, st>>>(p);
  else if (kv_format == DSV4_KV_V32)
    simple_attn_kernel<RowReader<DSV4_KV_V32>><<<grid, block, 0, st>>>(p);
  else if (d_qk == 512)
    simple_attn_kernel<RowReaderBf16<512>><<<grid, block, 0, st>>>(p);
  else
    simple_attn_kernel<RowReaderBf16<576>><<<grid, block, 0, st>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_combine(const Dsv4CombineArgs& a, cudaStream_t st) {
  // Four warps per (row, head) give n_rows * h_q / 2 CTAs; below about two CTAs per SM
  // (B200: 148 SMs) sixteen warps per (row, head) are used instead.
  const bool fine = static_cast<int64_t>(a.n_rows) * a.h_q < 600;
  const int parts = fine ? 16 : 4;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(a.n_rows, (a.h_q * parts + COMBINE_WARPS - 1) / COMBINE_WARPS);
  cfg.blockDim = dim3(COMBINE_WARPS * 32);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  cfg.attrs = attr;
  cfg.numAttrs = add_overlap_attribute(attr);
  return fine ? cudaLaunchKernelEx(&cfg, combine_kernel<1>, a)
              : cudaLaunchKernelEx(&cfg, combine_kernel<4>, a);
}

int combine_max_splits() { return COMBINE_MAX_SPLITS; }

cudaError_t launch_kv_store(const Dsv4StoreArgs& a, const int32_t* slots32, cudaStream_t st) {
  if (a.n_tokens <= 0) return cudaSuccess;
  constexpr int PER_BLOCK = STORE_WARPS * STORE_TOKENS;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((a.n_tokens + PER_BLOCK - 1) / PER_BLOCK);
  cfg.blockDim = dim3(STORE_WARPS * 32);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  cfg.attrs = attr;
  cfg.numAttrs = add_overlap_attribute(attr);
  return a.kv_format == DSV4_KV_MODEL1
             ? cudaLaunchKernelEx(&cfg, kv_store_kernel<DSV4_KV_MODEL1>, a, slots32)
             : cudaLaunchKernelEx(&cfg, kv_store_kernel<DSV4_KV_V32>, a, slots32);
}

cudaError_t launch_gather_dequant(const void* kv, int64_t stride, int kv_format, int num_blocks,
                                  int page_block, const int32_t* indices, int n, void* rows,
                                  int method, cudaStream_t st) {
  if (n <= 0) return cudaSuccess;
  const int blocks = (n + 7) / 8;
  const uint8_t* k = static_cast<const uint8_t*>(kv);
  __nv_bfloat16* r = static_cast<__nv_bfloat16*>(rows);
  if (kv_format == DSV4_KV_MODEL1)
    gather_dequant_kernel<DSV4_KV_MODEL1><<<blocks, 256, 0, st>>>(k, stride, page_block,
        num_blocks * page_block, indices, n, r, method);
  else
    gather_dequant_kernel<DSV4_KV_V32><<<blocks, 256, 0, st>>>(k, stride, page_block,
        num_blocks * page_block, indices, n, r, method);
  return cudaGetLastError();
}

}  // namespace dsv4
