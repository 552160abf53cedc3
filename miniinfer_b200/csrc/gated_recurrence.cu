// Recurrences whose state is one float32 per channel, S_t = a_t * S_(t-1) + b_t with a_t and b_t made from the
// token's own projections, and two small kernels for blocks that feed a sublayer from the residual stream itself:
//
//   token_shift         h[t] = x[t] + (x[t - 1] - x[t]) * shift, x[t - 1] of a request's first new token coming from the
//                       request's state (zeros at its start); without `shift` a plain copy into the compute type.
//   norm_scaled_add     x[t] <- x[t] + mult * w * y[t] / sqrt(mean(y[t]^2) + eps): the RMS norm of a sublayer's OUTPUT added
//                       to the residual stream, which may also be copied out in the compute type (the next sublayer's
//                       input) and whose old row, for the last new token of each request, may be kept as that request's
//                       token-shift state.
//   rglru_recurrence    the real-gated linear recurrent unit: r = sigmoid(r_logit + rb), i = sigmoid(i_logit + ib),
//                       log a = -8 r softplus(lam), S <- a S + sqrt(1 - a^2) i u, out = S * gelu_tanh(y + yb).
//   mingru_recurrence   z = sigmoid(z_logit + zb), S <- (1 - z) S + z c with c = x + 1/2 for x >= 0 and sigmoid(x) below,
//                       out = S * silu(g).
//
// A step brings, for each of its items, q_len[b] new tokens in rows q_start[b] .. of the activations; the item's state
// lives in row seq_slot[b] of the layer's state tensor, float32, zero when the request was admitted.  Everything behind
// the projections is float32: sigmoids, softplus, logarithms of the decays and their exponentials, sqrt(1 - a^2) (as
// -expm1(2 log a), which keeps its digits when a is near 1), the state.  Activations are read and written in the storage
// type.
//
// The recurrences walk an item's tokens in order.  In the flat form a thread owns a channel and walks all of the
// item's new tokens: results are bit-equal however the request was cut.  In the segmented form (long bfloat16 portions)
// the NW warps of a block share 32 channels and take a stretch of tokens each: every stretch first from a zero state,
// keeping the product of its decays and its end state; the stretches are chained through shared memory (S_end = A S_start
// + B, the map of a stretch being one multiply-add a channel); then every stretch again from its true start state,
// writing the outputs.  What a token gives a channel - decay, input, read-out factor, with their exponentials, logarithms
// and roots - is then made once, by a kernel of its own that runs over all tokens and channels at once and fills the
// GPU, and the two walks are a load and a multiply-add a token.
#include "common.cuh"

namespace {

__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float gelu_tanh_f(float z) {
  return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// ------------------------------------------------------------------------------------------------------------

// Four neighbouring values at a time where the rows allow it (a width that is a multiple of 4, 16-byte aligned rows).
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  return make_float4(lo.x, lo.y, hi.x, hi.y);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  uint2 raw;
  raw.x = *reinterpret_cast<const uint32_t*>(&lo);
  raw.y = *reinterpret_cast<const uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = raw;
}

template <typename TOut>
__global__ void __launch_bounds__(256)
token_shift_vec_kernel(TOut* __restrict__ out, const float* __restrict__ x, int W, const float* __restrict__ shift,
                       const float* __restrict__ state, long long state_stride, const int* __restrict__ token_item,
                       const int* __restrict__ q_start, const int* __restrict__ seq_slot) {
  const int t = blockIdx.x;
  const int item = token_item[t];
  const bool first = t == q_start[item];
  const int slot = seq_slot[item];
  mi::grid_dependency_sync();
  const float* row = x + (size_t)t * W;
  const float* before = shift ? (first ? state + (size_t)slot * state_stride : row - W) : nullptr;
  TOut* o = out + (size_t)t * W;
  for (int c = 4 * threadIdx.x; c < W; c += 4 * blockDim.x) {
    float4 v = load4(row + c);
    if (shift) {
      const float4 p = load4(before + c), s = load4(shift + c);
      v.x = fmaf(p.x - v.x, s.x, v.x); v.y = fmaf(p.y - v.y, s.y, v.y);
      v.z = fmaf(p.z - v.z, s.z, v.z); v.w = fmaf(p.w - v.w, s.w, v.w);
    }
    store4(o + c, v);
  }
}

// The same arithmetic as norm_scaled_add_kernel, value for value and sum for sum in another order of the additions only.
template <typename TY, typename TCopy>
__global__ void __launch_bounds__(256)
norm_scaled_add_vec_kernel(float* __restrict__ resid, const TY* __restrict__ y, const float* __restrict__ w, int W, float eps, float mult,
                           TCopy* __restrict__ copy, float* __restrict__ keep, long long keep_stride, const int* __restrict__ token_item,
                           const int* __restrict__ q_start, const int* __restrict__ q_len, const int* __restrict__ seq_slot) {
  __shared__ float scratch[33];
  const int t = blockIdx.x;
  float* kept = nullptr;
  if (keep) {
    const int item = token_item[t];
    if (t == q_start[item] + q_len[item] - 1) kept = keep + (size_t)seq_slot[item] * keep_stride;
  }
  mi::grid_dependency_sync();
  const TY* yr = y + (size_t)t * W;
  float ss = 0.f;
  for (int c = 4 * threadIdx.x; c < W; c += 4 * blockDim.x) {
    const float4 v = load4(yr + c);
    ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
  }
  const float rstd = rsqrtf(mi::block_sum(ss, scratch) / (float)W + eps);
  float* xr = resid + (size_t)t * W;
  for (int c = 4 * threadIdx.x; c < W; c += 4 * blockDim.x) {
    const float4 old = load4(xr + c), v = load4(yr + c), ww = load4(w + c);
    if (kept) store4(kept + c, old);
    float4 n;
    n.x = fmaf(mult, ww.x * (v.x * rstd), old.x); n.y = fmaf(mult, ww.y * (v.y * rstd), old.y);
    n.z = fmaf(mult, ww.z * (v.z * rstd), old.z); n.w = fmaf(mult, ww.w * (v.w * rstd), old.w);
    store4(xr + c, n);
    if (copy) store4(copy + (size_t)t * W + c, n);
  }
}

template <typename TOut>
__global__ void __launch_bounds__(256)
token_shift_kernel(TOut* __restrict__ out, const float* __restrict__ x, int W, const float* __restrict__ shift,
                   const float* __restrict__ state, long long state_stride, const int* __restrict__ token_item,
                   const int* __restrict__ q_start, const int* __restrict__ seq_slot) {
  const int t = blockIdx.x;
  const int item = token_item[t];
  const bool first = t == q_start[item];
  const int slot = seq_slot[item];
  mi::grid_dependency_sync();
  const float* row = x + (size_t)t * W;
  const float* before = shift ? (first ? state + (size_t)slot * state_stride : row - W) : nullptr;
  TOut* o = out + (size_t)t * W;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float v = row[c];
    if (shift) v = fmaf(before[c] - v, shift[c], v);
    o[c] = mi::from_float<TOut>(v);
  }
}

template <typename TY, typename TCopy>
__global__ void __launch_bounds__(256)
norm_scaled_add_kernel(float* __restrict__ resid, const TY* __restrict__ y, const float* __restrict__ w, int W, float eps, float mult,
                       TCopy* __restrict__ copy, float* __restrict__ keep, long long keep_stride, const int* __restrict__ token_item,
                       const int* __restrict__ q_start, const int* __restrict__ q_len, const int* __restrict__ seq_slot) {
  __shared__ float scratch[33];
  const int t = blockIdx.x;
  float* kept = nullptr;
  if (keep) {      // the step's description is written by no kernel: read before the wait
    const int item = token_item[t];
    if (t == q_start[item] + q_len[item] - 1) kept = keep + (size_t)seq_slot[item] * keep_stride;
  }
  mi::grid_dependency_sync();
  const TY* yr = y + (size_t)t * W;
  float ss = 0.f;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    const float v = mi::to_float(yr[c]);
    ss = fmaf(v, v, ss);
  }
  const float rstd = rsqrtf(mi::block_sum(ss, scratch) / (float)W + eps);
  float* xr = resid + (size_t)t * W;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    const float old = xr[c];
    if (kept) kept[c] = old;
    const float v = fmaf(mult, w[c] * (mi::to_float(yr[c]) * rstd), old);
    xr[c] = v;
    if (copy) copy[(size_t)t * W + c] = mi::from_float<TCopy>(v);
  }
}

// ------------------------------------------------------------------------------------------------------------
// The cells: what a token gives a channel - the decay a, the input b, and the factor g on the read-out.

template <typename T>
struct RglruCell {
  const T* u; int ldu;              // the convolved x branch [tokens, C]
  const float* gates; int ldg;      // a part's r logits, then its i logits: part b of token t at t * ldg + b * part_stride
  long long part_stride;            // 2 * bw for [tokens, parts, 2 bw]; tokens * 2 bw (with ldg = 2 bw) for [parts, tokens, 2 bw]
  const T* y; int ldy;              // the y branch as projected [tokens, C]
  const float *r_bias, *i_bias, *y_bias, *lam;
  int bw;
  // per channel, set by prepare()
  float rb, ib, yb, rate; long long goff;
  __device__ __forceinline__ void prepare(int c) {
    rb = r_bias[c]; ib = i_bias[c]; yb = y_bias ? y_bias[c] : 0.f;
    rate = -8.f * softplus_f(lam[c]);
    goff = (long long)(c / bw) * part_stride + c % bw;
  }
  __device__ __forceinline__ void ab(int row, int c, float& a, float& b) const {
    const float* g = gates + (size_t)row * ldg + goff;
    const float log_a = rate * sigmoid_f(g[0] + rb);
    a = expf(log_a);
    b = sqrtf(-expm1f(2.f * log_a)) * sigmoid_f(g[bw] + ib) * mi::to_float(u[(size_t)row * ldu + c]);
  }
  __device__ __forceinline__ float read_gate(int row, int c) const { return gelu_tanh_f(mi::to_float(y[(size_t)row * ldy + c]) + yb); }
};

template <typename T>
struct MingruCell {
  const T* proj; int ld;            // [tokens, 3 C]: z logits, x, g
  int C;
  const float *z_bias, *x_bias;
  float zb, xb;
  __device__ __forceinline__ void prepare(int c) { zb = z_bias ? z_bias[c] : 0.f; xb = x_bias ? x_bias[c] : 0.f; }
  __device__ __forceinline__ void ab(int row, int c, float& a, float& b) const {
    const T* p = proj + (size_t)row * ld + c;
    const float zl = mi::to_float(p[0]) + zb, x = mi::to_float(p[C]) + xb;
    a = sigmoid_f(-zl);                                  // 1 - z, with its own digits when z is near 1
    b = sigmoid_f(zl) * (x >= 0.f ? x + 0.5f : sigmoid_f(x));
  }
  __device__ __forceinline__ float read_gate(int row, int c) const {
    const float g = mi::to_float(proj[(size_t)row * ld + 2 * C + c]);
    return g / (1.f + expf(-g));
  }
};

// What a prepare kernel left: decays and inputs in float32, the read-out factor in the storage type, [tokens, C] each.
template <typename T>
struct PreparedCell {
  const float* a; const float* b; const T* g;
  int C;
  __device__ __forceinline__ void prepare(int) {}
  __device__ __forceinline__ void ab(int row, int c, float& a_, float& b_) const {
    a_ = a[(size_t)row * C + c];
    b_ = b[(size_t)row * C + c];
  }
  __device__ __forceinline__ float read_gate(int row, int c) const { return mi::to_float(g[(size_t)row * C + c]); }
};

constexpr int PREP_ROWS = 16;      // tokens a thread of the prepare kernel takes: what it keeps of its channel's weights serves them all

template <typename T, typename Cell>
__global__ void __launch_bounds__(128)
diag_prepare_kernel(Cell cell, float* __restrict__ a, float* __restrict__ b, T* __restrict__ g, int C, int rows) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int r0 = blockIdx.y * PREP_ROWS;
  if (c < C) cell.prepare(c);
  mi::grid_dependency_sync();
  if (c >= C) return;
#pragma unroll 4
  for (int r = r0; r < min(rows, r0 + PREP_ROWS); ++r) {
    float av, bv;
    cell.ab(r, c, av, bv);
    a[(size_t)r * C + c] = av;
    b[(size_t)r * C + c] = bv;
    g[(size_t)r * C + c] = mi::from_float<T>(cell.read_gate(r, c));
  }
}

template <typename T, typename Cell, int NW, bool SEG>
__global__ void __launch_bounds__(32 * NW)
diag_recurrence_kernel(Cell cell, T* __restrict__ out, int ldo, float* __restrict__ state, long long state_stride,
                       const int* __restrict__ q_start, const int* __restrict__ q_len, const int* __restrict__ seq_slot,
                       int C, int seg_min) {
  __shared__ float smA[SEG ? NW : 1][32], smB[SEG ? NW : 1][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int item = blockIdx.y;
  const int c = SEG ? blockIdx.x * 32 + lane : (blockIdx.x * NW + warp) * 32 + lane;
  const int n = q_len[item], row0 = q_start[item], slot = seq_slot[item];
  const bool active = c < C;
  if (active) cell.prepare(c);          // weights: fetched before the wait
  mi::grid_dependency_sync();
  const int nseg = (SEG && n >= seg_min * NW) ? NW : 1;          // the same for the whole block
  const int L = (n + nseg - 1) / nseg;
  const int t0 = SEG ? warp * L : 0, t1 = SEG ? min(n, t0 + L) : n;
  if (SEG && nseg > 1) {
    float A = 1.f, Bv = 0.f;
    if (active) {
#pragma unroll 4
      for (int t = t0; t < t1; ++t) {
        float a, b;
        cell.ab(row0 + t, c, a, b);
        A *= a;
        Bv = fmaf(a, Bv, b);
      }
    }
    smA[warp][lane] = A;
    smB[warp][lane] = Bv;
    __syncthreads();
  } else if (SEG && warp > 0) {
    return;
  }
  if (!active) return;
  float* st = state + (size_t)slot * state_stride + c;
  float S = *st;
  if (SEG && nseg > 1)
    for (int w = 0; w < warp; ++w) S = fmaf(smA[w][lane], S, smB[w][lane]);
  // eight tokens at a time: what they give the channel is fetched (and made) for all eight before the chain of
  // multiply-adds runs and the read-outs are stored, so the loads of a stretch are in flight together - a store
  // between two loads would hold the later one back, since the compiler cannot know that they do not overlap
  constexpr int U = 8;
  for (int t = t0; t < t1; t += U) {
    float av[U], bv[U], gv[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      av[u] = 1.f; bv[u] = 0.f; gv[u] = 0.f;
      if (t + u < t1) {
        cell.ab(row0 + t + u, c, av[u], bv[u]);
        gv[u] = cell.read_gate(row0 + t + u, c);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (t + u < t1) {
        S = fmaf(av[u], S, bv[u]);
        out[(size_t)(row0 + t + u) * ldo + c] = mi::from_float<T>(S * gv[u]);
      }
    }
  }
  if (t0 < n && t1 == n) *st = S;
}

constexpr int REC_NW = 32;       // warps of a block of the segmented form: stretches of an item's tokens
constexpr int REC_FLAT_NW = 4;   // warps of a block of the flat form: groups of 32 channels

template <typename T, typename Cell>
int launch_recurrence(Cell cell, T* out, int ldo, float* state, long long state_stride, const int* q_start, const int* q_len,
                      const int* seq_slot, int items, int C, int segmented, int seg_min, int rows, float* scratch, cudaStream_t stream) {
  if (segmented && scratch != nullptr && rows > 0) {
    // scratch: decays [rows, C] and inputs [rows, C] in float32, then the read-out factors [rows, C] in the storage type
    float* a = scratch;
    float* b = scratch + (size_t)rows * C;
    T* g = reinterpret_cast<T*>(scratch + 2 * (size_t)rows * C);
    mi::launch(diag_prepare_kernel<T, Cell>, dim3((C + 127) / 128, (rows + PREP_ROWS - 1) / PREP_ROWS), dim3(128), 0, stream, cell, a, b, g, C, rows);
    PreparedCell<T> prepared{a, b, g, C};
    mi::launch(diag_recurrence_kernel<T, PreparedCell<T>, REC_NW, true>, dim3((C + 31) / 32, items), dim3(32 * REC_NW), 0, stream, prepared, out, ldo,
               state, state_stride, q_start, q_len, seq_slot, C, seg_min);
  } else if (segmented)
    mi::launch(diag_recurrence_kernel<T, Cell, REC_NW, true>, dim3((C + 31) / 32, items), dim3(32 * REC_NW), 0, stream, cell, out, ldo, state,
               state_stride, q_start, q_len, seq_slot, C, seg_min);
  else
    mi::launch(diag_recurrence_kernel<T, Cell, REC_FLAT_NW, false>, dim3((C + 32 * REC_FLAT_NW - 1) / (32 * REC_FLAT_NW), items),
               dim3(32 * REC_FLAT_NW), 0, stream, cell, out, ldo, state, state_stride, q_start, q_len, seq_slot, C, seg_min);
  return 0;
}

}  // namespace

// out [T, W] in out_dtype; x [T, W] float32; shift [W] float32 or null; state rows float32, one per request slot (read only).
MI_API int mi_token_shift(void* out, int out_dtype, const float* x, int T, int W, const float* shift, const float* state,
                          long long state_stride, const int* token_item, const int* q_start, const int* seq_slot, cudaStream_t stream) {
  MI_REQUIRE(T >= 0 && W > 0, "token_shift: bad sizes T=%d W=%d", T, W);
  MI_REQUIRE(shift == nullptr || (state != nullptr && state_stride >= W), "token_shift: a shift needs state rows of at least %d values", W);
  if (T == 0) return 0;
  const bool vec = W % 4 == 0 && ((uintptr_t)out % 16) == 0 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)shift % 16) == 0 &&
                   ((uintptr_t)state % 16) == 0 && state_stride % 4 == 0;
  if (out_dtype == MI_BF16 && vec)
    mi::launch(token_shift_vec_kernel<__nv_bfloat16>, dim3(T), dim3(256), 0, stream, (__nv_bfloat16*)out, x, W, shift, state, state_stride, token_item, q_start, seq_slot);
  else if (out_dtype == MI_F32 && vec)
    mi::launch(token_shift_vec_kernel<float>, dim3(T), dim3(256), 0, stream, (float*)out, x, W, shift, state, state_stride, token_item, q_start, seq_slot);
  else if (out_dtype == MI_BF16)
    mi::launch(token_shift_kernel<__nv_bfloat16>, dim3(T), dim3(256), 0, stream, (__nv_bfloat16*)out, x, W, shift, state, state_stride, token_item, q_start, seq_slot);
  else if (out_dtype == MI_F32)
    mi::launch(token_shift_kernel<float>, dim3(T), dim3(256), 0, stream, (float*)out, x, W, shift, state, state_stride, token_item, q_start, seq_slot);
  else
    return mi_fail("token_shift: unknown dtype %d", out_dtype);
  MI_LAUNCH_OK("token_shift");
  return 0;
}

// resid [T, W] float32, updated in place; y [T, W] in y_dtype; w [W] float32; copy [T, W] in copy_dtype or null; keep: state
// rows (float32, one per request slot) that receive the OLD residual row of each item's last new token, or null.
MI_API int mi_norm_scaled_add(float* resid, const void* y, int y_dtype, const float* w, int T, int W, float eps, float mult, void* copy,
                              int copy_dtype, float* keep, long long keep_stride, const int* token_item, const int* q_start,
                              const int* q_len, const int* seq_slot, cudaStream_t stream) {
  MI_REQUIRE(T >= 0 && W > 0 && eps > 0.f, "norm_scaled_add: bad sizes T=%d W=%d or eps", T, W);
  MI_REQUIRE(keep == nullptr || keep_stride >= W, "norm_scaled_add: the kept rows are too short");
  MI_REQUIRE(copy == nullptr || copy_dtype == y_dtype, "norm_scaled_add: the copy has the sublayer output's type");
  if (T == 0) return 0;
  const bool vec = W % 4 == 0 && ((uintptr_t)resid % 16) == 0 && ((uintptr_t)y % 16) == 0 && ((uintptr_t)w % 16) == 0 &&
                   ((uintptr_t)copy % 16) == 0 && ((uintptr_t)keep % 16) == 0 && keep_stride % 4 == 0;
  if (y_dtype == MI_BF16 && vec)
    mi::launch(norm_scaled_add_vec_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(T), dim3(256), 0, stream, resid, (const __nv_bfloat16*)y, w, W, eps, mult,
               (__nv_bfloat16*)copy, keep, keep_stride, token_item, q_start, q_len, seq_slot);
  else if (y_dtype == MI_F32 && vec)
    mi::launch(norm_scaled_add_vec_kernel<float, float>, dim3(T), dim3(256), 0, stream, resid, (const float*)y, w, W, eps, mult, (float*)copy, keep,
               keep_stride, token_item, q_start, q_len, seq_slot);
  else if (y_dtype == MI_BF16)
    mi::launch(norm_scaled_add_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(T), dim3(256), 0, stream, resid, (const __nv_bfloat16*)y, w, W, eps, mult,
               (__nv_bfloat16*)copy, keep, keep_stride, token_item, q_start, q_len, seq_slot);
  else if (y_dtype == MI_F32)
    mi::launch(norm_scaled_add_kernel<float, float>, dim3(T), dim3(256), 0, stream, resid, (const float*)y, w, W, eps, mult, (float*)copy, keep,
               keep_stride, token_item, q_start, q_len, seq_slot);
  else
    return mi_fail("norm_scaled_add: unknown dtype %d", y_dtype);
  MI_LAUNCH_OK("norm_scaled_add");
  return 0;
}

MI_API int mi_recurrence_segment_warps() { return REC_NW; }

// out, u, y: [T, C] in dtype with row strides; gates float32: the 2 * (C / blocks) logits of part b of token t (r, then i) start at
// t * ldg + b * part_stride, so [T, blocks, .] and [blocks, T, .] both go; biases and lam [C] float32 (y_bias may be null);
// state rows float32 of at least C values.  segmented: the form with stretches side by side,
// taken by the items of at least seg_min * (warps of a block) new tokens; with scratch (3 * rows * C floats, rows = the
// step's tokens) what the tokens give the channels is prepared by a kernel of its own.
MI_API int mi_rglru_recurrence(void* out, int ldo, const void* u, int ldu, const float* gates, int ldg, long long part_stride, const void* y, int ldy, int dtype,
                               const float* r_bias, const float* i_bias, const float* y_bias, const float* lam, float* state,
                               long long state_stride, const int* q_start, const int* q_len, const int* seq_slot, int items, int C,
                               int blocks, int segmented, int seg_min, int rows, float* scratch, cudaStream_t stream) {
  MI_REQUIRE(items >= 0 && items <= 65535 && C > 0 && blocks > 0 && C % blocks == 0, "rglru: %d channels do not split into %d blocks", C, blocks);
  MI_REQUIRE(state_stride >= C && seg_min >= 1, "rglru: the state rows are too short");
  if (items == 0) return 0;
  if (dtype == MI_BF16) {
    RglruCell<__nv_bfloat16> cell{(const __nv_bfloat16*)u, ldu, gates, ldg, part_stride, (const __nv_bfloat16*)y, ldy, r_bias, i_bias, y_bias, lam, C / blocks};
    launch_recurrence<__nv_bfloat16>(cell, (__nv_bfloat16*)out, ldo, state, state_stride, q_start, q_len, seq_slot, items, C, segmented, seg_min, rows, scratch, stream);
  } else if (dtype == MI_F32) {
    RglruCell<float> cell{(const float*)u, ldu, gates, ldg, part_stride, (const float*)y, ldy, r_bias, i_bias, y_bias, lam, C / blocks};
    launch_recurrence<float>(cell, (float*)out, ldo, state, state_stride, q_start, q_len, seq_slot, items, C, segmented, seg_min, rows, scratch, stream);
  } else {
    return mi_fail("rglru: unknown dtype %d", dtype);
  }
  MI_LAUNCH_OK("rglru_recurrence");
  return 0;
}

// proj [T, 3 C] in dtype with row stride ld: z logits, x, g; biases [C] float32 or null.
MI_API int mi_mingru_recurrence(void* out, int ldo, const void* proj, int ld, int dtype, const float* z_bias, const float* x_bias,
                                float* state, long long state_stride, const int* q_start, const int* q_len, const int* seq_slot,
                                int items, int C, int segmented, int seg_min, int rows, float* scratch, cudaStream_t stream) {
  MI_REQUIRE(items >= 0 && items <= 65535 && C > 0 && ld >= 3 * C, "mingru: rows of %d values cannot hold three times %d channels", ld, C);
  MI_REQUIRE(state_stride >= C && seg_min >= 1, "mingru: the state rows are too short");
  if (items == 0) return 0;
  if (dtype == MI_BF16) {
    MingruCell<__nv_bfloat16> cell{(const __nv_bfloat16*)proj, ld, C, z_bias, x_bias};
    launch_recurrence<__nv_bfloat16>(cell, (__nv_bfloat16*)out, ldo, state, state_stride, q_start, q_len, seq_slot, items, C, segmented, seg_min, rows, scratch, stream);
  } else if (dtype == MI_F32) {
    MingruCell<float> cell{(const float*)proj, ld, C, z_bias, x_bias};
    launch_recurrence<float>(cell, (float*)out, ldo, state, state_stride, q_start, q_len, seq_slot, items, C, segmented, seg_min, rows, scratch, stream);
  } else {
    return mi_fail("mingru: unknown dtype %d", dtype);
  }
  MI_LAUNCH_OK("mingru_recurrence");
  return 0;
}
