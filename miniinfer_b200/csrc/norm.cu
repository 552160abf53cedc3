// RMSNorm with the residual add fused in front of it.
//
//   sum[r, :] = resid[row(r), :] (+ delta[row(r), :])         float32
//   out[r, :] = w * sum * rsqrt(mean(sum^2) + eps)            rounded once to the output type
//   resid[row(r), :] = sum                                    if write_back
//
// The reference adds in the model's type and rounds the normalised value before the weight
// multiply (kernels/triton/rms_norm.py:88-108, miniinfer/layers/layernorm.py:27-32); here the
// residual stream stays in float32 and the only rounding is the final one.
// `rows` selects rows (the final norm runs only on the rows whose logits are wanted).
#include "common.cuh"

namespace {

template <typename TOut, typename TDelta>
__global__ void add_rmsnorm_kernel(TOut* __restrict__ out, float* __restrict__ resid,
                                   const TDelta* __restrict__ delta, const float* __restrict__ w,
                                   const int* __restrict__ rows, int H, float eps, int write_back) {
  mi::grid_dependency_sync();
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  const int row = rows ? rows[r] : r;
  float* x = resid + (size_t)row * H;
  const TDelta* d = delta ? delta + (size_t)row * H : nullptr;
  float ss = 0.f;
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    float v = x[h];
    if (d) v += mi::to_float(d[h]);
    if (write_back && d) x[h] = v;
    ss += v * v;
  }
  const float total = mi::block_sum(ss, scratch);
  const float rstd = rsqrtf(total / (float)H + eps);
  TOut* o = out + (size_t)r * H;
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    float v = x[h];
    if (d && !write_back) v += mi::to_float(d[h]);
    o[h] = mi::from_float<TOut>(w[h] * (v * rstd));
  }
}

// The serving case in 16-byte steps: bf16 output and delta, H a multiple of 4, a row kept in
// registers between the two passes (up to 4 * 256 * VPT values).
template <int VPT>
__global__ void __launch_bounds__(256)
add_rmsnorm_bf16_vec_kernel(__nv_bfloat16* __restrict__ out, float* __restrict__ resid,
                            const __nv_bfloat16* __restrict__ delta, const float* __restrict__ w,
                            const int* __restrict__ rows, int H, float eps, int write_back) {
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  const int H4 = H / 4;
  // the norm weights and the row list are written by no kernel: fetched before the wait for the preceding kernel
  const int row = rows ? rows[r] : r;
  const float4* w4 = reinterpret_cast<const float4*>(w);
  float4 ww[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int h = threadIdx.x + i * 256;
    if (h < H4) ww[i] = w4[h];
  }
  mi::grid_dependency_sync();
  float4* x = reinterpret_cast<float4*>(resid + (size_t)row * H);
  const uint2* d = delta ? reinterpret_cast<const uint2*>(delta + (size_t)row * H) : nullptr;
  float4 v[VPT];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int h = threadIdx.x + i * 256;
    if (h < H4) {
      v[i] = x[h];
      if (d) {
        const uint2 raw = d[h];
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        v[i].x += a.x; v[i].y += a.y; v[i].z += b.x; v[i].w += b.y;
        if (write_back) x[h] = v[i];
      }
      ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
    }
  }
  const float total = mi::block_sum(ss, scratch);
  const float rstd = rsqrtf(total / (float)H + eps);
  uint2* o = reinterpret_cast<uint2*>(out + (size_t)r * H);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int h = threadIdx.x + i * 256;
    if (h < H4) {
      const __nv_bfloat162 lo = __floats2bfloat162_rn(ww[i].x * (v[i].x * rstd), ww[i].y * (v[i].y * rstd));
      const __nv_bfloat162 hi = __floats2bfloat162_rn(ww[i].z * (v[i].z * rstd), ww[i].w * (v[i].w * rstd));
      uint2 packed;
      packed.x = *reinterpret_cast<const uint32_t*>(&lo);
      packed.y = *reinterpret_cast<const uint32_t*>(&hi);
      o[h] = packed;
    }
  }
}

}  // namespace

MI_API int mi_add_rmsnorm(void* out, int out_dtype, float* resid, const void* delta, int delta_dtype,
                          const float* w, const int* rows, int R, int H, float eps, int write_back,
                          cudaStream_t stream) {
  MI_REQUIRE(R >= 0 && H > 0, "rmsnorm: bad sizes R=%d H=%d", R, H);
  MI_REQUIRE(eps > 0.f, "rmsnorm: eps must be positive");
  if (R == 0) return 0;
  const int threads = 256;  // fixed: the order of the reduction must not depend on the batch
  const bool aligned = ((uintptr_t)out % 8) == 0 && ((uintptr_t)resid % 16) == 0 && ((uintptr_t)delta % 8) == 0 && ((uintptr_t)w % 16) == 0;
  if (out_dtype == MI_BF16 && (delta == nullptr || delta_dtype == MI_BF16) && H % 4 == 0 && H <= 8192 && aligned) {
    const int vpt = (H / 4 + 255) / 256;
    if (vpt <= 1)
      mi::launch(add_rmsnorm_bf16_vec_kernel<1>, dim3(R), dim3(threads), 0, stream, (__nv_bfloat16*)out, resid, (const __nv_bfloat16*)delta, w, rows, H, eps, write_back);
    else if (vpt <= 2)
      mi::launch(add_rmsnorm_bf16_vec_kernel<2>, dim3(R), dim3(threads), 0, stream, (__nv_bfloat16*)out, resid, (const __nv_bfloat16*)delta, w, rows, H, eps, write_back);
    else if (vpt <= 4)
      mi::launch(add_rmsnorm_bf16_vec_kernel<4>, dim3(R), dim3(threads), 0, stream, (__nv_bfloat16*)out, resid, (const __nv_bfloat16*)delta, w, rows, H, eps, write_back);
    else
      mi::launch(add_rmsnorm_bf16_vec_kernel<8>, dim3(R), dim3(threads), 0, stream, (__nv_bfloat16*)out, resid, (const __nv_bfloat16*)delta, w, rows, H, eps, write_back);
    MI_LAUNCH_OK("add_rmsnorm");
    return 0;
  }
#define MI_NORM_LAUNCH(TO, TD) \
  mi::launch(add_rmsnorm_kernel<TO, TD>, dim3(R), dim3(threads), 0, stream, (TO*)out, resid, (const TD*)delta, w, rows, H, eps, write_back)
  if (out_dtype == MI_BF16 && delta_dtype == MI_BF16) MI_NORM_LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else if (out_dtype == MI_F32 && delta_dtype == MI_F32) MI_NORM_LAUNCH(float, float);
  else if (out_dtype == MI_BF16 && delta_dtype == MI_F32) MI_NORM_LAUNCH(__nv_bfloat16, float);
  else if (out_dtype == MI_F32 && delta_dtype == MI_BF16) MI_NORM_LAUNCH(float, __nv_bfloat16);
  else return mi_fail("rmsnorm: unknown dtypes out=%d delta=%d", out_dtype, delta_dtype);
#undef MI_NORM_LAUNCH
  MI_LAUNCH_OK("add_rmsnorm");
  return 0;
}

// ------------------------------------------------------------------------------------------------
// One root mean square, two weights: blocks whose mixer and feed-forward each have a norm of their own on the same
// residual rows.  sum = resid[row] (+ d1[row]) (+ d2[row]); out1 = w1 * sum * rstd; out2 = w2 * sum * rstd (if asked for).
// Also the plain RMSNorm behind a block that leaves two outputs pending (out2 null).
namespace {

template <typename TOut, typename TDelta>
__global__ void __launch_bounds__(256)
add_rmsnorm_pair_kernel(TOut* __restrict__ out1, TOut* __restrict__ out2, float* __restrict__ resid,
                        const TDelta* __restrict__ d1, const TDelta* __restrict__ d2, const float* __restrict__ w1,
                        const float* __restrict__ w2, const int* __restrict__ rows, int H, float eps, int write_back) {
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  const int row = rows ? rows[r] : r;
  mi::grid_dependency_sync();
  float* x = resid + (size_t)row * H;
  const TDelta* a = d1 ? d1 + (size_t)row * H : nullptr;
  const TDelta* b = d2 ? d2 + (size_t)row * H : nullptr;
  const bool any = a || b;
  float ss = 0.f;
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    float v = x[h];
    if (a && b) v += mi::to_float(a[h]) + mi::to_float(b[h]);     // the two outputs first, then the stream
    else if (a) v += mi::to_float(a[h]);
    else if (b) v += mi::to_float(b[h]);
    if (write_back && any) x[h] = v;
    ss += v * v;
  }
  const float total = mi::block_sum(ss, scratch);
  const float rstd = 1.f / sqrtf(total / (float)H + eps);
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    float v = x[h];
    if (any && !write_back) {
      if (a && b) v += mi::to_float(a[h]) + mi::to_float(b[h]);
      else if (a) v += mi::to_float(a[h]);
      else v += mi::to_float(b[h]);
    }
    const float n = v * rstd;
    out1[(size_t)r * H + h] = mi::from_float<TOut>(w1[h] * n);
    if (out2) out2[(size_t)r * H + h] = mi::from_float<TOut>(w2[h] * n);
  }
}

// out = scale * (w1 * a / rms(a) + w2 * b / rms(b)), each row normalised by its own root mean square: the meeting
// of two mixers that ran side by side on the same input.
template <typename T>
__global__ void __launch_bounds__(256)
rms_pair_sum_kernel(T* __restrict__ out, const T* __restrict__ a, const T* __restrict__ b, const float* __restrict__ w1,
                    const float* __restrict__ w2, int H, float eps, float scale) {
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  mi::grid_dependency_sync();
  const T* x = a + (size_t)r * H;
  const T* y = b + (size_t)r * H;
  float sa = 0.f, sb = 0.f;
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    const float u = mi::to_float(x[h]), v = mi::to_float(y[h]);
    sa += u * u;
    sb += v * v;
  }
  const float ta = mi::block_sum(sa, scratch);
  const float tb = mi::block_sum(sb, scratch);
  const float ra = 1.f / sqrtf(ta / (float)H + eps), rb = 1.f / sqrtf(tb / (float)H + eps);
  for (int h = threadIdx.x; h < H; h += blockDim.x)
    out[(size_t)r * H + h] = mi::from_float<T>(scale * (w1[h] * (mi::to_float(x[h]) * ra) + w2[h] * (mi::to_float(y[h]) * rb)));
}

}  // namespace

MI_API int mi_add_rmsnorm_pair(void* out1, void* out2, int out_dtype, float* resid, const void* d1, const void* d2, int delta_dtype,
                               const float* w1, const float* w2, const int* rows, int R, int H, float eps, int write_back,
                               cudaStream_t stream) {
  MI_REQUIRE(R >= 0 && H > 0 && eps > 0.f, "rmsnorm_pair: bad sizes R=%d H=%d or eps", R, H);
  MI_REQUIRE(out1 != nullptr && w1 != nullptr && (out2 == nullptr || w2 != nullptr), "rmsnorm_pair: an output without its weight");
  if (R == 0) return 0;
#define MI_NORM_LAUNCH(TO, TD) \
  mi::launch(add_rmsnorm_pair_kernel<TO, TD>, dim3(R), dim3(256), 0, stream, (TO*)out1, (TO*)out2, resid, (const TD*)d1, (const TD*)d2, w1, w2, rows, H, eps, write_back)
  if (out_dtype == MI_BF16 && delta_dtype == MI_BF16) MI_NORM_LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else if (out_dtype == MI_F32 && delta_dtype == MI_F32) MI_NORM_LAUNCH(float, float);
  else if (out_dtype == MI_BF16 && delta_dtype == MI_F32) MI_NORM_LAUNCH(__nv_bfloat16, float);
  else if (out_dtype == MI_F32 && delta_dtype == MI_BF16) MI_NORM_LAUNCH(float, __nv_bfloat16);
  else return mi_fail("rmsnorm_pair: unknown dtypes out=%d delta=%d", out_dtype, delta_dtype);
#undef MI_NORM_LAUNCH
  MI_LAUNCH_OK("add_rmsnorm_pair");
  return 0;
}

namespace {
template <typename T>
__global__ void scaled_pair_sum_kernel(T* __restrict__ out, const T* __restrict__ a, const T* __restrict__ b, size_t n, float sa, float sb) {
  mi::grid_dependency_sync();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    out[i] = mi::from_float<T>(fmaf(sa, mi::to_float(a[i]), sb * mi::to_float(b[i])));
}
}  // namespace

// out = sa * a + sb * b over n values, float32 arithmetic, one rounding (two mixers side by side, summed with constants).
MI_API int mi_scaled_pair_sum(void* out, const void* a, const void* b, int dtype, long long n, float sa, float sb, cudaStream_t stream) {
  MI_REQUIRE(n >= 0, "scaled_pair_sum: bad size %lld", n);
  if (n == 0) return 0;
  const size_t want = ((size_t)n + 255) / 256, most = (size_t)mi::sm_count() * 16;
  const dim3 grid((unsigned)(want < most ? want : most));
  if (dtype == MI_BF16)
    mi::launch(scaled_pair_sum_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)a, (const __nv_bfloat16*)b, (size_t)n, sa, sb);
  else if (dtype == MI_F32)
    mi::launch(scaled_pair_sum_kernel<float>, grid, dim3(256), 0, stream, (float*)out, (const float*)a, (const float*)b, (size_t)n, sa, sb);
  else return mi_fail("scaled_pair_sum: unknown dtype %d", dtype);
  MI_LAUNCH_OK("scaled_pair_sum");
  return 0;
}

MI_API int mi_rms_pair_sum(void* out, const void* a, const void* b, int dtype, const float* w1, const float* w2, int R, int H,
                           float eps, float scale, cudaStream_t stream) {
  MI_REQUIRE(R >= 0 && H > 0 && eps > 0.f, "rms_pair_sum: bad sizes R=%d H=%d or eps", R, H);
  if (R == 0) return 0;
  if (dtype == MI_BF16)
    mi::launch(rms_pair_sum_kernel<__nv_bfloat16>, dim3(R), dim3(256), 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)a, (const __nv_bfloat16*)b, w1, w2, H, eps, scale);
  else if (dtype == MI_F32)
    mi::launch(rms_pair_sum_kernel<float>, dim3(R), dim3(256), 0, stream, (float*)out, (const float*)a, (const float*)b, w1, w2, H, eps, scale);
  else return mi_fail("rms_pair_sum: unknown dtype %d", dtype);
  MI_LAUNCH_OK("rms_pair_sum");
  return 0;
}

// ------------------------------------------------------------------------------------------------
// Layer norm (mean and variance, weight and bias) with the residual add in front of it.
//
//   sum[r, :] = resid[row(r), :] + (d1[row(r), :] + d2[row(r), :])      float32; d1, d2 optional
//   out[r, :] = (sum - mean) * rsqrt(mean((sum - mean)^2) + eps) * w + b   rounded once to the output type
//   resid[row(r), :] = sum                                                 if write_back
//
// Two deltas because a layer whose mixer and feed-forward read the same normalised rows leaves two
// outputs to be added.  The row is kept in shared memory between the passes; the variance is the mean
// of the squared deviations (second pass), not E[x^2] - mean^2.
namespace {

template <typename TOut, typename TDelta>
__global__ void add_layernorm_kernel(TOut* __restrict__ out, float* __restrict__ resid,
                                     const TDelta* __restrict__ d1, const TDelta* __restrict__ d2,
                                     const float* __restrict__ w, const float* __restrict__ b,
                                     const int* __restrict__ rows, int H, float eps, int write_back) {
  extern __shared__ float ln_row[];
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  const int row = rows ? rows[r] : r;
  mi::grid_dependency_sync();
  float* x = resid + (size_t)row * H;
  const TDelta* a = d1 ? d1 + (size_t)row * H : nullptr;
  const TDelta* c = d2 ? d2 + (size_t)row * H : nullptr;
  float s = 0.f;
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    float v = x[h];
    if (a && c) v += mi::to_float(a[h]) + mi::to_float(c[h]);
    else if (a) v += mi::to_float(a[h]);
    else if (c) v += mi::to_float(c[h]);
    if (write_back && (a || c)) x[h] = v;
    ln_row[h] = v;
    s += v;
  }
  const float mean = mi::block_sum(s, scratch) / (float)H;
  float q = 0.f;
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    const float dv = ln_row[h] - mean;
    q += dv * dv;
  }
  const float rstd = 1.f / sqrtf(mi::block_sum(q, scratch) / (float)H + eps);
  TOut* o = out + (size_t)r * H;
  for (int h = threadIdx.x; h < H; h += blockDim.x)
    o[h] = mi::from_float<TOut>((ln_row[h] - mean) * rstd * w[h] + b[h]);
}


// Rows whose length is a multiple of 4, up to 8192: 16-byte steps, the row kept in registers between the passes.
template <typename TD> struct Delta4;
template <> struct Delta4<__nv_bfloat16> {
  static __device__ __forceinline__ float4 load(const __nv_bfloat16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
  }
};
template <> struct Delta4<float> {
  static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
};
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  uint2 packed;
  packed.x = *reinterpret_cast<const uint32_t*>(&lo);
  packed.y = *reinterpret_cast<const uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = packed;
}

template <typename TOut, typename TDelta, int VPT>
__global__ void __launch_bounds__(256)
add_layernorm_vec_kernel(TOut* __restrict__ out, float* __restrict__ resid, const TDelta* __restrict__ d1,
                         const TDelta* __restrict__ d2, const float* __restrict__ w, const float* __restrict__ b,
                         const int* __restrict__ rows, int H, float eps, int write_back) {
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  const int H4 = H / 4;
  const int row = rows ? rows[r] : r;       // the row list, weights and biases are written by no kernel
  float4 ww[VPT], bb[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int h = threadIdx.x + i * 256;
    if (h < H4) { ww[i] = reinterpret_cast<const float4*>(w)[h]; bb[i] = reinterpret_cast<const float4*>(b)[h]; }
  }
  mi::grid_dependency_sync();
  float* x = resid + (size_t)row * H;
  const TDelta* a = d1 ? d1 + (size_t)row * H : nullptr;
  const TDelta* c = d2 ? d2 + (size_t)row * H : nullptr;
  float4 v[VPT];
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int h = threadIdx.x + i * 256;
    if (h < H4) {
      v[i] = reinterpret_cast<const float4*>(x)[h];
      if (a || c) {
        float4 add = a ? Delta4<TDelta>::load(a + 4 * h) : make_float4(0.f, 0.f, 0.f, 0.f);
        if (a && c) { const float4 t = Delta4<TDelta>::load(c + 4 * h); add.x += t.x; add.y += t.y; add.z += t.z; add.w += t.w; }
        else if (c) add = Delta4<TDelta>::load(c + 4 * h);
        v[i].x += add.x; v[i].y += add.y; v[i].z += add.z; v[i].w += add.w;
        if (write_back) reinterpret_cast<float4*>(x)[h] = v[i];
      }
      s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    }
  }
  const float mean = mi::block_sum(s, scratch) / (float)H;
  float q = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int h = threadIdx.x + i * 256;
    if (h < H4) {
      const float dx = v[i].x - mean, dy = v[i].y - mean, dz = v[i].z - mean, dw = v[i].w - mean;
      q += (dx * dx + dy * dy) + (dz * dz + dw * dw);
    }
  }
  const float rstd = 1.f / sqrtf(mi::block_sum(q, scratch) / (float)H + eps);
  TOut* o = out + (size_t)r * H;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int h = threadIdx.x + i * 256;
    if (h < H4)
      store4(o + 4 * h, make_float4((v[i].x - mean) * rstd * ww[i].x + bb[i].x, (v[i].y - mean) * rstd * ww[i].y + bb[i].y,
                                    (v[i].z - mean) * rstd * ww[i].z + bb[i].z, (v[i].w - mean) * rstd * ww[i].w + bb[i].w));
  }
}

}  // namespace

MI_API int mi_add_layernorm(void* out, int out_dtype, float* resid, const void* d1, const void* d2, int delta_dtype,
                            const float* w, const float* b, const int* rows, int R, int H, float eps, int write_back,
                            cudaStream_t stream) {
  MI_REQUIRE(R >= 0 && H > 0 && H <= 12000, "layernorm: bad sizes R=%d H=%d (H up to 12000)", R, H);
  MI_REQUIRE(eps > 0.f, "layernorm: eps must be positive");
  if (R == 0) return 0;
  const int threads = 256;  // fixed: the order of the reductions must not depend on the batch
  const size_t smem = (size_t)H * sizeof(float);
  const bool vec = H % 4 == 0 && H <= 8192 && ((uintptr_t)out % 16) == 0 && ((uintptr_t)resid % 16) == 0 && ((uintptr_t)d1 % 16) == 0 &&
                   ((uintptr_t)d2 % 16) == 0 && ((uintptr_t)w % 16) == 0 && ((uintptr_t)b % 16) == 0;
  const int vpt = (H / 4 + 255) / 256;
#define MI_LN_VEC(TO, TD, V) \
  mi::launch(add_layernorm_vec_kernel<TO, TD, V>, dim3(R), dim3(threads), 0, stream, (TO*)out, resid, (const TD*)d1, (const TD*)d2, w, b, rows, H, eps, write_back)
#define MI_LN_LAUNCH(TO, TD)                                      \
  do {                                                            \
    if (vec && vpt <= 1) MI_LN_VEC(TO, TD, 1);                    \
    else if (vec && vpt <= 2) MI_LN_VEC(TO, TD, 2);               \
    else if (vec && vpt <= 4) MI_LN_VEC(TO, TD, 4);               \
    else if (vec) MI_LN_VEC(TO, TD, 8);                           \
    else mi::launch(add_layernorm_kernel<TO, TD>, dim3(R), dim3(threads), smem, stream, (TO*)out, resid, (const TD*)d1, (const TD*)d2, w, b, rows, H, eps, write_back); \
  } while (0)
  if (out_dtype == MI_BF16 && delta_dtype == MI_BF16) MI_LN_LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else if (out_dtype == MI_F32 && delta_dtype == MI_F32) MI_LN_LAUNCH(float, float);
  else if (out_dtype == MI_BF16 && delta_dtype == MI_F32) MI_LN_LAUNCH(__nv_bfloat16, float);
  else if (out_dtype == MI_F32 && delta_dtype == MI_BF16) MI_LN_LAUNCH(float, __nv_bfloat16);
  else return mi_fail("layernorm: unknown dtypes out=%d delta=%d", out_dtype, delta_dtype);
#undef MI_LN_LAUNCH
#undef MI_LN_VEC
  MI_LAUNCH_OK("add_layernorm");
  return 0;
}
