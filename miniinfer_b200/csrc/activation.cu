// Activations of the feed-forwards.  Gated: out[t, i] = act(gu[t, i]) * gu[t, I + i] - SwiGLU, silu(g) * u, or the clamped
// form of common.cuh (MiGlu) - in float32, one rounding
// (bfloat16: with the hardware's exponential and reciprocal; float32: exact division and expf).
// Stands where the reference runs a Triton kernel (kernels/triton/silu_mul.py:6-42).
#include "common.cuh"

namespace {

template <typename T>
__global__ void silu_mul_kernel(T* __restrict__ out, const T* __restrict__ gu, int I, size_t total, int kind, float limit) {
  mi::grid_dependency_sync();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / I;
    const int i = (int)(idx - t * I);
    const float g = mi::to_float(gu[t * 2 * I + i]);
    const float u = mi::to_float(gu[t * 2 * I + I + i]);
    out[idx] = mi::from_float<T>(sizeof(T) == 4 ? mi::glu_exact(g, u, kind, limit) : mi::glu_fast(g, u, kind, limit));
  }
}

// bf16 with I a multiple of 8: 16-byte loads and stores.
__global__ void silu_mul_bf16x8_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ gu, int I8, size_t total8, int kind, float limit) {
  mi::grid_dependency_sync();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total8; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / I8;
    const int i = (int)(idx - t * I8);
    const uint4 g = *reinterpret_cast<const uint4*>(gu + (t * 2 * I8 + i) * 8);
    const uint4 u = *reinterpret_cast<const uint4*>(gu + (t * 2 * I8 + I8 + i) * 8);
    const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&g);
    const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&u);
    uint4 r;
    __nv_bfloat162* rp = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 a = __bfloat1622float2(gp[k]), b = __bfloat1622float2(up[k]);
      rp[k] = __floats2bfloat162_rn(mi::glu_fast(a.x, b.x, kind, limit), mi::glu_fast(a.y, b.y, kind, limit));
    }
    *reinterpret_cast<uint4*>(out + idx * 8) = r;
  }
}

// out[i] = max(x[i], 0)^2, squared in float32 and rounded once; out may be x.
template <typename T>
__global__ void relu_squared_kernel(T* __restrict__ out, const T* __restrict__ x, size_t total) {
  mi::grid_dependency_sync();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const float v = fmaxf(mi::to_float(x[idx]), 0.f);
    out[idx] = mi::from_float<T>(v * v);
  }
}

__global__ void relu_squared_bf16x8_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ x, size_t total8) {
  mi::grid_dependency_sync();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total8; idx += (size_t)gridDim.x * blockDim.x) {
    const uint4 g = *reinterpret_cast<const uint4*>(x + idx * 8);
    const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&g);
    uint4 r;
    __nv_bfloat162* rp = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float2 a = __bfloat1622float2(gp[k]);
      a.x = fmaxf(a.x, 0.f); a.y = fmaxf(a.y, 0.f);
      rp[k] = __floats2bfloat162_rn(a.x * a.x, a.y * a.y);
    }
    *reinterpret_cast<uint4*>(out + idx * 8) = r;
  }
}

}  // namespace

// Squared ReLU over n values, in place if out == x.
MI_API int mi_relu_squared(void* out, const void* x, int dtype, long long n, cudaStream_t stream) {
  MI_REQUIRE(n >= 0, "relu_squared: bad size %lld", n);
  if (n == 0) return 0;
  const size_t total = (size_t)n;
  const int threads = 256;
  const size_t most = (size_t)mi::sm_count() * 16;
  if (dtype == MI_BF16 && total % 8 == 0 && ((uintptr_t)out % 16) == 0 && ((uintptr_t)x % 16) == 0) {
    const size_t total8 = total / 8, want = (total8 + threads - 1) / threads;
    mi::launch(relu_squared_bf16x8_kernel, dim3((unsigned)(want < most ? want : most)), dim3(threads), 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)x, total8);
  } else {
    const size_t want = (total + threads - 1) / threads;
    const dim3 grid((unsigned)(want < most ? want : most));
    if (dtype == MI_BF16) mi::launch(relu_squared_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)x, total);
    else if (dtype == MI_F32) mi::launch(relu_squared_kernel<float>, grid, dim3(threads), 0, stream, (float*)out, (const float*)x, total);
    else return mi_fail("relu_squared: unknown dtype %d", dtype);
  }
  MI_LAUNCH_OK("relu_squared");
  return 0;
}

// kind: a MiGlu; limit: the clamp of MI_GLU_CLAMPED.
MI_API int mi_glu_mul(void* out, const void* gu, int dtype, int T, int I, int kind, float limit, cudaStream_t stream) {
  MI_REQUIRE(T >= 0 && I > 0, "glu_mul: bad sizes T=%d I=%d", T, I);
  MI_REQUIRE(kind == MI_GLU_SILU || (kind == MI_GLU_CLAMPED && limit > 0.f), "glu_mul: unknown kind %d or a limit that is not positive", kind);
  if (T == 0) return 0;
  const size_t total = (size_t)T * I;
  const int threads = 256;
  const int most = mi::sm_count() * 16;
  const int blocks = (int)((total + threads - 1) / threads < most ? (total + threads - 1) / threads : most);
  if (dtype == MI_BF16 && I % 8 == 0 && ((uintptr_t)out % 16) == 0 && ((uintptr_t)gu % 16) == 0) {
    const size_t total8 = total / 8;
    const int b8 = (int)((total8 + threads - 1) / threads < most ? (total8 + threads - 1) / threads : most);
    mi::launch(silu_mul_bf16x8_kernel, dim3(b8), dim3(threads), 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)gu, I / 8, total8, kind, limit);
  } else if (dtype == MI_BF16)
    mi::launch(silu_mul_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)gu, I, total, kind, limit);
  else if (dtype == MI_F32)
    mi::launch(silu_mul_kernel<float>, dim3(blocks), dim3(threads), 0, stream, (float*)out, (const float*)gu, I, total, kind, limit);
  else
    return mi_fail("glu_mul: unknown dtype %d", dtype);
  MI_LAUNCH_OK("glu_mul");
  return 0;
}

MI_API int mi_silu_mul(void* out, const void* gu, int dtype, int T, int I, cudaStream_t stream) {
  return mi_glu_mul(out, gu, dtype, T, I, MI_GLU_SILU, 0.f, stream);
}
