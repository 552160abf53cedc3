// Hyper-connections: the residual stream is S streams, a row of `streams` holding them side by side
// ([token][stream][width], float32).  One kernel stands between two sublayers.  It
//
//   * brings the streams up to date with the output y of the sublayer before (optional):
//       x'[t] = sum_s mix[s, t] * x[s] + out[t] * y        all t from the old x; mix is indexed [from, to]
//     and writes them back (write_back), and
//   * reads for whoever comes next:  u = sum_t in[t] * x'[t]   (in null: every weight is 1, the plain sum), then
//       res = w * u / sqrt(mean(u^2) + eps)                 rounded once to the output type, or, with w null, res = u.
//
// All arithmetic is float32 in an order that depends on the row alone.  A block per row; u stays in shared memory
// between the two passes.  `rows` selects rows (the final norm on the wanted rows only).
#include "common.cuh"

namespace {

constexpr int HYPER_MAX_STREAMS = 8;

// VEC values of a row at a time: 16-byte accesses to the float32 streams when the width is a multiple of 4
template <int VEC> __device__ __forceinline__ void hyper_load(float (&v)[VEC], const float* p) {
  if constexpr (VEC == 4) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  } else {
    v[0] = p[0];
  }
}
template <int VEC> __device__ __forceinline__ void hyper_load(float (&v)[VEC], const __nv_bfloat16* p) {
  if constexpr (VEC == 4) {
    const uint2 t = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&t.x), b = *reinterpret_cast<const __nv_bfloat162*>(&t.y);
    v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
  } else {
    v[0] = __bfloat162float(p[0]);
  }
}
template <int VEC> __device__ __forceinline__ void hyper_store(float* p, const float (&v)[VEC]) {
  if constexpr (VEC == 4) *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  else p[0] = v[0];
}
template <int VEC> __device__ __forceinline__ void hyper_store(__nv_bfloat16* p, const float (&v)[VEC]) {
  if constexpr (VEC == 4) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    uint2 t;
    t.x = *reinterpret_cast<const unsigned*>(&a);
    t.y = *reinterpret_cast<const unsigned*>(&b);
    *reinterpret_cast<uint2*>(p) = t;
  } else {
    p[0] = __float2bfloat16_rn(v[0]);
  }
}

// SC: the number of streams when it is 1 to 4 (loops over streams unroll to exactly that), 0: any number up to the limit
template <typename TOut, typename TDelta, int SC, int VEC>
__global__ void __launch_bounds__(256)
hyper_connection_kernel(TOut* __restrict__ res, float* __restrict__ streams, const TDelta* __restrict__ y,
                        const float* __restrict__ mix, const float* __restrict__ outw, const float* __restrict__ inw,
                        const float* __restrict__ w, const int* __restrict__ rows, int S_any, int W, float eps, int write_back) {
  constexpr int MAXS = SC ? SC : HYPER_MAX_STREAMS;
  const int S = SC ? SC : S_any;
  extern __shared__ __align__(16) float hyper_u[];
  __shared__ float scratch[33];
  __shared__ float s_mix[HYPER_MAX_STREAMS * HYPER_MAX_STREAMS], s_out[HYPER_MAX_STREAMS], s_in[HYPER_MAX_STREAMS];
  // the weights: no kernel writes them
  if (threadIdx.x < S * S) s_mix[threadIdx.x] = y ? mix[threadIdx.x] : 0.f;
  if (threadIdx.x < S) {
    s_out[threadIdx.x] = y ? outw[threadIdx.x] : 0.f;
    s_in[threadIdx.x] = inw ? inw[threadIdx.x] : 1.f;
  }
  const int r = blockIdx.x;
  const int row = rows ? rows[r] : r;
  mi::grid_dependency_sync();
  __syncthreads();
  float* x = streams + (size_t)row * S * W;
  const TDelta* yr = y ? y + (size_t)row * W : nullptr;
  float ss = 0.f;
  for (int h = threadIdx.x * VEC; h < W; h += blockDim.x * VEC) {
    float old[MAXS][VEC], now[MAXS][VEC];
#pragma unroll
    for (int s = 0; s < MAXS; ++s) {
      if (s < S) {
        hyper_load<VEC>(old[s], x + (size_t)s * W + h);
      } else {
#pragma unroll
        for (int e = 0; e < VEC; ++e) old[s][e] = 0.f;
      }
    }
    if (yr) {
      float yv[VEC];
      hyper_load<VEC>(yv, yr + h);
#pragma unroll
      for (int t = 0; t < MAXS; ++t) {
        if (t >= S) continue;
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          float acc = 0.f;
#pragma unroll
          for (int s = 0; s < MAXS; ++s)
            if (s < S) acc = fmaf(s_mix[s * S + t], old[s][e], acc);
          now[t][e] = fmaf(s_out[t], yv[e], acc);
        }
        if (write_back) hyper_store<VEC>(x + (size_t)t * W + h, now[t]);
      }
    } else {
#pragma unroll
      for (int t = 0; t < MAXS; ++t)
#pragma unroll
        for (int e = 0; e < VEC; ++e) now[t][e] = old[t][e];
    }
    float u[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      u[e] = 0.f;
#pragma unroll
      for (int t = 0; t < MAXS; ++t)
        if (t < S) u[e] = fmaf(s_in[t], now[t][e], u[e]);
      ss = fmaf(u[e], u[e], ss);
    }
    hyper_store<VEC>(hyper_u + h, u);
  }
  TOut* o = res + (size_t)r * W;
  // every thread reads back the values it wrote itself
  if (w == nullptr) {
    for (int h = threadIdx.x * VEC; h < W; h += blockDim.x * VEC) {
      float u[VEC];
      hyper_load<VEC>(u, (const float*)hyper_u + h);
      hyper_store<VEC>(o + h, u);
    }
    return;
  }
  const float rstd = 1.f / sqrtf(mi::block_sum(ss, scratch) / (float)W + eps);
  for (int h = threadIdx.x * VEC; h < W; h += blockDim.x * VEC) {
    float u[VEC], wv[VEC];
    hyper_load<VEC>(u, (const float*)hyper_u + h);
    hyper_load<VEC>(wv, w + h);
#pragma unroll
    for (int e = 0; e < VEC; ++e) u[e] = wv[e] * (u[e] * rstd);
    hyper_store<VEC>(o + h, u);
  }
}

}  // namespace

MI_API int mi_hyper_connection(void* res, int res_dtype, float* streams, const void* y, int y_dtype, const float* mix,
                               const float* outw, const float* inw, const float* w, const int* rows, int R, int S, int W,
                               float eps, int write_back, cudaStream_t stream) {
  MI_REQUIRE(R >= 0 && W > 0 && S >= 1 && S <= HYPER_MAX_STREAMS, "hyper_connection: bad sizes R=%d W=%d streams=%d (up to %d)", R, W, S, HYPER_MAX_STREAMS);
  MI_REQUIRE(y == nullptr || (mix != nullptr && outw != nullptr), "hyper_connection: an update needs its mix matrix and out vector");
  MI_REQUIRE(w == nullptr || eps > 0.f, "hyper_connection: eps must be positive");
  if (R == 0) return 0;
  const size_t smem = (size_t)W * sizeof(float);
  MI_REQUIRE(smem <= 160 * 1024, "hyper_connection: rows of %d values do not fit shared memory", W);
  const bool vec = W % 4 == 0;
#define MI_HYPER_ONE(TO, TD, SC, VEC)                                                                                 \
  do {                                                                                                                \
    if (smem > 48 * 1024) cudaFuncSetAttribute(hyper_connection_kernel<TO, TD, SC, VEC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    mi::launch(hyper_connection_kernel<TO, TD, SC, VEC>, dim3(R), dim3(256), smem, stream, (TO*)res, streams, (const TD*)y, mix, outw, inw, w, rows, S, W, eps, write_back); \
  } while (0)
#define MI_HYPER(TO, TD)                                                                                              \
  do {                                                                                                                \
    if (!vec) MI_HYPER_ONE(TO, TD, 0, 1);                                                                             \
    else if (S == 1) MI_HYPER_ONE(TO, TD, 1, 4);                                                                      \
    else if (S == 2) MI_HYPER_ONE(TO, TD, 2, 4);                                                                      \
    else if (S == 3) MI_HYPER_ONE(TO, TD, 3, 4);                                                                      \
    else if (S == 4) MI_HYPER_ONE(TO, TD, 4, 4);                                                                      \
    else MI_HYPER_ONE(TO, TD, 0, 4);                                                                                  \
  } while (0)
  if (res_dtype == MI_BF16 && y_dtype == MI_BF16) MI_HYPER(__nv_bfloat16, __nv_bfloat16);
  else if (res_dtype == MI_F32 && y_dtype == MI_F32) MI_HYPER(float, float);
  else if (res_dtype == MI_BF16 && y_dtype == MI_F32) MI_HYPER(__nv_bfloat16, float);
  else if (res_dtype == MI_F32 && y_dtype == MI_BF16) MI_HYPER(float, __nv_bfloat16);
  else return mi_fail("hyper_connection: unknown dtypes res=%d y=%d", res_dtype, y_dtype);
#undef MI_HYPER
#undef MI_HYPER_ONE
  MI_LAUNCH_OK("hyper_connection");
  return 0;
}
