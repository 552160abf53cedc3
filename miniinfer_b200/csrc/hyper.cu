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

template <typename TOut, typename TDelta>
__global__ void __launch_bounds__(256)
hyper_connection_kernel(TOut* __restrict__ res, float* __restrict__ streams, const TDelta* __restrict__ y,
                        const float* __restrict__ mix, const float* __restrict__ outw, const float* __restrict__ inw,
                        const float* __restrict__ w, const int* __restrict__ rows, int S, int W, float eps, int write_back) {
  extern __shared__ float hyper_u[];
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
  for (int h = threadIdx.x; h < W; h += blockDim.x) {
    float old[HYPER_MAX_STREAMS], now[HYPER_MAX_STREAMS];
#pragma unroll
    for (int s = 0; s < HYPER_MAX_STREAMS; ++s) old[s] = s < S ? x[(size_t)s * W + h] : 0.f;
    if (yr) {
      const float yv = mi::to_float(yr[h]);
#pragma unroll
      for (int t = 0; t < HYPER_MAX_STREAMS; ++t) {
        if (t >= S) continue;
        float acc = 0.f;
#pragma unroll
        for (int s = 0; s < HYPER_MAX_STREAMS; ++s)
          if (s < S) acc = fmaf(s_mix[s * S + t], old[s], acc);
        now[t] = fmaf(s_out[t], yv, acc);
        if (write_back) x[(size_t)t * W + h] = now[t];
      }
    } else {
#pragma unroll
      for (int t = 0; t < HYPER_MAX_STREAMS; ++t) now[t] = old[t];
    }
    float u = 0.f;
#pragma unroll
    for (int t = 0; t < HYPER_MAX_STREAMS; ++t)
      if (t < S) u = fmaf(s_in[t], now[t], u);
    hyper_u[h] = u;
    ss = fmaf(u, u, ss);
  }
  TOut* o = res + (size_t)r * W;
  if (w == nullptr) {
    for (int h = threadIdx.x; h < W; h += blockDim.x) o[h] = mi::from_float<TOut>(hyper_u[h]);
    return;
  }
  const float rstd = 1.f / sqrtf(mi::block_sum(ss, scratch) / (float)W + eps);
  for (int h = threadIdx.x; h < W; h += blockDim.x) o[h] = mi::from_float<TOut>(w[h] * (hyper_u[h] * rstd));
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
#define MI_HYPER(TO, TD)                                                                                              \
  do {                                                                                                                \
    if (smem > 48 * 1024) cudaFuncSetAttribute(hyper_connection_kernel<TO, TD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    mi::launch(hyper_connection_kernel<TO, TD>, dim3(R), dim3(256), smem, stream, (TO*)res, streams, (const TD*)y, mix, outw, inw, w, rows, S, W, eps, write_back); \
  } while (0)
  if (res_dtype == MI_BF16 && y_dtype == MI_BF16) MI_HYPER(__nv_bfloat16, __nv_bfloat16);
  else if (res_dtype == MI_F32 && y_dtype == MI_F32) MI_HYPER(float, float);
  else if (res_dtype == MI_BF16 && y_dtype == MI_F32) MI_HYPER(__nv_bfloat16, float);
  else if (res_dtype == MI_F32 && y_dtype == MI_BF16) MI_HYPER(float, __nv_bfloat16);
  else return mi_fail("hyper_connection: unknown dtypes res=%d y=%d", res_dtype, y_dtype);
#undef MI_HYPER
  MI_LAUNCH_OK("hyper_connection");
  return 0;
}
