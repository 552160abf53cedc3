// Token embedding: out[t, :] = scale * table[ids[t], :], written as float32 because the result is the
// start of the residual stream, which is kept in 32-bit (scale is 1 for models that do not scale).  With
// copies > 1 a row of out holds the looked-up row that many times side by side (residual streams that start equal).
// Stands where the reference indexes the table in torch (miniinfer/layers/embedding.py:23-27).
#include "common.cuh"

namespace {

template <typename T>
__global__ void embedding_kernel(float* __restrict__ out, const T* __restrict__ table,
                                 const int* __restrict__ ids, int H, float scale, int copies) {
  mi::grid_dependency_sync();
  const int t = blockIdx.x;
  const T* row = table + (size_t)ids[t] * H;
  float* o = out + (size_t)t * H * copies;
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    const float v = mi::to_float(row[h]) * scale;
    for (int c = 0; c < copies; ++c) o[(size_t)c * H + h] = v;
  }
}

}  // namespace

// ids must already be known to lie in [0, V): the caller builds them on the host and checks there.
MI_API int mi_embedding(float* out, const void* table, int table_dtype, const int* ids, int T, int H,
                        float scale, int copies, cudaStream_t stream) {
  MI_REQUIRE(T >= 0 && H > 0 && copies >= 1, "embedding: bad sizes T=%d H=%d copies=%d", T, H, copies);
  if (T == 0) return 0;
  const int threads = H >= 1024 ? 256 : 128;
  if (table_dtype == MI_BF16)
    mi::launch(embedding_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, out, (const __nv_bfloat16*)table, ids, H, scale, copies);
  else if (table_dtype == MI_F32)
    mi::launch(embedding_kernel<float>, dim3(T), dim3(threads), 0, stream, out, (const float*)table, ids, H, scale, copies);
  else
    return mi_fail("embedding: unknown table dtype %d", table_dtype);
  MI_LAUNCH_OK("embedding");
  return 0;
}
