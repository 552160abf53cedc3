// From the rows of a fused query / key / value product to what attention reads: one pass over a token's heads that
//
//   * divides each query and key head by its root mean square over the head, x / sqrt(mean(x^2) + eps),
//     in float32 (optionally times a weight per dimension), and writes the query heads, padded with
//     zeros to the cache's head size, into a packed buffer [token, head, cache head size]; with norm_whole the root
//     mean square is taken over all query heads of the token at once (and over all its key heads), before they are
//     split, and the weights have a value per head and dimension; a bias per projection column (float32) may be added
//     to queries, keys and values first;
//   * optionally rotates the first rot_dims values of each query and key head, after the norm, by the angles of the
//     token's position (a table row: cos of rot_dims / 2 angles, then their sines): value i pairs with value
//     i + rot_dims / 2 (halves) or value 2i with 2i + 1 (interleaved); (u, v) -> (u cos - v sin, v cos + u sin);
//   * mixes the token's value heads with the values another layer made for the same token,
//     v <- (1 - lambda) v + lambda v_other (lambda read from the device), or records them as that
//     other layer's values (v_mode 1), or leaves them alone (v_mode 0);
//   * stores key and value heads into the layer's pages at slot_mapping[token] (page * page_size +
//     offset), padded with zeros.  What is cached is the normalised key and the mixed value.
//
// Key heads have `dim` values and value heads `vdim`; the cache keeps both in rows of `hdp >= max(dim, vdim)`
// values, so a zero tail adds nothing to a score and its output columns are dropped by the attention
// kernels (out_hd).  A warp per (token, head): blocks of four warps, the heads of a token spread over blockIdx.y.
#include "common.cuh"

namespace {

constexpr int PREP_WARPS = 4;
constexpr int PREP_MAX_PER_LANE = 8;   // head sizes up to 256

template <typename T>
struct PrepArgs {
  const T* proj;          // [tokens, proj_stride]: queries at q_off, keys at k_off, values at v_off
  int proj_stride, q_off, k_off, v_off;
  int nh, nkv, dim, vdim, hdp;
  T* q_out;               // [tokens, nh * hdp]
  const float* q_w;       // [dim] ([nh * dim] with norm_whole) or null
  const float* k_w;       // [dim] ([nkv * dim] with norm_whole) or null
  const float* bias;      // indexed like the projection's columns (queries, keys, values): added before anything else; or null
  float eps;
  int normalise;          // 0: queries and keys pass unchanged
  int norm_whole;         // the root mean square runs over all query heads (all key heads) of a token, not a head
  const float* lambda;    // device scalar (v_mode 2)
  T* v_other;             // [tokens, nkv * vdim]: written (v_mode 1) or read (v_mode 2)
  int v_mode;
  const int* slot_mapping;  // null: nothing is stored
  T* kv_layer;            // [page, 2, nkv, page_size, hdp]
  int page_size;
  const float* rope;      // [positions, rot_dims] or null: no rotation
  const int* positions;   // [tokens]
  int rot_dims, interleaved;
};

template <typename T>
__global__ void __launch_bounds__(PREP_WARPS * 32)
qkv_prepare_kernel(PrepArgs<T> a) {
  __shared__ float stage[PREP_WARPS][32 * PREP_MAX_PER_LANE];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int tkn = blockIdx.x;
  const int pos = a.rope ? a.positions[tkn] : 0;
  const float lam = (a.v_mode == 2) ? *a.lambda : 0.f;       // a weight: no kernel writes it
  const int slot = a.slot_mapping ? a.slot_mapping[tkn] : -1;  // part of the step's description
  mi::grid_dependency_sync();
  const T* row = a.proj + (size_t)tkn * a.proj_stride;
  const int units = a.nh + 2 * a.nkv;
  const int page = slot >= 0 ? slot / a.page_size : 0, off = slot >= 0 ? slot % a.page_size : 0;
  // The norm over the whole projection: the block adds up the squares of all of the token's queries, then of all its keys,
  // once for its four heads - every block of the token the same squares in the same order, which depends on the sizes alone.
  float r_whole[2] = {1.f, 1.f};
  if (a.normalise && a.norm_whole) {
    __shared__ float scratch[33];
#pragma unroll
    for (int which = 0; which < 2; ++which) {
      const int n = (which ? a.nkv : a.nh) * a.dim, c0 = which ? a.k_off : a.q_off;
      float sw = 0.f;
      for (int d = threadIdx.x; d < n; d += PREP_WARPS * 32) {
        const float x = mi::to_float(row[c0 + d]) + (a.bias ? a.bias[c0 + d] : 0.f);
        sw = fmaf(x, x, sw);
      }
      r_whole[which] = 1.f / sqrtf(mi::block_sum(sw, scratch) / (float)n + a.eps);
    }
  }
  for (int u = blockIdx.y * PREP_WARPS + warp; u < units; u += PREP_WARPS * gridDim.y) {
    if (u < a.nh + a.nkv) {
      // a query head or a key head
      const bool is_q = u < a.nh;
      const int h = is_q ? u : u - a.nh;
      const int col0 = (is_q ? a.q_off : a.k_off) + h * a.dim;
      const T* src = row + col0;
      const float* w = is_q ? a.q_w : a.k_w;
      if (w && a.norm_whole) w += (size_t)h * a.dim;
      const float* bs = a.bias ? a.bias + col0 : nullptr;
      float v[PREP_MAX_PER_LANE];
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < PREP_MAX_PER_LANE; ++i) {
        const int d = lane + 32 * i;
        v[i] = d < a.dim ? mi::to_float(src[d]) + (bs ? bs[d] : 0.f) : 0.f;
        ss += v[i] * v[i];
      }
      float r = 1.f;
      if (a.normalise && a.norm_whole) r = r_whole[is_q ? 0 : 1];
      else if (a.normalise) r = 1.f / sqrtf(mi::warp_sum(ss) / (float)a.dim + a.eps);
      T* dst = nullptr;
      if (is_q) dst = a.q_out + ((size_t)tkn * a.nh + h) * a.hdp;
      else if (slot >= 0) dst = a.kv_layer + ((((size_t)page * 2 + 0) * a.nkv + h) * a.page_size + off) * a.hdp;
      if (a.rope) {
        // the normalised head through shared memory, so that every value meets its partner
        float* sh = stage[warp];
        const float* cs = a.rope + (size_t)pos * a.rot_dims;
        const int half = a.rot_dims / 2;
#pragma unroll
        for (int i = 0; i < PREP_MAX_PER_LANE; ++i) {
          const int d = lane + 32 * i;
          float y = v[i] * r;
          if (w && d < a.dim) y *= w[d];
          v[i] = y;
          if (d < a.dim) sh[d] = y;
        }
        __syncwarp();
#pragma unroll
        for (int i = 0; i < PREP_MAX_PER_LANE; ++i) {
          const int d = lane + 32 * i;
          if (d < a.rot_dims) {
            const bool first = a.interleaved ? !(d & 1) : d < half;
            const int pi = a.interleaved ? d >> 1 : (first ? d : d - half);
            const int partner = a.interleaved ? d ^ 1 : (first ? d + half : d - half);
            const float c = cs[pi], sn = cs[half + pi], other = sh[partner];
            v[i] = first ? v[i] * c - other * sn : v[i] * c + other * sn;
          }
        }
        __syncwarp();
        if (dst) {
#pragma unroll
          for (int i = 0; i < PREP_MAX_PER_LANE; ++i) {
            const int d = lane + 32 * i;
            if (d < a.hdp) dst[d] = mi::from_float<T>(d < a.dim ? v[i] : 0.f);
          }
        }
      } else if (dst) {
#pragma unroll
        for (int i = 0; i < PREP_MAX_PER_LANE; ++i) {
          const int d = lane + 32 * i;
          if (d < a.hdp) {
            float y = v[i] * r;
            if (w && d < a.dim) y *= w[d];
            dst[d] = mi::from_float<T>(d < a.dim ? y : 0.f);
          }
        }
      }
    } else {
      // a value head
      const int h = u - a.nh - a.nkv;
      const T* src = row + a.v_off + (size_t)h * a.vdim;
      const float* bs = a.bias ? a.bias + a.v_off + h * a.vdim : nullptr;
      T* other = a.v_other ? a.v_other + ((size_t)tkn * a.nkv + h) * a.vdim : nullptr;
      T* dst = slot >= 0 ? a.kv_layer + ((((size_t)page * 2 + 1) * a.nkv + h) * a.page_size + off) * a.hdp : nullptr;
#pragma unroll
      for (int i = 0; i < PREP_MAX_PER_LANE; ++i) {
        const int d = lane + 32 * i;
        if (d >= a.hdp) continue;
        float y = 0.f;
        if (d < a.vdim) {
          y = mi::to_float(src[d]) + (bs ? bs[d] : 0.f);
          if (a.v_mode == 1) other[d] = mi::from_float<T>(y);
          else if (a.v_mode == 2) y = (1.f - lam) * y + lam * mi::to_float(other[d]);
        }
        if (dst) dst[d] = mi::from_float<T>(y);
      }
    }
  }
}


// The same with two values a lane and load (4 bytes of bfloat16, 8 of float32), for the usual case that every size and
// offset is even: a warp's load covers whole 128-byte lines.
template <typename T> struct Pair;
template <> struct Pair<__nv_bfloat16> {
  static __device__ __forceinline__ float2 load(const __nv_bfloat16* p) { return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p)); }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float a, float b) { *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b); }
};
template <> struct Pair<float> {
  static __device__ __forceinline__ float2 load(const float* p) { return *reinterpret_cast<const float2*>(p); }
  static __device__ __forceinline__ void store(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
};

template <typename T>
__global__ void __launch_bounds__(PREP_WARPS * 32)
qkv_prepare_pairs_kernel(PrepArgs<T> a) {
  constexpr int NP = PREP_MAX_PER_LANE / 2;     // pairs a lane
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int tkn = blockIdx.x;
  const float lam = (a.v_mode == 2) ? *a.lambda : 0.f;
  const int slot = a.slot_mapping ? a.slot_mapping[tkn] : -1;
  mi::grid_dependency_sync();
  const T* row = a.proj + (size_t)tkn * a.proj_stride;
  const int units = a.nh + 2 * a.nkv;
  const int page = slot >= 0 ? slot / a.page_size : 0, off = slot >= 0 ? slot % a.page_size : 0;
  for (int u = blockIdx.y * PREP_WARPS + warp; u < units; u += PREP_WARPS * gridDim.y) {
    if (u < a.nh + a.nkv) {
      const bool is_q = u < a.nh;
      const int h = is_q ? u : u - a.nh;
      const T* src = row + (is_q ? a.q_off : a.k_off) + (size_t)h * a.dim;
      const float* w = is_q ? a.q_w : a.k_w;
      float2 v[NP];
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < NP; ++i) {
        const int d = 2 * lane + 64 * i;
        v[i] = d < a.dim ? Pair<T>::load(src + d) : make_float2(0.f, 0.f);
        ss += v[i].x * v[i].x + v[i].y * v[i].y;
      }
      float r = 1.f;
      if (a.normalise) r = 1.f / sqrtf(mi::warp_sum(ss) / (float)a.dim + a.eps);
      T* dst = nullptr;
      if (is_q) dst = a.q_out + ((size_t)tkn * a.nh + h) * a.hdp;
      else if (slot >= 0) dst = a.kv_layer + ((((size_t)page * 2 + 0) * a.nkv + h) * a.page_size + off) * a.hdp;
      if (dst) {
#pragma unroll
        for (int i = 0; i < NP; ++i) {
          const int d = 2 * lane + 64 * i;
          if (d < a.hdp) {
            float y0 = v[i].x * r, y1 = v[i].y * r;
            if (w && d < a.dim) { y0 *= w[d]; y1 *= w[d + 1]; }
            Pair<T>::store(dst + d, d < a.dim ? y0 : 0.f, d < a.dim ? y1 : 0.f);
          }
        }
      }
    } else {
      const int h = u - a.nh - a.nkv;
      const T* src = row + a.v_off + (size_t)h * a.vdim;
      T* other = a.v_other ? a.v_other + ((size_t)tkn * a.nkv + h) * a.vdim : nullptr;
      T* dst = slot >= 0 ? a.kv_layer + ((((size_t)page * 2 + 1) * a.nkv + h) * a.page_size + off) * a.hdp : nullptr;
#pragma unroll
      for (int i = 0; i < NP; ++i) {
        const int d = 2 * lane + 64 * i;
        if (d >= a.hdp) continue;
        float2 y = make_float2(0.f, 0.f);
        if (d < a.vdim) {
          y = Pair<T>::load(src + d);
          if (a.v_mode == 1) Pair<T>::store(other + d, y.x, y.y);
          else if (a.v_mode == 2) {
            const float2 o = Pair<T>::load(other + d);
            y.x = (1.f - lam) * y.x + lam * o.x;
            y.y = (1.f - lam) * y.y + lam * o.y;
          }
        }
        if (dst) Pair<T>::store(dst + d, y.x, y.y);
      }
    }
  }
}

}  // namespace

MI_API int mi_qkv_norm_mix_store(const void* proj, int dtype, int proj_stride, int q_off, int k_off, int v_off, int T, int nh,
                                 int nkv, int dim, int vdim, int hdp, void* q_out, const float* q_w, const float* k_w,
                                 float eps, int normalise, const float* lambda, void* v_other, int v_mode,
                                 const int* slot_mapping, void* kv_layer, int page_size, const float* rope, const int* positions,
                                 int rot_dims, int interleaved, const float* bias, int norm_whole, cudaStream_t stream) {
  MI_REQUIRE(rope == nullptr || (positions != nullptr && rot_dims > 0 && rot_dims % 2 == 0 && rot_dims <= dim),
             "qkv_prepare: a rotation needs positions and an even number of rotated values, at most dim=%d (got %d)", dim, rot_dims);
  MI_REQUIRE(T >= 0 && nh > 0 && nkv > 0 && dim > 0 && vdim > 0 && nh + 2 * nkv <= 4 * 65535, "qkv_prepare: bad sizes");
  MI_REQUIRE(hdp >= dim && hdp >= vdim && hdp <= 32 * PREP_MAX_PER_LANE, "qkv_prepare: cache head size %d must cover dim=%d and vdim=%d, up to %d",
             hdp, dim, vdim, 32 * PREP_MAX_PER_LANE);
  MI_REQUIRE(v_mode >= 0 && v_mode <= 2 && (v_mode == 0 || v_other != nullptr) && (v_mode != 2 || lambda != nullptr),
             "qkv_prepare: value mixing needs the other layer's values and lambda");
  MI_REQUIRE(slot_mapping == nullptr || (kv_layer != nullptr && page_size > 0), "qkv_prepare: a store needs the cache layer");
  if (T == 0) return 0;
  const size_t es = dtype == MI_BF16 ? 2 : 4;
  const bool pairs = rope == nullptr && bias == nullptr && !norm_whole && dim % 2 == 0 && vdim % 2 == 0 && hdp % 2 == 0 && proj_stride % 2 == 0 && q_off % 2 == 0 && k_off % 2 == 0 && v_off % 2 == 0 &&
                     ((uintptr_t)proj % (2 * es)) == 0 && ((uintptr_t)q_out % (2 * es)) == 0 && ((uintptr_t)kv_layer % (2 * es)) == 0 &&
                     ((uintptr_t)v_other % (2 * es)) == 0;
#define MI_PREP(TT)                                                                                          \
  do {                                                                                                       \
    PrepArgs<TT> a;                                                                                          \
    a.proj = (const TT*)proj; a.proj_stride = proj_stride; a.q_off = q_off; a.k_off = k_off; a.v_off = v_off; \
    a.nh = nh; a.nkv = nkv; a.dim = dim; a.vdim = vdim; a.hdp = hdp; a.q_out = (TT*)q_out; a.q_w = q_w; a.k_w = k_w; \
    a.eps = eps; a.normalise = normalise; a.lambda = lambda; a.v_other = (TT*)v_other; a.v_mode = v_mode;     \
    a.slot_mapping = slot_mapping; a.kv_layer = (TT*)kv_layer; a.page_size = page_size;                      \
    a.rope = rope; a.positions = positions; a.rot_dims = rot_dims; a.interleaved = interleaved;              \
    a.bias = bias; a.norm_whole = norm_whole;                                                                \
    if (pairs) mi::launch(qkv_prepare_pairs_kernel<TT>, dim3(T, (nh + 2 * nkv + PREP_WARPS - 1) / PREP_WARPS), dim3(PREP_WARPS * 32), 0, stream, a); \
    else mi::launch(qkv_prepare_kernel<TT>, dim3(T, (nh + 2 * nkv + PREP_WARPS - 1) / PREP_WARPS), dim3(PREP_WARPS * 32), 0, stream, a);                        \
  } while (0)
  if (dtype == MI_BF16) MI_PREP(__nv_bfloat16);
  else if (dtype == MI_F32) MI_PREP(float);
  else return mi_fail("qkv_prepare: unknown dtype %d", dtype);
#undef MI_PREP
  MI_LAUNCH_OK("qkv_prepare");
  return 0;
}
