// Linear attention with a decaying matrix state: gated linear attention (a decay per token and key channel) and
// retention (one fixed decay per head).  Per head, with the state S [dim, vdim], token after token:
//
//   S[i, :] <- g[i] * S[i, :] + k[i] * v[:]        g = the token's decay of key channel i, or the head's constant
//   o[:]     = sum_i q[i] * S[i, :]                 (the read-out sees the token's own write)
//   out[t, head, :] = o / sqrt(mean(o^2) + eps) * norm_w * act(gate[t, head, :])     norm_w optional, act = silu or sigmoid
//
// A step brings, for each of its items, q_len[b] new tokens in rows q_start[b] .. of the activations; the item's state
// is row seq_slot[b] of the layer's state tensor, float32, zero when the request was admitted.  Three kernels, as for
// the gated delta rule (recurrent.cu).  (1) linear_prepare, a warp per (token, head), all tokens at once: what does not
// depend on the state - q and k rotated by the token's position (optional; the first rot_dims values of a head, value i
// with value i + rot_dims / 2) and scaled, the decays g = sigmoid(z)^(1/tau) = exp(logsigmoid(z) / tau) from their
// logits z = a + bias, the values - as float32 rows.  (2) linear_recurrence, the only part that walks the tokens in
// order: a block per (item, head, group of value columns); thread (j, r) keeps rows r * DK .. r * DK + DK - 1 of
// CPT neighbouring columns of S in registers (four, so that a query, key and decay value fetched from shared memory
// serves four columns: with one column a thread the warps mostly waited on shared-memory loads), the R threads of
// a column are neighbouring lanes and add their partial sums by shuffles; the tokens' vectors come through shared
// memory in chunks, by asynchronous copies into two buffers.
// (3) linear_output, a warp per (token, head): root mean square over the head, weight, gate.
//
// Everything between the projections and the gate is float32: angles (a table made on the host), decays and their
// logarithms, the state and the sums over it, the norm.
#include "common.cuh"

namespace {

__device__ __forceinline__ float lin_sigmoid(float z) { return 1.f / (1.f + expf(-z)); }
// log(sigmoid(z)) without cancellation: min(z, 0) - log1p(exp(-|z|))
__device__ __forceinline__ float lin_log_sigmoid(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

template <typename T, typename TA>
struct LinPrepArgs {
  const T* q; int ldq;                   // head h at column h * dim
  const T* k; int ldk;
  const T* v; int ldv;                   // head h at column h * vdim
  const TA* a; int lda;                  // decay logits, head h at column h * dim; null: the decay is a constant a head
  const float* a_bias;                   // [heads * dim] or null
  float inv_tau;
  const float* rope;                     // [positions, rot_dims]: cos of rot_dims / 2 angles, then their sines; null: no rotation
  const int* positions;
  int rot_dims;
  float q_scale, k_scale;
  float* qn; float* kn;                  // [tokens, heads * dim]
  float* g;                              // [tokens, heads * dim]
  float* raw;                            // [tokens, heads * vdim]: the values as float32; the recurrence writes its read-outs over them
  int heads, dim, vdim;
};

template <typename T, typename TA>
__global__ void __launch_bounds__(128)
linear_prepare_kernel(LinPrepArgs<T, TA> a) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x;
  const int pos = a.rope ? a.positions[t] : 0;        // part of the step's description
  mi::grid_dependency_sync();
  const int half = a.rot_dims / 2;
  const float* cs = a.rope ? a.rope + (size_t)pos * a.rot_dims : nullptr;
  for (int h = blockIdx.y * 4 + warp; h < a.heads; h += 4 * gridDim.y) {
    const T* q = a.q + (size_t)t * a.ldq + (size_t)h * a.dim;
    const T* k = a.k + (size_t)t * a.ldk + (size_t)h * a.dim;
    float* qo = a.qn + ((size_t)t * a.heads + h) * a.dim;
    float* ko = a.kn + ((size_t)t * a.heads + h) * a.dim;
    for (int i = lane; i < a.dim; i += 32) {
      float x = mi::to_float(q[i]), y = mi::to_float(k[i]);
      if (cs && i < a.rot_dims) {
        const bool first = i < half;
        const int pi = first ? i : i - half, partner = first ? i + half : i - half;
        const float c = cs[pi], s = cs[half + pi];
        const float xo = mi::to_float(q[partner]), yo = mi::to_float(k[partner]);
        x = first ? x * c - xo * s : x * c + xo * s;
        y = first ? y * c - yo * s : y * c + yo * s;
      }
      qo[i] = x * a.q_scale;
      ko[i] = y * a.k_scale;
    }
    if (a.a) {
      for (int i = lane; i < a.dim; i += 32) {
        float z = mi::to_float(a.a[(size_t)t * a.lda + (size_t)h * a.dim + i]);
        if (a.a_bias) z += a.a_bias[h * a.dim + i];
        a.g[((size_t)t * a.heads + h) * a.dim + i] = expf(lin_log_sigmoid(z) * a.inv_tau);
      }
    }
    for (int j = lane; j < a.vdim; j += 32)
      a.raw[((size_t)t * a.heads + h) * a.vdim + j] = mi::to_float(a.v[(size_t)t * a.ldv + (size_t)h * a.vdim + j]);
  }
}

// 4 bytes from global to shared memory without a register in between; zeros if not `take`
__device__ __forceinline__ void lin_copy4(float* dst, const float* src, bool take) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
  const int bytes = take ? 4 : 0;
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}

// 16 bytes at a time (both addresses 16-byte aligned)
__device__ __forceinline__ void lin_copy16(float* dst, const float* src, bool take) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
  const int bytes = take ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}

constexpr int LIN_THREADS = 128;
constexpr int LIN_CHUNK = 16;            // tokens whose vectors are in shared memory at a time
constexpr int LIN_SEGMENTS = 16;
constexpr int LIN_SEGMENT_MIN = 96;      // tokens a stretch has at least

__host__ __device__ __forceinline__ int lin_segments(int n_new) { return max(1, min(LIN_SEGMENTS, n_new / LIN_SEGMENT_MIN)); }
__host__ __device__ __forceinline__ int lin_segment_len(int n_new, int nseg) {
  return ((n_new + nseg - 1) / nseg + LIN_CHUNK - 1) / LIN_CHUNK * LIN_CHUNK;
}

struct LinArgs {
  float* raw;                            // [tokens, heads * vdim]: the values in, the read-outs before norm and gate out
  const float* qn; const float* kn;
  const float* g;                        // per token and key channel (CHANNEL) ...
  const float* head_decay;               // ... or one constant a head
  float* state; long long state_stride;  // [slot][heads][dim][vdim]
  const int* q_start; const int* q_len; const int* seq_slot;
  int heads, dim, vdim, R;
  // stretches side by side (MODE 1, 2)
  float* seg_state;                      // [item, stretch][heads][dim][vdim]: a stretch's end state from a zero start (MODE 1
                                         // writes), then - after the carry kernel - the state it starts from (MODE 2 reads)
  float* seg_decay;                      // [item, stretch][heads][dim]: the product of the stretch's decays, row by row
};

// MODE 0: an item's tokens in order, from the stored state to the stored state (every sum in an order that depends on
// the position alone).  MODE 1 and 2, for long prompt portions in bfloat16: the tokens in stretches side by side.  The
// state after a token is linear in the state before it, and the map is diagonal: a stretch's end state is (the product
// of its decays, row by row) x (the state it starts from) + (its end state from a zero start).  MODE 1 walks every
// stretch from zero and keeps the end state and the product; the carry kernel chains the stretches; MODE 2 walks every
// stretch again from the state it really starts from and writes the read-outs.
template <int DK, int CPT, int MODE, bool CHANNEL>
__global__ void __launch_bounds__(LIN_THREADS)
linear_recurrence_kernel(LinArgs a) {
  extern __shared__ __align__(16) float sm[];
  constexpr int LD = DK + 4;             // a thread's stretch of a vector, padded: 16-byte loads without bank conflicts
  constexpr int NV = CHANNEL ? 3 : 2;    // vectors a token: q, k and, with decays per channel, g
  const int item = MODE == 0 ? blockIdx.y : blockIdx.y / LIN_SEGMENTS, head = blockIdx.x;
  const int seg = MODE == 0 ? 0 : blockIdx.y % LIN_SEGMENTS;
  int row0 = a.q_start[item], n_new = a.q_len[item];
  const int slot = a.seq_slot[item];
  const float hd = CHANNEL ? 1.f : a.head_decay[head];     // a constant of the model
  if (MODE != 0) {
    const int nseg = lin_segments(n_new);
    if (seg >= nseg) return;
    const int len = lin_segment_len(n_new, nseg);
    row0 += seg * len;
    n_new = max(0, min(len, n_new - seg * len));
  }
  const int R = a.R, dim = a.dim, vdim = a.vdim;
  const int cols = LIN_THREADS / R * CPT;                 // value columns of the block, CPT neighbouring ones a thread
  const int cl = threadIdx.x / R, r = threadIdx.x % R;
  const int col = blockIdx.z * cols + cl * CPT;            // the thread's first column
  const int vec = R * LD;                                  // floats of one padded vector
  const int tok_floats = NV * vec + cols;                  // q, k, (g,) the block's values
  mi::grid_dependency_sync();
  const size_t seg_at = ((size_t)(item * LIN_SEGMENTS + seg) * a.heads + head) * dim;
  float* st = MODE == 0 ? a.state + (size_t)slot * a.state_stride + (size_t)head * dim * vdim : a.seg_state + seg_at * vdim;
  float S[CPT][DK], P[MODE == 1 ? DK : 1];
#pragma unroll
  for (int i = 0; i < DK; ++i) {
    const int row = r * DK + i;
#pragma unroll
    for (int c = 0; c < CPT; ++c) S[c][i] = (MODE != 1 && col + c < vdim && row < dim) ? st[(size_t)row * vdim + col + c] : 0.f;
    if (MODE == 1) P[i] = 1.f;
  }
  // Rows past dim and columns past vdim are filled with zeros (a zero key and query row leave such a row of S at zero
  // and out of the sums).
  const int chunk_floats = LIN_CHUNK * tok_floats;
  // Sizes that are multiples of 4 move 16 bytes a copy (the scratch rows then start on 16-byte boundaries); the first
  // pass of the stretches does not read the queries.
  const bool vec4 = dim % 4 == 0 && vdim % 4 == 0 && cols % 4 == 0;
  const int per = R * DK / 4, per_shift = __ffs(per) - 1;          // 16-byte pieces of a padded vector: a power of two
  const int cq = cols / 4, cq_shift = __ffs(cq > 0 ? cq : 1) - 1;
  auto fetch = [&](int c0, float* buf) {
    const int n = min(LIN_CHUNK, n_new - c0);
    if (vec4) {
      for (int idx = threadIdx.x; idx < n * per; idx += LIN_THREADS) {
        const int tt = idx >> per_shift, i = (idx & (per - 1)) * 4;
        const size_t t = (size_t)(row0 + c0 + tt);
        float* base = buf + (size_t)tt * tok_floats + (i / DK) * LD + (i % DK);
        const bool in = i < dim;
        const size_t at = (t * a.heads + head) * dim + (in ? i : 0);
        if (MODE != 1) lin_copy16(base, a.qn + at, in);
        lin_copy16(base + vec, a.kn + at, in);
        if (CHANNEL) lin_copy16(base + 2 * vec, a.g + at, in);
      }
      for (int idx = threadIdx.x; idx < n * cq; idx += LIN_THREADS) {
        const int tt = idx >> cq_shift, j = (idx & (cq - 1)) * 4;
        const int c = blockIdx.z * cols + j;
        lin_copy16(buf + (size_t)tt * tok_floats + NV * vec + j, a.raw + (size_t)(row0 + c0 + tt) * (a.heads * vdim) + head * vdim + (c < vdim ? c : 0), c < vdim);
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
      return;
    }
    for (int idx = threadIdx.x; idx < n * R * DK; idx += LIN_THREADS) {
      const int tt = idx / (R * DK), i = idx % (R * DK);
      const size_t t = (size_t)(row0 + c0 + tt);
      float* base = buf + (size_t)tt * tok_floats + (i / DK) * LD + (i % DK);
      const bool in = i < dim;
      const size_t at = (t * a.heads + head) * dim + (in ? i : 0);
      lin_copy4(base, a.qn + at, in);
      lin_copy4(base + vec, a.kn + at, in);
      if (CHANNEL) lin_copy4(base + 2 * vec, a.g + at, in);
    }
    for (int idx = threadIdx.x; idx < n * cols; idx += LIN_THREADS) {
      const int tt = idx / cols, j = idx % cols;
      const int c = blockIdx.z * cols + j;
      lin_copy4(buf + (size_t)tt * tok_floats + NV * vec + j, a.raw + (size_t)(row0 + c0 + tt) * (a.heads * vdim) + head * vdim + (c < vdim ? c : 0), c < vdim);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  if (n_new > 0) fetch(0, sm);
  for (int c0 = 0, ci = 0; c0 < n_new; c0 += LIN_CHUNK, ++ci) {
    const int n = min(LIN_CHUNK, n_new - c0);
    float* cur = sm + (size_t)(ci & 1) * chunk_floats;
    if (c0 + LIN_CHUNK < n_new) {
      fetch(c0 + LIN_CHUNK, sm + (size_t)((ci + 1) & 1) * chunk_floats);      // that buffer's chunk was finished before the barrier below
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    // One token: the state's rows of this thread decay and take the token's key x value; returns the thread's part of
    // the read-out (MODE 1: nothing is read out).
    auto token = [&](int tt, float (&o)[CPT]) {
      const float* base = cur + (size_t)tt * tok_floats;
      const float4* qv = reinterpret_cast<const float4*>(base + r * LD);
      const float4* kv = reinterpret_cast<const float4*>(base + vec + r * LD);
      const float4* gv = reinterpret_cast<const float4*>(base + 2 * vec + r * LD);
      float vj[CPT];
      if constexpr (CPT == 4) {
        const float4 v4 = *reinterpret_cast<const float4*>(base + NV * vec + cl * 4);
        vj[0] = v4.x; vj[1] = v4.y; vj[2] = v4.z; vj[3] = v4.w;
      } else {
#pragma unroll
        for (int c = 0; c < CPT; ++c) vj[c] = base[NV * vec + cl * CPT + c];
      }
      float os[CPT][4];
#pragma unroll
      for (int c = 0; c < CPT; ++c) os[c][0] = os[c][1] = os[c][2] = os[c][3] = 0.f;
#pragma unroll
      for (int i = 0; i < DK / 4; ++i) {
        const float4 k4 = kv[i];
        float4 g4 = make_float4(hd, hd, hd, hd), q4 = make_float4(0.f, 0.f, 0.f, 0.f);
        if (CHANNEL) g4 = gv[i];
        if (MODE != 1) q4 = qv[i];
#pragma unroll
        for (int c = 0; c < CPT; ++c) {
          float* Sc = S[c] + 4 * i;
          Sc[0] = fmaf(g4.x, Sc[0], k4.x * vj[c]); Sc[1] = fmaf(g4.y, Sc[1], k4.y * vj[c]);
          Sc[2] = fmaf(g4.z, Sc[2], k4.z * vj[c]); Sc[3] = fmaf(g4.w, Sc[3], k4.w * vj[c]);
          if (MODE != 1) {
            os[c][0] = fmaf(q4.x, Sc[0], os[c][0]); os[c][1] = fmaf(q4.y, Sc[1], os[c][1]);
            os[c][2] = fmaf(q4.z, Sc[2], os[c][2]); os[c][3] = fmaf(q4.w, Sc[3], os[c][3]);
          }
        }
        if (MODE == 1) {
          P[4 * i] *= g4.x; P[4 * i + 1] *= g4.y; P[4 * i + 2] *= g4.z; P[4 * i + 3] *= g4.w;
        }
      }
#pragma unroll
      for (int c = 0; c < CPT; ++c) o[c] = (os[c][0] + os[c][1]) + (os[c][2] + os[c][3]);
    };
    float* orow = a.raw + (size_t)(row0 + c0) * (a.heads * vdim) + head * vdim + col;
    constexpr int GROUP = 8;                 // tokens whose read-outs are added up together
    if (DK == 16 && n == LIN_CHUNK) {          // (more rows a thread leave no registers for eight tokens at once)
      // A whole chunk: its tokens unrolled, eight at a time, and the threads of a column add up the read-outs of all
      // eight together - independent chains of shuffles instead of one after every token.  Token by token the sums
      // are those of the loop below, in the same order.
#pragma unroll
      for (int t0 = 0; t0 < LIN_CHUNK; t0 += GROUP) {
        float oj[GROUP][CPT];
#pragma unroll
        for (int tt = 0; tt < GROUP; ++tt) token(t0 + tt, oj[tt]);
        if (MODE != 1) {
          for (int o = R >> 1; o > 0; o >>= 1) {
#pragma unroll
            for (int tt = 0; tt < GROUP; ++tt)
#pragma unroll
              for (int c = 0; c < CPT; ++c) oj[tt][c] += __shfl_xor_sync(0xffffffffu, oj[tt][c], o);
          }
          if (r == 0) {
#pragma unroll
            for (int tt = 0; tt < GROUP; ++tt)
#pragma unroll
              for (int c = 0; c < CPT; ++c)
                if (col + c < vdim) orow[(size_t)(t0 + tt) * (a.heads * vdim) + c] = oj[tt][c];
          }
        }
      }
    } else {
      for (int tt = 0; tt < n; ++tt) {
        float oj[CPT];
        token(tt, oj);
        if (MODE != 1) {                        // the first pass of the stretches keeps the state only
          for (int o = R >> 1; o > 0; o >>= 1) {
#pragma unroll
            for (int c = 0; c < CPT; ++c) oj[c] += __shfl_xor_sync(0xffffffffu, oj[c], o);
          }
          if (r == 0) {
#pragma unroll
            for (int c = 0; c < CPT; ++c)
              if (col + c < vdim) orow[(size_t)tt * (a.heads * vdim) + c] = oj[c];
          }
        }
      }
    }
    __syncthreads();      // everyone is done with this buffer before the fetch after next fills it
  }
  if (MODE != 2) {
#pragma unroll
    for (int i = 0; i < DK; ++i) {
      const int row = r * DK + i;
      if (row >= dim) continue;
#pragma unroll
      for (int c = 0; c < CPT; ++c)
        if (col + c < vdim) st[(size_t)row * vdim + col + c] = S[c][i];
      if (MODE == 1 && col == 0) a.seg_decay[seg_at + row] = P[i];
    }
  }
}

// Chains an item's stretches, a thread per (row i, column j) of a head's state: carry_0 = the stored state,
// carry_(s+1)[i, j] = decay_s[i] * carry_s[i, j] + end_s[i, j].  The carries replace the end states in seg_state; the
// last becomes the stored state.
__global__ void __launch_bounds__(256)
linear_carry_kernel(float* __restrict__ seg_state, const float* __restrict__ seg_decay, float* __restrict__ state,
                    long long state_stride, const int* __restrict__ q_len, const int* __restrict__ seq_slot, int heads, int dim, int vdim) {
  const int head = blockIdx.x, item = blockIdx.y;
  const int nseg = lin_segments(q_len[item]);
  const int slot = seq_slot[item];
  mi::grid_dependency_sync();
  float* st = state + (size_t)slot * state_stride + (size_t)head * dim * vdim;
  for (int e = blockIdx.z * blockDim.x + threadIdx.x; e < dim * vdim; e += gridDim.z * blockDim.x) {
    const int i = e / vdim;
    // every stretch's end state and decay first, all loads in flight at once; then the chain, which is arithmetic only
    float end[LIN_SEGMENTS], dec[LIN_SEGMENTS];
#pragma unroll
    for (int s = 0; s < LIN_SEGMENTS; ++s) {
      const size_t at = ((size_t)(item * LIN_SEGMENTS + s) * heads + head) * dim;
      end[s] = s < nseg ? seg_state[at * vdim + e] : 0.f;
      dec[s] = s < nseg ? seg_decay[at + i] : 1.f;
    }
    float c = st[e];
#pragma unroll
    for (int s = 0; s < LIN_SEGMENTS; ++s) {
      if (s >= nseg) break;
      const size_t at = ((size_t)(item * LIN_SEGMENTS + s) * heads + head) * dim;
      seg_state[at * vdim + e] = c;
      c = fmaf(dec[s], c, end[s]);
    }
    st[e] = c;
  }
}

template <typename T>
__global__ void __launch_bounds__(128)
linear_output_kernel(T* __restrict__ out, int ldo, const float* __restrict__ raw, const T* __restrict__ gate, int ldg,
                     const float* __restrict__ norm_w, int heads, int vdim, float eps, int gate_silu) {
  mi::grid_dependency_sync();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x;
  for (int h = blockIdx.y * 4 + warp; h < heads; h += 4 * gridDim.y) {
    const float* o = raw + ((size_t)t * heads + h) * vdim;
    float ss = 0.f;
    for (int j = lane; j < vdim; j += 32) ss = fmaf(o[j], o[j], ss);
    ss = mi::warp_sum(ss);
    const float rstd = 1.f / sqrtf(ss / (float)vdim + eps);
    for (int j = lane; j < vdim; j += 32) {
      float y = o[j] * rstd;
      if (norm_w) y *= norm_w[j];
      if (gate) {
        const float gl = mi::to_float(gate[(size_t)t * ldg + h * vdim + j]);
        y *= gate_silu ? gl * lin_sigmoid(gl) : lin_sigmoid(gl);
      }
      out[(size_t)t * ldo + h * vdim + j] = mi::from_float<T>(y);
    }
  }
}

}  // namespace

// scratch: float32, tokens * heads * (2 * dim + (per-channel decays ? dim : 0) + vdim) values
MI_API long long mi_linear_attention_scratch_floats(int T, int heads, int dim, int vdim, int channel_decay) {
  return (long long)T * heads * ((long long)(channel_decay ? 3 : 2) * dim + vdim) + 16;
}

MI_API int mi_linear_attention_segments() { return LIN_SEGMENTS; }

// value columns a thread keeps beside one another: four while the state fits its registers
static int lin_cpt(int DK) { return DK <= 32 ? 4 : 1; }

static void lin_tiling(int dim, int* DK, int* R) {
  int dk = dim <= 128 ? 16 : 32, r = 1;
  for (;; dk *= 2) {
    r = 1;
    while (r * dk < dim) r *= 2;
    if (r <= 32 || dk == 128) break;
  }
  *DK = dk;
  *R = r;
}

// Blocks that walk one request's tokens in order (heads x groups of value columns): what a long prompt portion keeps
// busy without stretches side by side.
MI_API int mi_linear_attention_blocks(int heads, int dim, int vdim) {
  int DK, R;
  lin_tiling(dim, &DK, &R);
  const int cols = LIN_THREADS / (R > 32 ? 32 : R) * lin_cpt(DK);
  return heads * ((vdim + cols - 1) / cols);
}

// out [T, heads * vdim] (row stride ldo); q, k [T, heads * dim] and v, gate [T, heads * vdim] column ranges of wider rows
// of the activations' dtype; a: the decays' logits [T, heads * dim] float32 (row stride lda) with a_bias and inv_tau, or
// null - then head_decay [heads] holds one constant a head.  rope [positions, rot_dims] float32 or null.
// segments: null, or items * LIN_SEGMENTS * heads * dim * (vdim + 1) floats of scratch - then the items' tokens run in
// stretches side by side (bfloat16 only: the sums then depend on where a portion starts).
MI_API int mi_linear_attention(void* out, int ldo, const void* q, int ldq, const void* k, int ldk, const void* v, int ldv,
                               const void* gate, int ldg, int dtype, const float* a_in, int lda, const float* a_bias, float inv_tau,
                               const float* head_decay, const float* rope, const int* positions, int rot_dims, float q_scale,
                               float k_scale, const float* norm_w, float eps, int gate_silu, float* state, long long state_stride,
                               const int* q_start, const int* q_len, const int* seq_slot, int T, int items, int heads, int dim,
                               int vdim, float* scratch, float* segments, cudaStream_t stream) {
  MI_REQUIRE(T >= 0 && items >= 0 && items <= 65535 && heads > 0 && heads <= 65535, "linear_attention: bad counts T=%d items=%d heads=%d", T, items, heads);
  MI_REQUIRE(dim > 0 && vdim > 0 && dim <= 4096, "linear_attention: bad sizes dim=%d vdim=%d", dim, vdim);
  MI_REQUIRE((a_in != nullptr) != (head_decay != nullptr), "linear_attention: decays come per channel (logits) or per head (constants), one of the two");
  MI_REQUIRE(rope == nullptr || (positions != nullptr && rot_dims > 0 && rot_dims % 2 == 0 && rot_dims <= dim),
             "linear_attention: a rotation needs positions and an even number of rotated values, at most dim=%d (got %d)", dim, rot_dims);
  MI_REQUIRE(segments == nullptr || (dtype == MI_BF16 && items * LIN_SEGMENTS <= 65535), "linear_attention: stretches side by side are for bfloat16 activations");
  MI_REQUIRE(state_stride >= (long long)heads * dim * vdim, "linear_attention: the state rows are too short");
  MI_REQUIRE(scratch != nullptr && ((uintptr_t)scratch % 16) == 0, "linear_attention: the scratch buffer is missing or unaligned");
  MI_REQUIRE(eps > 0.f, "linear_attention: eps must be positive");
  if (items == 0 || T == 0) return 0;
  int DK, R;
  lin_tiling(dim, &DK, &R);
  MI_REQUIRE(R <= 32, "linear_attention: dim=%d is more than a block's threads can keep", dim);
  const bool channel = a_in != nullptr;
  const int cols = LIN_THREADS / R * lin_cpt(DK);
  const int tok_floats = (channel ? 3 : 2) * R * (DK + 4) + cols;
  const size_t smem = (size_t)2 * LIN_CHUNK * tok_floats * sizeof(float);
  MI_REQUIRE(smem <= 200 * 1024, "linear_attention: a chunk's vectors (%zu bytes) do not fit shared memory", smem);
  const size_t hd = (size_t)T * heads * dim;
  float* qn = scratch;
  float* kn = qn + hd;
  float* g = kn + hd;                                   // used with per-channel decays only
  float* raw = g + (channel ? hd : 0);
  raw += (4 - ((size_t)(raw - scratch) & 3)) & 3;
  const int hy = (heads + 3) / 4 > 16 ? 16 : (heads + 3) / 4;
  dim3 pgrid(T, hy), ogrid(T, hy);
  dim3 rgrid(heads, items, (vdim + cols - 1) / cols);
  LinArgs d;
  d.raw = raw; d.qn = qn; d.kn = kn; d.g = g; d.head_decay = head_decay;
  d.state = state; d.state_stride = state_stride; d.q_start = q_start; d.q_len = q_len; d.seq_slot = seq_slot;
  d.heads = heads; d.dim = dim; d.vdim = vdim; d.R = R;
  d.seg_state = segments;
  d.seg_decay = segments ? segments + (size_t)items * LIN_SEGMENTS * heads * dim * vdim : nullptr;
#define MI_LIN_REC(DKV, CPTV, CH)                                                                                          \
  do {                                                                                                               \
    if (!segments) {                                                                                                 \
      if (smem > 48 * 1024) cudaFuncSetAttribute(linear_recurrence_kernel<DKV, CPTV, 0, CH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      mi::launch(linear_recurrence_kernel<DKV, CPTV, 0, CH>, rgrid, dim3(LIN_THREADS), smem, stream, d);                   \
    } else {                                                                                                         \
      if (smem > 48 * 1024) {                                                                                        \
        cudaFuncSetAttribute(linear_recurrence_kernel<DKV, CPTV, 1, CH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        cudaFuncSetAttribute(linear_recurrence_kernel<DKV, CPTV, 2, CH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      }                                                                                                              \
      dim3 sgrid(heads, items * LIN_SEGMENTS, rgrid.z);                                                              \
      mi::launch(linear_recurrence_kernel<DKV, CPTV, 1, CH>, sgrid, dim3(LIN_THREADS), smem, stream, d);                   \
      const int cz = (dim * vdim + 255) / 256 > 64 ? 64 : (dim * vdim + 255) / 256;                                    \
      mi::launch(linear_carry_kernel, dim3(heads, items, cz), dim3(256), 0, stream, d.seg_state, (const float*)d.seg_decay, state, \
                 state_stride, q_len, seq_slot, heads, dim, vdim);                                                   \
      mi::launch(linear_recurrence_kernel<DKV, CPTV, 2, CH>, sgrid, dim3(LIN_THREADS), smem, stream, d);                   \
    }                                                                                                                \
  } while (0)
#define MI_LIN_DK(CH)                                                                                                \
  do {                                                                                                               \
    if (DK == 16) MI_LIN_REC(16, 4, CH);                                                                             \
    else if (DK == 32) MI_LIN_REC(32, 4, CH);                                                                        \
    else if (DK == 64) MI_LIN_REC(64, 1, CH);                                                                        \
    else MI_LIN_REC(128, 1, CH);                                                                                     \
  } while (0)
#define MI_LIN_ALL(TT)                                                                                               \
  do {                                                                                                               \
    LinPrepArgs<TT, float> p;                                                                                        \
    p.q = (const TT*)q; p.ldq = ldq; p.k = (const TT*)k; p.ldk = ldk; p.v = (const TT*)v; p.ldv = ldv;               \
    p.a = a_in; p.lda = lda; p.a_bias = a_bias; p.inv_tau = inv_tau; p.rope = rope; p.positions = positions;         \
    p.rot_dims = rot_dims; p.q_scale = q_scale; p.k_scale = k_scale; p.qn = qn; p.kn = kn; p.g = g; p.raw = raw;     \
    p.heads = heads; p.dim = dim; p.vdim = vdim;                                                                     \
    mi::launch(linear_prepare_kernel<TT, float>, pgrid, dim3(128), 0, stream, p);                                    \
    if (channel) MI_LIN_DK(true);                                                                                    \
    else MI_LIN_DK(false);                                                                                           \
    mi::launch(linear_output_kernel<TT>, ogrid, dim3(128), 0, stream, (TT*)out, ldo, (const float*)raw, (const TT*)gate, ldg, \
               norm_w, heads, vdim, eps, gate_silu);                                                                 \
  } while (0)
  if (dtype == MI_BF16) MI_LIN_ALL(__nv_bfloat16);
  else if (dtype == MI_F32) MI_LIN_ALL(float);
  else return mi_fail("linear_attention: unknown dtype %d", dtype);
#undef MI_LIN_ALL
#undef MI_LIN_DK
#undef MI_LIN_REC
  MI_LAUNCH_OK("linear_attention");
  return 0;
}
