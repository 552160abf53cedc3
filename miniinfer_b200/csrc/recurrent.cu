// Mixers that carry a state from token to token instead of reading a cache of keys: the short causal convolution
// in front of them, the selective scan (a diagonal state-space recurrence whose step size, input and output maps
// depend on the token) and the gated delta rule (a matrix state per head that decays per key channel and is
// corrected towards the new value along the new key).
//
// A step brings, for each of its items, q_len[b] new tokens in rows q_start[b] .. of the activations; the item's
// state lives in row seq_slot[b] of the layer's state tensor, float32, zero when the request was admitted.  A kernel
// walks an item's tokens in order, starting from the stored state and leaving the state after the last token, so the
// result at a position does not depend on how the request was cut into steps or on what else is in the batch.  All
// arithmetic of the recurrences - decays, their logarithms, softplus, exponentials, step sizes, gates, unit norms,
// the state and the sums over it - is float32; activations are read and written in the storage type.
#include "common.cuh"

namespace {

__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }

// ------------------------------------------------------------------------------------------------------------
// Short causal convolution over time, per channel: out[t, c] = act(bias[c] + sum_k w[c, taps - 1 - k] * in[t - k, c]),
// the inputs before the step's first token coming from the item's state (the last taps - 1 inputs of the request,
// oldest first, zeros before its start).  With in_bias, in[t, c] = x[t, c] + in_bias[c] (the bias of the projection that
// made x; the zeros before a request's start stay zeros), and the state keeps the inputs with it.  A thread per (token, channel).
constexpr int MAX_TAPS = 16;

template <typename T>
__global__ void __launch_bounds__(256)
causal_conv_kernel(T* __restrict__ out, int ldo, const T* __restrict__ x, int ldx, const float* __restrict__ w,
                   const float* __restrict__ bias, const float* __restrict__ in_bias, const float* __restrict__ state, long long state_stride,
                   const int* __restrict__ token_item, const int* __restrict__ q_start, const int* __restrict__ seq_slot,
                   int C, int taps, int silu) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int t = blockIdx.y;
  const int item = token_item[t];
  const int j = t - q_start[item];                         // index of the token among the item's new tokens
  const int slot = seq_slot[item];
  mi::grid_dependency_sync();
  if (c >= C) return;
  const float* st = state + (size_t)slot * state_stride;   // [taps - 1][C]
  float acc = bias ? bias[c] : 0.f;
  const float ib = in_bias ? in_bias[c] : 0.f;
  for (int k = taps - 1; k >= 0; --k) {                    // oldest input first
    const int jj = j - k;
    const float v = jj >= 0 ? mi::to_float(x[(size_t)(t - k) * ldx + c]) + ib : st[(size_t)(taps - 1 + jj) * C + c];
    acc = fmaf(w[(size_t)c * taps + (taps - 1 - k)], v, acc);
  }
  if (silu) acc = silu_f(acc);
  out[(size_t)t * ldo + c] = mi::from_float<T>(acc);
}

// After the convolution has run: the state becomes the last taps - 1 inputs of the request.  A thread per (item, channel).
template <typename T>
__global__ void __launch_bounds__(256)
conv_state_kernel(float* __restrict__ state, long long state_stride, const T* __restrict__ x, int ldx, const float* __restrict__ in_bias,
                  const int* __restrict__ q_start, const int* __restrict__ q_len, const int* __restrict__ seq_slot,
                  int C, int taps) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int item = blockIdx.y;
  const int row0 = q_start[item], n = q_len[item], slot = seq_slot[item];
  mi::grid_dependency_sync();
  if (c >= C) return;
  float* st = state + (size_t)slot * state_stride;
  float keep[MAX_TAPS];
  const int S = taps - 1;
  const float ib = in_bias ? in_bias[c] : 0.f;
#pragma unroll
  for (int r = 0; r < MAX_TAPS; ++r) {
    if (r >= S) break;
    const int jj = n - S + r;                               // index among the new tokens; negative: an older input
    keep[r] = jj >= 0 ? mi::to_float(x[(size_t)(row0 + jj) * ldx + c]) + ib : st[(size_t)(S + jj) * C + c];
  }
#pragma unroll
  for (int r = 0; r < MAX_TAPS; ++r) {
    if (r >= S) break;
    st[(size_t)r * C + c] = keep[r];
  }
}

// ------------------------------------------------------------------------------------------------------------
// Selective scan.  Per channel c and state index n, token after token:
//   dt = softplus(dt_in[t, c] + dt_bias[c]);  S[c, n] <- exp(dt * A[c, n]) * S[c, n] + dt * u[t, c] * B[t, n]
//   y[t, c] = (sum_n S[c, n] * C[t, n] + D[c] * u[t, c]) * silu(z[t, c]),      A = -exp(A_log)
// A channel's states are dealt to P neighbouring lanes, SPT to each (up to 32 * SPT states); their partial sums meet by shuffles.
constexpr int SPT = 4;
constexpr int SCAN_CHUNK = 16;    // tokens whose inputs are fetched together (32 was measured slower: 1.63 against 1.36 ms for two layers of 2048 tokens)
constexpr int SCAN_THREADS = 64;

// The float32 path takes the library's functions; the bfloat16 path the hardware's exponential, logarithm and
// reciprocal, whose errors (a few units in the last place of float32) are far below the rounding of the activations.
template <typename T> struct Math {
  static __device__ __forceinline__ float exp(float x) { return expf(x); }
  static __device__ __forceinline__ float softplus(float z) { return softplus_f(z); }
  static __device__ __forceinline__ float silu(float z) { return silu_f(z); }
};
template <> struct Math<__nv_bfloat16> {
  static __device__ __forceinline__ float exp(float x) { return __expf(x); }
  static __device__ __forceinline__ float softplus(float z) { return z > 20.f ? z : __logf(1.f + __expf(z)); }
  static __device__ __forceinline__ float silu(float z) { return __fdividef(z, 1.f + __expf(-z)); }
};

template <typename T>
struct ScanArgs {
  T* y; int ldy;
  const T* u; int ldu;          // the convolved, activated input
  const T* dt_in; int lddt;     // the step-size projection, before bias and softplus
  const T* bc; int ldbc;        // B at column b_off, C at column c_off of the same rows
  int b_off, c_off;
  const T* z; int ldz;          // the gate's input
  const float* dt_bias; const float* A_log; const float* D;
  float* state; long long state_stride;   // [slot][inner][N]
  const int* q_start; const int* q_len; const int* seq_slot;
  int inner, N, P;
  // segments (MODE 1, 2): an item's new tokens in up to SCAN_SEGMENTS stretches that run side by side
  float* seg_state;     // [item, segment][inner][N]: MODE 1 writes a stretch's end state from a zero start; the carry kernel
                        // turns it, in place, into the state the stretch starts from; MODE 2 reads that
  float* seg_dt;        // [item, segment][inner]: the stretch's sum of step sizes (its decay is exp(A * sum))
};

constexpr int SCAN_SEGMENTS = 16;
constexpr int SCAN_SEGMENT_MIN = 128;   // tokens a stretch has at least

__device__ __forceinline__ int scan_segments(int n_new) { return max(1, min(SCAN_SEGMENTS, n_new / SCAN_SEGMENT_MIN)); }
// tokens a stretch of an item (a multiple of the chunk, so that chunks do not straddle stretches)
__device__ __forceinline__ int scan_segment_len(int n_new, int nseg) { return ((n_new + nseg - 1) / nseg + SCAN_CHUNK - 1) / SCAN_CHUNK * SCAN_CHUNK; }

// MODE 0: an item's tokens in order, from the stored state to the stored state (every sum in an order that depends on
// the position alone: the 32-bit path, and steps of few tokens).  MODE 1 and 2, for long prompt portions in bfloat16:
// the item's tokens in stretches side by side - first every stretch from a zero state (1: no output, end state and sum
// of step sizes kept), then, after the carry kernel has chained the stretches, again from the state it really starts from
// (2: the outputs).  S_t = a_t S_(t-1) + b_t is linear in S, so a stretch's end state is its decay times the state it
// starts from plus its end state from zero.
template <typename T, int MODE>
__global__ void __launch_bounds__(SCAN_THREADS)
selective_scan_kernel(ScanArgs<T> a) {
  const int item = blockIdx.y;
  const int per_block = SCAN_THREADS / a.P;
  const int c = blockIdx.x * per_block + threadIdx.x / a.P;
  const int part = threadIdx.x % a.P;
  int row0 = a.q_start[item], n_new = a.q_len[item];
  const int slot = a.seq_slot[item];
  const int seg = MODE == 0 ? 0 : blockIdx.z;
  if (MODE != 0) {
    const int nseg = scan_segments(n_new);
    if (seg >= nseg) return;
    const int len = scan_segment_len(n_new, nseg);
    row0 += seg * len;
    n_new = max(0, min(len, n_new - seg * len));
  }
  const bool live = c < a.inner;
  const int cc = live ? c : 0;
  float A[SPT];
#pragma unroll
  for (int i = 0; i < SPT; ++i) {
    const int n = part * SPT + i;
    A[i] = n < a.N ? -expf(a.A_log[(size_t)cc * a.N + n]) : 0.f;
  }
  const float dtb = a.dt_bias[cc], Dc = a.D[cc];
  mi::grid_dependency_sync();
  float* st = MODE == 0 ? a.state + (size_t)slot * a.state_stride + (size_t)cc * a.N
                        : a.seg_state + ((size_t)(item * SCAN_SEGMENTS + seg) * a.inner + cc) * a.N;
  float S[SPT];
#pragma unroll
  for (int i = 0; i < SPT; ++i) {
    const int n = part * SPT + i;
    S[i] = (MODE != 1 && live && n < a.N) ? st[n] : 0.f;
  }
  float dt_sum = 0.f;
  // The tokens go by in chunks: a chunk's B and C rows into shared memory and its step sizes, inputs and gates into
  // registers, all loads issued together, and only then the recurrence over the chunk - so the latency of the loads is
  // paid once a chunk and not once a token.
  extern __shared__ float bc_s[];               // [SCAN_CHUNK][2][N]
  const int N = a.N;
  for (int c0 = 0; c0 < n_new; c0 += SCAN_CHUNK) {
    const int n = min(SCAN_CHUNK, n_new - c0);
    __syncthreads();                            // the chunk before has been read
    for (int i0 = threadIdx.x; i0 < n * N; i0 += 4 * SCAN_THREADS) {      // eight loads in flight a thread
      float bv[4], cv[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int idx = min(i0 + q * SCAN_THREADS, n * N - 1);
        const T* brow = a.bc + (size_t)(row0 + c0 + idx / N) * a.ldbc;
        bv[q] = mi::to_float(brow[a.b_off + idx % N]);
        cv[q] = mi::to_float(brow[a.c_off + idx % N]);
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int idx = i0 + q * SCAN_THREADS;
        if (idx < n * N) {
          bc_s[((idx / N) * 2 + 0) * N + idx % N] = bv[q];
          bc_s[((idx / N) * 2 + 1) * N + idx % N] = cv[q];
        }
      }
    }
    float dtv[SCAN_CHUNK], uv[SCAN_CHUNK], zv[SCAN_CHUNK];
#pragma unroll
    for (int tt = 0; tt < SCAN_CHUNK; ++tt) {
      const size_t t = (size_t)(row0 + c0 + min(tt, n - 1));
      dtv[tt] = mi::to_float(a.dt_in[t * a.lddt + cc]);
      uv[tt] = mi::to_float(a.u[t * a.ldu + cc]);
      zv[tt] = mi::to_float(a.z[t * a.ldz + cc]);
    }
    __syncthreads();
    // four tokens at a time: first what does not depend on the state - step sizes, decays, gates, all independent of one
    // another - then the recurrence itself, which is multiply-adds only
#pragma unroll
    for (int t4 = 0; t4 < SCAN_CHUNK; t4 += 4) {
      if (t4 < n) {
        float dA[4][SPT], du[4], gz[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float dt = Math<T>::softplus(dtv[t4 + q] + dtb);
          if (MODE == 1 && t4 + q < n) dt_sum += dt;
          du[q] = dt * uv[t4 + q];
          gz[q] = Math<T>::silu(zv[t4 + q]);
#pragma unroll
          for (int i = 0; i < SPT; ++i) dA[q][i] = Math<T>::exp(dt * A[i]);
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int tt = t4 + q;
          if (tt < n) {
            const float* Bv = bc_s + (tt * 2 + 0) * N;
            const float* Cv = bc_s + (tt * 2 + 1) * N;
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < SPT; ++i) {
              const int nn = part * SPT + i;
              if (nn < N) {
                S[i] = fmaf(dA[q][i], S[i], du[q] * Bv[nn]);
                acc = fmaf(S[i], Cv[nn], acc);
              }
            }
            if (MODE != 1) {                         // the first pass of the stretches keeps the state only
              for (int o = a.P >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
              if (live && part == 0)
                a.y[(size_t)(row0 + c0 + tt) * a.ldy + cc] = mi::from_float<T>((acc + Dc * uv[tt]) * gz[q]);
            }
          }
        }
      }
    }
  }
  if (live && MODE != 2) {
#pragma unroll
    for (int i = 0; i < SPT; ++i) {
      const int n = part * SPT + i;
      if (n < a.N) st[n] = S[i];
    }
    if (MODE == 1 && part == 0) a.seg_dt[(size_t)(item * SCAN_SEGMENTS + seg) * a.inner + cc] = dt_sum;
  }
}

// Chains an item's stretches: carry_0 = the stored state, carry_(s+1) = exp(A * dt_sum_s) * carry_s + end_s; the carries
// replace the end states in seg_state, the last one becomes the stored state.  A thread per (item, channel, state index).
__global__ void __launch_bounds__(256)
scan_carry_kernel(float* __restrict__ seg_state, const float* __restrict__ seg_dt, const float* __restrict__ A_log,
                  float* __restrict__ state, long long state_stride, const int* __restrict__ q_len,
                  const int* __restrict__ seq_slot, int inner, int N) {
  const int item = blockIdx.y;
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  const int nseg = scan_segments(q_len[item]);
  const int slot = seq_slot[item];
  mi::grid_dependency_sync();
  if (idx >= inner * N) return;
  const int c = idx / N;
  const float A = -expf(A_log[idx]);
  float* st = state + (size_t)slot * state_stride + idx;
  float carry = *st;
  for (int s = 0; s < nseg; ++s) {
    float* e = seg_state + (size_t)(item * SCAN_SEGMENTS + s) * inner * N + idx;
    const float end = *e;
    *e = carry;
    carry = fmaf(expf(A * seg_dt[(size_t)(item * SCAN_SEGMENTS + s) * inner + c]), carry, end);
  }
  *st = carry;
}

// ------------------------------------------------------------------------------------------------------------
// Gated delta rule.  Per head, with the state S [dim, vdim], token after token:
//   qh = q / sqrt(sum q^2 + 1e-6) * dim^-1/2,  kh = k / sqrt(sum k^2 + 1e-6)       (q, k of the head's q/k head)
//   g[i] = exp(-exp(A_log[head]) * softplus(a[t, head, i] + dt_bias[head, i])),    beta = sigmoid(b[t, head])
//   S[i, :] <- g[i] * S[i, :];   u = beta * (v - S^T kh);   S <- S + kh u^T;   o = S^T qh
//   out[t, head, :] = o / sqrt(mean(o^2) + eps) * norm_w * sigmoid(gate[t, head, :])
// Three kernels.  (1) delta_prepare, a warp per (token, head), all tokens at once: everything of a token that does not
// depend on the state - unit q and k, decays, beta - as float32 rows.  (2) delta_recurrence, the only part that walks
// the tokens in order: a block per (item, head, group of value columns).  Thread (j, r) keeps rows r * DK .. r * DK + DK - 1
// of column j of S in registers; the R threads of a column are neighbouring lanes and add their partial sums by
// shuffles.  Columns do not depend on one another, so a head's columns are dealt to several blocks; the tokens' vectors
// go through shared memory in chunks.  The raw read-outs go to a float32 buffer.  (3) delta_output, a warp per
// (token, head): root mean square over the head, weight, gate.
template <typename T>
struct DeltaPrepArgs {
  const T* q; const T* k; int ldqk;      // rows of the convolved q and k: q/k head g at column g * dim
  const T* a; int lda;                   // decay input, head h at column h * dim
  const T* b; int ldb;                   // beta logits, head h at column h
  const float* dt_bias; const float* A_log;
  float* qn; float* kn;                  // [tokens, kv_heads * dim]
  float* g;                              // [tokens, heads * dim]
  float* beta;                           // [tokens, heads]
  const T* v; int ldv;                   // values, head h at column h * vdim
  float* raw;                            // [tokens, heads * vdim]: receives the values as float32 (the recurrence reads a
                                         // token's values from here and writes its read-outs over them)
  int T_, heads, kv_heads, dim, vdim;
};

template <typename T>
__global__ void __launch_bounds__(128)
delta_prepare_kernel(DeltaPrepArgs<T> a) {
  mi::grid_dependency_sync();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x;
  const int units = a.kv_heads + a.heads;
  for (int u = blockIdx.y * 4 + warp; u < units; u += 4 * gridDim.y) {
    if (u < a.kv_heads) {
      const T* q = a.q + (size_t)t * a.ldqk + (size_t)u * a.dim;
      const T* k = a.k + (size_t)t * a.ldqk + (size_t)u * a.dim;
      float sq = 0.f, sk = 0.f;
      for (int i = lane; i < a.dim; i += 32) {
        const float x = mi::to_float(q[i]), y = mi::to_float(k[i]);
        sq = fmaf(x, x, sq);
        sk = fmaf(y, y, sk);
      }
      sq = mi::warp_sum(sq);
      sk = mi::warp_sum(sk);
      const float fq = rsqrtf((float)a.dim) / sqrtf(sq + 1e-6f), fk = 1.f / sqrtf(sk + 1e-6f);
      for (int i = lane; i < a.dim; i += 32) {
        a.qn[((size_t)t * a.kv_heads + u) * a.dim + i] = mi::to_float(q[i]) * fq;
        a.kn[((size_t)t * a.kv_heads + u) * a.dim + i] = mi::to_float(k[i]) * fk;
      }
    } else {
      const int h = u - a.kv_heads;
      const float neg_rate = -expf(a.A_log[h]);
      for (int i = lane; i < a.dim; i += 32) {
        const float z = mi::to_float(a.a[(size_t)t * a.lda + (size_t)h * a.dim + i]) + a.dt_bias[h * a.dim + i];
        a.g[((size_t)t * a.heads + h) * a.dim + i] = expf(neg_rate * softplus_f(z));
      }
      if (lane == 0) a.beta[(size_t)t * a.heads + h] = sigmoid_f(mi::to_float(a.b[(size_t)t * a.ldb + h]));
      for (int j = lane; j < a.vdim; j += 32)
        a.raw[((size_t)t * a.heads + h) * a.vdim + j] = mi::to_float(a.v[(size_t)t * a.ldv + (size_t)h * a.vdim + j]);
    }
  }
}

// 4 bytes from global to shared memory without a register in between; zeros if not `take`
__device__ __forceinline__ void copy4(float* dst, const float* src, bool take) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
  const int bytes = take ? 4 : 0;
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}

constexpr int DELTA_THREADS = 128;
constexpr int DELTA_CHUNK = 16;       // tokens whose vectors are in shared memory at a time

template <typename T>
struct DeltaArgs {
  float* raw;                            // [tokens, heads * vdim]: the values in, the read-outs before norm and gate out
  const float* qn; const float* kn; const float* g; const float* beta;
  float* state; long long state_stride;  // [slot][heads][dim][vdim]
  const int* q_start; const int* q_len; const int* seq_slot;
  int heads, kv_heads, dim, vdim, R;
  // stretches side by side (MODE 1, 2)
  float* seg_state;                      // [item, stretch][heads][dim][vdim]: a stretch's end state from a zero start (MODE 1
                                         // writes), then - after the carry kernel - the state it starts from (MODE 2 reads)
  float* seg_map;                        // [item, stretch][heads][dim (k)][dim (i)]: the stretch's map of its start state,
                                         // transposed: end = map * start + end_from_zero
};

constexpr int DELTA_SEGMENTS = 16;
constexpr int DELTA_SEGMENT_MIN = 96;    // tokens a stretch has at least

__host__ __device__ __forceinline__ int delta_segments(int n_new) { return max(1, min(DELTA_SEGMENTS, n_new / DELTA_SEGMENT_MIN)); }
__host__ __device__ __forceinline__ int delta_segment_len(int n_new, int nseg) {
  return ((n_new + nseg - 1) / nseg + DELTA_CHUNK - 1) / DELTA_CHUNK * DELTA_CHUNK;
}

// MODE 0: an item's tokens in order, from the stored state to the stored state.  MODE 1 and 2, for long prompt portions in
// bfloat16: the tokens in stretches side by side.  The state after a token is linear in the state before it - S <-
// (I - beta k k^T) diag(g) S + beta k v^T - so a stretch's end state is (its map) x (the state it starts from) + (its end state
// from a zero start).  MODE 1 walks every stretch twice over, in one launch: the value columns from zero with the real
// values, and dim more columns that start as the identity with zero values - they end as the stretch's map.  The carry
// kernel chains the stretches; MODE 2 walks every stretch again from the state it really starts from and writes the
// read-outs.
template <typename T, int DK, int MODE>
__global__ void __launch_bounds__(DELTA_THREADS)
delta_recurrence_kernel(DeltaArgs<T> a) {
  extern __shared__ __align__(16) float sm[];
  constexpr int LD = DK + 4;             // a thread's stretch of a vector, padded: 16-byte loads without bank conflicts
  const int item = MODE == 0 ? blockIdx.y : blockIdx.y / DELTA_SEGMENTS, head = blockIdx.x;
  const int seg = MODE == 0 ? 0 : blockIdx.y % DELTA_SEGMENTS;
  const int kvh = head / (a.heads / a.kv_heads);
  int row0 = a.q_start[item], n_new = a.q_len[item];
  const int slot = a.seq_slot[item];
  if (MODE != 0) {
    const int nseg = delta_segments(n_new);
    if (seg >= nseg) return;
    const int len = delta_segment_len(n_new, nseg);
    row0 += seg * len;
    n_new = max(0, min(len, n_new - seg * len));
  }
  const int R = a.R, dim = a.dim, vdim = a.vdim;
  const int cols = DELTA_THREADS / R;
  const int cl = threadIdx.x / R, r = threadIdx.x % R;
  const int col = blockIdx.z * cols + cl;
  const bool map_col = MODE == 1 && col >= vdim;             // a column of the stretch's map: starts as a unit vector, zero values
  const bool live = col < vdim + (MODE == 1 ? dim : 0);
  const int vec = R * LD;                                    // floats of one padded vector
  const int tok_floats = 3 * vec + cols + 4;                 // q, k, g, the block's values, beta
  mi::grid_dependency_sync();
  const size_t seg_at = ((size_t)(item * DELTA_SEGMENTS + seg) * a.heads + head) * dim;
  float* st = MODE == 0 ? a.state + (size_t)slot * a.state_stride + (size_t)head * dim * vdim : a.seg_state + seg_at * vdim;
  float S[DK];
#pragma unroll
  for (int i = 0; i < DK; ++i) {
    const int row = r * DK + i;
    if (MODE == 1) S[i] = (map_col && row == col - vdim) ? 1.f : 0.f;
    else S[i] = (live && row < dim) ? st[(size_t)row * vdim + col] : 0.f;
  }
  // The chunks' vectors come by asynchronous copies into two buffers: while a chunk is worked on, the next one is on
  // its way.  Rows past dim and columns past vdim are filled with zeros (a zero key row and decay leave such a row of S
  // at zero).
  const int chunk_floats = DELTA_CHUNK * tok_floats;
  auto fetch = [&](int c0, float* buf) {
    const int n = min(DELTA_CHUNK, n_new - c0);
    for (int idx = threadIdx.x; idx < n * R * DK; idx += DELTA_THREADS) {
      const int tt = idx / (R * DK), i = idx % (R * DK);
      const size_t t = (size_t)(row0 + c0 + tt);
      float* base = buf + (size_t)tt * tok_floats + (i / DK) * LD + (i % DK);
      const bool in = i < dim;
      copy4(base, a.qn + (t * a.kv_heads + kvh) * dim + (in ? i : 0), in);
      copy4(base + vec, a.kn + (t * a.kv_heads + kvh) * dim + (in ? i : 0), in);
      copy4(base + 2 * vec, a.g + (t * a.heads + head) * dim + (in ? i : 0), in);
    }
    for (int idx = threadIdx.x; idx < n * cols; idx += DELTA_THREADS) {
      const int tt = idx / cols, j = idx % cols;
      const int c = blockIdx.z * cols + j;
      copy4(buf + (size_t)tt * tok_floats + 3 * vec + j, a.raw + (size_t)(row0 + c0 + tt) * (a.heads * vdim) + head * vdim + (c < vdim ? c : 0), c < vdim);
    }
    for (int tt = threadIdx.x; tt < n; tt += DELTA_THREADS)
      copy4(buf + (size_t)tt * tok_floats + 3 * vec + cols, a.beta + (size_t)(row0 + c0 + tt) * a.heads + head, true);
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  if (n_new > 0) fetch(0, sm);
  for (int c0 = 0, ci = 0; c0 < n_new; c0 += DELTA_CHUNK, ++ci) {
    const int n = min(DELTA_CHUNK, n_new - c0);
    float* cur = sm + (size_t)(ci & 1) * chunk_floats;
    if (c0 + DELTA_CHUNK < n_new) {
      fetch(c0 + DELTA_CHUNK, sm + (size_t)((ci + 1) & 1) * chunk_floats);      // that buffer's chunk was finished before the barrier below
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    for (int tt = 0; tt < n; ++tt) {
      const float* base = cur + (size_t)tt * tok_floats;
      const float4* qv = reinterpret_cast<const float4*>(base + r * LD);
      const float4* kv = reinterpret_cast<const float4*>(base + vec + r * LD);
      const float4* gv = reinterpret_cast<const float4*>(base + 2 * vec + r * LD);
      float ks[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < DK / 4; ++i) {
        const float4 g4 = gv[i], k4 = kv[i];
        S[4 * i] *= g4.x; S[4 * i + 1] *= g4.y; S[4 * i + 2] *= g4.z; S[4 * i + 3] *= g4.w;
        ks[0] = fmaf(k4.x, S[4 * i], ks[0]); ks[1] = fmaf(k4.y, S[4 * i + 1], ks[1]);
        ks[2] = fmaf(k4.z, S[4 * i + 2], ks[2]); ks[3] = fmaf(k4.w, S[4 * i + 3], ks[3]);
      }
      float kS = (ks[0] + ks[1]) + (ks[2] + ks[3]);
      for (int o = R >> 1; o > 0; o >>= 1) kS += __shfl_xor_sync(0xffffffffu, kS, o);
      const float u = base[3 * vec + cols] * (base[3 * vec + cl] - kS);
      float os[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < DK / 4; ++i) {
        const float4 k4 = kv[i], q4 = qv[i];
        S[4 * i] = fmaf(k4.x, u, S[4 * i]); S[4 * i + 1] = fmaf(k4.y, u, S[4 * i + 1]);
        S[4 * i + 2] = fmaf(k4.z, u, S[4 * i + 2]); S[4 * i + 3] = fmaf(k4.w, u, S[4 * i + 3]);
        os[0] = fmaf(q4.x, S[4 * i], os[0]); os[1] = fmaf(q4.y, S[4 * i + 1], os[1]);
        os[2] = fmaf(q4.z, S[4 * i + 2], os[2]); os[3] = fmaf(q4.w, S[4 * i + 3], os[3]);
      }
      if (MODE != 1) {                        // the first pass of the stretches keeps the state only
        float oj = (os[0] + os[1]) + (os[2] + os[3]);
        for (int o = R >> 1; o > 0; o >>= 1) oj += __shfl_xor_sync(0xffffffffu, oj, o);
        if (live && r == 0) a.raw[(size_t)(row0 + c0 + tt) * (a.heads * vdim) + head * vdim + col] = oj;
      }
    }
    __syncthreads();      // everyone is done with this buffer before the fetch after next fills it
  }
  if (MODE != 2) {
#pragma unroll
    for (int i = 0; i < DK; ++i) {
      const int row = r * DK + i;
      if (!live || row >= dim) continue;
      if (map_col) a.seg_map[(seg_at + (col - vdim)) * dim + row] = S[i];    // transposed: [start row k = col - vdim][end row i]
      else st[(size_t)row * vdim + col] = S[i];
    }
  }
}

// Chains an item's stretches, a block per (head, item, group of value columns), a thread per (row i, column j):
// carry_0 = the stored state, carry_(s+1)[i, j] = sum_k map_s[i, k] carry_s[k, j] + end_s[i, j].  The carries replace
// the end states in seg_state; the last becomes the stored state.
constexpr int CARRY_KT = 128;   // rows of the map in shared memory at a time (the whole map up to dim 128)

__global__ void __launch_bounds__(1024)
delta_carry_kernel(float* __restrict__ seg_state, const float* __restrict__ seg_map, float* __restrict__ state,
                   long long state_stride, const int* __restrict__ q_len, const int* __restrict__ seq_slot, int heads, int dim,
                   int vdim, int dimp, int TJ) {
  extern __shared__ float carry_s[];             // [dim][TJ], then a tile of the map [CARRY_KT][dim]
  float* map_s = carry_s + dim * TJ;
  const int head = blockIdx.x, item = blockIdx.y;
  const int i = threadIdx.x % dimp, jl = threadIdx.x / dimp;
  const int j = blockIdx.z * TJ + jl;
  const int nseg = delta_segments(q_len[item]);
  const int slot = seq_slot[item];
  mi::grid_dependency_sync();
  const bool valid = i < dim && j < vdim;
  float* st = state + (size_t)slot * state_stride + (size_t)head * dim * vdim;
  float c = valid ? st[(size_t)i * vdim + j] : 0.f;
  for (int s = 0; s < nseg; ++s) {
    const size_t at = ((size_t)(item * DELTA_SEGMENTS + s) * heads + head) * dim;
    float* e = seg_state + at * vdim;
    const float* m = seg_map + at * dim;
    if (i < dim) carry_s[i * TJ + jl] = c;
    __syncthreads();
    float acc = 0.f;
    if (valid) {
      acc = e[(size_t)i * vdim + j];
      e[(size_t)i * vdim + j] = c;
    }
    // the map goes through shared memory in tiles of CARRY_KT of its rows (k), fetched by all threads together
    for (int k0 = 0; k0 < dim; k0 += CARRY_KT) {
      const int kn = min(CARRY_KT, dim - k0);
      for (int i0 = threadIdx.x; i0 < kn * dim; i0 += 8 * blockDim.x) {       // eight loads in flight a thread
        float mv[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) mv[q] = m[(size_t)k0 * dim + min(i0 + q * (int)blockDim.x, kn * dim - 1)];
#pragma unroll
        for (int q = 0; q < 8; ++q)
          if (i0 + q * (int)blockDim.x < kn * dim) map_s[i0 + q * blockDim.x] = mv[q];
      }
      __syncthreads();
      if (valid)
        for (int k = 0; k < kn; ++k) acc = fmaf(map_s[k * dim + i], carry_s[(k0 + k) * TJ + jl], acc);
      __syncthreads();
    }
    c = acc;
  }
  if (valid) st[(size_t)i * vdim + j] = c;
}

template <typename T>
__global__ void __launch_bounds__(128)
delta_output_kernel(T* __restrict__ out, int ldo, const float* __restrict__ raw, const T* __restrict__ gate, int ldg,
                    const float* __restrict__ norm_w, int heads, int vdim, float eps) {
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
      const float gl = mi::to_float(gate[(size_t)t * ldg + h * vdim + j]);
      out[(size_t)t * ldo + h * vdim + j] = mi::from_float<T>(o[j] * rstd * norm_w[j] * sigmoid_f(gl));
    }
  }
}

}  // namespace

MI_API int mi_causal_conv(void* out, int ldo, const void* x, int ldx, int dtype, const float* w, const float* bias, const float* in_bias,
                          float* state, long long state_stride, const int* token_item, const int* q_start, const int* q_len,
                          const int* seq_slot, int T, int items, int C, int taps, int silu, cudaStream_t stream) {
  MI_REQUIRE(T >= 0 && items >= 0 && C > 0 && taps >= 1 && taps <= MAX_TAPS, "causal_conv: bad sizes C=%d taps=%d (taps up to %d)", C, taps, MAX_TAPS);
  MI_REQUIRE(T <= 65535 && items <= 65535, "causal_conv: more than 65535 tokens or items in one launch");
  MI_REQUIRE(state_stride >= (long long)(taps - 1) * C, "causal_conv: the state rows are too short");
  if (T == 0) return 0;
  dim3 grid((C + 255) / 256, T), sgrid((C + 255) / 256, items);
  if (dtype == MI_BF16) {
    mi::launch(causal_conv_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, (__nv_bfloat16*)out, ldo, (const __nv_bfloat16*)x, ldx, w, bias, in_bias,
               (const float*)state, state_stride, token_item, q_start, seq_slot, C, taps, silu);
    if (taps > 1) mi::launch(conv_state_kernel<__nv_bfloat16>, sgrid, dim3(256), 0, stream, state, state_stride, (const __nv_bfloat16*)x, ldx, in_bias,
                             q_start, q_len, seq_slot, C, taps);
  } else if (dtype == MI_F32) {
    mi::launch(causal_conv_kernel<float>, grid, dim3(256), 0, stream, (float*)out, ldo, (const float*)x, ldx, w, bias, in_bias,
               (const float*)state, state_stride, token_item, q_start, seq_slot, C, taps, silu);
    if (taps > 1) mi::launch(conv_state_kernel<float>, sgrid, dim3(256), 0, stream, state, state_stride, (const float*)x, ldx, in_bias,
                             q_start, q_len, seq_slot, C, taps);
  } else {
    return mi_fail("causal_conv: unknown dtype %d", dtype);
  }
  MI_LAUNCH_OK("causal_conv");
  return 0;
}

MI_API int mi_selective_scan_segments() { return SCAN_SEGMENTS; }

MI_API int mi_selective_scan(void* y, int ldy, const void* u, int ldu, const void* dt_in, int lddt, const void* bc, int ldbc,
                             int b_off, int c_off, const void* z, int ldz, int dtype, const float* dt_bias, const float* A_log,
                             const float* D, float* state, long long state_stride, const int* q_start, const int* q_len,
                             const int* seq_slot, int items, int inner, int N, float* segments, cudaStream_t stream) {
  // segments: null, or items * SCAN_SEGMENTS * inner * (N + 1) floats of scratch - then the items' tokens run in stretches
  // side by side (bfloat16 only: the sums then depend on where a portion starts)
  MI_REQUIRE(segments == nullptr || dtype == MI_BF16, "selective_scan: stretches side by side are for bfloat16 activations");
  MI_REQUIRE(items >= 0 && items <= 65535 && inner > 0 && N > 0 && N <= 32 * SPT, "selective_scan: bad sizes inner=%d state=%d (state up to %d)", inner, N, 32 * SPT);
  MI_REQUIRE(state_stride >= (long long)inner * N, "selective_scan: the state rows are too short");
  if (items == 0) return 0;
  int P = 1;
  while (P * SPT < N) P *= 2;
  const int per_block = SCAN_THREADS / P;
  const size_t smem = (size_t)SCAN_CHUNK * 2 * N * sizeof(float);
  dim3 grid((inner + per_block - 1) / per_block, items);
#define MI_SCAN(TT)                                                                                               \
  do {                                                                                                            \
    ScanArgs<TT> a;                                                                                               \
    a.y = (TT*)y; a.ldy = ldy; a.u = (const TT*)u; a.ldu = ldu; a.dt_in = (const TT*)dt_in; a.lddt = lddt;        \
    a.bc = (const TT*)bc; a.ldbc = ldbc; a.b_off = b_off; a.c_off = c_off; a.z = (const TT*)z; a.ldz = ldz;       \
    a.dt_bias = dt_bias; a.A_log = A_log; a.D = D; a.state = state; a.state_stride = state_stride;                \
    a.q_start = q_start; a.q_len = q_len; a.seq_slot = seq_slot; a.inner = inner; a.N = N; a.P = P;               \
    a.seg_state = segments; a.seg_dt = segments ? segments + (size_t)items * SCAN_SEGMENTS * inner * N : nullptr; \
    if (!segments) {                                                                                              \
      mi::launch(selective_scan_kernel<TT, 0>, grid, dim3(SCAN_THREADS), smem, stream, a);                        \
    } else {                                                                                                      \
      dim3 sgrid(grid.x, items, SCAN_SEGMENTS);                                                                   \
      mi::launch(selective_scan_kernel<TT, 1>, sgrid, dim3(SCAN_THREADS), smem, stream, a);                       \
      mi::launch(scan_carry_kernel, dim3((inner * N + 255) / 256, items), dim3(256), 0, stream, a.seg_state, (const float*)a.seg_dt, \
                 A_log, state, state_stride, q_len, seq_slot, inner, N);                                          \
      mi::launch(selective_scan_kernel<TT, 2>, sgrid, dim3(SCAN_THREADS), smem, stream, a);                       \
    }                                                                                                             \
  } while (0)
  if (dtype == MI_BF16) MI_SCAN(__nv_bfloat16);
  else if (dtype == MI_F32) MI_SCAN(float);
  else return mi_fail("selective_scan: unknown dtype %d", dtype);
#undef MI_SCAN
  MI_LAUNCH_OK("selective_scan");
  return 0;
}

// scratch: float32, tokens * (2 * kv_heads * dim + heads * dim + heads + heads * vdim) values (mi_gated_delta_scratch_floats)
MI_API long long mi_gated_delta_scratch_floats(int T, int heads, int kv_heads, int dim, int vdim) {
  return (long long)T * ((long long)2 * kv_heads * dim + (long long)heads * dim + heads + (long long)heads * vdim);
}

MI_API int mi_gated_delta_segments() { return DELTA_SEGMENTS; }

// Blocks that walk one request's tokens in order (heads x groups of value columns): what a long prompt portion keeps
// busy without stretches side by side.
MI_API int mi_gated_delta_blocks(int heads, int dim, int vdim) {
  int DK = dim <= 128 ? 16 : 32, R = 1;
  for (;; DK *= 2) {
    R = 1;
    while (R * DK < dim) R *= 2;
    if (R <= 32 || DK == 128) break;
  }
  const int cols = DELTA_THREADS / (R > 32 ? 32 : R);
  return heads * ((vdim + cols - 1) / cols);
}

MI_API int mi_gated_delta(void* out, int ldo, const void* q, const void* k, int ldqk, const void* v, int ldv, const void* a_in, int lda,
                          const void* b_in, int ldb, const void* gate, int ldg, int dtype, const float* dt_bias, const float* A_log,
                          const float* norm_w, float eps, float* state, long long state_stride, const int* q_start, const int* q_len,
                          const int* seq_slot, int T, int items, int heads, int kv_heads, int dim, int vdim, float* scratch,
                          float* segments, cudaStream_t stream) {
  // segments: null, or items * DELTA_SEGMENTS * heads * dim * (vdim + dim) floats of scratch - then the items' tokens run
  // in stretches side by side (bfloat16 only: the sums then depend on where a portion starts; dim up to 256)
  MI_REQUIRE(segments == nullptr || (dtype == MI_BF16 && dim <= 256 && items * DELTA_SEGMENTS <= 65535),
             "gated_delta: stretches side by side are for bfloat16 activations and dim up to 256");
  MI_REQUIRE(T >= 0 && items >= 0 && items <= 65535 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0, "gated_delta: bad head counts %d / %d", heads, kv_heads);
  MI_REQUIRE(dim > 0 && vdim > 0 && dim <= 4096 && heads <= 65535, "gated_delta: bad sizes dim=%d vdim=%d", dim, vdim);
  MI_REQUIRE(state_stride >= (long long)heads * dim * vdim, "gated_delta: the state rows are too short");
  MI_REQUIRE(scratch != nullptr && ((uintptr_t)scratch % 16) == 0, "gated_delta: the scratch buffer is missing or unaligned");
  if (items == 0 || T == 0) return 0;
  // rows of a column a thread keeps (DK) and threads a column (R, a power of two up to 32)
  int DK = dim <= 128 ? 16 : 32, R = 1;      // measured on B200 at 128 x 128: 16 rows a thread are faster than 32
  for (;; DK *= 2) {
    R = 1;
    while (R * DK < dim) R *= 2;
    if (R <= 32 || DK == 128) break;
  }
  MI_REQUIRE(R <= 32, "gated_delta: dim=%d is more than a block's threads can keep", dim);
  const int cols = DELTA_THREADS / R;
  const int tok_floats = 3 * R * (DK + 4) + cols + 4;
  const size_t smem = (size_t)2 * DELTA_CHUNK * tok_floats * sizeof(float);
  MI_REQUIRE(smem <= 200 * 1024, "gated_delta: a chunk's vectors (%zu bytes) do not fit shared memory", smem);
  float* qn = scratch;
  float* kn = qn + (size_t)T * kv_heads * dim;
  float* g = kn + (size_t)T * kv_heads * dim;
  float* beta = g + (size_t)T * heads * dim;
  float* raw = beta + (((size_t)T * heads + 3) / 4) * 4;
  dim3 pgrid(T, (heads + kv_heads + 3) / 4 > 16 ? 16 : (heads + kv_heads + 3) / 4);
  dim3 ogrid(T, (heads + 3) / 4 > 16 ? 16 : (heads + 3) / 4);
  dim3 rgrid(heads, items, (vdim + cols - 1) / cols);
#define MI_DELTA(TT, DKV)                                                                                         \
  do {                                                                                                            \
    DeltaArgs<TT> d;                                                                                              \
    d.raw = raw; d.qn = qn; d.kn = kn; d.g = g; d.beta = beta;                                                    \
    d.state = state; d.state_stride = state_stride; d.q_start = q_start; d.q_len = q_len; d.seq_slot = seq_slot;  \
    d.heads = heads; d.kv_heads = kv_heads; d.dim = dim; d.vdim = vdim; d.R = R;                                  \
    d.seg_state = segments; d.seg_map = segments ? segments + (size_t)items * DELTA_SEGMENTS * heads * dim * vdim : nullptr; \
    if (!segments) {                                                                                              \
      if (smem > 48 * 1024) cudaFuncSetAttribute(delta_recurrence_kernel<TT, DKV, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      mi::launch(delta_recurrence_kernel<TT, DKV, 0>, rgrid, dim3(DELTA_THREADS), smem, stream, d);               \
    } else {                                                                                                      \
      if (smem > 48 * 1024) {                                                                                     \
        cudaFuncSetAttribute(delta_recurrence_kernel<TT, DKV, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        cudaFuncSetAttribute(delta_recurrence_kernel<TT, DKV, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      }                                                                                                           \
      dim3 g1(heads, items * DELTA_SEGMENTS, (vdim + dim + cols - 1) / cols), g2(heads, items * DELTA_SEGMENTS, rgrid.z); \
      const int dimp = (dim + 31) / 32 * 32, TJ = 1024 / dimp;                                                    \
      mi::launch(delta_recurrence_kernel<TT, DKV, 1>, g1, dim3(DELTA_THREADS), smem, stream, d);                  \
      const size_t csmem = (size_t)dim * (TJ + (dim < CARRY_KT ? dim : CARRY_KT)) * sizeof(float);                \
      if (csmem > 48 * 1024) cudaFuncSetAttribute(delta_carry_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)csmem); \
      mi::launch(delta_carry_kernel, dim3(heads, items, (vdim + TJ - 1) / TJ), dim3(dimp * TJ), csmem, stream,    \
                 d.seg_state, (const float*)d.seg_map, state, state_stride, q_len, seq_slot, heads, dim, vdim, dimp, TJ); \
      mi::launch(delta_recurrence_kernel<TT, DKV, 2>, g2, dim3(DELTA_THREADS), smem, stream, d);                  \
    }                                                                                                             \
  } while (0)
#define MI_DELTA_ALL(TT)                                                                                          \
  do {                                                                                                            \
    DeltaPrepArgs<TT> p;                                                                                          \
    p.q = (const TT*)q; p.k = (const TT*)k; p.ldqk = ldqk; p.a = (const TT*)a_in; p.lda = lda; p.b = (const TT*)b_in; p.ldb = ldb; \
    p.dt_bias = dt_bias; p.A_log = A_log; p.qn = qn; p.kn = kn; p.g = g; p.beta = beta; p.T_ = T; p.heads = heads;  \
    p.kv_heads = kv_heads; p.dim = dim; p.v = (const TT*)v; p.ldv = ldv; p.raw = raw; p.vdim = vdim;                  \
    mi::launch(delta_prepare_kernel<TT>, pgrid, dim3(128), 0, stream, p);                                         \
    if (DK == 16) MI_DELTA(TT, 16);                                                                               \
    else if (DK == 32) MI_DELTA(TT, 32);                                                                          \
    else if (DK == 64) MI_DELTA(TT, 64);                                                                          \
    else MI_DELTA(TT, 128);                                                                                       \
    mi::launch(delta_output_kernel<TT>, ogrid, dim3(128), 0, stream, (TT*)out, ldo, (const float*)raw, (const TT*)gate, ldg, norm_w, heads, vdim, eps); \
  } while (0)
  if (dtype == MI_BF16) MI_DELTA_ALL(__nv_bfloat16);
  else if (dtype == MI_F32) MI_DELTA_ALL(float);
  else return mi_fail("gated_delta: unknown dtype %d", dtype);
#undef MI_DELTA_ALL
#undef MI_DELTA
  MI_LAUNCH_OK("gated_delta");
  return 0;
}
