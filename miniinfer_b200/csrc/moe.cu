// Routed experts (a mixture of small SwiGLU feed-forward layers of which each token uses `top`), in
// a product and five kernels, without a word read back by the host, so that a step can be recorded as a graph:
//
//   route    (the logits z = W_router h come from the engine's matrix product, accumulated in float32; bfloat16 operands
//            multiply exactly in float32, so this is the 32-bit sum of the rounded inputs.)  One warp per token: scores
//            s = sigmoid(z), choice = s + correction; the `top` experts of largest choice (ties: the lower
//            index); weights = their s divided by (the sum of those s + 1e-20).  Or (mode 1) the `top` largest logits
//            are chosen and the weights are the softmax over the chosen logits alone.
//   align    one block: counts the (token, choice) pairs of every expert, gives each expert a range of
//            rows rounded up to the row tile, and every pair a row in its expert's range.  Rows nobody
//            owns are marked -1, tiles nobody owns too; the grid of the products is sized for the worst case.
//   gate-up  grouped product: a block takes one row tile (rows of ONE expert, gathered from the tokens'
//            normalised rows) and a slice of that expert's gate and up rows, and writes silu(g) * u.
//   down     grouped product of those rows with the expert's down matrix, written as float32.
//   combine  out[token] = sum over its choices, in the order of the choices, of weight * down row.
//
// A pair's products depend on its own row and its expert's weights only (sums over k in a fixed order), and a
// token's sum runs over its choices in order, so a token's output does not depend on the rest of the batch.
// bfloat16: mma.m16n8k16 with float32 accumulation - row tiles of 64 through shared memory by cp.async (three slices of K
// in flight), row tiles of 16 with the weights streamed into registers; float32: plain FMA in the order of k.
#include "common.cuh"

namespace {

constexpr int MAX_EXPERTS = 256;
constexpr int ROUTE_WARPS = 8;

// A warp per token: a lane keeps the scores of the experts lane, lane + 32, ... (up to eight) and the warp picks the
// `top` largest choices one after the other.
__global__ void __launch_bounds__(ROUTE_WARPS * 32)
moe_route_kernel(const float* __restrict__ z, int z_stride, int Tn, const float* __restrict__ corr, int E, int top, int mode,
                 int* __restrict__ idx_out, float* __restrict__ w_out) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x * ROUTE_WARPS + warp;
  float c_fix[MAX_EXPERTS / 32];
#pragma unroll
  for (int i = 0; i < MAX_EXPERTS / 32; ++i) c_fix[i] = (corr && lane + 32 * i < E) ? corr[lane + 32 * i] : 0.f;   // a weight: fetched before the wait
  mi::grid_dependency_sync();
  if (t >= Tn) return;
  float score[MAX_EXPERTS / 32], choice[MAX_EXPERTS / 32];
#pragma unroll
  for (int i = 0; i < MAX_EXPERTS / 32; ++i) {
    const int e = lane + 32 * i;
    const float ze = e < E ? z[(size_t)t * z_stride + e] : 0.f;
    score[i] = e < E ? (mode == 1 ? ze : 1.f / (1.f + expf(-ze))) : 0.f;
    choice[i] = e < E ? score[i] + c_fix[i] : -INFINITY;
  }
  float sum = 0.f;
  float mine = 0.f;   // lane k keeps the score of choice k
  float first = 0.f;  // mode 1: the largest logit, which is the first choice
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY, best_s = 0.f;
    int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < MAX_EXPERTS / 32; ++i)
      if (choice[i] > best) { best = choice[i]; bi = lane + 32 * i; best_s = score[i]; }    // indices grow: the first of equals stays
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const float os = __shfl_xor_sync(0xffffffffu, best_s, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; best_s = os; }
    }
    if (mode == 1) {
      if (k == 0) first = best_s;
      best_s = expf(best_s - first);
    }
    sum += best_s;
    if (lane == k) mine = best_s;
    if (lane == 0) idx_out[(size_t)t * top + k] = bi;
#pragma unroll
    for (int i = 0; i < MAX_EXPERTS / 32; ++i)
      if (lane + 32 * i == bi) choice[i] = -INFINITY;
  }
  if (lane < top) w_out[(size_t)t * top + lane] = mode == 1 ? mine / sum : mine / (sum + 1e-20f);
}

__global__ void __launch_bounds__(1024)
moe_align_kernel(const int* __restrict__ topk_idx, int n_pairs, int E, int TM, int* __restrict__ sorted_pair,
                 int* __restrict__ pos_of, int* __restrict__ tile_expert, int max_rows, int max_tiles) {
  __shared__ int count[MAX_EXPERTS];
  __shared__ int start[MAX_EXPERTS + 1];
  mi::grid_dependency_sync();
  for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
  for (int i = threadIdx.x; i < max_rows; i += blockDim.x) sorted_pair[i] = -1;
  for (int i = threadIdx.x; i < max_tiles; i += blockDim.x) tile_expert[i] = -1;
  __syncthreads();
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) atomicAdd(&count[topk_idx[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0;
    for (int e = 0; e < E; ++e) {
      start[e] = at;
      at += (count[e] + TM - 1) / TM * TM;
    }
    start[E] = at;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x)
    for (int tile = start[e] / TM; tile < start[e + 1] / TM; ++tile) tile_expert[tile] = e;
  // rows inside an expert's range are handed out in the order of the pairs, so the layout is the same every time
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    if (count[e] == 0) continue;
    int at = start[e];
    for (int i = 0; i < n_pairs; ++i)
      if (topk_idx[i] == e) { sorted_pair[at] = i; pos_of[i] = at; ++at; }
  }
}

// the same without the serial walk, for steps with many pairs: a pair's row inside its expert's range comes from
// an atomic counter (which row a pair gets then varies from run to run; its values do not depend on the row)
__global__ void __launch_bounds__(1024)
moe_align_atomic_kernel(const int* __restrict__ topk_idx, int n_pairs, int E, int TM, int* __restrict__ sorted_pair,
                        int* __restrict__ pos_of, int* __restrict__ tile_expert, int max_rows, int max_tiles) {
  __shared__ int count[MAX_EXPERTS];
  __shared__ int start[MAX_EXPERTS + 1];
  __shared__ int cursor[MAX_EXPERTS];
  mi::grid_dependency_sync();
  for (int e = threadIdx.x; e < E; e += blockDim.x) { count[e] = 0; cursor[e] = 0; }
  for (int i = threadIdx.x; i < max_rows; i += blockDim.x) sorted_pair[i] = -1;
  for (int i = threadIdx.x; i < max_tiles; i += blockDim.x) tile_expert[i] = -1;
  __syncthreads();
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) atomicAdd(&count[topk_idx[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0;
    for (int e = 0; e < E; ++e) {
      start[e] = at;
      at += (count[e] + TM - 1) / TM * TM;
    }
    start[E] = at;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x)
    for (int tile = start[e] / TM; tile < start[e + 1] / TM; ++tile) tile_expert[tile] = e;
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
    const int e = topk_idx[i];
    const int at = start[e] + atomicAdd(&cursor[e], 1);
    sorted_pair[at] = i;
    pos_of[i] = at;
  }
}

// ---------------------------------------------------------------------------------------------- products

struct GroupedArgs {
  const void* a;          // rows: gathered by pair (row = pair / top) if gather, else row = position
  int a_stride;
  const void* w;          // [E, n_rows_per_expert, K]
  void* out;              // [max_rows, N]
  const int* sorted_pair;
  const int* tile_expert;
  int N, K, top, gather;
  long long w_expert_stride;   // elements between two experts' matrices
  int glu;                     // the gated activation of the gate-and-up product (a MiGlu) and its limit
  float limit;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

constexpr int GBK = 64;          // k per stage
constexpr int GLDS = GBK + 8;    // shared-memory row stride in elements (odd number of 16-byte units)
constexpr int WN_COLS = 32;      // columns of a warp's tile

// WM x WN warps; a warp owns 16 rows x 32 columns (of gate and of up, if SWIGLU).  Block tile: 16 WM rows x 32 WN columns.
// STAGES slices of 64 elements of K are in flight: with few rows an expert the kernel streams weights, and what a block
// has asked for is what keeps the memory busy - narrow tiles take more stages.
template <int WM, int WN, bool SWIGLU, int STAGES>
__global__ void __launch_bounds__(WM * WN * 32)
moe_gemm_bf16_kernel(GroupedArgs a) {
  constexpr int TM = 16 * WM, BN = WN_COLS * WN, THREADS = WM * WN * 32;
  constexpr int NB = SWIGLU ? 2 : 1;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* as = reinterpret_cast<__nv_bfloat16*>(smem_raw);        // [STAGES][TM][GLDS]
  __nv_bfloat16* bs = as + STAGES * TM * GLDS;                           // [STAGES][NB][BN][GLDS]
  __shared__ int s_row[TM];
  const int tile = blockIdx.y, n0 = blockIdx.x * BN;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int wm = warp % WM, wn = warp / WM;
  const int g = lane >> 2, t = lane & 3, lm = lane >> 3, lr = lane & 7;
  mi::grid_dependency_sync();
  const int e = a.tile_expert[tile];
  if (e < 0) return;
  for (int r = threadIdx.x; r < TM; r += THREADS) {
    const int pair = a.sorted_pair[tile * TM + r];
    s_row[r] = pair < 0 ? -1 : (a.gather ? pair / a.top : tile * TM + r);
  }
  __syncthreads();
  const __nv_bfloat16* A = (const __nv_bfloat16*)a.a;
  const __nv_bfloat16* W = (const __nv_bfloat16*)a.w + (size_t)e * a.w_expert_stride;
  const int K = a.K, N = a.N;
  constexpr int CH = GBK / 8;   // 16-byte chunks of a staged row

  auto load = [&](int stage, int k0) {
    __nv_bfloat16* ad = as + stage * TM * GLDS;
    for (int idx = threadIdx.x; idx < TM * CH; idx += THREADS) {
      const int r = idx / CH, c = idx % CH;
      const int row = s_row[r];
      const bool valid = row >= 0 && k0 + c * 8 < K;
      cp_async16(ad + r * GLDS + c * 8, valid ? A + (size_t)row * a.a_stride + k0 + c * 8 : A, valid);
    }
#pragma unroll
    for (int b = 0; b < NB; ++b) {
      __nv_bfloat16* bd = bs + (stage * NB + b) * BN * GLDS;
      for (int idx = threadIdx.x; idx < BN * CH; idx += THREADS) {
        const int r = idx / CH, c = idx % CH;
        const bool valid = n0 + r < N && k0 + c * 8 < K;
        cp_async16(bd + r * GLDS + c * 8, valid ? W + ((size_t)b * N + n0 + r) * K + k0 + c * 8 : W, valid);
      }
    }
  };

  float acc[NB][4][4];
#pragma unroll
  for (int b = 0; b < NB; ++b)
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[b][i][c] = 0.f;

  const int nk = (K + GBK - 1) / GBK;
#pragma unroll
  for (int st = 0; st < STAGES - 1; ++st) {
    if (st < nk) load(st, st * GBK);
    cp_async_commit();
  }
  for (int kb = 0; kb < nk; ++kb) {
    const int stage = kb % STAGES;
    cp_async_wait<STAGES - 2>();       // slice kb has landed
    __syncthreads();                   // ... for every thread; and everyone is done with slice kb - 1, whose stage is asked for next
    {
      const int nxt = kb + STAGES - 1;
      if (nxt < nk) load(nxt % STAGES, nxt * GBK);
      cp_async_commit();
    }
    const __nv_bfloat16* at = as + stage * TM * GLDS + (wm * 16 + (lm & 1) * 8 + lr) * GLDS + (lm >> 1) * 8;
#pragma unroll
    for (int k = 0; k < GBK / 16; ++k) {
      uint32_t af[4];
      ldmatrix_x4(af, at + k * 16);
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        const __nv_bfloat16* bt = bs + (stage * NB + b) * BN * GLDS + (wn * WN_COLS + (lm >> 1) * 8 + lr) * GLDS + k * 16 + (lm & 1) * 8;
#pragma unroll
        for (int nb = 0; nb < 2; ++nb) {
          uint32_t bf[4];
          ldmatrix_x4(bf, bt + nb * 16 * GLDS);
          mma_bf16(acc[b][2 * nb], af, bf[0], bf[1]);
          mma_bf16(acc[b][2 * nb + 1], af, bf[2], bf[3]);
        }
      }
    }
  }
  cp_async_wait<0>();

  // rows g and g + 8 of the warp's 16, columns wn * 32 + i * 8 + 2 t (+1)
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = wm * 16 + g + 8 * h;
    if (s_row[r] < 0) continue;
    const size_t orow = (size_t)(tile * TM + r) * N;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int n = n0 + wn * WN_COLS + i * 8 + 2 * t;
      if (n >= N) continue;
      if (SWIGLU) {
        const float y0 = mi::glu_fast(acc[0][i][2 * h], acc[1][i][2 * h], a.glu, a.limit);
        const float y1 = mi::glu_fast(acc[0][i][2 * h + 1], acc[1][i][2 * h + 1], a.glu, a.limit);
        __nv_bfloat16* o = (__nv_bfloat16*)a.out + orow + n;
        o[0] = __float2bfloat16_rn(y0);
        if (n + 1 < N) o[1] = __float2bfloat16_rn(y1);
      } else {
        float* o = (float*)a.out + orow + n;
        o[0] = acc[0][i][2 * h];
        if (n + 1 < N) o[1] = acc[0][i][2 * h + 1];
      }
    }
  }
}

// Few rows an expert (a decode step): the time goes into reading each expert's matrices once, so the weights go from
// global memory straight to the registers of the warp that multiplies them - 16-byte loads that bypass L1, four slices
// of K asked for before the first is used - as in the engine's few-row product for dense matrices.  A block of eight
// warps owns a row tile of 16 rows and 8 * (8 / KS) output columns; KS warps share a group of 8 columns (of gate and
// of up, if SWIGLU) and deal the 32-element slices of K among them, and their partial tiles are added through shared
// memory in the order of the warps, so a value is a function of (N, K) alone.  The k index inside a slice is permuted
// the same way for both operands, so that a thread's 16-byte load is its fragment of two consecutive MMAs.
__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

constexpr int SW = 8;       // warps of a block of the streaming product

template <bool SWIGLU, int KS>
__global__ void __launch_bounds__(SW * 32)
moe_stream_bf16_kernel(GroupedArgs a) {
  constexpr int NB = SWIGLU ? 2 : 1, GROUPS = SW / KS, U = 4;
  __shared__ float red[SW][16][NB * 8 + 1];
  __shared__ int s_row[16];
  const int tile = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int group = warp / KS, kpart = warp % KS;
  const int n0 = (blockIdx.x * GROUPS + group) * 8;
  mi::grid_dependency_sync();
  const int e = a.tile_expert[tile];
  if (e < 0) return;
  if (threadIdx.x < 16) {
    const int pair = a.sorted_pair[tile * 16 + threadIdx.x];
    s_row[threadIdx.x] = pair < 0 ? -1 : (a.gather ? pair / a.top : tile * 16 + (int)threadIdx.x);
  }
  __syncthreads();
  const int K = a.K, N = a.N;
  const __nv_bfloat16* A = (const __nv_bfloat16*)a.a;
  const __nv_bfloat16* W = (const __nv_bfloat16*)a.w + (size_t)e * a.w_expert_stride;
  const int ra = s_row[g], rb = s_row[g + 8];
  const __nv_bfloat16* xa = ra >= 0 ? A + (size_t)ra * a.a_stride : nullptr;
  const __nv_bfloat16* xb = rb >= 0 ? A + (size_t)rb * a.a_stride : nullptr;
  const bool col_ok = n0 + g < N;
  const __nv_bfloat16* wrow[NB];
#pragma unroll
  for (int b = 0; b < NB; ++b) wrow[b] = W + ((size_t)b * N + n0 + g) * K;
  float acc[NB][4];
#pragma unroll
  for (int b = 0; b < NB; ++b)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[b][c] = 0.f;
  const uint4 zero = make_uint4(0, 0, 0, 0);
  const int nkb = (K + 31) / 32;
  for (int kb0 = kpart; kb0 < nkb; kb0 += KS * U) {
    uint4 wv[U][NB], va[U], vb[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int k = (kb0 + u * KS) * 32 + 8 * t;
      const bool ok = kb0 + u * KS < nkb && k < K;
#pragma unroll
      for (int b = 0; b < NB; ++b) wv[u][b] = (ok && col_ok) ? ld_stream16(wrow[b] + k) : zero;
      va[u] = (ok && xa) ? __ldg(reinterpret_cast<const uint4*>(xa + k)) : zero;
      vb[u] = (ok && xb) ? __ldg(reinterpret_cast<const uint4*>(xb + k)) : zero;
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint32_t aa[4] = {va[u].x, va[u].y, va[u].z, va[u].w}, ab[4] = {vb[u].x, vb[u].y, vb[u].z, vb[u].w};
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        const uint32_t ww[4] = {wv[u][b].x, wv[u][b].y, wv[u][b].z, wv[u][b].w};
#pragma unroll
        for (int m = 0; m < 2; ++m) {
          const uint32_t af[4] = {aa[2 * m], ab[2 * m], aa[2 * m + 1], ab[2 * m + 1]};
          mma_bf16(acc[b], af, ww[2 * m], ww[2 * m + 1]);
        }
      }
    }
  }
#pragma unroll
  for (int b = 0; b < NB; ++b) {
    red[warp][g][b * 8 + 2 * t] = acc[b][0];
    red[warp][g][b * 8 + 2 * t + 1] = acc[b][1];
    red[warp][g + 8][b * 8 + 2 * t] = acc[b][2];
    red[warp][g + 8][b * 8 + 2 * t + 1] = acc[b][3];
  }
  __syncthreads();
  // 16 rows x 8 columns per group: a thread each, the KS partial tiles added in the order of the warps
  for (int idx = threadIdx.x; idx < GROUPS * 128; idx += SW * 32) {
    const int grp = idx / 128, r = (idx % 128) / 8, c = idx % 8;
    const int n = (blockIdx.x * GROUPS + grp) * 8 + c;
    if (s_row[r] < 0 || n >= N) continue;
    float v[NB];
#pragma unroll
    for (int b = 0; b < NB; ++b) {
      v[b] = 0.f;
#pragma unroll
      for (int k = 0; k < KS; ++k) v[b] += red[grp * KS + k][r][b * 8 + c];
    }
    const size_t o = (size_t)(tile * 16 + r) * N + n;
    if (SWIGLU) ((__nv_bfloat16*)a.out)[o] = __float2bfloat16_rn(mi::glu_fast(v[0], v[NB - 1], a.glu, a.limit));
    else ((float*)a.out)[o] = v[0];
  }
}

// float32: 16 rows x 64 columns per block of 256 threads, a thread one row x 4 columns; sums in the order of k
constexpr int FTM = 16, FBN = 64, FBK = 16;

template <bool SWIGLU>
__global__ void __launch_bounds__(256)
moe_gemm_f32_kernel(GroupedArgs a) {
  constexpr int NB = SWIGLU ? 2 : 1;
  __shared__ float as[FTM][FBK + 1];
  __shared__ float bs[NB][FBN][FBK + 1];
  __shared__ int s_row[FTM];
  const int tile = blockIdx.y, n0 = blockIdx.x * FBN;
  mi::grid_dependency_sync();
  const int e = a.tile_expert[tile];
  if (e < 0) return;
  if (threadIdx.x < FTM) {
    const int pair = a.sorted_pair[tile * FTM + threadIdx.x];
    s_row[threadIdx.x] = pair < 0 ? -1 : (a.gather ? pair / a.top : tile * FTM + (int)threadIdx.x);
  }
  __syncthreads();
  const float* A = (const float*)a.a;
  const float* W = (const float*)a.w + (size_t)e * a.w_expert_stride;
  const int K = a.K, N = a.N;
  const int r = threadIdx.x / 16, cg = threadIdx.x % 16;
  float acc[NB][4];
#pragma unroll
  for (int b = 0; b < NB; ++b)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[b][c] = 0.f;
  for (int k0 = 0; k0 < K; k0 += FBK) {
    {
      const int rr = threadIdx.x / FBK, kk = threadIdx.x % FBK;     // 16 x 16 = 256 values of A
      const int row = s_row[rr];
      as[rr][kk] = (row >= 0 && k0 + kk < K) ? A[(size_t)row * a.a_stride + k0 + kk] : 0.f;
    }
#pragma unroll
    for (int b = 0; b < NB; ++b)
      for (int idx = threadIdx.x; idx < FBN * FBK; idx += 256) {
        const int rr = idx / FBK, kk = idx % FBK;
        bs[b][rr][kk] = (n0 + rr < N && k0 + kk < K) ? W[((size_t)b * N + n0 + rr) * K + k0 + kk] : 0.f;
      }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < FBK; ++kk) {
      const float av = as[r][kk];
#pragma unroll
      for (int b = 0; b < NB; ++b)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[b][c] = fmaf(av, bs[b][cg * 4 + c][kk], acc[b][c]);
    }
    __syncthreads();
  }
  if (s_row[r] < 0) return;
  float* o = (float*)a.out + (size_t)(tile * FTM + r) * N;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const int n = n0 + cg * 4 + c;
    if (n < N) o[n] = SWIGLU ? mi::glu_exact(acc[0][c], acc[NB - 1][c], a.glu, a.limit) : acc[0][c];
  }
}

template <typename TOut, typename TY>
__global__ void __launch_bounds__(256)
moe_combine_kernel(TOut* __restrict__ out, const TY* __restrict__ y, const int* __restrict__ pos_of,
                   const float* __restrict__ w, int top, int N, const TOut* __restrict__ shared,
                   const float* __restrict__ shared_logit, int logit_stride) {
  mi::grid_dependency_sync();
  const int t = blockIdx.x;
  // an expert every token runs through: its row joins the sum, times the sigmoid of the token's gate logit if there is one
  const float sw = shared ? (shared_logit ? 1.f / (1.f + expf(-shared_logit[(size_t)t * logit_stride])) : 1.f) : 0.f;
  for (int n = threadIdx.x; n < N; n += blockDim.x) {
    float acc = 0.f;
    for (int k = 0; k < top; ++k) acc = fmaf(w[(size_t)t * top + k], mi::to_float(y[(size_t)pos_of[(size_t)t * top + k] * N + n]), acc);
    if (shared) acc = fmaf(sw, mi::to_float(shared[(size_t)t * N + n]), acc);
    out[(size_t)t * N + n] = mi::from_float<TOut>(acc);
  }
}

// The tokens' rows put in the order of the experts' rows: xs[pos] = x[pair / top] for the rows that a pair owns, zeros
// for the others; 16 bytes a thread.  (The tcgen05 product reads its rows by TMA, which wants them side by side.)
__global__ void __launch_bounds__(256)
moe_gather_kernel(__nv_bfloat16* __restrict__ xs, const __nv_bfloat16* __restrict__ x, const int* __restrict__ sorted_pair,
                  int top, int H8) {
  mi::grid_dependency_sync();
  const int pos = blockIdx.x;
  const int pair = sorted_pair[pos];
  uint4* dst = reinterpret_cast<uint4*>(xs) + (size_t)pos * H8;
  const uint4* src = pair >= 0 ? reinterpret_cast<const uint4*>(x) + (size_t)(pair / top) * H8 : nullptr;
  for (int i = threadIdx.x; i < H8; i += blockDim.x) dst[i] = src ? src[i] : make_uint4(0, 0, 0, 0);
}

template <int WM, int WN, bool SWIGLU, int STAGES>
int launch_bf16(const GroupedArgs& a, int tiles, cudaStream_t stream) {
  constexpr int TM = 16 * WM, BN = WN_COLS * WN;
  const size_t smem = (size_t)STAGES * (TM + (SWIGLU ? 2 : 1) * BN) * GLDS * sizeof(__nv_bfloat16);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(moe_gemm_bf16_kernel<WM, WN, SWIGLU, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return mi_fail("moe_gemm: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  mi::launch(moe_gemm_bf16_kernel<WM, WN, SWIGLU, STAGES>, dim3((a.N + BN - 1) / BN, tiles), dim3(WM * WN * 32), smem, stream, a);
  return 0;
}

}  // namespace

// Rows of a row tile for a step with `n_pairs` (token, choice) pairs: 16 while an expert gets few rows, 64 beyond.
MI_API int mi_moe_row_tile(int n_pairs, int E, int dtype) {
  if (dtype == MI_F32) return FTM;
  return n_pairs >= 32 * E ? 64 : 16;
}

// z: the router's logits in float32, rows of z_stride >= E values (a product of the engine's own: W_router h with float32
// accumulation).  mode 0: sigmoid scores, chosen by score + correction, weights the scores over their sum; mode 1: the
// largest logits are chosen (correction, if given, added for the choice), weights the softmax over the chosen logits.
MI_API int mi_moe_route(const float* z, int z_stride, int T, const float* correction, int E, int top, int mode, int* idx_out, float* w_out,
                        cudaStream_t stream) {
  MI_REQUIRE((mode == 0 || mode == 1) && z_stride >= E, "moe_route: mode %d is not known or rows of %d logits are too short", mode, z_stride);
  MI_REQUIRE(T >= 0 && E > 0 && E <= MAX_EXPERTS, "moe_route: experts=%d must lie in 1..%d", E, MAX_EXPERTS);
  MI_REQUIRE(top > 0 && top <= E && top <= 32, "moe_route: top=%d must lie in 1..min(experts, 32)", top);
  if (T == 0) return 0;
  mi::launch(moe_route_kernel, dim3((T + ROUTE_WARPS - 1) / ROUTE_WARPS), dim3(ROUTE_WARPS * 32), 0, stream, z, z_stride, T, correction, E, top, mode, idx_out, w_out);
  MI_LAUNCH_OK("moe_route");
  return 0;
}

MI_API int mi_moe_align(const int* topk_idx, int n_pairs, int E, int TM, int* sorted_pair, int* pos_of, int* tile_expert,
                        int max_rows, int max_tiles, cudaStream_t stream) {
  MI_REQUIRE(E > 0 && E <= MAX_EXPERTS && TM > 0 && max_rows == max_tiles * TM, "moe_align: bad sizes");
  MI_REQUIRE(max_rows >= n_pairs + E * (TM - 1), "moe_align: %d rows cannot hold %d pairs of %d experts in tiles of %d", max_rows, n_pairs, E, TM);
  if (n_pairs == 0) return 0;
  if (n_pairs <= 256)
    mi::launch(moe_align_kernel, dim3(1), dim3(1024), 0, stream, topk_idx, n_pairs, E, TM, sorted_pair, pos_of, tile_expert, max_rows, max_tiles);
  else
    mi::launch(moe_align_atomic_kernel, dim3(1), dim3(1024), 0, stream, topk_idx, n_pairs, E, TM, sorted_pair, pos_of, tile_expert, max_rows, max_tiles);
  MI_LAUNCH_OK("moe_align");
  return 0;
}

// swiglu 1: out[row, :N] = act(a w_gate^T) * (a w_up^T), the expert's matrix holding N gate rows and then N up rows,
// rows gathered from the tokens, the gated activation `glu` (a MiGlu) with its `limit`; swiglu 0: out[row, :N] = a w^T in
// float32, rows by position.
MI_API int mi_moe_gemm(const void* a_rows, int dtype, int a_stride, const void* w, void* out, const int* sorted_pair,
                       const int* tile_expert, int max_tiles, int TM, int N, int K, int top, int swiglu, int glu, float limit,
                       cudaStream_t stream) {
  MI_REQUIRE(glu == MI_GLU_SILU || (glu == MI_GLU_CLAMPED && limit > 0.f), "moe_gemm: unknown activation %d or a limit that is not positive", glu);
  MI_REQUIRE(N > 0 && K > 0 && max_tiles >= 0 && max_tiles <= 65535, "moe_gemm: bad sizes N=%d K=%d tiles=%d", N, K, max_tiles);
  if (max_tiles == 0) return 0;
  GroupedArgs g;
  g.a = a_rows; g.a_stride = a_stride; g.w = w; g.out = out; g.sorted_pair = sorted_pair; g.tile_expert = tile_expert;
  g.N = N; g.K = K; g.top = top; g.gather = swiglu ? 1 : 0; g.glu = glu; g.limit = limit;
  g.w_expert_stride = (long long)(swiglu ? 2 : 1) * N * K;
  if (dtype == MI_F32) {
    MI_REQUIRE(TM == FTM, "moe_gemm: the float32 product takes row tiles of %d", FTM);
    const dim3 grid((N + FBN - 1) / FBN, max_tiles);
    if (swiglu) mi::launch(moe_gemm_f32_kernel<true>, grid, dim3(256), 0, stream, g);
    else mi::launch(moe_gemm_f32_kernel<false>, grid, dim3(256), 0, stream, g);
  } else if (dtype == MI_BF16) {
    MI_REQUIRE(K % 8 == 0 && a_stride % 8 == 0, "moe_gemm: K=%d and the row stride %d must be multiples of 8 in bfloat16", K, a_stride);
    MI_REQUIRE(((uintptr_t)a_rows % 16) == 0 && ((uintptr_t)w % 16) == 0, "moe_gemm: operands must be 16-byte aligned");
    int rc;
    if (TM == 64) rc = swiglu ? launch_bf16<4, 2, true, 3>(g, max_tiles, stream) : launch_bf16<4, 2, false, 3>(g, max_tiles, stream);
    else if (TM == 16) {
      // few rows an expert: the weights are streamed once, straight into registers; K is dealt to eight warps where it
      // is long, to four (two groups of columns a block) where it is short
      MI_REQUIRE((N + 7) / 8 <= 65535 * 2, "moe_gemm: too many columns for one launch");
      rc = 0;
      if (K >= 1024) {
        const dim3 grid((N + 7) / 8, max_tiles);
        if (swiglu) mi::launch(moe_stream_bf16_kernel<true, 8>, grid, dim3(SW * 32), 0, stream, g);
        else mi::launch(moe_stream_bf16_kernel<false, 8>, grid, dim3(SW * 32), 0, stream, g);
      } else {
        const dim3 grid((N + 15) / 16, max_tiles);
        if (swiglu) mi::launch(moe_stream_bf16_kernel<true, 4>, grid, dim3(SW * 32), 0, stream, g);
        else mi::launch(moe_stream_bf16_kernel<false, 4>, grid, dim3(SW * 32), 0, stream, g);
      }
    }
    else return mi_fail("moe_gemm: row tiles of 16 or 64 in bfloat16, got %d", TM);
    if (rc) return rc;
  } else {
    return mi_fail("moe_gemm: unknown dtype %d", dtype);
  }
  MI_LAUNCH_OK("moe_gemm");
  return 0;
}

MI_API int mi_moe_gather(void* xs, const void* x, const int* sorted_pair, int rows, int top, int H, cudaStream_t stream) {
  MI_REQUIRE(rows >= 0 && top > 0 && H > 0 && H % 8 == 0, "moe_gather: rows of %d values (a multiple of 8 in bfloat16)", H);
  MI_REQUIRE(((uintptr_t)xs % 16) == 0 && ((uintptr_t)x % 16) == 0, "moe_gather: operands must be 16-byte aligned");
  if (rows == 0) return 0;
  mi::launch(moe_gather_kernel, dim3(rows), dim3(256), 0, stream, (__nv_bfloat16*)xs, (const __nv_bfloat16*)x, sorted_pair, top, H / 8);
  MI_LAUNCH_OK("moe_gather");
  return 0;
}

// y: the down rows, float32 (y_dtype MI_F32) or bfloat16.  shared (or null): rows [T, N] of out's type that every token adds,
// times sigmoid(shared_logit[t * logit_stride]) if shared_logit is given.
MI_API int mi_moe_combine(void* out, int out_dtype, const void* y, int y_dtype, const int* pos_of, const float* weights, int T, int top, int N,
                          const void* shared, const float* shared_logit, int logit_stride, cudaStream_t stream) {
  MI_REQUIRE(T >= 0 && top > 0 && N > 0, "moe_combine: bad sizes");
  if (T == 0) return 0;
  if (out_dtype == MI_BF16 && y_dtype == MI_F32)
    mi::launch(moe_combine_kernel<__nv_bfloat16, float>, dim3(T), dim3(256), 0, stream, (__nv_bfloat16*)out, (const float*)y, pos_of, weights, top, N, (const __nv_bfloat16*)shared, shared_logit, logit_stride);
  else if (out_dtype == MI_BF16 && y_dtype == MI_BF16)
    mi::launch(moe_combine_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(T), dim3(256), 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)y, pos_of, weights, top, N, (const __nv_bfloat16*)shared, shared_logit, logit_stride);
  else if (out_dtype == MI_F32 && y_dtype == MI_F32)
    mi::launch(moe_combine_kernel<float, float>, dim3(T), dim3(256), 0, stream, (float*)out, (const float*)y, pos_of, weights, top, N, (const float*)shared, shared_logit, logit_stride);
  else
    return mi_fail("moe_combine: unknown dtypes %d, %d", out_dtype, y_dtype);
  MI_LAUNCH_OK("moe_combine");
  return 0;
}
