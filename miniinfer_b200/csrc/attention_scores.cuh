// Scores that are shaped before the weights are made, for the bfloat16 attention kernels, which all keep an online
// softmax in base 2 (a running maximum m, weights 2^(s - m), a running sum l, the output divided by l at the end).
//
//   softcap > 0   a scaled score x = scale * q.k becomes softcap * tanh(x / softcap);
//   sigmoid       the weight of a visible key is sigmoid(x + bias[head]) and nothing is normalised over the keys.
//
// The kernels keep their arithmetic: a shaped score enters as the base-2 logarithm of its weight, s = log2(sigmoid(x + b))
// = -log2(1 + 2^(-(x + b) log2 e)), so 2^(s - m) is the weight times 2^(-m), the partial outputs of blocks, warps and
// chunks merge with the factors 2^(m_part - m) as they always do, and at the very end the output is multiplied with 2^m
// where the softmax divides by l.  tanh is 1 - 2 / (1 + 2^(2 y log2 e)): its absolute error of about 1e-7 times the cap is
// far below what rounding the weights to bfloat16 leaves.
#pragma once

#include <cuda_runtime.h>

namespace mi {

struct ScoreShape {
  float scale;          // of q.k
  float softcap;        // 0: none
  const float* bias;    // [heads] float32: sigmoid weights; null: softmax
};

__device__ __forceinline__ float ex2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float lg2_fast(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// raw = q.k; returns the base-2 logit the online softmax takes.  `head_bias` is bias[head] (ignored for softmax).
__device__ __forceinline__ float shaped_logit2(float raw, float scale, float softcap, bool sigmoid, float head_bias) {
  constexpr float LOG2E = 1.4426950408889634f;
  float x = raw * scale;
  if (softcap > 0.f) {
    const float e = ex2_fast(fminf(x * (2.f * LOG2E / softcap), 60.f));      // beyond, tanh is 1 to the last bit
    x = softcap * (1.f - __fdividef(2.f, 1.f + e));
  }
  if (!sigmoid) return x * LOG2E;
  return -lg2_fast(1.f + ex2_fast(-(x + head_bias) * LOG2E));
}

// The weight itself, sigmoid(cap(scale * raw) + head_bias), for kernels that keep sigmoid weights as they are: they lie in
// (0, 1), so nothing has to be held against a running maximum.
__device__ __forceinline__ float shaped_sigmoid_weight(float raw, float scale, float softcap, float head_bias) {
  constexpr float LOG2E = 1.4426950408889634f;
  float x = raw * scale;
  if (softcap > 0.f) {
    const float e = ex2_fast(fminf(x * (2.f * LOG2E / softcap), 60.f));
    x = softcap * (1.f - __fdividef(2.f, 1.f + e));
  }
  return __fdividef(1.f, 1.f + ex2_fast(fminf(-(x + head_bias) * LOG2E, 80.f)));      // beyond 2^80 the weight is nothing
}

}  // namespace mi
