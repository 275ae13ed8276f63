// Sigmoid arithmetic shared by the forward and backward kernels.
#pragma once

#include "ptx.cuh"

namespace sigattn {

constexpr float kLog2e = 1.4426950408889634f;

// sigmoid(x) with x given in the base-2 domain (t = x * log2(e)).
// e = 2^-|t| in (0,1] (one MUFU op); sigmoid = (t < 0 ? e : 1) / (1 + e).  This keeps RELATIVE
// accuracy for strongly negative logits (the default bias is -log(T), so a typical probability
// is ~1/T), which 0.5 + 0.5 tanh(x/2) does not.  1/(1+e) on [0,1] is a minimax polynomial on
// the FMA pipe (packed f32x2) instead of a second MUFU op: the MUFU unit (16 results / clock /
// SM) and the instruction issue slots are what bound the kernels.  Maximum relative error of
// the polynomial: 3.0e-4 (degree 4, used for fp16, whose own rounding is 4.9e-4) and 1.7e-3
// (degree 3, used for bf16, rounding 3.9e-3).
template <bool kBF16>
__device__ __forceinline__ float2 rcp1p_poly(float2 e) {
  float2 r;
  if constexpr (kBF16) {
    r = make_float2(-0.2218334674835205f, -0.2218334674835205f);
    r = __ffma2_rn(r, e, make_float2(0.6655056476593018f, 0.6655056476593018f));
    r = __ffma2_rn(r, e, make_float2(-0.9428054094314575f, -0.9428054094314575f));
    r = __ffma2_rn(r, e, make_float2(0.9982667565345764f, 0.9982667565345764f));
  } else {
    r = make_float2(0.1522425264120102f, 0.1522425264120102f);
    r = __ffma2_rn(r, e, make_float2(-0.5328524708747864f, -0.5328524708747864f));
    r = __ffma2_rn(r, e, make_float2(0.8658902645111084f, 0.8658902645111084f));
    r = __ffma2_rn(r, e, make_float2(-0.9848342537879944f, -0.9848342537879944f));
    r = __ffma2_rn(r, e, make_float2(0.9997026324272156f, 0.9997026324272156f));
  }
  return r;
}

// Two sigmoids at once; t holds the logits times log2(e).
template <bool kBF16>
__device__ __forceinline__ float2 sigmoid2_from_log2(float2 t) {
  float2 e = make_float2(ex2_approx(-fabsf(t.x)), ex2_approx(-fabsf(t.y)));
  const float2 r = rcp1p_poly<kBF16>(e);
  e.x = t.x < 0.0f ? e.x : 1.0f;
  e.y = t.y < 0.0f ? e.y : 1.0f;
  return __fmul2_rn(e, r);
}

// The same when both logits are known to be negative (the usual case under the default bias):
// no absolute value and no select.
template <bool kBF16>
__device__ __forceinline__ float2 sigmoid2_from_log2_neg(float2 t) {
  const float2 e = make_float2(ex2_approx(t.x), ex2_approx(t.y));
  return __fmul2_rn(e, rcp1p_poly<kBF16>(e));
}

// Far below zero the series sigmoid(x) = e - e^2 + e^3 - ... (e = exp(x)) needs very few terms.  The
// kernels evaluate their logits shifted up by kDeepShift (in the base-2 domain, folded into the bias
// they add anyway), u = t + kDeepShift, so that "every logit of the warp is below -kDeepShift" is the
// same sign-bit test as warp_all_negative(); that is the usual case under the default bias -log(T)
// (a typical probability is 1/T).  With e' = 2^u = 2^kDeepShift e:
//   fp16: p = e' (a + e' (b + e' c)),  a = 2^-5, b = -2^-10, c = 2^-15   (relative error < e^3 <= 3.1e-5)
//   bf16: p = e' (a + e' b)                                             (relative error < e^2 <= 9.8e-4)
// i.e. two or three packed operations after the exponential instead of four or five.
constexpr float kDeepShift = 5.0f;
template <bool kBF16>
__device__ __forceinline__ float2 sigmoid2_from_shifted_log2_deep(float2 u) {
  const float2 e = make_float2(ex2_approx(u.x), ex2_approx(u.y));
  constexpr float a = 0.03125f, b = -0.0009765625f, c = 0.000030517578125f;
  float2 r;
  if constexpr (kBF16) {
    r = __ffma2_rn(e, make_float2(b, b), make_float2(a, a));
  } else {
    r = __ffma2_rn(e, make_float2(c, c), make_float2(b, b));
    r = __ffma2_rn(r, e, make_float2(a, a));
  }
  return __fmul2_rn(e, r);
}

// True when every one of a warp's logits t[0..N) (all 32 lanes) is negative: AND of the sign bits.
template <int N>
__device__ __forceinline__ bool warp_all_negative(const float2 (&t)[N]) {
  uint32_t sgn = 0x80000000u;
#pragma unroll
  for (int i = 0; i < N; ++i) sgn &= __float_as_uint(t[i].x) & __float_as_uint(t[i].y);
  return __all_sync(0xffffffffu, (int)sgn < 0) != 0;
}

}  // namespace sigattn
