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

// ---------------------------------------------------------------- cheaper forms for the deep regime
// 2^u for u <= 0 without the MUFU unit: floor(u) by the magic-number addition (rounded down, so the low
// mantissa bits of the sum hold the integer part), a minimax polynomial of the fraction (degree 3:
// relative error 7.5e-5, used for fp16; degree 2: 1.7e-3, used for bf16, whose own rounding is 3.9e-3) and
// the exponent inserted by an integer shift-add.  Inputs below -125 give 2^-125 (the caller's result
// underflows to zero in 16 bits either way).  The kernels evaluate a small fraction of their
// exponentials this way: the MUFU unit (16 results / clock / SM) is the scarcest resource of the sigmoid
// warps, and a few exponentials per chunk fit into otherwise idle FMA / ALU issue slots.
template <bool kBF16>
__device__ __forceinline__ float2 ex2_emulated2(float2 u) {
  u.x = fmaxf(u.x, -125.0f);
  u.y = fmaxf(u.y, -125.0f);
  constexpr float kMagic = 12582912.0f;  // 2^23 + 2^22
  float2 y;
  const float2 magic2 = make_float2(kMagic, kMagic);
  asm("add.rm.ftz.f32x2 %0, %1, %2;"
      : "=l"(*reinterpret_cast<unsigned long long*>(&y))
      : "l"(*reinterpret_cast<const unsigned long long*>(&u)), "l"(*reinterpret_cast<const unsigned long long*>(&magic2)));
  const float2 yb = __fadd2_rn(y, make_float2(-kMagic, -kMagic));
  const float2 r = __fadd2_rn(u, make_float2(-yb.x, -yb.y));  // fraction in [0, 1)
  float2 p;
  if constexpr (kBF16) {
    p = __ffma2_rn(make_float2(0.3371894061565399f, 0.3371894061565399f), r, make_float2(0.657636284828186f, 0.657636284828186f));
    p = __ffma2_rn(p, r, make_float2(1.0017247200012207f, 1.0017247200012207f));
  } else {
    p = __ffma2_rn(make_float2(0.07802452147006989f, 0.07802452147006989f), r, make_float2(0.22606715559959412f, 0.22606715559959412f));
    p = __ffma2_rn(p, r, make_float2(0.6958335638046265f, 0.6958335638046265f));
    p = __ffma2_rn(p, r, make_float2(0.9999251961708069f, 0.9999251961708069f));
  }
  float2 o;
  o.x = __int_as_float(__float_as_int(p.x) + (__float_as_int(y.x) << 23));
  o.y = __int_as_float(__float_as_int(p.y) + (__float_as_int(y.y) << 23));
  return o;
}

// Packed 16-bit arithmetic (two elements per instruction and lane).
template <bool kBF16>
__device__ __forceinline__ uint32_t hfma2(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  if constexpr (kBF16) asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  else                 asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
template <bool kBF16>
__device__ __forceinline__ uint32_t hmul2(uint32_t a, uint32_t b) {
  uint32_t d;
  if constexpr (kBF16) asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  else                 asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// The deep-regime series of sigmoid2_from_shifted_log2_deep() evaluated in the 16-bit type the result is
// stored in anyway: e' = 2^u is rounded to 16 bits first and the series runs on packed pairs,
//   fp16: p = e' (a + e' (b + e' c)),   bf16: p = e' (a + e' b),   a = 2^-5, b = -2^-10, c = 2^-15,
// which halves the instructions after the exponential (one conversion, two or three packed operations
// per PAIR of elements).  Relative error: two roundings of the 16-bit type instead of one.
// `emulate` selects the FMA-pipe exponential for this pair.
template <bool kBF16>
__device__ __forceinline__ uint32_t sigmoid2_deep_packed(float2 u, bool emulate) {
  const float2 e = emulate ? ex2_emulated2<kBF16>(u) : make_float2(ex2_approx(u.x), ex2_approx(u.y));
  const uint32_t eh = pack2<kBF16>(e.x, e.y);
  if constexpr (kBF16) {
    return hmul2<true>(eh, hfma2<true>(eh, 0xBA80BA80u, 0x3D003D00u));
  } else {
    uint32_t w = hfma2<false>(eh, 0x02000200u, 0x94009400u);
    w = hfma2<false>(w, eh, 0x28002800u);
    return hmul2<false>(eh, w);
  }
}

// Accurate form (the reference's TRITON_SIGMOID_ACCURATE mode, src/triton_sigmoid/kernel_utils.py:190-193,
// 236-237, selects tl.sigmoid there): exponential and reciprocal both on the MUFU unit, no polynomial;
// relative error ~2^-22.  Twice the MUFU work of the default form.
__device__ __forceinline__ float2 sigmoid2_accurate_from_log2(float2 t) {
  float2 e = make_float2(ex2_approx(-fabsf(t.x)), ex2_approx(-fabsf(t.y)));
  const float2 r = make_float2(rcp_approx(1.0f + e.x), rcp_approx(1.0f + e.y));
  e.x = t.x < 0.0f ? e.x : 1.0f;
  e.y = t.y < 0.0f ? e.y : 1.0f;
  return __fmul2_rn(e, r);
}

}  // namespace sigattn
