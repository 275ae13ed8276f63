// Sigmoid arithmetic shared by the forward and backward kernels.
#pragma once

#include "ptx.cuh"

namespace sigattn {

constexpr float kLog2e = 1.4426950408889634f;

// sigmoid(x) with x given in the base-2 domain (t = x * log2(e)).
// e = 2^-|t| in (0,1] (one MUFU op); sigmoid = (t < 0 ? e : 1) / (1 + e).  This keeps RELATIVE
// accuracy for strongly negative logits (the default bias is -log(T), so a typical probability
// is ~1/T), which 0.5 + 0.5 tanh(x/2) does not.  1/(1+e) on [0,1] is a minimax polynomial on
// the FMA pipe instead of a second MUFU op: the MUFU unit (16 results / clock / SM) is what
// bounds this kernel.  Maximum relative error of the polynomial: 5.1e-5 (degree 5, used for
// fp16, whose own rounding is 4.9e-4) and 3.0e-4 (degree 4, used for bf16, rounding 3.9e-3).
#ifndef SIG_POLY_MODE
#define SIG_POLY_MODE 0
#endif

// coefficients, highest degree first; {c, c} pairs for the packed f32x2 form
__constant__ float2 kPolyF16[6] = {{-0.1044827550649643f, -0.1044827550649643f}, {0.41793352365493774f, 0.41793352365493774f},
                                   {-0.7705690264701843f, -0.7705690264701843f}, {0.9534193277359009f, 0.9534193277359009f},
                                   {-0.9962754845619202f, -0.9962754845619202f}, {0.9999489784240723f, 0.9999489784240723f}};
__constant__ float2 kPolyBF16[5] = {{0.1522425264120102f, 0.1522425264120102f}, {-0.5328524708747864f, -0.5328524708747864f},
                                    {0.8658902645111084f, 0.8658902645111084f}, {-0.9848342537879944f, -0.9848342537879944f},
                                    {0.9997026324272156f, 0.9997026324272156f}};

template <bool kBF16>
__device__ __forceinline__ float2 rcp1p_poly(float2 e) {
  float2 r;
#if SIG_POLY_MODE == 2
  if constexpr (kBF16) {
    r = kPolyBF16[0];
#pragma unroll
    for (int i = 1; i < 5; ++i) r = __ffma2_rn(r, e, kPolyBF16[i]);
  } else {
    r = kPolyF16[0];
#pragma unroll
    for (int i = 1; i < 6; ++i) r = __ffma2_rn(r, e, kPolyF16[i]);
  }
#elif SIG_POLY_MODE == 1
  if constexpr (kBF16) {
    r = make_float2(0.1522425264120102f, 0.1522425264120102f);
    r.x = fmaf(r.x, e.x, -0.5328524708747864f); r.y = fmaf(r.y, e.y, -0.5328524708747864f);
    r.x = fmaf(r.x, e.x, 0.8658902645111084f);  r.y = fmaf(r.y, e.y, 0.8658902645111084f);
    r.x = fmaf(r.x, e.x, -0.9848342537879944f); r.y = fmaf(r.y, e.y, -0.9848342537879944f);
    r.x = fmaf(r.x, e.x, 0.9997026324272156f);  r.y = fmaf(r.y, e.y, 0.9997026324272156f);
  } else {
    r = make_float2(-0.1044827550649643f, -0.1044827550649643f);
    r.x = fmaf(r.x, e.x, 0.41793352365493774f); r.y = fmaf(r.y, e.y, 0.41793352365493774f);
    r.x = fmaf(r.x, e.x, -0.7705690264701843f); r.y = fmaf(r.y, e.y, -0.7705690264701843f);
    r.x = fmaf(r.x, e.x, 0.9534193277359009f);  r.y = fmaf(r.y, e.y, 0.9534193277359009f);
    r.x = fmaf(r.x, e.x, -0.9962754845619202f); r.y = fmaf(r.y, e.y, -0.9962754845619202f);
    r.x = fmaf(r.x, e.x, 0.9999489784240723f);  r.y = fmaf(r.y, e.y, 0.9999489784240723f);
  }
#else
  if constexpr (kBF16) {
    r = make_float2(0.1522425264120102f, 0.1522425264120102f);
    r = __ffma2_rn(r, e, make_float2(-0.5328524708747864f, -0.5328524708747864f));
    r = __ffma2_rn(r, e, make_float2(0.8658902645111084f, 0.8658902645111084f));
    r = __ffma2_rn(r, e, make_float2(-0.9848342537879944f, -0.9848342537879944f));
    r = __ffma2_rn(r, e, make_float2(0.9997026324272156f, 0.9997026324272156f));
  } else {
    r = make_float2(-0.1044827550649643f, -0.1044827550649643f);
    r = __ffma2_rn(r, e, make_float2(0.41793352365493774f, 0.41793352365493774f));
    r = __ffma2_rn(r, e, make_float2(-0.7705690264701843f, -0.7705690264701843f));
    r = __ffma2_rn(r, e, make_float2(0.9534193277359009f, 0.9534193277359009f));
    r = __ffma2_rn(r, e, make_float2(-0.9962754845619202f, -0.9962754845619202f));
    r = __ffma2_rn(r, e, make_float2(0.9999489784240723f, 0.9999489784240723f));
  }
#endif
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

}  // namespace sigattn
