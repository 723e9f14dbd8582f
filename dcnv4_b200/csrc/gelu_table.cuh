// GELU of 16-bit values by table lookup, shared by the kernels that apply the activation to data
// already rounded to fp16 / bf16 (linear.cu, bias_act.cu).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdint>

namespace dcnb200 {

// GELU by table.  The activation is applied to a value already rounded to the 16-bit storage
// type, so there are only 65536 possible inputs; for 2^-12 <= |h| < 8 the result is read from a
// table that every CTA fills in its prologue with the erf formula, which makes it bit-identical
// to evaluating erff per element.  Outside that range (about one pre-activation in a thousand
// even for a freshly initialised network) a warp-uniform branch evaluates the rest: below
// 2^-12 the Maclaurin series of the normal CDF is exact to fp32 rounding, and from 8 upward
// GELU(h) is h (or -0 for negative h) in 16-bit precision.
// Layout: entry [d + sign * kSpan], d = (bits & 0x7fff) - kLo.
template <typename T> struct GeluLut;
template <> struct GeluLut<__half> {
  static constexpr uint32_t kLo = 0x0C00, kSpan = 0x3C00;  // 2^-12 .. 8, 10-bit mantissa (60 KB)
};
template <> struct GeluLut<__nv_bfloat16> {
  static constexpr uint32_t kLo = 0x3980, kSpan = 0x0780;  // 2^-12 .. 8, 7-bit mantissa
};
template <typename T>
constexpr int gelu_lut_bytes() { return (int)(2 * GeluLut<T>::kSpan * 2 + 1023) / 1024 * 1024; }

// Two fp32 values rounded (nearest even) into one packed 16-bit pair, and back.
template <typename T> __device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  const __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}
template <typename T> __device__ __forceinline__ float2 unpack2(uint32_t u);
template <> __device__ __forceinline__ float2 unpack2<__half>(uint32_t u) {
  return __half22float2(*reinterpret_cast<const __half2*>(&u));
}
template <> __device__ __forceinline__ float2 unpack2<__nv_bfloat16>(uint32_t u) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u));
}

// GELU outside the table's range, for one 16-bit value with bits `hb` and value `hf`.
template <typename T>
__device__ __forceinline__ uint32_t gelu_outside_table(uint32_t hb, float hf) {
  // small |h|: h * Phi(h), Phi(h) = 1/2 + h/sqrt(2 pi) - h^3/(6 sqrt(2 pi)) + O(h^5)
  const float small_v = hf * fmaf(hf, fmaf(hf * hf, -0.066490380f, 0.39894228f), 0.5f);
  // |h| >= 8: h for h > 0, -0 for h < 0; NaN and -inf come out as NaN like the erf formula
  const float big_v = hf * (hf > 0.f ? 1.f : 0.f);
  return pack2<T>((hb & 0x7FFFu) < GeluLut<T>::kLo ? small_v : big_v, 0.f) & 0xFFFFu;
}
// GELU of eight 16-bit values packed in four registers, in place; see GeluLut.  Must be called
// by the whole warp: all table reads are issued first, then ONE vote decides whether any lane
// holds a value outside the table, so the common path has no branch between the lookups.
template <typename T>
__device__ __forceinline__ void gelu_lut8(uint32_t (&h)[4], const uint16_t* lut) {
  constexpr uint32_t kLo = GeluLut<T>::kLo, kSpan = GeluLut<T>::kSpan;
  uint32_t t[8];
  bool any_out = false;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t x0 = h[i] & 0xFFFFu, x1 = h[i] >> 16;
    const uint32_t d0 = (x0 & 0x7FFFu) - kLo, d1 = (x1 & 0x7FFFu) - kLo;
    t[2 * i] = lut[min(d0, kSpan - 1) + (x0 >> 15) * kSpan];
    t[2 * i + 1] = lut[min(d1, kSpan - 1) + (x1 >> 15) * kSpan];
    any_out |= (d0 >= kSpan) | (d1 >= kSpan);
  }
  if (__any_sync(0xffffffffu, any_out)) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t x0 = h[i] & 0xFFFFu, x1 = h[i] >> 16;
      const float2 f = unpack2<T>(h[i]);
      if ((x0 & 0x7FFFu) - kLo >= kSpan) t[2 * i] = gelu_outside_table<T>(x0, f.x);
      if ((x1 & 0x7FFFu) - kLo >= kSpan) t[2 * i + 1] = gelu_outside_table<T>(x1, f.y);
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = t[2 * i] | (t[2 * i + 1] << 16);
}

// Fill the table cooperatively: thread `tid` of `n_threads`.  The caller synchronises afterwards.
// One erff serves both signs: erff is odd, so 1 + erff(-z) == 1 - erff(z) exactly.
template <typename T>
__device__ __forceinline__ void gelu_lut_fill(uint16_t* lut, uint32_t tid, uint32_t n_threads) {
  for (uint32_t d = tid; d < GeluLut<T>::kSpan; d += n_threads) {
    const float x = unpack2<T>(GeluLut<T>::kLo + d).x;
    const float e = erff(x * 0.70710678118654752440f);
    lut[d] = (uint16_t)(pack2<T>(0.5f * x * (1.0f + e), 0.f) & 0xFFFFu);
    lut[d + GeluLut<T>::kSpan] = (uint16_t)(pack2<T>(0.5f * -x * (1.0f - e), 0.f) & 0xFFFFu);
  }
}

}  // namespace dcnb200
