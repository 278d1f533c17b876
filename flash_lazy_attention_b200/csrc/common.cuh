// Shared definitions of libflashlazy: parameter blocks, dtype helpers, the scalar
// alpha-entmax arithmetic used by every kernel family.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/fla.h"

namespace fla {

enum Mode : int { ENTMAX = 0, LAZY = 1 };

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

struct View4 {
  void* ptr;
  int64_t s[4];
};

// One parameter block for every attention kernel (SIMT and tensor-core families).
struct AttnParams {
  int B, H, L, D;
  int Hkv, n_rep;   // grouped-query attention: k, v (and dk, dv) have Hkv = H / n_rep heads; query head h reads head h / n_rep
  int causal;
  const int* varlen;
  float scale;  // 1/sqrt(D)
  View4 q, k, v, o, dout, dq, dk, dv;
  // entmax
  float alpha;
  int niter;
  float* tau;        // [B,H,L] thresholds (entmax) -- (alpha-1)*score units
  float* aux_o;      // entmax [B,H,L,D]: U.V;  lazy [B,H,L,2D]: fp32 O | sum of V over the ReLU support
  float* aux_s;      // [B,H,L]
  uint32_t* block_mask;
  int mask_words;
  // lazy
  const float* bias;
  int64_t bias_stride;
  const float* tau_h;  // [H]
  int window;
  float* lse;  // [B,H,L] base-2 log-sum-exp of the scores (log2(e) times the natural one)
  float* dbias;
  int64_t dbias_stride;
  float* dtau;
  // dbias and dtau are summed over the whole batch by many CTAs.  The kernels add into 64-bit fixed-point
  // accumulators (integer addition is associative: the sums do not depend on the order in which the CTAs arrive),
  // and a last small kernel converts them into the fp32 outputs above.  NULL: not wanted.
  unsigned long long* dbias_acc;   // [H, dbias_acc_stride], distances < L
  int64_t dbias_acc_stride;
  unsigned long long* dtau_acc;    // [H]
  // backward scratch
  float* delta;  // [B,H,L]
  int flags;        // FLA_FLAG_* of fla_attn_geom
};


template <typename T>
__device__ __forceinline__ float to_f32(T x);
template <>
__device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ float to_f32<__half>(__half x) { return __half2float(x); }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T>
__device__ __forceinline__ T from_f32(float x);
template <>
__device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

// Round an fp32 value to the precision of T (what "P.to(v.dtype)" does before the PV product).
template <typename T>
__device__ __forceinline__ float round_to(float x) { return to_f32<T>(from_f32<T>(x)); }

// Fixed-point form of a dbias / dtau contribution: 32 fractional bits (resolution 2.3e-10; the 64-bit range holds
// sums up to 2e9 in magnitude).
constexpr float kFixedScale = 4294967296.f;
__device__ __forceinline__ unsigned long long to_fixed(float v) {
  return (unsigned long long)__float2ll_rn(v * kFixedScale);
}

// ---- alpha-entmax scalar arithmetic -------------------------------------------------------
// With e = 1/(alpha-1) and d = X - tau > 0:   p = d^e,  p' = d^(e-1),  p'' = d^(e-2).
// Kind 0: alpha = 1.5 (e = 2), kind 1: alpha = 2 (e = 1), kind 2: any alpha in (1,2].
__host__ __device__ inline int alpha_kind(float alpha) {
  return alpha == 1.5f ? 0 : (alpha == 2.0f ? 1 : 2);
}

template <int KIND, bool FAST = true>
__device__ __forceinline__ float pow_e(float d, float e) {
  if (KIND == 0) return d * d;
  if (KIND == 1) return d;
  return FAST ? exp2f(e * __log2f(d)) : powf(d, e);
}

// p = d^e and u = p^(2-alpha) = d^(e-1) for d > 0.
template <int KIND>
__device__ __forceinline__ void p_and_u(float d, float e, float& p, float& u) {
  if (KIND == 0) { p = d * d; u = d; }
  else if (KIND == 1) { p = d; u = 1.f; }
  else { float l = __log2f(d); p = exp2f(e * l); u = exp2f((e - 1.f) * l); }
}

// Safeguarded update of the threshold from the sums over the support at the current tau:
//   s0 = sum d^e, s1 = sum d^(e-1), s2 = sum d^(e-2)   (s2 only used when e >= 2)
// f = s0 - 1, f' = -e s1, f'' = e(e-1) s2.  Halley when e >= 2 (f'' bounded), Newton
// otherwise; [lo, hi] is the running bracket; a step leaving it is replaced by its midpoint.
// Starting from the left end of the bracket both iterations increase monotonically to the
// root because f is convex and decreasing.  Returns the new tau and updates the bracket.
__device__ __forceinline__ float tau_update(float tau, float s0, float s1, float s2, float e,
                                            float& lo, float& hi, bool* regular = nullptr) {
  float f = s0 - 1.f;
  if (f >= 0.f) lo = tau; else hi = tau;
  float f1 = -e * s1;
  float step;
  if (e >= 2.f) {
    float f2 = e * (e - 1.f) * s2;
    float den = 2.f * f1 * f1 - f * f2;
    step = 2.f * f * f1 / den;
  } else {
    step = f / f1;
  }
  float t = tau - step;
  const bool inside = t >= lo && t <= hi;
  if (!inside) t = 0.5f * (lo + hi);
  if (regular) *regular = inside;   // false: the step was replaced by a bisection
  return t;
}

// alpha = 1.5 only: a longer first step for the threshold iteration.  At tau0 = max - 1 the excesses
// d = X - tau0 > 0 of a row have count c, sum s1 and sum of squares s0.  Modelling them as a
// generalised Pareto tail with those two moments (shape xi, scale sigma: mean sigma/(1-xi), second
// moment 2 sigma^2/((1-xi)(1-2 xi))) gives, for a threshold raised by t, the model value of
// sum (d - t)_+^2 in closed form; its root in t replaces the Halley step, which falls short by
// 0.1-0.3 on rows with hundreds of excesses where the model lands within a few 1e-2.  Returns the
// step, or a negative number when the moments do not admit the model (few excesses, all equal, too
// heavy a tail): the caller then keeps the Halley step.  The result is only a starting point: the
// iteration that follows is the safeguarded one, and converges from either side.
__device__ __forceinline__ float gpd_first_step(float s0, float s1, float c) {
  if (!(c >= 8.f) || !(s1 > 0.f) || !(s0 > 1.f)) return -1.f;
  const float m1 = s1 / c, m2 = s0 / c;
  const float R = m2 / (m1 * m1);
  if (!(R > 1.05f) || !(R < 12.f)) return -1.f;
  float xi = (R - 2.f) / (2.f * R - 2.f);
  if (fabsf(xi) < 1e-3f) xi = xi < 0.f ? -1e-3f : 1e-3f;
  const float sigma = m1 * (1.f - xi);
  const float k2 = 2.f * c / ((1.f - xi) * (1.f - 2.f * xi));
  const float k1 = 2.f * c / (1.f - xi);
  const float inv_xi = 1.f / xi, inv_sigma = 1.f / sigma;
  float t = 0.f;
#pragma unroll 1
  for (int it = 0; it < 12; ++it) {   // Newton on a convex decreasing function from its left
    const float sg = sigma + xi * t;
    const float z = sg * inv_sigma;
    if (!(z > 1e-6f)) break;
    // approximate log / exp / divide: the result is only a starting point
    const float surv = exp2f(-__log2f(z) * inv_xi);
    const float g = k2 * surv * sg * sg - 1.f;
    const float gp = -k1 * surv * sg;
    const float tn = t - __fdividef(g, gp);
    if (!(tn >= t)) break;
    const bool small = tn - t <= 1e-4f;
    t = tn;
    if (small) break;
  }
  return (t > 0.f && t < 1.f) ? t : -1.f;
}

}  // namespace fla
