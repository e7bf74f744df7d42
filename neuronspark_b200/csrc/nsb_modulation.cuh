// Modulation of the selective scans: raw projections + per-channel biases -> beta, alpha,
// v_th (, omega), as NeuronSpark's SNNBlock computes them between its input projections and
// its scan (atomic_ops/snn_block.py:52-76; first-order form
// archive/atomic_ops_v75_pre/snn_block.py:41-47):
//
//   beta  = sigmoid(raw_beta + b_beta)          alpha = softplus(raw_alpha + b_alpha)
//   v_th  = v_th_min + |raw_th + b_th|          omega = softplus(raw_omega + b_omega)
//   r2 = beta^2 + omega^2;  if r2 > 0.999^2: (beta, omega) *= 0.999 * rsqrt(r2)
//   u = alpha * I
//
// These device functions are shared by the fused scan kernels and by the stand-alone
// modulation kernel, and are written with explicit rounded operations only (no expression
// the compiler may contract or reassociate), so that both produce the same bits from the
// same inputs. The transcendental parts use the hardware approximations (ex2, rcp, rsqrt)
// on arguments whose range makes them safe; relative error of beta, alpha, omega against a
// correctly rounded evaluation stays below 1e-6 (the exponential's argument rounding
// dominates), v_th is exact.
#pragma once

#include <cuda_runtime.h>

namespace nsb {
namespace mod {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRmax = 0.999f;
constexpr float kRmaxSq = (float)(0.999 * 0.999);

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float rcp_approx(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float rsqrt_approx(float x) {
  float y;
  asm("rsqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// t = exp(-|z|) in (0, 1]
__device__ __forceinline__ float exp_neg_abs(float z) { return ex2_approx(__fmul_rn(-fabsf(z), kLog2e)); }

// sigmoid(z) = z >= 0 ? 1/(1+t) : t/(1+t), t = exp(-|z|): never overflows.
__device__ __forceinline__ float sigmoid_from_t(float z, float t) {
  const float r = rcp_approx(__fadd_rn(1.0f, t));
  return z >= 0.0f ? r : __fmul_rn(t, r);
}
__device__ __forceinline__ float sigmoid(float z) { return sigmoid_from_t(z, exp_neg_abs(z)); }

// log1p(t) for t in [0, 1]: 2*atanh(s) with s = t/(2+t) <= 1/3, odd series to s^13
// (truncation 1.4e-8 relative).
__device__ __forceinline__ float log1p_unit(float t) {
  const float s = __fmul_rn(t, rcp_approx(__fadd_rn(2.0f, t)));
  const float s2 = __fmul_rn(s, s);
  float p = 2.0f / 13.0f;
  p = __fmaf_rn(p, s2, 2.0f / 11.0f);
  p = __fmaf_rn(p, s2, 2.0f / 9.0f);
  p = __fmaf_rn(p, s2, 2.0f / 7.0f);
  p = __fmaf_rn(p, s2, 2.0f / 5.0f);
  p = __fmaf_rn(p, s2, 2.0f / 3.0f);
  p = __fmaf_rn(p, s2, 2.0f);
  return __fmul_rn(s, p);
}

// softplus(z) = max(z, 0) + log1p(exp(-|z|)); equals z for z > 20 in fp32, which is the
// reference's threshold form. `t` is exp(-|z|), for the caller that also wants sigmoid(z).
__device__ __forceinline__ float softplus_from_t(float z, float t) {
  return __fadd_rn(fmaxf(z, 0.0f), log1p_unit(t));
}
__device__ __forceinline__ float softplus(float z) { return softplus_from_t(z, exp_neg_abs(z)); }

// Stability rescale of (beta, omega): radius sqrt(beta^2 + omega^2) capped at 0.999.
// Returns the scale applied (1 when inactive) and r2 of the unscaled pair.
__device__ __forceinline__ float rf_rescale(float& beta, float& omega, float& r2) {
  r2 = __fadd_rn(__fmul_rn(beta, beta), __fmul_rn(omega, omega));
  float scale = 1.0f;
  if (r2 > kRmaxSq) scale = __fmul_rn(kRmax, rsqrt_approx(r2));
  beta = __fmul_rn(beta, scale);
  omega = __fmul_rn(omega, scale);
  return scale;
}

// What a thread keeps per owned column: the biases of its channel.
template <int V>
struct Bias {
  float beta[V], alpha[V], th[V], omega[V];
};

// Forward modulation of one element. RF selects the second-order form.
template <bool RF>
__device__ __forceinline__ void forward(float raw_beta, float raw_alpha, float raw_th, float raw_omega, float cur,
                                        float bb, float ba, float bt, float bo, float v_th_min, float& beta,
                                        float& u, float& vth, float& omega) {
  beta = sigmoid(__fadd_rn(raw_beta, bb));
  const float alpha = softplus(__fadd_rn(raw_alpha, ba));
  vth = __fadd_rn(v_th_min, fabsf(__fadd_rn(raw_th, bt)));
  if constexpr (RF) {
    omega = softplus(__fadd_rn(raw_omega, bo));
    float r2;
    rf_rescale(beta, omega, r2);
  } else {
    omega = 0.0f;
  }
  u = __fmul_rn(alpha, cur);
}

}  // namespace mod
}  // namespace nsb
