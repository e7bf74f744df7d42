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
// the compiler may contract or reassociate), so that every kernel variant produces the same
// bits from the same inputs. The transcendental parts use the hardware approximations (ex2, rcp, rsqrt)
// on arguments whose range makes them safe; against a correctly rounded evaluation beta stays
// within 1e-6 relative (the exponential's argument rounding dominates), alpha and omega within
// 1e-6 relative or 2.5e-7 absolute, whichever is larger (see softplus), v_th is exact.
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

// ---------------------------------------------------------------------------------------
// Lane packs. The modulation is issue-bound, so where a thread owns an even number of
// columns the additions, multiplications and fused multiply-adds run two lanes at a time on
// the packed fp32x2 instructions of sm_100 (half the issue slots); the exponentials,
// reciprocals, comparisons and selects stay per lane. Pack<1> is the same arithmetic on
// one lane. For both to give the same bits from the same inputs the formulas obey one
// rule: NO ADDITION TAKES THE RESULT OF A MULTIPLICATION AS AN OPERAND unless it is written
// as a fused multiply-add - the assembler contracts a packed multiply followed by a packed
// add into a packed FMA even when both carry .rn (measured), and never contracts the scalar
// forms, so any other shape would round differently in the two packs.
// ---------------------------------------------------------------------------------------
template <int N>
struct Pack;

template <>
struct Pack<1> {
  float v;
  __device__ __forceinline__ static Pack load(const float* p) { return {p[0]}; }
  __device__ __forceinline__ void store(float* p) const { p[0] = v; }
  __device__ __forceinline__ static Pack splat(float c) { return {c}; }
  __device__ __forceinline__ friend Pack add(Pack a, Pack b) { return {__fadd_rn(a.v, b.v)}; }
  __device__ __forceinline__ friend Pack mul(Pack a, Pack b) { return {__fmul_rn(a.v, b.v)}; }
  __device__ __forceinline__ friend Pack fma(Pack a, Pack b, Pack c) { return {__fmaf_rn(a.v, b.v, c.v)}; }
  template <typename F>
  __device__ __forceinline__ Pack map(F f) const { return {f(v)}; }
  template <typename F>
  __device__ __forceinline__ friend Pack zip(Pack a, Pack b, Pack c, F f) { return {f(a.v, b.v, c.v)}; }
};

template <>
struct Pack<2> {
  unsigned long long v;
  __device__ __forceinline__ static Pack make(float lo, float hi) {
    Pack r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r.v) : "f"(lo), "f"(hi));
    return r;
  }
  __device__ __forceinline__ void get(float& lo, float& hi) const { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
  __device__ __forceinline__ static Pack load(const float* p) { return make(p[0], p[1]); }
  __device__ __forceinline__ void store(float* p) const { get(p[0], p[1]); }
  __device__ __forceinline__ static Pack splat(float c) { return make(c, c); }
  __device__ __forceinline__ friend Pack add(Pack a, Pack b) {
    Pack r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r.v) : "l"(a.v), "l"(b.v));
    return r;
  }
  __device__ __forceinline__ friend Pack mul(Pack a, Pack b) {
    Pack r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r.v) : "l"(a.v), "l"(b.v));
    return r;
  }
  __device__ __forceinline__ friend Pack fma(Pack a, Pack b, Pack c) {
    Pack r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r.v) : "l"(a.v), "l"(b.v), "l"(c.v));
    return r;
  }
  template <typename F>
  __device__ __forceinline__ Pack map(F f) const {
    float lo, hi;
    get(lo, hi);
    return make(f(lo), f(hi));
  }
  template <typename F>
  __device__ __forceinline__ friend Pack zip(Pack a, Pack b, Pack c, F f) {
    float a0, a1, b0, b1, c0, c1;
    a.get(a0, a1);
    b.get(b0, b1);
    c.get(c0, c1);
    return make(f(a0, b0, c0), f(a1, b1, c1));
  }
};

// t = exp(-|z|) in (0, 1]   (the product feeds the exponential only)
template <class P>
__device__ __forceinline__ P exp_neg_abs(P z) {
  return z.map([](float x) { return ex2_approx(__fmul_rn(-fabsf(x), kLog2e)); });
}

// sigmoid(z) = z >= 0 ? 1/(1+t) : t/(1+t), t = exp(-|z|): never overflows.
template <class P>
__device__ __forceinline__ P sigmoid_from_t(P z, P t) {
  const P r = add(P::splat(1.0f), t).map([](float x) { return rcp_approx(x); });
  return zip(z, r, mul(t, r), [](float zz, float rr, float tr) { return zz >= 0.0f ? rr : tr; });
}
template <class P>
__device__ __forceinline__ P sigmoid(P z) {
  return sigmoid_from_t(z, exp_neg_abs(z));
}

// softplus(z) = max(z, 0) + log1p(t), t = exp(-|z|) in (0, 1], with log1p(t) = ln2 * lg2(1 + t) on
// the hardware logarithm: three instructions, absolute error <= 2.5e-7 (lg2.approx is good to
// 2^-22.6 absolute on [1, 2]; forming 1 + t costs another 6e-8). Relative accuracy is therefore lost
// where softplus itself is small (z < -2: 1e-6 at z = -1.7, 1e-5 at z = -4), which is harmless for
// what it feeds - alpha and omega enter the membrane update through products and sums with O(1)
// terms - and it buys 17 % on the resonate-and-fire forward (measured against the 2*atanh(t/(2+t))
// series to s^13, which was relative-accurate to 2e-7 and cost 8 more instructions per softplus).
// Equals z for z > 20 in fp32: the reference's threshold form.
template <class P>
__device__ __forceinline__ P softplus_from_t(P z, P t) {
  const P l = add(P::splat(1.0f), t).map([](float x) {
    float y;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
  });
  return fma(l, P::splat(0.6931471805599453f), z.map([](float x) { return fmaxf(x, 0.0f); }));
}

// Stability rescale of (beta, omega): radius sqrt(beta^2 + omega^2) capped at 0.999.
// r2 = fma(beta, beta, omega*omega). Returns the scale applied (1 when inactive).
template <class P>
__device__ __forceinline__ P rf_rescale(P& beta, P& omega, P& r2) {
  r2 = fma(beta, beta, mul(omega, omega));
  const P scale = r2.map([](float x) { return x > kRmaxSq ? __fmul_rn(kRmax, rsqrt_approx(x)) : 1.0f; });
  beta = mul(beta, scale);
  omega = mul(omega, scale);
  return scale;
}

// What a thread keeps per owned column: the biases of its channel.
template <int V>
struct Bias {
  float beta[V], alpha[V], th[V], omega[V];
};

// Forward modulation of N = 1 or 2 lanes with the intermediates its adjoint needs:
// b0 = unscaled beta, alpha, sa = sigmoid(z_alpha) = d softplus, o0 = unscaled omega,
// so = sigmoid(z_omega). RF selects the second-order form. u = alpha * I is a per-lane
// multiply (it feeds the scan's rounded add, which must never be contracted with it).
template <bool RF, int N>
__device__ __forceinline__ void forward_full(const float* raw_beta, const float* raw_alpha, const float* raw_th,
                                             const float* raw_omega, const float* cur, const float* bb,
                                             const float* ba, const float* bt, const float* bo, float v_th_min,
                                             float* beta, float* u, float* vth, float* omega, float* b0,
                                             float* alpha, float* sa, float* o0, float* so) {
  using P = Pack<N>;
  P be = sigmoid(add(P::load(raw_beta), P::load(bb)));
  be.store(b0);
  const P za = add(P::load(raw_alpha), P::load(ba));
  const P ta = exp_neg_abs(za);
  const P al = softplus_from_t(za, ta);
  al.store(alpha);
  sigmoid_from_t(za, ta).store(sa);
  add(P::splat(v_th_min), add(P::load(raw_th), P::load(bt)).map([](float x) { return fabsf(x); })).store(vth);
  if constexpr (RF) {
    const P zo = add(P::load(raw_omega), P::load(bo));
    const P to = exp_neg_abs(zo);
    P om = softplus_from_t(zo, to);
    om.store(o0);
    sigmoid_from_t(zo, to).store(so);
    P r2;
    rf_rescale(be, om, r2);
    om.store(omega);
  } else {
#pragma unroll
    for (int i = 0; i < N; ++i) omega[i] = o0[i] = so[i] = 0.0f;
  }
  be.store(beta);
#pragma unroll
  for (int i = 0; i < N; ++i) u[i] = __fmul_rn(alpha[i], cur[i]);
}

// The same for the V lanes of a thread (pairs where V is even). Inputs and outputs may alias
// lane by lane (raw_beta with beta, cur with u, raw_th with vth, raw_omega with omega).
template <bool RF, int V>
__device__ __forceinline__ void forward_lanes(float (&b)[V], const float (&ra)[V], float (&th)[V], float (&om)[V],
                                              float (&dr)[V], const Bias<V>& bias, float v_th_min, float (&b0)[V],
                                              float (&al)[V], float (&sa)[V], float (&o0)[V], float (&so)[V]) {
  constexpr int N = V % 2 == 0 ? 2 : 1;
#pragma unroll
  for (int j = 0; j < V; j += N)
    forward_full<RF, N>(&b[j], &ra[j], &th[j], &om[j], &dr[j], &bias.beta[j], &bias.alpha[j], &bias.th[j],
                        &bias.omega[j], v_th_min, &b[j], &dr[j], &th[j], &om[j], &b0[j], &al[j], &sa[j], &o0[j],
                        &so[j]);
}

}  // namespace mod
}  // namespace nsb
