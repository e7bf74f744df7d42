/*
 * CPU oracle for the PLIF scan family, the FP16 boundary codec and the
 * divisive-normalisation lateral inhibition.
 *
 * TEST INFRASTRUCTURE ONLY. This file restates, in plain C, the sequential
 * semantics of NeuronSpark's operators so that the CUDA kernels can be checked
 * against it. Nothing in the shipped package may call into it; only the test
 * suite, the smoke check and the benchmark's CPU-baseline leg do.
 *
 * Parity status: PINNED for the forward scans, the sigmoid-surrogate backward,
 * the codec and the normaliser (checked in the test suite against vectors
 * produced by running the reference's own Python on CPU). The arctangent
 * surrogate has no counterpart in the reference's fused kernels; it is pinned
 * to its published definition instead: g'(x) = (a/2) / (1 + (pi/2 * a * x)^2)
 * written here by hand must equal, to 1e-5, what torch autograd derives from
 * the primitive g(x) = atan(pi/2 * a * x) / pi + 1/2 through the reference
 * test's time loop (fixture scan_ai_bwd_atan of tests/golden/make_golden.py).
 *
 * Arithmetic contract: every state update is one rounded fp32 multiply
 * followed by one rounded fp32 add (no fused multiply-add), which is what the
 * reference's eager PyTorch time loop does. Build with -ffp-contract=off.
 *
 * Layout: time-major [T, cols] with cols = batch * channels, identical to the
 * reference's (K, *shape) tensors (atomic_ops/parallel_scan.py:713-714).
 */
#include <math.h>
#include <stdint.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_SURR_SIGMOID 0
#define ORC_SURR_ATAN 1

int orc_version(void) { return 1; }

int orc_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

void orc_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

/* Columns are independent; they are cut into blocks so that the inner loop
 * runs over contiguous lanes (vectorisable) while time advances outside. */
#define COL_BLOCK 256

/* ------------------------------------------------------------------ */
/* Selective scan, u-form.                                             */
/* Follows atomic_ops/parallel_scan.py:209-213 (kernel docstring) and  */
/* the executable CPU loop at :1667-1677 with omega = 0:               */
/*   v_pre = beta[k]*v + u[k]; s = (v_pre >= v_th[k]);                 */
/*   v = v_pre - v_th[k]*s                                             */
/* spike / vpost / vlast may each be NULL.                             */
/* ------------------------------------------------------------------ */
void orc_plif_selective_fwd(const float *beta, const float *u, const float *vth,
                            const float *v_init, float *spike, float *vpost,
                            float *vlast, int64_t T, int64_t cols) {
#pragma omp parallel for schedule(static)
  for (int64_t c0 = 0; c0 < cols; c0 += COL_BLOCK) {
    int64_t n = cols - c0 < COL_BLOCK ? cols - c0 : COL_BLOCK;
    float v[COL_BLOCK];
    for (int64_t j = 0; j < n; ++j) v[j] = v_init[c0 + j];
    for (int64_t k = 0; k < T; ++k) {
      const int64_t off = k * cols + c0;
      for (int64_t j = 0; j < n; ++j) {
        float bv = beta[off + j] * v[j];
        float vpre = bv + u[off + j];
        float s = vpre >= vth[off + j] ? 1.0f : 0.0f;
        float vs = vth[off + j] * s;
        v[j] = vpre - vs;
        if (spike) spike[off + j] = s;
        if (vpost) vpost[off + j] = v[j];
      }
    }
    if (vlast)
      for (int64_t j = 0; j < n; ++j) vlast[c0 + j] = v[j];
  }
}

/* ------------------------------------------------------------------ */
/* Selective scan, alpha*I form: the write gain and the current are    */
/* separate inputs, as in SelectivePLIFNode.single_step_forward        */
/* (atomic_ops/selective_plif.py:127,130,137):                         */
/*   v_pre = beta*v + alpha*x  (three roundings)                       */
/* ------------------------------------------------------------------ */
void orc_plif_selective_ai_fwd(const float *beta, const float *cur,
                               const float *gain, const float *vth,
                               const float *v_init, float *spike, float *vpost,
                               float *vlast, int64_t T, int64_t cols) {
#pragma omp parallel for schedule(static)
  for (int64_t c0 = 0; c0 < cols; c0 += COL_BLOCK) {
    int64_t n = cols - c0 < COL_BLOCK ? cols - c0 : COL_BLOCK;
    float v[COL_BLOCK];
    for (int64_t j = 0; j < n; ++j) v[j] = v_init[c0 + j];
    for (int64_t k = 0; k < T; ++k) {
      const int64_t off = k * cols + c0;
      for (int64_t j = 0; j < n; ++j) {
        float bv = beta[off + j] * v[j];
        float ai = gain[off + j] * cur[off + j];
        float vpre = bv + ai;
        float s = vpre >= vth[off + j] ? 1.0f : 0.0f;
        float vs = vth[off + j] * s;
        v[j] = vpre - vs;
        if (spike) spike[off + j] = s;
        if (vpost) vpost[off + j] = v[j];
      }
    }
    if (vlast)
      for (int64_t j = 0; j < n; ++j) vlast[c0 + j] = v[j];
  }
}

/* ------------------------------------------------------------------ */
/* Row-parameter scan: beta and v_th constant over time, one value per */
/* column. Follows atomic_ops/parallel_scan.py:330-343 (materialising) */
/* and :508-523 (spike + V_last only).                                 */
/* ------------------------------------------------------------------ */
void orc_plif_rowparam_fwd(const float *beta_row, const float *u,
                           const float *vth_row, const float *v_init,
                           float *spike, float *vpost, float *vlast, int64_t T,
                           int64_t cols) {
#pragma omp parallel for schedule(static)
  for (int64_t c0 = 0; c0 < cols; c0 += COL_BLOCK) {
    int64_t n = cols - c0 < COL_BLOCK ? cols - c0 : COL_BLOCK;
    float v[COL_BLOCK];
    for (int64_t j = 0; j < n; ++j) v[j] = v_init[c0 + j];
    for (int64_t k = 0; k < T; ++k) {
      const int64_t off = k * cols + c0;
      for (int64_t j = 0; j < n; ++j) {
        float bv = beta_row[c0 + j] * v[j];
        float vpre = bv + u[off + j];
        float s = vpre >= vth_row[c0 + j] ? 1.0f : 0.0f;
        float vs = vth_row[c0 + j] * s;
        v[j] = vpre - vs;
        if (spike) spike[off + j] = s;
        if (vpost) vpost[off + j] = v[j];
      }
    }
    if (vlast)
      for (int64_t j = 0; j < n; ++j) vlast[c0 + j] = v[j];
  }
}

/* Surrogate derivative, evaluated in double so that the oracle is the
 * "true" value the fp32 kernels are compared against.
 * Sigmoid: atomic_ops/parallel_scan.py:291-296 (argument of exp clamped at
 * 88). Arctangent: derivative of atan(pi/2*a*x)/pi + 1/2 (checked against
 * autograd through that primitive by the golden fixture scan_ai_bwd_atan). */
static inline double surr_grad(double x, double a, int kind) {
  if (kind == ORC_SURR_ATAN) {
    double z = 1.5707963267948966 * a * x;
    return 0.5 * a / (1.0 + z * z);
  }
  double nax = -a * x;
  if (nax > 88.0) nax = 88.0;
  double sig = 1.0 / (1.0 + exp(nax));
  return a * sig * (1.0 - sig);
}

/* ------------------------------------------------------------------ */
/* Reverse-time surrogate-gradient pass of the selective scan.         */
/* Transcribes the recurrence of atomic_ops/parallel_scan.py:246-256   */
/* with x = V_post - v_th*(1 - s) = V_pre - v_th (:292). The spike in  */
/* the reset path is a constant (detached), which is the semantics of  */
/* the autograd loop at exp/verify_fused_plif.py:111-124.              */
/*                                                                     */
/* The forward states are recomputed here in fp32 exactly as the       */
/* forward does; the adjoint arithmetic runs in double. u-form: u set,  */
/* cur/gain NULL, g_u receives the gradient. alpha*I form: u NULL,     */
/* cur/gain set, g_cur = gpre*gain and g_gain = gpre*cur.              */
/* ------------------------------------------------------------------ */
static void selective_bwd_core(const float *beta, const float *u,
                               const float *cur, const float *gain,
                               const float *vth, const float *v_init,
                               const float *g_spike, const float *g_vpost,
                               float *g_beta, float *g_u, float *g_cur,
                               float *g_gain, float *g_vth, float *g_vinit,
                               int64_t T, int64_t cols, double a, int kind) {
  /* Columns are processed in blocks of BWD_BLOCK so that the inner loops run
   * over contiguous lanes; V_prev[k] and x[k] of a block are kept for the
   * reverse pass. */
#define BWD_BLOCK 32
#pragma omp parallel
  {
    float *vp = (float *)__builtin_malloc(sizeof(float) * (size_t)(T > 0 ? T : 1) * BWD_BLOCK * 2);
    float *xs = vp + (size_t)(T > 0 ? T : 1) * BWD_BLOCK;
#pragma omp for schedule(dynamic, 4)
    for (int64_t c0 = 0; c0 < cols; c0 += BWD_BLOCK) {
      const int64_t n = cols - c0 < BWD_BLOCK ? cols - c0 : BWD_BLOCK;
      float v[BWD_BLOCK];
      double acc[BWD_BLOCK];
      for (int64_t j = 0; j < n; ++j) v[j] = v_init[c0 + j];
      for (int64_t k = 0; k < T; ++k) {
        const int64_t o = k * cols + c0;
        for (int64_t j = 0; j < n; ++j) {
          float uu = u ? u[o + j] : gain[o + j] * cur[o + j];
          float bv = beta[o + j] * v[j];
          float vpre = bv + uu;
          vp[k * BWD_BLOCK + j] = v[j];
          xs[k * BWD_BLOCK + j] = vpre - vth[o + j];
          float s = vpre >= vth[o + j] ? 1.0f : 0.0f;
          float vs = vth[o + j] * s;
          v[j] = vpre - vs;
        }
      }
      for (int64_t j = 0; j < n; ++j) acc[j] = 0.0;
      for (int64_t k = T - 1; k >= 0; --k) {
        const int64_t o = k * cols + c0;
        for (int64_t j = 0; j < n; ++j) {
          const double x = (double)xs[k * BWD_BLOCK + j];
          const double s = x >= 0.0 ? 1.0 : 0.0;
          const double sg = surr_grad(x, a, kind);
          const double gs = g_spike ? (double)g_spike[o + j] : 0.0;
          const double tot = (g_vpost ? (double)g_vpost[o + j] : 0.0) + acc[j];
          const double gpre = gs * sg + tot;
          if (g_beta) g_beta[o + j] = (float)(gpre * (double)vp[k * BWD_BLOCK + j]);
          if (u) {
            if (g_u) g_u[o + j] = (float)gpre;
          } else {
            if (g_cur) g_cur[o + j] = (float)(gpre * (double)gain[o + j]);
            if (g_gain) g_gain[o + j] = (float)(gpre * (double)cur[o + j]);
          }
          if (g_vth) g_vth[o + j] = (float)(-gs * sg - tot * s);
          acc[j] = gpre * (double)beta[o + j];
        }
      }
      if (g_vinit)
        for (int64_t j = 0; j < n; ++j) g_vinit[c0 + j] = (float)acc[j];
    }
    __builtin_free(vp);
  }
#undef BWD_BLOCK
}

void orc_plif_selective_bwd(const float *beta, const float *u, const float *vth,
                            const float *v_init, const float *g_spike,
                            const float *g_vpost, float *g_beta, float *g_u,
                            float *g_vth, float *g_vinit, int64_t T,
                            int64_t cols, double alpha, int kind) {
  selective_bwd_core(beta, u, 0, 0, vth, v_init, g_spike, g_vpost, g_beta, g_u,
                     0, 0, g_vth, g_vinit, T, cols, alpha, kind);
}

void orc_plif_selective_ai_bwd(const float *beta, const float *cur,
                               const float *gain, const float *vth,
                               const float *v_init, const float *g_spike,
                               const float *g_vpost, float *g_beta,
                               float *g_cur, float *g_gain, float *g_vth,
                               float *g_vinit, int64_t T, int64_t cols,
                               double alpha, int kind) {
  selective_bwd_core(beta, 0, cur, gain, vth, v_init, g_spike, g_vpost, g_beta,
                     0, g_cur, g_gain, g_vth, g_vinit, T, cols, alpha, kind);
}

/* ------------------------------------------------------------------ */
/* Reverse pass of the row-parameter scan: grad_u per step, grad_beta  */
/* and grad_v_th reduced over time per column                          */
/* (atomic_ops/parallel_scan.py:393-413; with g_vpost == NULL this is  */
/* the recompute variant :592-612 whose V_post gradient is zero).      */
/* ------------------------------------------------------------------ */
void orc_plif_rowparam_bwd(const float *beta_row, const float *u,
                           const float *vth_row, const float *v_init,
                           const float *g_spike, const float *g_vpost,
                           float *g_beta_row, float *g_u, float *g_vth_row,
                           float *g_vinit, int64_t T, int64_t cols,
                           double alpha, int kind) {
#pragma omp parallel for schedule(dynamic, 16)
  for (int64_t c = 0; c < cols; ++c) {
    float *vp = (float *)__builtin_malloc(sizeof(float) * (size_t)T * 2);
    float *xs = vp + T;
    const float b = beta_row[c], th = vth_row[c];
    float v = v_init[c];
    for (int64_t k = 0; k < T; ++k) {
      float bv = b * v;
      float vpre = bv + u[k * cols + c];
      vp[k] = v;
      xs[k] = vpre - th;
      float s = vpre >= th ? 1.0f : 0.0f;
      float vs = th * s;
      v = vpre - vs;
    }
    double acc = 0.0, gb = 0.0, gt = 0.0;
    for (int64_t k = T - 1; k >= 0; --k) {
      const int64_t o = k * cols + c;
      double s = xs[k] >= 0.0f ? 1.0 : 0.0;
      double sg = surr_grad((double)xs[k], alpha, kind);
      double gs = g_spike ? (double)g_spike[o] : 0.0;
      double tot = (g_vpost ? (double)g_vpost[o] : 0.0) + acc;
      double gpre = gs * sg + tot;
      if (g_u) g_u[o] = (float)gpre;
      gb += gpre * (double)vp[k];
      gt += -gs * sg - tot * s;
      acc = gpre * (double)b;
    }
    if (g_vinit) g_vinit[c] = (float)acc;
    if (g_beta_row) g_beta_row[c] = (float)gb;
    if (g_vth_row) g_vth_row[c] = (float)gt;
    __builtin_free(vp);
  }
}

/* ------------------------------------------------------------------ */
/* Resonate-and-fire (second-order) scan.                              */
/* Forward: the reference's executable CPU loop,                       */
/* atomic_ops/parallel_scan.py:1667-1677:                              */
/*   v_pre = beta*v - omega*w + u     ((beta*v) - (omega*w)) + u       */
/*   w_new = omega*v + beta*w         only V is reset, W is not        */
/* vpost / wout / spike may be NULL.                                   */
/* ------------------------------------------------------------------ */
void orc_plif_rf_fwd(const float *beta, const float *omega, const float *u,
                     const float *vth, const float *v_init, const float *w_init,
                     float *spike, float *vpost, float *wout, float *vlast,
                     float *wlast, int64_t T, int64_t cols) {
#pragma omp parallel for schedule(static)
  for (int64_t c0 = 0; c0 < cols; c0 += COL_BLOCK) {
    int64_t n = cols - c0 < COL_BLOCK ? cols - c0 : COL_BLOCK;
    float v[COL_BLOCK], w[COL_BLOCK];
    for (int64_t j = 0; j < n; ++j) {
      v[j] = v_init[c0 + j];
      w[j] = w_init[c0 + j];
    }
    for (int64_t k = 0; k < T; ++k) {
      const int64_t off = k * cols + c0;
      for (int64_t j = 0; j < n; ++j) {
        float bv = beta[off + j] * v[j];
        float ow = omega[off + j] * w[j];
        float d = bv - ow;
        float vpre = d + u[off + j];
        float ov = omega[off + j] * v[j];
        float bw = beta[off + j] * w[j];
        float wn = ov + bw;
        float s = vpre >= vth[off + j] ? 1.0f : 0.0f;
        float vs = vth[off + j] * s;
        v[j] = vpre - vs;
        w[j] = wn;
        if (spike) spike[off + j] = s;
        if (vpost) vpost[off + j] = v[j];
        if (wout) wout[off + j] = w[j];
      }
    }
    for (int64_t j = 0; j < n; ++j) {
      if (vlast) vlast[c0 + j] = v[j];
      if (wlast) wlast[c0 + j] = w[j];
    }
  }
}

/* Reverse pass of the resonate-and-fire scan with the two coupled adjoint   */
/* accumulators of atomic_ops/parallel_scan.py:835-848 (hard spike constant  */
/* in the reset path; a gradient arriving for W is ignored, as :1114 does).  */
void orc_plif_rf_bwd(const float *beta, const float *omega, const float *u,
                     const float *vth, const float *v_init, const float *w_init,
                     const float *g_spike, const float *g_vpost, float *g_beta,
                     float *g_omega, float *g_u, float *g_vth, float *g_vinit,
                     float *g_winit, int64_t T, int64_t cols, double a, int kind) {
#define RF_BLOCK 32
#pragma omp parallel
  {
    const size_t tt = (size_t)(T > 0 ? T : 1) * RF_BLOCK;
    float *vp = (float *)__builtin_malloc(sizeof(float) * tt * 3);
    float *wp = vp + tt, *xs = wp + tt;
#pragma omp for schedule(dynamic, 4)
    for (int64_t c0 = 0; c0 < cols; c0 += RF_BLOCK) {
      const int64_t n = cols - c0 < RF_BLOCK ? cols - c0 : RF_BLOCK;
      float v[RF_BLOCK], w[RF_BLOCK];
      double av[RF_BLOCK], aw[RF_BLOCK];
      for (int64_t j = 0; j < n; ++j) {
        v[j] = v_init[c0 + j];
        w[j] = w_init[c0 + j];
      }
      for (int64_t k = 0; k < T; ++k) {
        const int64_t o = k * cols + c0;
        for (int64_t j = 0; j < n; ++j) {
          float bv = beta[o + j] * v[j];
          float ow = omega[o + j] * w[j];
          float d = bv - ow;
          float vpre = d + u[o + j];
          float ov = omega[o + j] * v[j];
          float bw = beta[o + j] * w[j];
          vp[k * RF_BLOCK + j] = v[j];
          wp[k * RF_BLOCK + j] = w[j];
          xs[k * RF_BLOCK + j] = vpre - vth[o + j];
          float s = vpre >= vth[o + j] ? 1.0f : 0.0f;
          float vs = vth[o + j] * s;
          v[j] = vpre - vs;
          w[j] = ov + bw;
        }
      }
      for (int64_t j = 0; j < n; ++j) av[j] = aw[j] = 0.0;
      for (int64_t k = T - 1; k >= 0; --k) {
        const int64_t o = k * cols + c0;
        for (int64_t j = 0; j < n; ++j) {
          const double x = (double)xs[k * RF_BLOCK + j];
          const double s = x >= 0.0 ? 1.0 : 0.0;
          const double sg = surr_grad(x, a, kind);
          const double gs = g_spike ? (double)g_spike[o + j] : 0.0;
          const double tv = (g_vpost ? (double)g_vpost[o + j] : 0.0) + av[j];
          const double tw = aw[j];
          const double gpre = gs * sg + tv;
          const double vpr = (double)vp[k * RF_BLOCK + j], wpr = (double)wp[k * RF_BLOCK + j];
          const double b = (double)beta[o + j], om = (double)omega[o + j];
          if (g_beta) g_beta[o + j] = (float)(gpre * vpr + tw * wpr);
          if (g_omega) g_omega[o + j] = (float)(tw * vpr - gpre * wpr);
          if (g_u) g_u[o + j] = (float)gpre;
          if (g_vth) g_vth[o + j] = (float)(-gs * sg - tv * s);
          av[j] = gpre * b + tw * om;
          aw[j] = tw * b - gpre * om;
        }
      }
      for (int64_t j = 0; j < n; ++j) {
        if (g_vinit) g_vinit[c0 + j] = (float)av[j];
        if (g_winit) g_winit[c0 + j] = (float)aw[j];
      }
    }
    __builtin_free(vp);
  }
#undef RF_BLOCK
}

/* ------------------------------------------------------------------ */
/* FP16 boundary codec.                                                */
/* ------------------------------------------------------------------ */

/* fp32 -> IEEE binary16 bit pattern, round to nearest even, after the
 * reference's clamp to +-65504 (atomic_ops/fp16_codec.py:32). NaN keeps a
 * quiet-NaN pattern (clamp passes NaN through in PyTorch). */
static inline uint16_t f32_to_f16_bits(float f) {
  if (f > 65504.0f) f = 65504.0f;
  if (f < -65504.0f) f = -65504.0f;
  uint32_t x;
  memcpy(&x, &f, 4);
  uint32_t sign = (x >> 16) & 0x8000u;
  uint32_t ax = x & 0x7fffffffu;
  if (ax > 0x7f800000u) return (uint16_t)(sign | 0x7e00u);
  if (ax >= 0x38800000u) { /* normal half range (>= 2^-14) */
    uint32_t mant = ax & 0x7fffffu;
    uint32_t e = (ax >> 23) - 112u; /* rebias 127 -> 15 */
    uint32_t h = (e << 10) | (mant >> 13);
    uint32_t rem = mant & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) h += 1u;
    return (uint16_t)(sign | h);
  }
  if (ax < 0x33000000u) return (uint16_t)sign; /* < 2^-25 rounds to zero */
  /* subnormal half: value = m * 2^-24 with m in [0,1024) */
  uint32_t e = ax >> 23;
  uint32_t mant = (ax & 0x7fffffu) | 0x800000u;
  uint32_t shift = 126u - e; /* 14..24 */
  uint32_t h = mant >> shift;
  uint32_t rem = mant & ((1u << shift) - 1u);
  uint32_t half = 1u << (shift - 1u);
  if (rem > half || (rem == half && (h & 1u))) h += 1u;
  return (uint16_t)(sign | h);
}

/* Encode: emb [B, S, D] -> frames [S*16, B, D]; frame t*16+k carries bit
 * (15-k) of the half pattern, i.e. sign first, then E4..E0, M9..M0
 * (atomic_ops/fp16_codec.py:17-46). */
void orc_fp16_encode(const float *emb, float *frames, int64_t B, int64_t S,
                     int64_t D) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t b = 0; b < B; ++b)
    for (int64_t s = 0; s < S; ++s)
      for (int64_t d = 0; d < D; ++d) {
        uint16_t h = f32_to_f16_bits(emb[(b * S + s) * D + d]);
        for (int k = 0; k < 16; ++k)
          frames[((s * 16 + k) * B + b) * D + d] =
              (float)((h >> (15 - k)) & 1u);
      }
}

/* Optional emulation of a low-precision frame dtype: the reference computes
 * the decode formula in the dtype of the spike tensor, so with bf16 frames the
 * mantissa sum and 1+m are each rounded to bf16. mode 0 = fp32 (exact),
 * 1 = bf16. (fp16 frames need no emulation: every intermediate is exact.) */
static inline float round_bf16(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  if ((x & 0x7fffffffu) > 0x7f800000u) return f;
  uint32_t r = x + 0x7fffu + ((x >> 16) & 1u);
  r &= 0xffff0000u;
  float o;
  memcpy(&o, &r, 4);
  return o;
}

/* Decode: frames [S*16, B, D] (any real values, normally {0,1}) ->
 * value [B, S, D] (atomic_ops/fp16_codec.py:49-98). An all-ones exponent
 * decodes as an ordinary normal number (no inf/nan), as in the reference. */
void orc_fp16_decode(const float *frames, float *out, int64_t B, int64_t S,
                     int64_t D, int mode) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t b = 0; b < B; ++b)
    for (int64_t s = 0; s < S; ++s)
      for (int64_t d = 0; d < D; ++d) {
        float bit[16];
        for (int k = 0; k < 16; ++k)
          bit[k] = frames[((s * 16 + k) * B + b) * D + d];
        float sign = 1.0f - 2.0f * bit[0];
        float e = 0.0f;
        static const float ew[5] = {16.f, 8.f, 4.f, 2.f, 1.f};
        for (int i = 0; i < 5; ++i) e += bit[1 + i] * ew[i];
        float m = 0.0f;
        for (int i = 0; i < 10; ++i) m += bit[6 + i] * ldexpf(1.0f, -(i + 1));
        if (mode == 1) {
          sign = round_bf16(sign);
          e = round_bf16(e);
          m = round_bf16(m);
        }
        float val;
        if (e > 0.0f) {
          float opm = 1.0f + m;
          float p = sign * exp2f(e - 15.0f);
          if (mode == 1) {
            opm = round_bf16(opm);
            p = round_bf16(p);
          }
          val = p * opm;
        } else {
          val = (sign * 6.103515625e-05f) * m;
        }
        if (mode == 1) val = round_bf16(val);
        out[(b * S + s) * D + d] = val;
      }
}

/* Gradient of the decode formula w.r.t. each frame (autograd of
 * atomic_ops/fp16_codec.py:72-98; torch.where routes the gradient to the
 * selected branch only, and exp_val > 0 itself carries no gradient):
 *   d/d sign-bit      = -2 * |val| taken with sign = +1
 *   d/d exp-bit i     = val * ln2 * w_i   (normal branch), 0 (subnormal)
 *   d/d mantissa-bit j= sign * scale * 2^-(j+1), scale = 2^(e-15) or 2^-14 */
void orc_fp16_decode_bwd(const float *frames, const float *g_out,
                         float *g_frames, int64_t B, int64_t S, int64_t D) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t b = 0; b < B; ++b)
    for (int64_t s = 0; s < S; ++s)
      for (int64_t d = 0; d < D; ++d) {
        float bit[16];
        for (int k = 0; k < 16; ++k)
          bit[k] = frames[((s * 16 + k) * B + b) * D + d];
        float g = g_out[(b * S + s) * D + d];
        float sign = 1.0f - 2.0f * bit[0];
        float e = 0.0f;
        static const float ew[5] = {16.f, 8.f, 4.f, 2.f, 1.f};
        for (int i = 0; i < 5; ++i) e += bit[1 + i] * ew[i];
        float m = 0.0f;
        for (int i = 0; i < 10; ++i) m += bit[6 + i] * ldexpf(1.0f, -(i + 1));
        float gs, ge[5], gm[10];
        if (e > 0.0f) {
          float p = exp2f(e - 15.0f);
          gs = -2.0f * p * (1.0f + m) * g;
          for (int i = 0; i < 5; ++i)
            ge[i] = g * sign * (1.0f + m) * p * 0.6931471805599453f * ew[i];
          for (int j = 0; j < 10; ++j)
            gm[j] = g * sign * p * ldexpf(1.0f, -(j + 1));
        } else {
          gs = -2.0f * 6.103515625e-05f * m * g;
          for (int i = 0; i < 5; ++i) ge[i] = 0.0f;
          for (int j = 0; j < 10; ++j)
            gm[j] = g * sign * 6.103515625e-05f * ldexpf(1.0f, -(j + 1));
        }
        int64_t base = (s * 16 * B + b) * D + d;
        int64_t fs = B * D;
        g_frames[base] = gs;
        for (int i = 0; i < 5; ++i) g_frames[base + (1 + i) * fs] = ge[i];
        for (int j = 0; j < 10; ++j) g_frames[base + (6 + j) * fs] = gm[j];
      }
}

/* Binary residual: encode(decode(a) + decode(b)), frames [T*16, B, D]
 * (atomic_ops/fp16_codec.py:115-164).
 * mode 0: fp32 throughout (what fp32 and fp16 frames give: every intermediate is exact there).
 * mode 1: bf16 frames evaluated op by op, as eager PyTorch does (_binary_residual_naive, or
 *         _binary_residual_fwd called directly): mantissa sum, 1+m, each decoded value and their
 *         sum are rounded to bf16.
 * mode 2: bf16 frames through the reference's torch.compile'd residual (:168-170), observed on a
 *         B200 with torch 2.11: the decode stays in fp32 inside the fused kernel and only the
 *         sum, which is materialised as a bf16 tensor between two kernels, is rounded to bf16. */
void orc_binary_residual(const float *fa, const float *fb, float *out,
                         int64_t B, int64_t S, int64_t D, int mode) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t b = 0; b < B; ++b)
    for (int64_t s = 0; s < S; ++s)
      for (int64_t d = 0; d < D; ++d) {
        float val[2];
        const float *src[2] = {fa, fb};
        for (int w = 0; w < 2; ++w) {
          float bit[16];
          for (int k = 0; k < 16; ++k)
            bit[k] = src[w][((s * 16 + k) * B + b) * D + d];
          float sign = 1.0f - 2.0f * bit[0];
          float e = 0.0f;
          static const float ew[5] = {16.f, 8.f, 4.f, 2.f, 1.f};
          for (int i = 0; i < 5; ++i) e += bit[1 + i] * ew[i];
          float m = 0.0f;
          for (int i = 0; i < 10; ++i)
            m += bit[6 + i] * ldexpf(1.0f, -(i + 1));
          if (mode == 1) m = round_bf16(m);
          if (e > 0.0f) {
            float opm = 1.0f + m;
            if (mode == 1) opm = round_bf16(opm);
            val[w] = (sign * exp2f(e - 15.0f)) * opm;
          } else {
            val[w] = (sign * 6.103515625e-05f) * m;
          }
          if (mode == 1) val[w] = round_bf16(val[w]);
        }
        float sum = val[0] + val[1];
        if (mode == 1 || mode == 2) sum = round_bf16(sum);
        uint16_t h = f32_to_f16_bits(sum);
        for (int k = 0; k < 16; ++k)
          out[((s * 16 + k) * B + b) * D + d] = (float)((h >> (15 - k)) & 1u);
      }
}

/* Backward of binary_encode_ste: mean over the 16 frames of a token
 * (atomic_ops/fp16_codec.py:220-224). g_frames [S*16,B,D] -> g [B,S,D]. */
void orc_encode_ste_bwd(const float *g_frames, float *g, int64_t B, int64_t S,
                        int64_t D) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t b = 0; b < B; ++b)
    for (int64_t s = 0; s < S; ++s)
      for (int64_t d = 0; d < D; ++d) {
        float acc = 0.0f;
        for (int k = 0; k < 16; ++k)
          acc += g_frames[((s * 16 + k) * B + b) * D + d];
        g[(b * S + s) * D + d] = acc / 16.0f;
      }
}

/* ------------------------------------------------------------------ */
/* Lateral inhibition (divisive normalisation, = RMSNorm).             */
/* Forward: atomic_ops/lateral_inhibition.py:208-212 / kernel :66-77.  */
/* Backward: kernel :100-117 and the row reduction at :169.            */
/* Reductions run in double.                                           */
/* ------------------------------------------------------------------ */
void orc_li_fwd(const float *x, const float *gain, float *out, int64_t rows,
                int64_t D, double eps) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    double ss = 0.0;
    for (int64_t d = 0; d < D; ++d)
      ss += (double)x[r * D + d] * (double)x[r * D + d];
    double rrms = 1.0 / sqrt(ss / (double)D + eps);
    for (int64_t d = 0; d < D; ++d)
      out[r * D + d] = (float)((double)x[r * D + d] * rrms * (double)gain[d]);
  }
}

void orc_li_bwd(const float *g_out, const float *x, const float *gain,
                float *g_x, double *g_gain, int64_t rows, int64_t D,
                double eps) {
  for (int64_t d = 0; d < D; ++d) g_gain[d] = 0.0;
  for (int64_t r = 0; r < rows; ++r) {
    double ss = 0.0;
    for (int64_t d = 0; d < D; ++d)
      ss += (double)x[r * D + d] * (double)x[r * D + d];
    double rrms = 1.0 / sqrt(ss / (double)D + eps);
    double dot = 0.0;
    for (int64_t d = 0; d < D; ++d) {
      double xh = (double)x[r * D + d] * rrms;
      dot += (double)g_out[r * D + d] * (double)gain[d] * xh;
    }
    dot /= (double)D;
    for (int64_t d = 0; d < D; ++d) {
      double xh = (double)x[r * D + d] * rrms;
      double dg = (double)g_out[r * D + d] * (double)gain[d];
      g_x[r * D + d] = (float)((dg - xh * dot) * rrms);
      g_gain[d] += (double)g_out[r * D + d] * xh;
    }
  }
}

/* ------------------------------------------------------------------ */
/* Modulation: raw projections + per-channel biases -> scan inputs.    */
/* Follows atomic_ops/snn_block.py:52-76 (_fused_modulation_rf) and    */
/* archive/atomic_ops_v75_pre/snn_block.py:41-47 (_fused_modulation):  */
/*   beta  = sigmoid(raw_beta + b_beta)                                */
/*   alpha = softplus(raw_alpha + b_alpha)      (threshold 20)         */
/*   v_th  = v_th_min + |raw_th + b_th|                                */
/*   omega = softplus(raw_omega + b_omega)                 (RF only)   */
/*   r2 = beta*beta + omega*omega;                         (RF only)   */
/*   scale = r2 > 0.999^2 ? 0.999 * rsqrt(max(r2, 1e-12)) : 1          */
/*   beta *= scale; omega *= scale                                     */
/*   u = alpha * I                                                     */
/* Every +, * is one rounded fp32 operation in the order written; the  */
/* transcendental functions are evaluated in double and rounded once   */
/* (the reference's eager CPU evaluation agrees with that to 1-2 ulp,  */
/* which is what the golden-vector test allows).                       */
/* rows = T*batch, ch = channels; biases are [ch]. raw_omega == NULL   */
/* selects the first-order form. mod_round: 0 = keep fp32, 1 = round   */
/* beta/u/v_th/omega to bf16, 2 = to fp16 (a reference run with bf16   */
/* parameters materialises them in that dtype).                        */
/* ------------------------------------------------------------------ */
static inline float orc_sigmoidf(float z) { return (float)(1.0 / (1.0 + exp(-(double)z))); }
static inline float orc_softplusf(float z) {
  return z > 20.0f ? z : (float)log1p(exp((double)z));
}
static inline float round_f16(float f);
static inline float orc_mod_round(float f, int mode);

void orc_modulation_fwd(const float *raw_beta, const float *raw_alpha,
                        const float *raw_th, const float *raw_omega,
                        const float *cur, const float *b_beta,
                        const float *b_alpha, const float *b_th,
                        const float *b_omega, float v_th_min, int64_t rows,
                        int64_t ch, int mod_round, float *beta, float *u,
                        float *vth, float *omega) {
  const float rmax = 0.999f;
  const float rmax_sq = (float)(0.999 * 0.999);
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    for (int64_t c = 0; c < ch; ++c) {
      const int64_t i = r * ch + c;
      float b = orc_sigmoidf(raw_beta[i] + b_beta[c]);
      const float a = orc_softplusf(raw_alpha[i] + b_alpha[c]);
      const float th = v_th_min + fabsf(raw_th[i] + b_th[c]);
      if (raw_omega) {
        float o = orc_softplusf(raw_omega[i] + b_omega[c]);
        const float bb = b * b, oo = o * o;
        const float r2 = bb + oo;
        float scale = 1.0f;
        if (r2 > rmax_sq) {
          const float cl = r2 < 1e-12f ? 1e-12f : r2;
          const float rs = (float)(1.0 / sqrt((double)cl));
          scale = rmax * rs;
        }
        b = b * scale;
        o = o * scale;
        omega[i] = orc_mod_round(o, mod_round);
      }
      beta[i] = orc_mod_round(b, mod_round);
      u[i] = orc_mod_round(a * cur[i], mod_round);
      vth[i] = orc_mod_round(th, mod_round);
    }
  }
}

/* Adjoint of the above in double. Upstream gradients g_beta, g_u, g_vth,    */
/* g_omega (NULL with the first-order form) are those of the modulated      */
/* values; outputs are the gradients of the raw projections and of I, and   */
/* the bias gradients summed over rows ([ch], double accumulation).         */
/*   d sigmoid = s(1-s);  d softplus(z) = sigmoid(z);  d|z| = sign(z)        */
/*   scale active: beta = c*b0/r, omega = c*o0/r with r = sqrt(b0^2+o0^2):   */
/*     g_b0 = scale*(g_beta - (g_beta*b0 + g_omega*o0)*b0/r2), same for o0   */
void orc_modulation_bwd(const float *raw_beta, const float *raw_alpha,
                        const float *raw_th, const float *raw_omega,
                        const float *cur, const float *b_beta,
                        const float *b_alpha, const float *b_th,
                        const float *b_omega, int64_t rows, int64_t ch,
                        const float *g_beta, const float *g_u,
                        const float *g_vth, const float *g_omega,
                        float *g_raw_beta, float *g_raw_alpha, float *g_raw_th,
                        float *g_raw_omega, float *g_cur, double *gb_beta,
                        double *gb_alpha, double *gb_th, double *gb_omega) {
  const double rmax = (double)0.999f;
  const float rmax_sq = (float)(0.999 * 0.999);
  for (int64_t c = 0; c < ch; ++c) {
    gb_beta[c] = gb_alpha[c] = gb_th[c] = 0.0;
    if (raw_omega) gb_omega[c] = 0.0;
  }
#pragma omp parallel for schedule(static)
  for (int64_t c = 0; c < ch; ++c) {
    double sb = 0.0, sa = 0.0, st = 0.0, so = 0.0;
    for (int64_t r = 0; r < rows; ++r) {
      const int64_t i = r * ch + c;
      const float zb = raw_beta[i] + b_beta[c];
      const float za = raw_alpha[i] + b_alpha[c];
      const float zt = raw_th[i] + b_th[c];
      const double b0 = 1.0 / (1.0 + exp(-(double)zb));
      const double alpha = za > 20.0f ? (double)za : log1p(exp((double)za));
      double gb0 = g_beta[i];
      if (raw_omega) {
        const float zo = raw_omega[i] + b_omega[c];
        const double o0 = zo > 20.0f ? (double)zo : log1p(exp((double)zo));
        /* the branch is taken on the fp32 value the forward compares */
        const float b0f = (float)b0, o0f = (float)o0;
        const float r2f = b0f * b0f + o0f * o0f;
        double go0 = g_omega[i];
        if (r2f > rmax_sq) {
          const double r2 = b0 * b0 + o0 * o0;
          const double scale = rmax / sqrt(r2);
          const double dot = (gb0 * b0 + go0 * o0) / r2;
          const double nb = scale * (gb0 - dot * b0);
          const double no = scale * (go0 - dot * o0);
          gb0 = nb;
          go0 = no;
        }
        const double dsp = zo > 20.0f ? 1.0 : 1.0 / (1.0 + exp(-(double)zo));
        const double gzo = go0 * dsp;
        g_raw_omega[i] = (float)gzo;
        so += gzo;
      }
      const double gzb = gb0 * b0 * (1.0 - b0);
      const double dsa = za > 20.0f ? 1.0 : 1.0 / (1.0 + exp(-(double)za));
      const double gza = (double)g_u[i] * (double)cur[i] * dsa;
      const double sgn = zt > 0.0f ? 1.0 : (zt < 0.0f ? -1.0 : 0.0);
      const double gzt = (double)g_vth[i] * sgn;
      g_raw_beta[i] = (float)gzb;
      g_raw_alpha[i] = (float)gza;
      g_raw_th[i] = (float)gzt;
      g_cur[i] = (float)((double)g_u[i] * alpha);
      sb += gzb;
      sa += gza;
      st += gzt;
    }
    gb_beta[c] = sb;
    gb_alpha[c] = sa;
    gb_th[c] = st;
    if (raw_omega) gb_omega[c] = so;
  }
}

static inline float round_f16(float f) {
  const uint16_t h = f32_to_f16_bits(f);
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  const uint32_t e = (h >> 10) & 0x1Fu, m = h & 0x3FFu;
  float out;
  if (e == 0) {
    out = ldexpf((float)m, -24);
  } else if (e == 31) {
    out = m ? NAN : INFINITY;
  } else {
    out = ldexpf((float)(m | 0x400u), (int)e - 25);
  }
  uint32_t bits;
  memcpy(&bits, &out, 4);
  bits |= sign;
  memcpy(&out, &bits, 4);
  return out;
}
static inline float orc_mod_round(float f, int mode) {
  return mode == 1 ? round_bf16(f) : (mode == 2 ? round_f16(f) : f);
}

/* ------------------------------------------------------------------ */
/* Linear recurrence V[k] = beta[k]*V[k-1] + u[k]                      */
/* (atomic_ops/parallel_scan.py:65-141; public linear_recurrence       */
/* :1282-1302). Forward in fp32, one rounded multiply and one rounded  */
/* add per step; adjoint in double:                                    */
/*   g += dV[k]; grad_u[k] = g; grad_beta[k] = g*V[k-1]; g *= beta[k]  */
/* ------------------------------------------------------------------ */
void orc_linear_recurrence_fwd(const float *beta, const float *u,
                               const float *vinit, float *vout, int64_t T,
                               int64_t cols) {
#pragma omp parallel for schedule(static)
  for (int64_t c = 0; c < cols; ++c) {
    float v = vinit[c];
    for (int64_t k = 0; k < T; ++k) {
      const float bv = beta[k * cols + c] * v;
      v = bv + u[k * cols + c];
      vout[k * cols + c] = v;
    }
  }
}

void orc_linear_recurrence_bwd(const float *beta, const float *u,
                               const float *vinit, const float *g_v,
                               float *g_beta, float *g_u, float *g_vinit,
                               int64_t T, int64_t cols) {
#pragma omp parallel for schedule(static)
  for (int64_t c = 0; c < cols; ++c) {
    /* forward states in fp32, as the forward computes them */
    float v = vinit[c];
    float *vprev = (float *)g_u; /* reuse the output column as scratch for V[k-1] */
    for (int64_t k = 0; k < T; ++k) {
      vprev[k * cols + c] = v;
      const float bv = beta[k * cols + c] * v;
      v = bv + u[k * cols + c];
    }
    double g = 0.0;
    for (int64_t k = T - 1; k >= 0; --k) {
      g += (double)g_v[k * cols + c];
      const double vp = (double)vprev[k * cols + c];
      g_u[k * cols + c] = (float)g;
      g_beta[k * cols + c] = (float)(g * vp);
      g *= (double)beta[k * cols + c];
    }
    g_vinit[c] = (float)g;
  }
}

/* ------------------------------------------------------------------ */
/* MoE combine (atomic_ops/moe_kernels.py:1-13, 210-224): double       */
/* accumulation, rounded once.                                         */
/* ------------------------------------------------------------------ */
void orc_moe_combine_fwd(const float *shared, const float *experts,
                         const float *w, float *out, int64_t N, int64_t D,
                         int64_t E) {
#pragma omp parallel for schedule(static)
  for (int64_t n = 0; n < N; ++n)
    for (int64_t d = 0; d < D; ++d) {
      double acc = shared[n * D + d];
      for (int64_t e = 0; e < E; ++e)
        acc += (double)experts[(e * N + n) * D + d] * (double)w[n * E + e];
      out[n * D + d] = (float)acc;
    }
}

void orc_moe_combine_bwd(const float *g_out, const float *experts,
                         const float *w, float *g_experts, float *g_w,
                         int64_t N, int64_t D, int64_t E) {
#pragma omp parallel for schedule(static)
  for (int64_t n = 0; n < N; ++n)
    for (int64_t e = 0; e < E; ++e) {
      double dot = 0.0;
      for (int64_t d = 0; d < D; ++d) {
        const double g = g_out[n * D + d];
        g_experts[(e * N + n) * D + d] = (float)(g * (double)w[n * E + e]);
        dot += g * (double)experts[(e * N + n) * D + d];
      }
      g_w[n * E + e] = (float)dot;
    }
}
