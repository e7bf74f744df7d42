// PLIF scan kernels (forward and reverse-time backward) for sm_100a.
//
// Work decomposition. Every (batch, channel) column is an independent
// sequential recurrence over T steps, so parallelism comes from columns only.
// A warp owns 32*V consecutive columns (V = lanes per thread) and walks time in
// tiles of C steps. Each warp runs its OWN shared-memory ring: lane 0 issues one
// 2-D TMA tile load per input stream ([C rows x 32*V columns]) into the next
// free stage and all 32 lanes wait on that stage's mbarrier. Because producer
// and consumers are the same warp, a __syncwarp() is the only release needed
// before a stage is refilled: there are no CTA-wide barriers anywhere, warps
// drift freely, and a CTA is just a container whose size is chosen so that the
// grid balances over the SMs.
//
// The membrane state lives in fp32 registers. The charge step is a rounded
// multiply followed by a rounded add (never an FMA) so that spikes agree bit
// for bit with an eager fp32 time loop.
//
// The backward does not read a stored V_post: the forward writes one fp32
// checkpoint row per tile and the backward, walking tiles last to first,
// recomputes the C states of a tile from its checkpoint with the forward's
// exact arithmetic, then runs the adjoint recurrence over the same tile.
#pragma once

#include <algorithm>

#include "nsb_common.cuh"

namespace nsb {

enum { MODE_U = 0, MODE_AI = 1, MODE_ROW = 2 };

struct FwdArgs {
  const void* beta = nullptr;   // streams ([T, cols], stream dtype)
  const void* drive = nullptr;  // u (MODE_U / MODE_ROW) or cur (MODE_AI)
  const void* gain = nullptr;   // MODE_AI only
  const void* vth = nullptr;
  const float* beta_row = nullptr;  // MODE_ROW
  const float* vth_row = nullptr;
  const float* v_init = nullptr;
  void* spike = nullptr;
  uint32_t* packed = nullptr;
  void* vpost = nullptr;
  float* ckpt = nullptr;
  float* vlast = nullptr;
  long long T = 0, cols = 0;
  int mode = MODE_U;
  int tile = 8;  // C
  cudaStream_t stream = nullptr;
};

struct BwdArgs {
  const void* beta = nullptr;
  const void* drive = nullptr;
  const void* gain = nullptr;
  const void* vth = nullptr;
  const float* beta_row = nullptr;
  const float* vth_row = nullptr;
  const float* ckpt = nullptr;
  const void* g_spike = nullptr;
  const void* g_vpost = nullptr;
  void* g_beta = nullptr;   // stream dtype (selective)
  void* g_drive = nullptr;  // grad wrt u / cur
  void* g_gain = nullptr;
  void* g_vth = nullptr;
  float* g_beta_row = nullptr;  // MODE_ROW
  float* g_vth_row = nullptr;
  float* g_vinit = nullptr;
  long long T = 0, cols = 0;
  int mode = MODE_U;
  int tile = 8;
  int surrogate = NSB_SURR_SIGMOID;
  float alpha = 4.0f;
  cudaStream_t stream = nullptr;
};

// Per-dtype front doors (one translation unit each, to keep compile time flat).
int scan_fwd_f32(const FwdArgs& a);
int scan_fwd_bf16(const FwdArgs& a);
int scan_fwd_f16(const FwdArgs& a);
int scan_bwd_f32(const BwdArgs& a);
int scan_bwd_bf16(const BwdArgs& a);
int scan_bwd_f16(const BwdArgs& a);

#ifdef __CUDACC__

// ----------------------------------------------------------------- launch plan

struct Plan {
  int wpc = 1, stages = 2, grid = 0;
  size_t smem = 0;
};

// Chooses warps per CTA and ring depth for `nwarps` independent warps.
// stage_bytes: shared memory of one ring stage of one warp; regs: registers per
// thread of the kernel. The score models one or more waves of CTAs over the SMs
// of a bandwidth-bound kernel: a full wave costs its warps per SM, a partial
// last wave costs the warps of its busiest SM but never less than a latency
// floor, and configurations that keep too few bytes in flight are penalised.
inline Plan make_plan(const DeviceInfo& d, long long nwarps, size_t stage_bytes, int regs,
                      const Tuning& tune, int max_stages_useful) {
  Plan best;
  double best_score = 1e300;
  const int reserved = d.reserved_smem_per_cta > 0 ? d.reserved_smem_per_cta : 1024;
  const int reg_warps = std::max(1, 65536 / (std::max(regs, 16) * 32));
  for (int wpc = 1; wpc <= 8; ++wpc) {
    if (tune.warps_per_cta > 0 && wpc != tune.warps_per_cta) continue;
    for (int st = 2; st <= 6; ++st) {
      if (tune.stages > 0 && st != tune.stages) continue;
      if (tune.stages <= 0 && st > std::max(2, max_stages_useful)) continue;
      const size_t smem = (size_t)wpc * st * (stage_bytes + 8) + 256;
      if (smem > (size_t)d.max_smem_optin) continue;
      long long res = std::min<long long>(32, d.smem_per_sm / (long long)(smem + reserved));
      res = std::min<long long>(res, 64 / wpc);
      res = std::min<long long>(res, reg_warps / wpc);
      if (res < 1) continue;
      const long long ctas = (nwarps + wpc - 1) / wpc;
      const long long cap = res * d.sm_count;
      const long long nf = ctas / cap, rem = ctas % cap;
      const double floor_warps = 4.0;
      double units = (double)nf * (double)(res * wpc);
      if (rem) units += std::max<double>((double)((rem + d.sm_count - 1) / d.sm_count) * wpc, floor_warps);
      // bytes in flight per SM while streaming (all stages but the one being read)
      const double resident_warps = (double)std::min<long long>(cap, ctas) * wpc / d.sm_count;
      const double inflight = resident_warps * (st - 1) * (double)stage_bytes;
      const double want = 64.0 * 1024.0;
      double score = units * (inflight >= want ? 1.0 : (0.5 + 0.5 * want / std::max(inflight, 1.0)));
      score *= 1.0 + 0.002 * st + 0.001 * wpc;  // mild preference for small configs on ties
      if (score < best_score) {
        best_score = score;
        best.wpc = wpc;
        best.stages = st;
        best.grid = (int)ctas;
        best.smem = smem;
      }
    }
  }
  return best;
}

// ------------------------------------------------------------------- forward

struct FwdParams {
  const void* s[4];  // stream base pointers (direct path), order as in smem
  const float* beta_row;
  const float* vth_row;
  const float* v_init;
  void* spike;
  uint32_t* packed;
  void* vpost;
  float* ckpt;
  float* vlast;
  long long T, cols, words_per_row;
  int ntiles, stages;
  uint32_t* err;
};

template <int MODE>
struct ModeTraits {
  static constexpr int kFwdStreams = MODE == MODE_ROW ? 1 : (MODE == MODE_AI ? 4 : 3);
  // index of each role inside the stage / pointer table (-1 = absent)
  static constexpr int kBeta = MODE == MODE_ROW ? -1 : 0;
  static constexpr int kDrive = MODE == MODE_ROW ? 0 : 1;
  static constexpr int kGain = MODE == MODE_AI ? 2 : -1;
  static constexpr int kVth = MODE == MODE_ROW ? -1 : (MODE == MODE_AI ? 3 : 2);
};

// One charge / fire / soft-reset step. Returns the spike; x_out = v_pre - v_th.
__device__ __forceinline__ bool plif_step(float& v, float beta, float drive, float vth, float& x_out,
                                          float& vpre_out) {
  const float vpre = __fadd_rn(__fmul_rn(beta, v), drive);
  const float x = __fsub_rn(vpre, vth);
  const bool s = vpre >= vth;
  v = s ? x : vpre;
  x_out = x;
  vpre_out = vpre;
  return s;
}

template <typename ST, int MODE, bool PACKED, int V, int C, bool TMA>
__global__ void plif_fwd_kernel(const FwdParams p, const __grid_constant__ CUtensorMap tm0,
                                const __grid_constant__ CUtensorMap tm1,
                                const __grid_constant__ CUtensorMap tm2,
                                const __grid_constant__ CUtensorMap tm3) {
  using MT = ModeTraits<MODE>;
  using E = Elem<ST>;
  constexpr int NS = MT::kFwdStreams;
  constexpr int TILE_ELEMS = C * 32 * V;
  constexpr uint32_t TILE_BYTES = TILE_ELEMS * sizeof(ST);
  constexpr uint32_t STAGE_BYTES = NS * TILE_BYTES;
  extern __shared__ __align__(128) uint8_t smem_raw[];

  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int wpc = blockDim.x >> 5;
  const long long col0 = ((long long)blockIdx.x * wpc + warp) * (32 * V);
  if (col0 >= p.cols) return;

  long long colj[V];
  bool valid[V];
  float v[V], brow[V], trow[V];
#pragma unroll
  for (int j = 0; j < V; ++j) {
    colj[j] = PACKED ? col0 + 32 * j + lane : col0 + V * lane + j;
    valid[j] = colj[j] < p.cols;
    v[j] = valid[j] ? p.v_init[colj[j]] : 0.0f;
    brow[j] = 0.0f;
    trow[j] = 0.0f;
    if (MODE == MODE_ROW && valid[j]) {
      brow[j] = p.beta_row[colj[j]];
      trow[j] = p.vth_row[colj[j]];
    }
  }

  const int stages = p.stages;
  uint32_t bar0 = 0, data0 = 0;
  const uint8_t* data_ptr = nullptr;
  if constexpr (TMA) {
    const uint32_t base = smem_u32(smem_raw);
    bar0 = base + (uint32_t)(warp * stages) * 8u;
    const uint32_t data_base = (base + (uint32_t)(wpc * stages) * 8u + 127u) & ~127u;
    data0 = data_base + (uint32_t)(warp * stages) * STAGE_BYTES;
    data_ptr = smem_raw + (data0 - base);
    if (lane == 0) {
      for (int s = 0; s < stages; ++s) mbar_init(bar0 + 8u * s, 1);
      mbar_init_fence();
      proxy_async_fence();
    }
    __syncwarp();
  }

  auto issue = [&](int tile, int s) {
    if constexpr (TMA) {
      const uint32_t bar = bar0 + 8u * s;
      const uint32_t dst = data0 + (uint32_t)s * STAGE_BYTES;
      mbar_arrive_expect_tx(bar, STAGE_BYTES);
      tma_load_2d(dst, &tm0, (int)col0, tile * C, bar);
      if (NS > 1) tma_load_2d(dst + TILE_BYTES, &tm1, (int)col0, tile * C, bar);
      if (NS > 2) tma_load_2d(dst + 2 * TILE_BYTES, &tm2, (int)col0, tile * C, bar);
      if (NS > 3) tma_load_2d(dst + 3 * TILE_BYTES, &tm3, (int)col0, tile * C, bar);
    }
  };

  const int ntiles = p.ntiles;
  if constexpr (TMA) {
    if (lane == 0) {
      const int pre = ntiles < stages ? ntiles : stages;
      for (int s = 0; s < pre; ++s) issue(s, s);
    }
  }

  // Fetches element (stream, step k, lane-slot j) of the current tile as fp32.
  // The direct path stages KB steps of every stream in registers at a time.
  constexpr int KB = TMA ? C : 8;
  const ST* stage_ptr = nullptr;
  ST regs[TMA ? 1 : NS * KB * V] = {};
  auto get = [&](int stream, int k, int j) -> float {
    if constexpr (TMA) {
      const int idx = PACKED ? (k * 32 * V + 32 * j + lane) : (k * 32 * V + V * lane + j);
      return E::to_f32(stage_ptr[stream * TILE_ELEMS + idx]);
    } else {
      return E::to_f32(regs[(stream * KB + (k % KB)) * V + j]);
    }
  };

  int s_idx = 0;
  uint32_t phase = 0;
  bool failed = false;
  for (int i = 0; i < ntiles; ++i) {
    const long long t0 = (long long)i * C;
    const int nsteps = (p.T - t0) < C ? (int)(p.T - t0) : C;
    if constexpr (TMA) {
      const bool ok = mbar_wait_bounded(bar0 + 8u * s_idx, phase, p.err, 1u);
      if (!__any_sync(0xffffffffu, ok)) {
        failed = true;
        break;
      }
      stage_ptr = reinterpret_cast<const ST*>(data_ptr + (size_t)s_idx * STAGE_BYTES);
    }

    if (p.ckpt) {
#pragma unroll
      for (int j = 0; j < V; ++j)
        if (valid[j]) p.ckpt[(long long)i * p.cols + colj[j]] = v[j];
    }

    uint32_t words[V];
#pragma unroll
    for (int j = 0; j < V; ++j) words[j] = 0u;

#pragma unroll
    for (int k = 0; k < C; ++k) {
      if constexpr (!TMA) {
        if (k % KB == 0) {
#pragma unroll
          for (int st = 0; st < NS; ++st) {
            const ST* g = static_cast<const ST*>(p.s[st]);
#pragma unroll
            for (int kk = 0; kk < KB; ++kk)
#pragma unroll
              for (int j = 0; j < V; ++j)
                regs[(st * KB + kk) * V + j] =
                    (k + kk < nsteps && valid[j]) ? g[(t0 + k + kk) * p.cols + colj[j]] : E::zero();
          }
        }
      }
      if (k < nsteps) {
        bool sp[V];
#pragma unroll
        for (int j = 0; j < V; ++j) {
          const float b = MODE == MODE_ROW ? brow[j] : get(MT::kBeta < 0 ? 0 : MT::kBeta, k, j);
          const float th = MODE == MODE_ROW ? trow[j] : get(MT::kVth < 0 ? 0 : MT::kVth, k, j);
          float drive = get(MT::kDrive, k, j);
          if (MODE == MODE_AI) drive = __fmul_rn(get(MT::kGain < 0 ? 0 : MT::kGain, k, j), drive);
          float x, vpre;
          sp[j] = plif_step(v[j], b, drive, th, x, vpre);
        }
        const long long row = (t0 + k) * p.cols;
        if constexpr (!PACKED && V > 1) {
          // the V columns of a thread are contiguous: one vector store per output
          if (valid[0]) {
            if (p.spike) {
              Vec<ST, V> o;
#pragma unroll
              for (int j = 0; j < V; ++j) o.v[j] = sp[j] ? E::one() : E::zero();
              *reinterpret_cast<Vec<ST, V>*>(static_cast<ST*>(p.spike) + row + colj[0]) = o;
            }
            if (p.vpost) {
              Vec<ST, V> o;
#pragma unroll
              for (int j = 0; j < V; ++j) o.v[j] = E::from_f32(v[j]);
              *reinterpret_cast<Vec<ST, V>*>(static_cast<ST*>(p.vpost) + row + colj[0]) = o;
            }
          }
        } else {
#pragma unroll
          for (int j = 0; j < V; ++j) {
            if (valid[j]) {
              if (p.spike) static_cast<ST*>(p.spike)[row + colj[j]] = sp[j] ? E::one() : E::zero();
              if (p.vpost) static_cast<ST*>(p.vpost)[row + colj[j]] = E::from_f32(v[j]);
            }
          }
        }
        if constexpr (PACKED) {
#pragma unroll
          for (int j = 0; j < V; ++j) {
            const uint32_t w = __ballot_sync(0xffffffffu, sp[j] && valid[j]);
            if (lane == k) words[j] = w;
          }
        }
      }
    }

    if constexpr (PACKED) {
      if (p.packed && lane < nsteps) {
#pragma unroll
        for (int j = 0; j < V; ++j) {
          const long long widx = col0 / 32 + j;
          if (widx < p.words_per_row) p.packed[(t0 + lane) * p.words_per_row + widx] = words[j];
        }
      }
    }

    if constexpr (TMA) {
      __syncwarp();
      if (lane == 0 && i + stages < ntiles) issue(i + stages, s_idx);
      if (++s_idx == stages) {
        s_idx = 0;
        phase ^= 1u;
      }
    }
  }

  if constexpr (TMA) {
    if (failed) {
      // Give every load that may still be in flight a bounded chance to land
      // before the CTA's shared memory is released.
      for (int s = 0; s < stages; ++s) mbar_wait_bounded(bar0 + 8u * s, (s < s_idx) ? (phase ^ 1u) : phase, nullptr, 0u);
      return;
    }
  }
#pragma unroll
  for (int j = 0; j < V; ++j)
    if (valid[j]) p.vlast[colj[j]] = v[j];
}

// ------------------------------------------------------------------ backward

struct BwdParams {
  const void* s[6];  // stream base pointers (direct path), smem order
  const float* beta_row;
  const float* vth_row;
  const float* ckpt;
  void* g_beta;
  void* g_drive;
  void* g_gain;
  void* g_vth;
  float* g_beta_row;
  float* g_vth_row;
  float* g_vinit;
  long long T, cols;
  int ntiles, stages, has_gv, nstreams;
  float alpha;
  uint32_t* err;
};

template <int SURR>
__device__ __forceinline__ float surrogate_grad(float x, float alpha, float c1, float c2) {
  if (SURR == NSB_SURR_ATAN) {
    // (alpha/2) / (1 + (pi/2 * alpha * x)^2);  c1 = pi/2*alpha, c2 = alpha/2
    const float z = c1 * x;
    return __fdividef(c2, fmaf(z, z, 1.0f));
  } else {
    // alpha * sig * (1 - sig) = alpha * e / (1 + e)^2 with e = exp(-alpha*|x|) in (0, 1]
    // (even in x, so no overflow and no clamp);  c1 = -alpha*log2(e)
    const float e = exp2f(c1 * fabsf(x));
    const float r = __fdividef(1.0f, 1.0f + e);
    return alpha * e * r * r;
  }
}

template <typename ST, int MODE, int SURR, int V, int C, bool TMA>
__global__ void plif_bwd_kernel(const BwdParams p, const __grid_constant__ CUtensorMap tm0,
                                const __grid_constant__ CUtensorMap tm1,
                                const __grid_constant__ CUtensorMap tm2,
                                const __grid_constant__ CUtensorMap tm3,
                                const __grid_constant__ CUtensorMap tm4,
                                const __grid_constant__ CUtensorMap tm5,
                                const __grid_constant__ CUtensorMap tm_ckpt) {
  using MT = ModeTraits<MODE>;
  using E = Elem<ST>;
  constexpr int NF = MT::kFwdStreams;  // forward inputs; then g_spike, then optional g_vpost
  constexpr int kGS = NF, kGV = NF + 1;
  constexpr int TILE_ELEMS = C * 32 * V;
  constexpr uint32_t TILE_BYTES = TILE_ELEMS * sizeof(ST);
  constexpr uint32_t CKPT_BYTES = 32 * V * sizeof(float);
  extern __shared__ __align__(128) uint8_t smem_raw[];

  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int wpc = blockDim.x >> 5;
  const long long col0 = ((long long)blockIdx.x * wpc + warp) * (32 * V);
  if (col0 >= p.cols) return;

  const int nstreams = p.nstreams;  // NF + 1 + has_gv
  const bool has_gv = p.has_gv != 0;
  const uint32_t stage_bytes = (uint32_t)nstreams * TILE_BYTES + CKPT_BYTES;

  long long colj[V];
  bool valid[V];
  float brow[V], trow[V], acc[V], accb[V], acct[V];
#pragma unroll
  for (int j = 0; j < V; ++j) {
    colj[j] = col0 + V * lane + j;
    valid[j] = colj[j] < p.cols;
    acc[j] = accb[j] = acct[j] = 0.0f;
    brow[j] = trow[j] = 0.0f;
    if (MODE == MODE_ROW && valid[j]) {
      brow[j] = p.beta_row[colj[j]];
      trow[j] = p.vth_row[colj[j]];
    }
  }

  const int stages = p.stages;
  uint32_t bar0 = 0, data0 = 0;
  const uint8_t* data_ptr = nullptr;
  if constexpr (TMA) {
    const uint32_t base = smem_u32(smem_raw);
    bar0 = base + (uint32_t)(warp * stages) * 8u;
    const uint32_t data_base = (base + (uint32_t)(wpc * stages) * 8u + 127u) & ~127u;
    data0 = data_base + (uint32_t)(warp * stages) * stage_bytes;
    data_ptr = smem_raw + (data0 - base);
    if (lane == 0) {
      for (int s = 0; s < stages; ++s) mbar_init(bar0 + 8u * s, 1);
      mbar_init_fence();
      proxy_async_fence();
    }
    __syncwarp();
  }

  auto issue = [&](int tile, int s) {
    if constexpr (TMA) {
      const uint32_t bar = bar0 + 8u * s;
      const uint32_t dst = data0 + (uint32_t)s * stage_bytes;
      mbar_arrive_expect_tx(bar, stage_bytes);
      const int x = (int)col0, y = tile * C;
      tma_load_2d(dst, &tm0, x, y, bar);
      tma_load_2d(dst + TILE_BYTES, &tm1, x, y, bar);
      if (nstreams > 2) tma_load_2d(dst + 2 * TILE_BYTES, &tm2, x, y, bar);
      if (nstreams > 3) tma_load_2d(dst + 3 * TILE_BYTES, &tm3, x, y, bar);
      if (nstreams > 4) tma_load_2d(dst + 4 * TILE_BYTES, &tm4, x, y, bar);
      if (nstreams > 5) tma_load_2d(dst + 5 * TILE_BYTES, &tm5, x, y, bar);
      tma_load_2d(dst + (uint32_t)nstreams * TILE_BYTES, &tm_ckpt, x, tile, bar);
    }
  };

  const int ntiles = p.ntiles;
  if constexpr (TMA) {
    if (lane == 0) {
      const int pre = ntiles < stages ? ntiles : stages;
      for (int s = 0; s < pre; ++s) issue(ntiles - 1 - s, s);
    }
  }

  const ST* stage_ptr = nullptr;
  ST regs[TMA ? 1 : (NF + 2) * C * V] = {};
  auto get = [&](int stream, int k, int j) -> float {
    if constexpr (TMA) {
      return E::to_f32(stage_ptr[stream * TILE_ELEMS + k * 32 * V + V * lane + j]);
    } else {
      return E::to_f32(regs[(stream * C + k) * V + j]);
    }
  };

  const float alpha = p.alpha;
  const float c1 = SURR == NSB_SURR_ATAN ? 1.5707963267948966f * alpha : -alpha * 1.4426950408889634f;
  const float c2 = 0.5f * alpha;

  int s_idx = 0;
  uint32_t phase = 0;
  bool failed = false;
  for (int n = 0; n < ntiles; ++n) {
    const int i = ntiles - 1 - n;
    const long long t0 = (long long)i * C;
    const int nsteps = (p.T - t0) < C ? (int)(p.T - t0) : C;
    float v[V];
    if constexpr (TMA) {
      const bool ok = mbar_wait_bounded(bar0 + 8u * s_idx, phase, p.err, 2u);
      if (!__any_sync(0xffffffffu, ok)) {
        failed = true;
        break;
      }
      const uint8_t* sp8 = data_ptr + (size_t)s_idx * stage_bytes;
      stage_ptr = reinterpret_cast<const ST*>(sp8);
      const float* ck = reinterpret_cast<const float*>(sp8 + (size_t)nstreams * TILE_BYTES);
#pragma unroll
      for (int j = 0; j < V; ++j) v[j] = ck[V * lane + j];
    } else {
#pragma unroll
      for (int st = 0; st < NF + 2; ++st) {
        const ST* g = static_cast<const ST*>(p.s[st]);
        const bool present = st < nstreams;
#pragma unroll
        for (int k = 0; k < C; ++k)
#pragma unroll
          for (int j = 0; j < V; ++j)
            regs[(st * C + k) * V + j] =
                (present && k < nsteps && valid[j]) ? g[(t0 + k) * p.cols + colj[j]] : E::zero();
      }
#pragma unroll
      for (int j = 0; j < V; ++j) v[j] = valid[j] ? p.ckpt[(long long)i * p.cols + colj[j]] : 0.0f;
    }

    // recompute the tile forward, keeping V[k-1] and x[k] = V_pre[k] - V_th[k]
    float vprev[C][V], xs[C][V];
#pragma unroll
    for (int k = 0; k < C; ++k) {
#pragma unroll
      for (int j = 0; j < V; ++j) {
        vprev[k][j] = v[j];
        xs[k][j] = 0.0f;
        if (k < nsteps) {
          const float b = MODE == MODE_ROW ? brow[j] : get(MT::kBeta < 0 ? 0 : MT::kBeta, k, j);
          const float th = MODE == MODE_ROW ? trow[j] : get(MT::kVth < 0 ? 0 : MT::kVth, k, j);
          float drive = get(MT::kDrive, k, j);
          if (MODE == MODE_AI) drive = __fmul_rn(get(MT::kGain < 0 ? 0 : MT::kGain, k, j), drive);
          float vpre;
          plif_step(v[j], b, drive, th, xs[k][j], vpre);
        }
      }
    }

    // adjoint recurrence, last step of the tile first
#pragma unroll
    for (int kk = 0; kk < C; ++kk) {
      const int k = C - 1 - kk;
      if (k < nsteps) {
        float o_beta[V], o_drive[V], o_gain[V], o_vth[V];
#pragma unroll
        for (int j = 0; j < V; ++j) {
          const float x = xs[k][j];
          const bool s = x >= 0.0f;
          const float sg = surrogate_grad<SURR>(x, alpha, c1, c2);
          const float gs = get(kGS, k, j);
          const float tot = has_gv ? acc[j] + get(kGV, k, j) : acc[j];
          const float gssg = gs * sg;
          const float gpre = gssg + tot;
          const float b = MODE == MODE_ROW ? brow[j] : get(MT::kBeta < 0 ? 0 : MT::kBeta, k, j);
          const float gvth = s ? (-gssg - tot) : -gssg;
          o_beta[j] = gpre * vprev[k][j];
          o_vth[j] = gvth;
          if (MODE == MODE_AI) {
            o_drive[j] = gpre * get(MT::kGain < 0 ? 0 : MT::kGain, k, j);
            o_gain[j] = gpre * get(MT::kDrive, k, j);
          } else {
            o_drive[j] = gpre;
            o_gain[j] = 0.0f;
          }
          if (MODE == MODE_ROW) {
            accb[j] += o_beta[j];
            acct[j] += gvth;
          }
          acc[j] = gpre * b;
        }
        const long long off = (t0 + k) * p.cols + colj[0];
        auto store = [&](void* dst, const float (&val)[V]) {
          if (!dst) return;
          if constexpr (V > 1) {
            if (valid[0]) {
              Vec<ST, V> o;
#pragma unroll
              for (int j = 0; j < V; ++j) o.v[j] = E::from_f32(val[j]);
              *reinterpret_cast<Vec<ST, V>*>(static_cast<ST*>(dst) + off) = o;
            }
          } else {
            if (valid[0]) static_cast<ST*>(dst)[off] = E::from_f32(val[0]);
          }
        };
        if (MODE != MODE_ROW) {
          store(p.g_beta, o_beta);
          store(p.g_vth, o_vth);
        }
        store(p.g_drive, o_drive);
        if (MODE == MODE_AI) store(p.g_gain, o_gain);
      }
    }

    if constexpr (TMA) {
      __syncwarp();
      if (lane == 0 && i - stages >= 0) issue(i - stages, s_idx);
      if (++s_idx == stages) {
        s_idx = 0;
        phase ^= 1u;
      }
    }
  }

  if constexpr (TMA) {
    if (failed) {
      for (int s = 0; s < stages; ++s) mbar_wait_bounded(bar0 + 8u * s, (s < s_idx) ? (phase ^ 1u) : phase, nullptr, 0u);
      return;
    }
  }
#pragma unroll
  for (int j = 0; j < V; ++j) {
    if (valid[j]) {
      if (p.g_vinit) p.g_vinit[colj[j]] = acc[j];
      if (MODE == MODE_ROW) {
        if (p.g_beta_row) p.g_beta_row[colj[j]] = accb[j];
        if (p.g_vth_row) p.g_vth_row[colj[j]] = acct[j];
      }
    }
  }
}

// -------------------------------------------------------------- host launchers

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <typename ST, int MODE, bool PACKED, int V, int C, bool TMA>
int launch_fwd_one(const FwdArgs& a, const DeviceInfo& dev, const Tuning& tune) {
  using MT = ModeTraits<MODE>;
  constexpr int NS = MT::kFwdStreams;
  auto kern = plif_fwd_kernel<ST, MODE, PACKED, V, C, TMA>;
  FwdParams p = {};
  const void* streams[4] = {nullptr, nullptr, nullptr, nullptr};
  if (MODE == MODE_ROW) {
    streams[0] = a.drive;
  } else if (MODE == MODE_AI) {
    streams[0] = a.beta; streams[1] = a.drive; streams[2] = a.gain; streams[3] = a.vth;
  } else {
    streams[0] = a.beta; streams[1] = a.drive; streams[2] = a.vth;
  }
  for (int i = 0; i < 4; ++i) p.s[i] = streams[i];
  p.beta_row = a.beta_row; p.vth_row = a.vth_row; p.v_init = a.v_init;
  p.spike = a.spike; p.packed = a.packed; p.vpost = a.vpost; p.ckpt = a.ckpt; p.vlast = a.vlast;
  p.T = a.T; p.cols = a.cols; p.words_per_row = (a.cols + 31) / 32;
  p.ntiles = (int)((a.T + C - 1) / C);
  p.err = device_error_word_ptr();

  const long long nwarps = (a.cols + 32 * V - 1) / (32 * V);
  CUtensorMap tm[4];
  memset(tm, 0, sizeof tm);
  Plan plan;
  LaunchInfo& li = last_launch();
  if (TMA) {
    for (int i = 0; i < NS; ++i) {
      int r = make_tensor_map_2d(&tm[i], streams[i], Elem<ST>::kDtype, (uint64_t)a.T, (uint64_t)a.cols, C,
                                 32 * V);
      if (r != NSB_OK) return r;
    }
    cudaFuncAttributes fa;
    NSB_CUDA_TRY(cudaFuncGetAttributes(&fa, kern), "cudaFuncGetAttributes(fwd)");
    const size_t stage_bytes = (size_t)NS * C * 32 * V * sizeof(ST);
    plan = make_plan(dev, nwarps, stage_bytes, fa.numRegs, tune, std::min(4, p.ntiles));
    if (plan.grid == 0) return NSB_ERR_UNSUPPORTED;
    NSB_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)plan.smem),
                 "cudaFuncSetAttribute(fwd)");
  } else {
    plan.wpc = tune.warps_per_cta > 0 ? tune.warps_per_cta : 4;
    plan.stages = 1;
    plan.grid = (int)((nwarps + plan.wpc - 1) / plan.wpc);
    plan.smem = 0;
  }
  p.stages = plan.stages;
  kern<<<plan.grid, plan.wpc * 32, plan.smem, a.stream>>>(p, tm[0], tm[1], tm[2], tm[3]);
  NSB_CUDA_TRY(cudaGetLastError(), "launch plif_fwd_kernel");
  li.used_tma = TMA; li.warps_per_cta = plan.wpc; li.stages = plan.stages; li.lanes_per_thread = V;
  li.grid = plan.grid; li.smem_bytes = (int)plan.smem; li.tile_steps = C; li.launches = 1;
  return NSB_OK;
}

template <typename ST, int MODE, int SURR, int V, int C, bool TMA>
int launch_bwd_one(const BwdArgs& a, const DeviceInfo& dev, const Tuning& tune) {
  using MT = ModeTraits<MODE>;
  constexpr int NF = MT::kFwdStreams;
  auto kern = plif_bwd_kernel<ST, MODE, SURR, V, C, TMA>;
  BwdParams p = {};
  const void* streams[6] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  if (MODE == MODE_ROW) {
    streams[0] = a.drive;
  } else if (MODE == MODE_AI) {
    streams[0] = a.beta; streams[1] = a.drive; streams[2] = a.gain; streams[3] = a.vth;
  } else {
    streams[0] = a.beta; streams[1] = a.drive; streams[2] = a.vth;
  }
  streams[NF] = a.g_spike;
  streams[NF + 1] = a.g_vpost;
  const int has_gv = a.g_vpost != nullptr;
  const int nstreams = NF + 1 + has_gv;
  for (int i = 0; i < 6; ++i) p.s[i] = streams[i];
  p.beta_row = a.beta_row; p.vth_row = a.vth_row; p.ckpt = a.ckpt;
  p.g_beta = a.g_beta; p.g_drive = a.g_drive; p.g_gain = a.g_gain; p.g_vth = a.g_vth;
  p.g_beta_row = a.g_beta_row; p.g_vth_row = a.g_vth_row; p.g_vinit = a.g_vinit;
  p.T = a.T; p.cols = a.cols;
  p.ntiles = (int)((a.T + C - 1) / C);
  p.has_gv = has_gv; p.nstreams = nstreams; p.alpha = a.alpha;
  p.err = device_error_word_ptr();

  const long long nwarps = (a.cols + 32 * V - 1) / (32 * V);
  CUtensorMap tm[7];
  memset(tm, 0, sizeof tm);
  Plan plan;
  if (TMA) {
    for (int i = 0; i < nstreams; ++i) {
      int r = make_tensor_map_2d(&tm[i], streams[i], Elem<ST>::kDtype, (uint64_t)a.T, (uint64_t)a.cols, C,
                                 32 * V);
      if (r != NSB_OK) return r;
    }
    int r = make_tensor_map_2d(&tm[6], a.ckpt, NSB_F32, (uint64_t)p.ntiles, (uint64_t)a.cols, 1, 32 * V);
    if (r != NSB_OK) return r;
    cudaFuncAttributes fa;
    NSB_CUDA_TRY(cudaFuncGetAttributes(&fa, kern), "cudaFuncGetAttributes(bwd)");
    const size_t stage_bytes = (size_t)nstreams * C * 32 * V * sizeof(ST) + 32 * V * sizeof(float);
    plan = make_plan(dev, nwarps, stage_bytes, fa.numRegs, tune, std::min(3, p.ntiles));
    if (plan.grid == 0) return NSB_ERR_UNSUPPORTED;
    NSB_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)plan.smem),
                 "cudaFuncSetAttribute(bwd)");
  } else {
    plan.wpc = tune.warps_per_cta > 0 ? tune.warps_per_cta : 4;
    plan.stages = 1;
    plan.grid = (int)((nwarps + plan.wpc - 1) / plan.wpc);
    plan.smem = 0;
  }
  p.stages = plan.stages;
  kern<<<plan.grid, plan.wpc * 32, plan.smem, a.stream>>>(p, tm[0], tm[1], tm[2], tm[3], tm[4], tm[5], tm[6]);
  NSB_CUDA_TRY(cudaGetLastError(), "launch plif_bwd_kernel");
  LaunchInfo& li = last_launch();
  li.used_tma = TMA; li.warps_per_cta = plan.wpc; li.stages = plan.stages; li.lanes_per_thread = V;
  li.grid = plan.grid; li.smem_bytes = (int)plan.smem; li.tile_steps = C; li.launches = 1;
  return NSB_OK;
}

// The TMA path needs 16-byte aligned bases and row pitch, int32 coordinates and
// an sm_100 device; anything else takes the direct-load kernel.
template <typename ST>
inline bool tma_ok_common(const DeviceInfo& dev, long long T, long long cols, const Tuning& tune) {
  if (tune.force_direct) return false;
  if (dev.cc_major != 10) return false;
  if ((cols * (long long)sizeof(ST)) % 16 != 0) return false;
  if (cols >= (1ll << 31) || T >= (1ll << 31)) return false;
  return true;
}

template <typename ST>
int scan_fwd_dispatch(const FwdArgs& a) {
  DeviceInfo dev;
  int r = get_device_info(&dev);
  if (r != NSB_OK) return r;
  if (dev.cc_major != 10) return NSB_ERR_UNSUPPORTED;
  const Tuning tune = get_tuning();
  bool tma = tma_ok_common<ST>(dev, a.T, a.cols, tune);
  const void* ptrs[] = {a.beta, a.drive, a.gain, a.vth, a.spike, a.vpost, a.ckpt};
  for (const void* q : ptrs) tma = tma && aligned16(q);
  const bool packed = a.packed != nullptr;
  const int V = tune.lanes_per_thread > 0 ? tune.lanes_per_thread : 2;
  const int C = a.tile;

#define NSB_FWD_CASE(MODE_, PACKED_, V_, C_)                                           \
  if (a.mode == MODE_ && packed == PACKED_ && V == V_ && C == C_)                      \
    return launch_fwd_one<ST, MODE_, PACKED_, V_, C_, true>(a, dev, tune);
#define NSB_FWD_CASES_V(MODE_, PACKED_)                                                \
  NSB_FWD_CASE(MODE_, PACKED_, 1, 8) NSB_FWD_CASE(MODE_, PACKED_, 2, 8)                \
  NSB_FWD_CASE(MODE_, PACKED_, 4, 8) NSB_FWD_CASE(MODE_, PACKED_, 1, 16)               \
  NSB_FWD_CASE(MODE_, PACKED_, 2, 16) NSB_FWD_CASE(MODE_, PACKED_, 4, 16)
  if (tma) {
    NSB_FWD_CASES_V(MODE_U, false) NSB_FWD_CASES_V(MODE_U, true)
    NSB_FWD_CASES_V(MODE_AI, false) NSB_FWD_CASES_V(MODE_AI, true)
    NSB_FWD_CASES_V(MODE_ROW, false) NSB_FWD_CASES_V(MODE_ROW, true)
    return NSB_ERR_INVALID_ARG;
  }
#undef NSB_FWD_CASES_V
#undef NSB_FWD_CASE
#define NSB_FWD_DIRECT(MODE_, C_)                                                      \
  if (a.mode == MODE_ && C == C_)                                                      \
    return packed ? launch_fwd_one<ST, MODE_, true, 1, C_, false>(a, dev, tune)        \
                  : launch_fwd_one<ST, MODE_, false, 1, C_, false>(a, dev, tune);
  NSB_FWD_DIRECT(MODE_U, 8) NSB_FWD_DIRECT(MODE_U, 16)
  NSB_FWD_DIRECT(MODE_AI, 8) NSB_FWD_DIRECT(MODE_AI, 16)
  NSB_FWD_DIRECT(MODE_ROW, 8) NSB_FWD_DIRECT(MODE_ROW, 16)
#undef NSB_FWD_DIRECT
  return NSB_ERR_INVALID_ARG;
}

template <typename ST>
int scan_bwd_dispatch(const BwdArgs& a) {
  DeviceInfo dev;
  int r = get_device_info(&dev);
  if (r != NSB_OK) return r;
  if (dev.cc_major != 10) return NSB_ERR_UNSUPPORTED;
  const Tuning tune = get_tuning();
  bool tma = tma_ok_common<ST>(dev, a.T, a.cols, tune);
  const void* ptrs[] = {a.beta, a.drive, a.gain, a.vth, a.ckpt, a.g_spike, a.g_vpost,
                        a.g_beta, a.g_drive, a.g_gain, a.g_vth};
  for (const void* q : ptrs) tma = tma && aligned16(q);
  const int V = tune.lanes_per_thread > 0 ? tune.lanes_per_thread : 2;
  const int C = a.tile;

#define NSB_BWD_CASE(MODE_, SURR_, V_, C_)                                             \
  if (a.mode == MODE_ && a.surrogate == SURR_ && V == V_ && C == C_)                   \
    return launch_bwd_one<ST, MODE_, SURR_, V_, C_, true>(a, dev, tune);
#define NSB_BWD_CASES_V(MODE_, SURR_)                                                  \
  NSB_BWD_CASE(MODE_, SURR_, 1, 8) NSB_BWD_CASE(MODE_, SURR_, 2, 8)                    \
  NSB_BWD_CASE(MODE_, SURR_, 1, 16) NSB_BWD_CASE(MODE_, SURR_, 2, 16)
  if (tma && V <= 2) {
    NSB_BWD_CASES_V(MODE_U, NSB_SURR_SIGMOID) NSB_BWD_CASES_V(MODE_U, NSB_SURR_ATAN)
    NSB_BWD_CASES_V(MODE_AI, NSB_SURR_SIGMOID) NSB_BWD_CASES_V(MODE_AI, NSB_SURR_ATAN)
    NSB_BWD_CASES_V(MODE_ROW, NSB_SURR_SIGMOID) NSB_BWD_CASES_V(MODE_ROW, NSB_SURR_ATAN)
    return NSB_ERR_INVALID_ARG;
  }
#undef NSB_BWD_CASES_V
#undef NSB_BWD_CASE
#define NSB_BWD_DIRECT(MODE_, SURR_, C_)                                               \
  if (a.mode == MODE_ && a.surrogate == SURR_ && C == C_)                              \
    return launch_bwd_one<ST, MODE_, SURR_, 1, C_, false>(a, dev, tune);
#define NSB_BWD_DIRECT_S(MODE_)                                                        \
  NSB_BWD_DIRECT(MODE_, NSB_SURR_SIGMOID, 8) NSB_BWD_DIRECT(MODE_, NSB_SURR_SIGMOID, 16) \
  NSB_BWD_DIRECT(MODE_, NSB_SURR_ATAN, 8) NSB_BWD_DIRECT(MODE_, NSB_SURR_ATAN, 16)
  NSB_BWD_DIRECT_S(MODE_U) NSB_BWD_DIRECT_S(MODE_AI) NSB_BWD_DIRECT_S(MODE_ROW)
#undef NSB_BWD_DIRECT_S
#undef NSB_BWD_DIRECT
  return NSB_ERR_INVALID_ARG;
}

#endif  // __CUDACC__

}  // namespace nsb
