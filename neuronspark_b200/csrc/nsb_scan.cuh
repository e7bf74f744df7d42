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
#include <type_traits>

#include "nsb_codec.cuh"
#include "nsb_common.cuh"
#include "nsb_modulation.cuh"

namespace nsb {

// MODE_MOD / MODE_RFMOD are MODE_AI / MODE_RF with the modulation fused into the load path: they
// stream the RAW projections (raw_beta, I, raw_alpha, raw_th [, raw_omega]) and form beta, u = alpha*I,
// v_th (, omega) per element in registers (nsb_modulation.cuh).
// MODE_LIN is the linear recurrence V[k] = beta[k]*V[k-1] + u[k] (no threshold, no reset): the u-form
// scan with an infinite threshold whose dense output is V instead of the spikes and whose incoming
// gradient is that of V.
// MODE_ROWRES (forward only) is MODE_ROW followed by the binary residual of the FP16 codec: every 16
// steps the column's spikes are one half bit pattern; it is decoded, added to the value decoded from
// the 16 frames of a second input stream, re-encoded, and those frames are the output.
// MODE_ROWPAT (forward only) is MODE_ROW whose output is PACKED IN TIME: the 16 spikes of a token
// and column leave as one uint16 - the IEEE half bit pattern they spell, frame 0 = sign - in a
// [T/16, cols] array, 2 bytes per value where dense frames take 16 elements. With a second
// pattern array given, the binary residual is applied to the two patterns first (as MODE_ROWRES
// does on frames). It streams the drive only.
// MODE_RF is the second-order resonate-and-fire scan: it streams beta, u, omega, v_th
// (omega in the slot the gain*cur form uses for the gain) and carries two states, V and W.
enum { MODE_U = 0, MODE_AI = 1, MODE_ROW = 2, MODE_RF = 3, MODE_MOD = 4, MODE_RFMOD = 5, MODE_ROWRES = 6, MODE_LIN = 7,
       // forward-only variants of MODE_MOD / MODE_RFMOD that also accumulate the moments of u = alpha*I (for
       // the adaptive surrogate slope). Separate kernels: compiled into the same kernel, as a run-time or a
       // per-tile choice, the extra accumulators cost 25-85 registers and a third of the resident warps.
       MODE_MODS = 8, MODE_RFMODS = 9, MODE_ROWPAT = 10 };

struct FwdArgs {
  const void* beta = nullptr;   // streams ([T, cols], stream dtype)
  const void* drive = nullptr;  // u (MODE_U / MODE_ROW) or cur (MODE_AI)
  const void* gain = nullptr;   // MODE_AI: gain; MODE_RF: omega; modulated modes: raw_alpha
  const void* vth = nullptr;
  const void* extra = nullptr;  // MODE_RFMOD: raw_omega
  const float* bias[4] = {nullptr, nullptr, nullptr, nullptr};  // modulated modes: b_beta, b_alpha, b_th, b_omega ([channels])
  long long channels = 0;                                         // cols is a multiple of it
  float v_th_min = 0.0f;
  // modulated modes, optional: adaptive surrogate slope from the moments of u = alpha*I, which the
  // kernel accumulates while it streams (u_stats: 2 doubles per warp of the launch)
  double* u_stats = nullptr;
  float* alpha_out = nullptr;
  float alpha0 = 4.0f, sigma0 = 0.4f;
  const float* beta_row = nullptr;  // MODE_ROW
  const float* vth_row = nullptr;
  const float* v_init = nullptr;
  const float* w_init = nullptr;  // MODE_RF
  void* w_out = nullptr;          // MODE_RF, optional dense W
  float* ckpt_w = nullptr;        // MODE_RF
  float* wlast = nullptr;         // MODE_RF
  void* spike = nullptr;
  uint32_t* packed = nullptr;
  void* vpost = nullptr;
  float* ckpt = nullptr;
  float* vlast = nullptr;
  long long T = 0, cols = 0;
  int mode = MODE_U;
  int tile = 8;  // C
  int residual_compiled = 0;  // MODE_ROWRES, bf16 frames: rounding of the residual (NSB_RESIDUAL_*)
  const uint16_t* pat_in = nullptr;  // MODE_ROWPAT: optional [T/16, cols] patterns to add
  uint16_t* pat_out = nullptr;       // MODE_ROWPAT: [T/16, cols] patterns out
  int frame_dtype = NSB_F32;         // MODE_ROWPAT: the frame dtype whose residual roundings apply
  float* split_scratch = nullptr;    // optional: nsb_time_split_scratch_floats(cols) floats; enables the time split
  cudaStream_t stream = nullptr;
};

struct BwdArgs {
  const void* beta = nullptr;
  const void* drive = nullptr;
  const void* gain = nullptr;
  const void* vth = nullptr;
  const void* extra = nullptr;  // MODE_RFMOD: raw_omega
  const float* bias[4] = {nullptr, nullptr, nullptr, nullptr};
  long long channels = 0;
  float v_th_min = 0.0f;
  void* g_extra = nullptr;                                 // MODE_RFMOD: grad raw_omega
  float* g_bias[4] = {nullptr, nullptr, nullptr, nullptr};  // modulated modes: per-column sums over time ([cols])
  const float* beta_row = nullptr;
  const float* vth_row = nullptr;
  const float* ckpt = nullptr;
  const float* ckpt_w = nullptr;  // MODE_RF
  float* g_winit = nullptr;       // MODE_RF
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
  const float* alpha_dev = nullptr;  // when set, the surrogate slope is read from device memory
  float* split_scratch = nullptr;    // optional: nsb_time_split_scratch_floats(cols) floats; enables the time split
  unsigned int* chain_sync = nullptr;  // optional: chain_scratch_words(cols) words; enables chained chunks (backward)
  cudaStream_t stream = nullptr;
};

// Per-dtype front doors (one translation unit each, to keep compile time flat).
int scan_fwd_f32(const FwdArgs& a);
int scan_fwd_bf16(const FwdArgs& a);
int scan_fwd_f16(const FwdArgs& a);
int scan_bwd_f32(const BwdArgs& a);
int scan_bwd_bf16(const BwdArgs& a);
int scan_bwd_f16(const BwdArgs& a);
// The modulated modes (MODE_MOD, MODE_RFMOD) are instantiated in their own translation units.
int scan_mod_fwd_f32(const FwdArgs& a);
int scan_mod_fwd_bf16(const FwdArgs& a);
int scan_mod_fwd_f16(const FwdArgs& a);
int scan_pat_fwd_f32(const FwdArgs& a);  // MODE_ROWPAT, same translation units
int scan_pat_fwd_bf16(const FwdArgs& a);
int scan_pat_fwd_f16(const FwdArgs& a);
int scan_res_fwd_f32(const FwdArgs& a);  // MODE_ROWRES, same translation units
int scan_res_fwd_bf16(const FwdArgs& a);
int scan_res_fwd_f16(const FwdArgs& a);
int scan_lin_fwd_f32(const FwdArgs& a);  // MODE_LIN, same translation units as the modulated modes
int scan_lin_fwd_bf16(const FwdArgs& a);
int scan_lin_fwd_f16(const FwdArgs& a);
int scan_lin_bwd_f32(const BwdArgs& a);
int scan_lin_bwd_bf16(const BwdArgs& a);
int scan_lin_bwd_f16(const BwdArgs& a);
int scan_mod_bwd_f32(const BwdArgs& a);
int scan_mod_bwd_bf16(const BwdArgs& a);
int scan_mod_bwd_f16(const BwdArgs& a);

// ----------------------------------------------------------------- launch plan

// What the planner needs to know about one scan launch.
struct PlanQuery {
  long long T = 0, cols = 0;
  int elem_size = 2;   // bytes per streamed element
  int nstreams = 4;    // TMA-loaded [T, cols] streams per stage
  int tile = 8;        // steps per tile (C)
  bool backward = false;
  int max_lanes = 4;   // largest lanes-per-thread the kernel family is built for
  int stash = 0;       // fp32 values per element of a tile that each warp keeps in shared memory
  int stash_2lanes = -1;  // the same when a thread owns 2 lanes, where that differs (-1: it does not)
  int modulated = 0;   // 0 plain scan, 1 first-order modulation fused in, 2 resonate-and-fire modulation
};

struct Plan {
  int lanes = 2;  // V: columns per thread; a warp owns 32*V columns
  int wpc = 1, stages = 2, grid = 0;
  size_t smem = 0;
  double cost = 0.0;  // model cost in "warp-times", lower is better
};

// Chooses lanes per thread, warps per CTA and ring depth. Pure host arithmetic
// (no CUDA calls), so it can be unit-tested without a GPU.
Plan plan_scan(const DeviceInfo& dev, const PlanQuery& q, const Tuning& tune);

// Time split of a forward scan over few columns (nseg == 1: none). Host arithmetic (nsb_plan.cu).
struct TimeSplit {
  int nseg = 1, seg_tiles = 0, warm_tiles = 0;
  int allow_rescans = 0;  // segments one warp may have to rescan before the split costs more than it saves
};
// family: 0 = row-parameter scans (split wherever the model below says it pays); 1 = scans with per-step
// parameters, 2 = those with the modulation fused in (split only on request: nsb_set_time_split with a
// segment count above 1)
TimeSplit plan_time_split(const DeviceInfo& dev, long long T, long long cols, int tile, int lanes, int wpc,
                          bool backward, int family);
TimeSplit& last_time_split();  // of the calling thread's last forward launch
// Warps that take the tiles of a column group in turn in a forward scan with the modulation fused in over
// few columns (1 = none). Host arithmetic (nsb_plan.cu).
int plan_rotation(const DeviceInfo& dev, long long column_warps, int ntiles);
bool get_rotation_forced();  // a count set through nsb_set_scan_rotation is used whether or not all CTAs fit
int& last_rotation();  // of the calling thread's last forward launch
// What earlier split launches of one neuron had to rescan, fed back into the automatic choice. `neuron`
// is any pointer that names the call site (the per-row parameter vector). _allows: false while that
// neuron's dynamics forget too slowly for the split to pay. _record: queues the copy of the launch's two
// counter words {segments rescanned, most by one warp} to the host.
bool time_split_automatic();
bool split_feedback_allows(const void* neuron, long long T, long long cols, bool backward);
void split_feedback_record(const void* neuron, long long T, long long cols, bool backward,
                           const unsigned int* dev_words, int allow_rescans, cudaStream_t stream);
// floats of scratch a time-split launch over `cols` columns may need (boundary states + a counter)
long long time_split_scratch_floats(long long cols);

// Chained chunks of a backward launch of `grid` CTAs of which `slots` fit on the GPU at once: the number of
// chunks of the time axis (1 = none). Host arithmetic (nsb_plan.cu).
int plan_chain_chunks(bool eligible, int ntiles, int target_tiles);
void set_last_chain_chunks(int q);
int last_chain_chunks();  // of the process's last backward launch
long long chain_scratch_words(long long cols);

// Device description of a B200 for planning when no GPU is present.
DeviceInfo b200_device_info();

#ifdef __CUDACC__

// ------------------------------------------------------- per-thread vector I/O

// Moves the V consecutive elements a thread owns with one instruction and
// converts them to / from fp32 (widening is exact, narrowing rounds to nearest
// even; two 16-bit values are converted per instruction).
template <typename ST, int V>
struct VecIO {
  __device__ static __forceinline__ void load(const ST* p, float (&out)[V]) {
    const Vec<ST, V> t = *reinterpret_cast<const Vec<ST, V>*>(p);
    if constexpr (sizeof(ST) == 2 && V % 2 == 0) {
      const uint32_t* w = reinterpret_cast<const uint32_t*>(&t);
#pragma unroll
      for (int i = 0; i < V / 2; ++i) {
        if constexpr (Elem<ST>::kDtype == NSB_BF16) {
          out[2 * i] = __uint_as_float(w[i] << 16);
          out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        } else {
          const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
          out[2 * i] = f.x;
          out[2 * i + 1] = f.y;
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < V; ++j) out[j] = Elem<ST>::to_f32(t.v[j]);
    }
  }
  __device__ static __forceinline__ void store(ST* p, const float (&in)[V]) {
    Vec<ST, V> t;
    if constexpr (sizeof(ST) == 2 && V % 2 == 0) {
      uint32_t* w = reinterpret_cast<uint32_t*>(&t);
#pragma unroll
      for (int i = 0; i < V / 2; ++i) {
        if constexpr (Elem<ST>::kDtype == NSB_BF16) {
          const __nv_bfloat162 h = __floats2bfloat162_rn(in[2 * i], in[2 * i + 1]);
          w[i] = *reinterpret_cast<const uint32_t*>(&h);
        } else {
          const __half2 h = __floats2half2_rn(in[2 * i], in[2 * i + 1]);
          w[i] = *reinterpret_cast<const uint32_t*>(&h);
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < V; ++j) t.v[j] = Elem<ST>::from_f32(in[j]);
    }
    *reinterpret_cast<Vec<ST, V>*>(p) = t;
  }
  // {0,1} spikes in the stream dtype
  __device__ static __forceinline__ void store_spikes(ST* p, const bool (&s)[V]) {
    Vec<ST, V> t;
    if constexpr (sizeof(ST) == 2 && V % 2 == 0) {
      constexpr uint32_t one = Elem<ST>::kDtype == NSB_BF16 ? 0x3F80u : 0x3C00u;
      uint32_t* w = reinterpret_cast<uint32_t*>(&t);
#pragma unroll
      for (int i = 0; i < V / 2; ++i) w[i] = (s[2 * i] ? one : 0u) | (s[2 * i + 1] ? (one << 16) : 0u);
    } else {
#pragma unroll
      for (int j = 0; j < V; ++j) t.v[j] = s[j] ? Elem<ST>::one() : Elem<ST>::zero();
    }
    *reinterpret_cast<Vec<ST, V>*>(p) = t;
  }
};

// One fp32 value kept in the four bytes of the two 16-bit elements a thread owns in a staged tile
// (a slot whose input has been consumed and whose output is not written yet). The access has the
// type VecIO uses on the same address, so the compiler orders it with those loads and stores.
template <typename ST>
__device__ __forceinline__ void slot_put(ST* p, float x) {
  static_assert(sizeof(ST) == 2, "a slot is two 16-bit elements");
  Vec<ST, 2> t;
  *reinterpret_cast<uint32_t*>(&t) = __float_as_uint(x);
  *reinterpret_cast<Vec<ST, 2>*>(p) = t;
}
template <typename ST>
__device__ __forceinline__ float slot_get(const ST* p) {
  static_assert(sizeof(ST) == 2, "a slot is two 16-bit elements");
  const Vec<ST, 2> t = *reinterpret_cast<const Vec<ST, 2>*>(p);
  return __uint_as_float(*reinterpret_cast<const uint32_t*>(&t));
}

// Lane-wise fp32 arithmetic on the V values of a thread.
//
// NSB_X2=1 routes pairs through the packed two-wide fp32 instructions of sm_100
// (mul/add/fma .f32x2). It is OFF by default: measured on B200 with CUDA 12.9, a
// packed multiply followed by a packed add is contracted into a packed fused
// multiply-add even when both carry an explicit .rn (as CUDA intrinsics and as
// inline PTX alike), which changes the last bit of the membrane state in ~30 % of
// the elements and so breaks bit-exact parity with an eager fp32 time loop. The
// scalar __fmul_rn / __fadd_rn forms are never contracted. (Writing the add as
// fma.rn.f32x2(a, one, b) is contracted too when `one` is the literal 1.0; with a 1.0 the
// assembler cannot see - a __constant__ the host could rewrite - the packed form is bit-exact,
// all parity tests pass, and it is no faster than the scalar one: resonate-and-fire with
// modulation, forward 3.94 against 4.00 ms, backward 7.90 against 7.80 ms. The contracted,
// inexact form would run 7.23 ms: what it saves is the add, not the issue slot.)
#ifndef NSB_X2
#define NSB_X2 0
#endif

__device__ __forceinline__ unsigned long long pack_f2(float lo, float hi) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack_f2(unsigned long long p, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(p));
}

template <int V>
__device__ __forceinline__ void vmul(float (&r)[V], const float (&a)[V], const float (&b)[V]) {
  if constexpr (NSB_X2 && V % 2 == 0) {
#pragma unroll
    for (int i = 0; i < V / 2; ++i) {
      unsigned long long t;
      asm("mul.rn.f32x2 %0, %1, %2;"
          : "=l"(t)
          : "l"(pack_f2(a[2 * i], a[2 * i + 1])), "l"(pack_f2(b[2 * i], b[2 * i + 1])));
      unpack_f2(t, r[2 * i], r[2 * i + 1]);
    }
  } else {
#pragma unroll
    for (int j = 0; j < V; ++j) r[j] = __fmul_rn(a[j], b[j]);
  }
}
template <int V>
__device__ __forceinline__ void vmuls(float (&r)[V], const float (&a)[V], float s) {
  float b[V];
#pragma unroll
  for (int j = 0; j < V; ++j) b[j] = s;
  vmul<V>(r, a, b);
}
template <int V>
__device__ __forceinline__ void vadd(float (&r)[V], const float (&a)[V], const float (&b)[V]) {
  if constexpr (NSB_X2 && V % 2 == 0) {
#pragma unroll
    for (int i = 0; i < V / 2; ++i) {
      unsigned long long t;
      asm("add.rn.f32x2 %0, %1, %2;"
          : "=l"(t)
          : "l"(pack_f2(a[2 * i], a[2 * i + 1])), "l"(pack_f2(b[2 * i], b[2 * i + 1])));
      unpack_f2(t, r[2 * i], r[2 * i + 1]);
    }
  } else {
#pragma unroll
    for (int j = 0; j < V; ++j) r[j] = __fadd_rn(a[j], b[j]);
  }
}
template <int V>
__device__ __forceinline__ void vsub(float (&r)[V], const float (&a)[V], const float (&b)[V]) {
  float nb[V];
#pragma unroll
  for (int j = 0; j < V; ++j) nb[j] = -b[j];
  vadd<V>(r, a, nb);
}
template <int V>
__device__ __forceinline__ void vfma(float (&r)[V], const float (&a)[V], const float (&b)[V],
                                     const float (&c)[V]) {
  if constexpr (NSB_X2 && V % 2 == 0) {
#pragma unroll
    for (int i = 0; i < V / 2; ++i) {
      unsigned long long t;
      asm("fma.rn.f32x2 %0, %1, %2, %3;"
          : "=l"(t)
          : "l"(pack_f2(a[2 * i], a[2 * i + 1])), "l"(pack_f2(b[2 * i], b[2 * i + 1])),
            "l"(pack_f2(c[2 * i], c[2 * i + 1])));
      unpack_f2(t, r[2 * i], r[2 * i + 1]);
    }
  } else {
#pragma unroll
    for (int j = 0; j < V; ++j) r[j] = fmaf(a[j], b[j], c[j]);
  }
}

// ------------------------------------------------------------------- forward

struct FwdParams {
  const void* s[5];  // stream base pointers (direct path), order as in smem
  const float* bias[4];  // modulated modes: b_beta, b_alpha, b_th, b_omega
  long long channels;
  float v_th_min;
  double* u_stats;  // modulated modes, optional: per-warp (sum, sum of squares) of u
  const float* beta_row;
  const float* vth_row;
  const float* v_init;
  const float* w_init;
  void* spike;
  uint32_t* packed;
  void* vpost;
  void* w_out;
  float* ckpt;
  float* ckpt_w;
  float* vlast;
  float* wlast;
  long long T, cols, words_per_row;
  int ntiles, stages;
  int defer;  // 1: a stage is refilled one tile after its outputs were handed to TMA
  uint32_t* err;
  unsigned long long wait_ns;  // limit of the bounded barrier waits
  int residual_compiled;
  const uint16_t* pat_in;
  uint16_t* pat_out;
  int frame_dtype;
  // Time split (few columns): nseg > 1 cuts the scan into nseg segments of seg_tiles tiles that
  // run side by side (grid.y); a segment after the first starts warm_tiles tiles early from V = 0
  // and keeps only what it computes from its own start on. vspec / vend are [nseg, cols]: the
  // state a segment reached at its own start, and at its end. fixup = 1 is the second launch,
  // which checks every vspec against the exact state and redoes the segments that differ.
  int nseg, seg_tiles, warm_tiles, fixup;
  float* vspec;
  float* vend;
  float* wspec;  // the same for the second state of the resonate-and-fire scans
  float* wend;
  unsigned int* fix_count;
  // Rotation (few columns, modulation fused in): rot > 1 warps of a CTA own the same 32*V columns and take
  // the tiles in turn; the membrane state goes from warp to warp through shared memory (see plif_fwd_body).
  int rot;
};

template <int MODE_>
struct ModeTraits {
  static constexpr bool kStats = MODE_ == MODE_MODS || MODE_ == MODE_RFMODS;
  static constexpr int MODE = MODE_ == MODE_MODS ? MODE_MOD : (MODE_ == MODE_RFMODS ? MODE_RFMOD : MODE_);
  static constexpr bool kSecond = MODE == MODE_RF || MODE == MODE_RFMOD;  // carries the second state W
  static constexpr bool kMod = MODE == MODE_MOD || MODE == MODE_RFMOD;    // modulation fused into the loads
  static constexpr bool kRow = MODE == MODE_ROW || MODE == MODE_ROWRES || MODE == MODE_ROWPAT;  // per-column beta / v_th
  static constexpr int kFwdStreams =
      (MODE == MODE_ROW || MODE == MODE_ROWPAT) ? 1 : ((MODE == MODE_ROWRES || MODE == MODE_LIN) ? 2 : (MODE == MODE_RFMOD ? 5 : ((MODE == MODE_AI || MODE == MODE_RF || MODE == MODE_MOD) ? 4 : 3)));
  // index of each role inside the stage / pointer table (roles that a mode
  // does not stream alias slot 0 and are never read)
  static constexpr int kBeta = 0;
  static constexpr int kDrive = kRow ? 0 : 1;
  static constexpr int kRes = 1;  // MODE_ROWRES: the frames added to the scan's spikes
  static constexpr int kGain = kFwdStreams >= 4 ? 2 : 0;
  static constexpr int kVth = (kRow || MODE == MODE_LIN) ? 0 : (kFwdStreams >= 4 ? 3 : 2);
  static constexpr int kOmega = MODE == MODE_RFMOD ? 4 : (MODE == MODE_RF ? 2 : 0);
};

// One charge / fire / soft-reset step on the V lanes of a thread:
//   v_pre = beta*v + drive (multiply and add rounded separately),
//   x = v_pre - v_th, spike = v_pre >= v_th, v = spike ? x : v_pre.
template <int V>
__device__ __forceinline__ void plif_step(float (&v)[V], const float (&beta)[V], const float (&drive)[V],
                                          const float (&vth)[V], float (&x)[V], bool (&s)[V]) {
  float bv[V], vpre[V];
  vmul<V>(bv, beta, v);
  vadd<V>(vpre, bv, drive);
  vsub<V>(x, vpre, vth);
#pragma unroll
  for (int j = 0; j < V; ++j) {
    s[j] = vpre[j] >= vth[j];
    v[j] = s[j] ? x[j] : vpre[j];
  }
}

// Moves bit m of the low 32/V bits of x to bit V*m (V = 1, 2 or 4).
template <int V>
__device__ __forceinline__ uint32_t spread_bits(uint32_t x) {
  if constexpr (V == 2) {
    x &= 0xFFFFu;
    x = (x | (x << 8)) & 0x00FF00FFu;
    x = (x | (x << 4)) & 0x0F0F0F0Fu;
    x = (x | (x << 2)) & 0x33333333u;
    x = (x | (x << 1)) & 0x55555555u;
  } else if constexpr (V == 4) {
    x &= 0xFFu;
    x = (x | (x << 12)) & 0x000F000Fu;
    x = (x | (x << 6)) & 0x03030303u;
    x = (x | (x << 3)) & 0x11111111u;
  }
  return x;
}

// Resonate-and-fire step: v_pre = (beta*v - omega*w) + u, w' = omega*v + beta*w, every
// product and sum rounded separately; only V is reset.
template <int V>
__device__ __forceinline__ void rf_step(float (&v)[V], float (&w)[V], const float (&beta)[V],
                                        const float (&omega)[V], const float (&u)[V], const float (&vth)[V],
                                        float (&x)[V], bool (&s)[V]) {
  float bv[V], ow[V], d[V], vpre[V], ov[V], bw[V], wn[V];
  vmul<V>(bv, beta, v);
  vmul<V>(ow, omega, w);
  vsub<V>(d, bv, ow);
  vadd<V>(vpre, d, u);
  vmul<V>(ov, omega, v);
  vmul<V>(bw, beta, w);
  vadd<V>(wn, ov, bw);
  vsub<V>(x, vpre, vth);
#pragma unroll
  for (int j = 0; j < V; ++j) {
    s[j] = vpre[j] >= vth[j];
    v[j] = s[j] ? x[j] : vpre[j];
    w[j] = wn[j];
  }
}

// The forward scan. A device function so that it can sit behind two kernel entry points: one
// without a register limit (ptxas' own choice; giving it an explicit 255 made it spend 30-100 more
// registers on every variant), one held to 160 registers.
template <typename ST, int MODE, bool PACKED, int V, int C, bool TMA, bool SPLIT = false, bool ROT = false>
__device__ __forceinline__ void plif_fwd_body(const FwdParams& p, const CUtensorMap& tm0, const CUtensorMap& tm1,
                                              const CUtensorMap& tm2, const CUtensorMap& tm3,
                                              const CUtensorMap& tm4, const CUtensorMap& tm_spike) {
  using MT = ModeTraits<MODE>;
  using E = Elem<ST>;
  using IO = VecIO<ST, V>;
  constexpr int NS = MT::kFwdStreams;
  constexpr int TILE_ELEMS = C * 32 * V;
  constexpr uint32_t TILE_BYTES = TILE_ELEMS * sizeof(ST);
  constexpr uint32_t STAGE_BYTES = NS * TILE_BYTES;
  constexpr bool VEC = TMA;  // a thread's V columns are contiguous and aligned
  // Dense spikes leave through shared memory + TMA only in the kernels built for them; a
  // bit-packing kernel that is also asked for dense spikes writes them from registers.
  constexpr bool DENSE_TMA = VEC && !PACKED;
  // MODE_ROWPAT is built with PACKED = true (no dense output path) but packs in time, not by ballot
  constexpr bool BALLOT = PACKED && MODE != MODE_ROWPAT;
  // Bit packing: a 32-column word belongs to the 32/V lanes that own those columns.
  constexpr int G = 32 / V;
  constexpr int NSLOT = (C + G - 1) / G;
  extern __shared__ __align__(128) uint8_t smem_raw[];

  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int wpc = blockDim.x >> 5;
  // ---- rotation. The modulation of a tile (two thirds of a modulated scan's instructions) depends on
  // nothing but the tile's inputs; only the few instructions of the recurrence itself form the serial
  // chain over T. With few columns there are too few warps to fill the issue slots (2.5 per scheduler at
  // 49 152 columns), so R warps share a column group: warp r takes tiles r, r+R, r+2R, ..., evaluates a
  // tile's modulation, THEN waits for the state its predecessor left after the tile before, runs the tile's
  // steps, and hands the state on - through 2*32*V floats of shared memory and one counter per warp, which
  // its predecessor advances each time it has a state for it (bounded wait like every other). Arithmetic
  // and its order per column are those of the one-warp scan: the results are the same bits.
  static_assert(!ROT || (!SPLIT && TMA && !ModeTraits<MODE>::kStats), "rotation: tiled copies, no time split, no moments");
  const int R = ROT ? p.rot : 1;
  const int rw = ROT ? warp % R : 0;
  const long long col0 = ROT ? ((long long)blockIdx.x * (wpc / R) + warp / R) * (32 * V)
                             : ((long long)blockIdx.x * wpc + warp) * (32 * V);
  uint32_t hbar_mine = 0, hbar_next = 0;  // rotation: this warp's counter of states received and its successor's,
  volatile uint32_t* hfail = nullptr;      // the group's give-up flag,
  float* hstate = nullptr;                 // and the state in transit: V then W, 32*V floats each
  if constexpr (ROT) {
    constexpr uint32_t kHandHeader = 48u;  // up to 4 counters (8 bytes apart), the flag
    const uint32_t base = smem_u32(smem_raw);
    const uint32_t data_base = (base + (uint32_t)(wpc * p.stages) * 8u + 127u) & ~127u;
    const uint32_t hand = data_base + (uint32_t)(wpc * p.stages) * STAGE_BYTES +
                          (uint32_t)(warp / R) * (kHandHeader + 8u * 32u * V);
    hbar_mine = hand + 8u * (uint32_t)rw;
    hbar_next = hand + 8u * (uint32_t)((rw + 1) % R);
    hfail = reinterpret_cast<volatile uint32_t*>(smem_raw + (hand + 32u - base));
    hstate = reinterpret_cast<float*>(smem_raw + (hand + kHandHeader - base));
    if (lane == 0) {
      smem_flag_publish(hbar_mine, 0u);
      if (rw == 0) *hfail = 0u;
    }
    __syncthreads();  // (before any warp leaves: every thread of the CTA takes part)
  }
  if (col0 >= p.cols) return;

  long long colj[V];
  bool valid[V];
  float v[V], w[V], brow[V], trow[V];
#pragma unroll
  for (int j = 0; j < V; ++j) {
    colj[j] = col0 + V * lane + j;
    valid[j] = colj[j] < p.cols;
    v[j] = valid[j] ? p.v_init[colj[j]] : 0.0f;
    w[j] = (MT::kSecond && valid[j]) ? p.w_init[colj[j]] : 0.0f;
    brow[j] = 0.0f;
    trow[j] = 0.0f;
    if (MT::kRow && valid[j]) {
      brow[j] = p.beta_row[colj[j]];
      trow[j] = p.vth_row[colj[j]];
    }
  }
  mod::Bias<V> bias = {};
  if constexpr (MT::kMod) {
#pragma unroll
    for (int j = 0; j < V; ++j) {
      if (valid[j]) {
        const long long ch = colj[j] % p.channels;
        bias.beta[j] = p.bias[0][ch];
        bias.alpha[j] = p.bias[1][ch];
        bias.th[j] = p.bias[2][ch];
        if (MT::kSecond) bias.omega[j] = p.bias[3][ch];
      }
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
      if (NS > 4) tma_load_2d(dst + 4 * TILE_BYTES, &tm4, (int)col0, tile * C, bar);
    }
  };

  const int ntiles_total = p.ntiles;

  // The direct path stages KB steps of every stream in registers at a time.
  constexpr int KB = TMA ? C : 8;
  const ST* sp = nullptr;  // this thread's first element inside the current stage
  ST regs[TMA ? 1 : NS * KB * V] = {};
  auto fetch = [&](int stream, int k, float (&out)[V]) {
    if constexpr (VEC) {
      IO::load(sp + stream * TILE_ELEMS + k * (32 * V), out);
    } else {
#pragma unroll
      for (int j = 0; j < V; ++j) out[j] = E::to_f32(regs[(stream * KB + (k % KB)) * V + j]);
    }
  };

  const long long row_elems = p.cols;
  long long t0 = 0;
  int s_idx = 0;
  uint32_t phase = 0;
  bool failed = false;

  // Outputs that leave through per-step global stores (V_post, W, and dense spikes of a
  // bit-packing kernel). When a call asks for none of them the step loop is compiled
  // without their address arithmetic and predicated stores (they were ~40 % of the
  // instructions of a step, which is what bounds a launch with one warp per SM).
  double st_s = 0.0, st_q = 0.0;  // modulated modes: this thread's moments of u
  const bool any_direct = p.vpost != nullptr || (MT::kSecond && p.w_out != nullptr) ||
                          (!DENSE_TMA && p.spike != nullptr);

  // MODE_ROWPAT with a residual: the patterns to add to the tokens of the current tile and of the
  // next one. They come straight from global memory (2 bytes per token and column), requested a
  // whole tile ahead so that the serial scan never waits for them.
  constexpr int TOK = (MODE == MODE_ROWPAT) ? (C / 16 > 0 ? C / 16 : 1) : 1;
  Vec<uint16_t, V> pin_cur[TOK] = {}, pin_nxt[TOK] = {};
  auto load_patterns = [&](int tile_idx, Vec<uint16_t, V> (&dst)[TOK]) {
    if constexpr (MODE == MODE_ROWPAT) {
#pragma unroll
      for (int q = 0; q < TOK; ++q) {
        const long long tok = (long long)tile_idx * TOK + q;
        if (tok * 16 >= p.T) break;
        if constexpr (VEC) {
          if (valid[0]) dst[q] = *reinterpret_cast<const Vec<uint16_t, V>*>(p.pat_in + tok * row_elems + colj[0]);
        } else {
#pragma unroll
          for (int j = 0; j < V; ++j)
            if (valid[j]) dst[q].v[j] = p.pat_in[tok * row_elems + colj[j]];
        }
      }
    }
  };

  // Rotation: what happens between a tile's modulation and its first step (state_in, called from inside
  // the tile), and after its last step (state_out).
  int cur_tile = 0;               // absolute index of the tile in hand
  uint32_t cur_handoff = 0, sent = 0;  // states this warp has received / handed on
  bool rot_failed = false;
  auto state_in = [&]() {
    if constexpr (ROT) {
      if (cur_tile > 0) {
        bool ok = smem_flag_wait_bounded(hbar_mine, ++cur_handoff, p.err, 1u, p.wait_ns);
        ok = ok && *hfail == 0u;  // (a predecessor that gave up still advances the counter, with the flag set)
        if (!__all_sync(0xffffffffu, ok)) {
          rot_failed = true;  // this tile's results are wasted; the loop ends after it
        } else {
#pragma unroll
          for (int j = 0; j < V; ++j) {
            v[j] = hstate[V * lane + j];
            if (MT::kSecond) w[j] = hstate[32 * V + V * lane + j];
          }
        }
      }
      if (p.ckpt && valid[0]) {
        VecIO<float, V>::store(p.ckpt + (long long)cur_tile * row_elems + colj[0], v);
        if (MT::kSecond) VecIO<float, V>::store(p.ckpt_w + (long long)cur_tile * row_elems + colj[0], w);
      }
    }
  };
  auto state_out = [&](bool gave_up) {
    if constexpr (ROT) {
      if (gave_up) {
        *hfail = 1u;
      } else {
#pragma unroll
        for (int j = 0; j < V; ++j) {
          hstate[V * lane + j] = v[j];
          if (MT::kSecond) hstate[32 * V + V * lane + j] = w[j];
        }
      }
      __syncwarp();
      ++sent;
      if (lane == 0) smem_flag_publish(hbar_next, gave_up ? 0x7fffffffu : sent);
    }
  };

  // emit_tag = false: a warm-up tile of a time-split scan; the state advances, nothing is written
  auto tile = [&](auto full_tag, auto direct_tag, auto emit_tag, int nsteps) {
    constexpr bool FULL = decltype(full_tag)::value;
    constexpr bool EMIT = decltype(emit_tag)::value;
    constexpr bool DIRECT = decltype(direct_tag)::value && EMIT;
    constexpr bool STATS = MT::kStats;  // accumulate the moments of u
    // On the vector path dense spikes are written over the consumed drive tile in
    // shared memory and leave through one TMA store per tile (which also clips the
    // ragged edges), so the step loop carries no global address arithmetic for them.
    ST* o_spike = (DIRECT && !DENSE_TMA && MODE != MODE_ROWRES && p.spike)
                      ? static_cast<ST*>(p.spike) + t0 * row_elems + colj[0] : nullptr;
    uint32_t hb[V];  // MODE_ROWRES / MODE_ROWPAT: the spikes of the current token as a half bit pattern
#pragma unroll
    for (int j = 0; j < V; ++j) hb[j] = 0u;
    ST* o_vpost = (DIRECT && p.vpost) ? static_cast<ST*>(p.vpost) + t0 * row_elems + colj[0] : nullptr;
    ST* o_wout = (DIRECT && MT::kSecond && p.w_out) ? static_cast<ST*>(p.w_out) + t0 * row_elems + colj[0] : nullptr;
    uint32_t keep[NSLOT][V];  // raw ballots of the step(s) this lane is responsible for
    // modulated modes: steps whose modulation is evaluated together, and its results
    constexpr int CH = (MT::kMod && TMA) ? ((16 / V) < C ? (16 / V) : C) : 1;
    float mb[CH][V], mu[CH][V], mth[CH][V], mom[CH][V];
#pragma unroll
    for (int q = 0; q < NSLOT; ++q)
#pragma unroll
      for (int j = 0; j < V; ++j) keep[q][j] = 0u;
#pragma unroll
    for (int k = 0; k < C; ++k) {
      if (!FULL && k >= nsteps) break;
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
                    (k + kk < nsteps && valid[j]) ? g[(t0 + k + kk) * row_elems + colj[j]] : E::zero();
          }
        }
      }
      float b[V], th[V], dr[V], om[V], x[V];
      bool sp_[V];
      fetch(MT::kDrive, k, dr);
      if constexpr (MT::kRow) {
#pragma unroll
        for (int j = 0; j < V; ++j) {
          b[j] = brow[j];
          th[j] = trow[j];
        }
      } else if constexpr (MODE == MODE_LIN) {
        fetch(MT::kBeta, k, b);
#pragma unroll
        for (int j = 0; j < V; ++j) th[j] = __int_as_float(0x7f800000);  // +inf: never fires
      } else {
        fetch(MT::kBeta, k, b);
        fetch(MT::kVth, k, th);
      }
      if constexpr (MODE == MODE_AI) {
        float gn[V];
        fetch(MT::kGain, k, gn);
        vmul<V>(dr, gn, dr);
      }
      if constexpr (MT::kSecond) fetch(MT::kOmega, k, om);
      if constexpr (MT::kMod) {
        // Modulated modes: the raw projections of CH steps are turned into beta, u, v_th, omega
        // together, ahead of the steps that use them. The modulation is long chains of dependent
        // arithmetic with no dependence between steps; evaluated step by step, in between the
        // serial scan, a warp stalls on every link (measured: 1.6 wait + 1.1 scoreboard cycles
        // per instruction). CH steps at once give the scheduler CH*V independent chains.
        if (k % CH == 0) {
          float cs = 0.0f, cq = 0.0f;
#pragma unroll
          for (int kk = 0; kk < CH; ++kk) {
            // One lane per thread: two consecutive steps of the column go through the packed fp32x2
            // instructions together (the same bits as one at a time, see nsb_modulation.cuh; 49 152 columns,
            // same box: resonate-and-fire 1.41 -> 1.38 ms, first order 0.92 -> 0.91 ms).
            constexpr bool kTimePairs = V == 1 && CH % 2 == 0;
            if constexpr (kTimePairs) {
              if (kk % 2 == 0 && k + kk + 1 < C && (FULL || k + kk + 1 < nsteps)) {
                float rb[2], ra[2], rt[2], ro[2] = {0.0f, 0.0f}, cu[2], t1[V];
                float q0[2], q1[2], q2[2], q3[2], q4[2], be[2], uu[2], tt[2], oo[2];
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                  fetch(MT::kBeta, k + kk + e, t1); rb[e] = t1[0];
                  fetch(MT::kGain, k + kk + e, t1); ra[e] = t1[0];
                  fetch(MT::kVth, k + kk + e, t1); rt[e] = t1[0];
                  fetch(MT::kDrive, k + kk + e, t1); cu[e] = t1[0];
                  if constexpr (MT::kSecond) { fetch(MT::kOmega, k + kk + e, t1); ro[e] = t1[0]; }
                }
                const float bb[2] = {bias.beta[0], bias.beta[0]}, ba[2] = {bias.alpha[0], bias.alpha[0]};
                const float bt[2] = {bias.th[0], bias.th[0]}, bo[2] = {bias.omega[0], bias.omega[0]};
                mod::forward_full<MT::kSecond, 2>(rb, ra, rt, ro, cu, bb, ba, bt, bo, p.v_th_min, be, uu, tt, oo, q0,
                                                  q1, q2, q3, q4);
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                  mb[kk + e][0] = be[e];
                  mu[kk + e][0] = uu[e];
                  mth[kk + e][0] = tt[e];
                  mom[kk + e][0] = oo[e];
                  if constexpr (STATS) {
                    const float uj = valid[0] ? uu[e] : 0.0f;
                    cs += uj;
                    cq = fmaf(uj, uj, cq);
                  }
                }
                continue;
              }
              if (kk % 2 == 1 && (FULL || k + kk < nsteps)) continue;  // done with its partner
            }
            if (k + kk < C && (FULL || k + kk < nsteps)) {
              float ra[V], q0[V], q1[V], q2[V], q3[V], q4[V];
              fetch(MT::kBeta, k + kk, mb[kk]);
              fetch(MT::kVth, k + kk, mth[kk]);
              fetch(MT::kDrive, k + kk, mu[kk]);
              fetch(MT::kGain, k + kk, ra);
              if constexpr (MT::kSecond) fetch(MT::kOmega, k + kk, mom[kk]);
              mod::forward_lanes<MT::kSecond, V>(mb[kk], ra, mth[kk], mom[kk], mu[kk], bias, p.v_th_min, q0, q1,
                                                 q2, q3, q4);
              // moments of u (for the adaptive surrogate slope): fp32 within the chunk, double across
              // chunks (only in the kernels built for it).
              if constexpr (STATS) {
#pragma unroll
                for (int j = 0; j < V; ++j) {
                  const float uj = valid[j] ? mu[kk][j] : 0.0f;
                  cs += uj;
                  cq = fmaf(uj, uj, cq);
                }
              }
            }
          }
          if constexpr (STATS) {
            st_s += (double)cs;
            st_q += (double)cq;
          }
        }
#pragma unroll
        for (int j = 0; j < V; ++j) {
          b[j] = mb[k % CH][j];
          th[j] = mth[k % CH][j];
          dr[j] = mu[k % CH][j];
          om[j] = mom[k % CH][j];
        }
      }
      if constexpr (ROT) {
        if (k == 0) {
          // The tile's modulation has to be finished BEFORE the wait for the state, or nothing overlaps: left
          // to itself the compiler evaluates beta, u, v_th, omega of a step right before the step uses them,
          // i.e. after the wait (measured: 1.80 ms instead of 1.43 at 49 152 columns). Volatile statements
          // keep their order, so one that reads the values pins their evaluation in front of the wait.
          if constexpr (MT::kMod) {
#pragma unroll
            for (int kk = 0; kk < CH; ++kk)
              if (FULL || kk < nsteps) {
#pragma unroll
                for (int j = 0; j < V; ++j)
                  asm volatile("" ::"f"(mb[kk][j]), "f"(mu[kk][j]), "f"(mth[kk][j]), "f"(mom[kk][j]));
              }
          }
          state_in();  // now the state the tile starts from
        }
      }
      if constexpr (MT::kSecond) {
        rf_step<V>(v, w, b, om, dr, th, x, sp_);
      } else {
        plif_step<V>(v, b, dr, th, x, sp_);
      }

      if constexpr (MODE == MODE_ROWPAT) {
        // Step k is bit 15 - (k mod 16) of the token's half pattern; the patterns to add, if any,
        // were requested one tile ahead (pin_cur).
#pragma unroll
        for (int j = 0; j < V; ++j) hb[j] = (k % 16 == 0 ? 0u : hb[j]) | (sp_[j] ? (1u << (15 - k % 16)) : 0u);
        const long long tok_off = ((t0 + k) / 16) * row_elems;
        if (k % 16 == 15) {
          Vec<uint16_t, V> po;
#pragma unroll
          for (int j = 0; j < V; ++j) {
            uint32_t h = hb[j];
            if (p.pat_in)
              h = codec::residual_of_patterns(hb[j], pin_cur[k / 16].v[j], p.frame_dtype, p.residual_compiled != 0);
            po.v[j] = (uint16_t)h;
          }
          if constexpr (VEC) {
            if (valid[0] && EMIT) *reinterpret_cast<Vec<uint16_t, V>*>(p.pat_out + tok_off + colj[0]) = po;
          } else {
#pragma unroll
            for (int j = 0; j < V; ++j)
              if (valid[j] && EMIT) p.pat_out[tok_off + colj[j]] = po.v[j];
          }
        }
      }
      if constexpr (MODE == MODE_ROWRES) {
        // Step k is bit 15 - (k mod 16) of the token's half pattern (frame 0 = sign). After the
        // token's last step: decode it, add the value decoded from the 16 input frames, re-encode,
        // and write the 16 output frames over the token's (consumed) drive rows / to global memory.
#pragma unroll
        for (int j = 0; j < V; ++j) hb[j] = (k % 16 == 0 ? 0u : hb[j]) | (sp_[j] ? (1u << (15 - k % 16)) : 0u);
        if (k % 16 == 15) {
          const int k0 = k - 15;
          float fb[16][V];
          const ST* g_res = static_cast<const ST*>(p.s[MT::kRes]);
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            if constexpr (VEC) {
              IO::load(sp + MT::kRes * TILE_ELEMS + (k0 + i) * (32 * V), fb[i]);
            } else {
#pragma unroll
              for (int j = 0; j < V; ++j)
                fb[i][j] = valid[j] ? E::to_f32(g_res[(t0 + k0 + i) * row_elems + colj[j]]) : 0.0f;
            }
          }
          uint32_t h[V];
#pragma unroll
          for (int j = 0; j < V; ++j) {
            float b_[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) b_[i] = fb[i][j];
            h[j] = codec::residual_pattern_frames<E::kDtype>(hb[j], b_, p.residual_compiled != 0);
          }
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            bool ob[V];
#pragma unroll
            for (int j = 0; j < V; ++j) ob[j] = (h[j] >> (15 - i)) & 1u;
            if constexpr (VEC) {
              IO::store_spikes(const_cast<ST*>(sp) + MT::kDrive * TILE_ELEMS + (k0 + i) * (32 * V), ob);
            } else {
              ST* g_out = static_cast<ST*>(p.spike);
#pragma unroll
              for (int j = 0; j < V; ++j)
                if (valid[j] && EMIT) g_out[(t0 + k0 + i) * row_elems + colj[j]] = ob[j] ? E::one() : E::zero();
            }
          }
        }
      } else if constexpr (VEC) {
        if constexpr (DENSE_TMA && MODE == MODE_LIN)  // the dense output of the linear recurrence is V
          IO::store(const_cast<ST*>(sp) + MT::kDrive * TILE_ELEMS + k * (32 * V), v);
        else if constexpr (DENSE_TMA)
          IO::store_spikes(const_cast<ST*>(sp) + MT::kDrive * TILE_ELEMS + k * (32 * V), sp_);
        if constexpr (DIRECT) {
          // a thread's V columns are all valid or all invalid
          if (!DENSE_TMA && o_spike && valid[0]) IO::store_spikes(o_spike + (size_t)k * row_elems, sp_);
          if (o_vpost && valid[0]) IO::store(o_vpost + (size_t)k * row_elems, v);
          if (MT::kSecond && o_wout && valid[0]) IO::store(o_wout + (size_t)k * row_elems, w);
        }
      } else {
#pragma unroll
        for (int j = 0; j < V; ++j) {
          if (DIRECT && valid[j]) {
            const size_t off = (size_t)k * row_elems + (colj[j] - colj[0]);
            if (o_spike) o_spike[off] = MODE == MODE_LIN ? E::from_f32(v[j]) : (sp_[j] ? E::one() : E::zero());
            if (o_vpost) o_vpost[off] = E::from_f32(v[j]);
            if (MT::kSecond && o_wout) o_wout[off] = E::from_f32(w[j]);
          }
        }
      }
      if constexpr (BALLOT && EMIT) {
        // one ballot per lane slot j: bit l = spike of column col0 + V*l + j. Lane (k mod G) of
        // every group of G lanes keeps the V ballots of step k and interleaves them into the
        // word it stores once the tile is done.
#pragma unroll
        for (int j = 0; j < V; ++j) {
          const uint32_t b = __ballot_sync(0xffffffffu, sp_[j] && valid[j]);
          if ((lane % G) == (k % G)) keep[k / G][j] = b;
        }
      }
    }
    if constexpr (BALLOT) {
      if (EMIT && p.packed) {
        const long long widx = col0 / 32 + lane / G;
#pragma unroll
        for (int q = 0; q < NSLOT; ++q) {
          const int kk = q * G + (lane % G);
          // columns 32*w .. 32*w+31 (w = lane / G) are lanes G*w .. G*w+G-1: bit (V*m + j) of the
          // word is bit (G*w + m) of ballot j
          uint32_t word = 0u;
#pragma unroll
          for (int j = 0; j < V; ++j) word |= spread_bits<V>(keep[q][j] >> (G * (lane / G) % 32)) << j;
          if (kk < nsteps && widx < p.words_per_row) p.packed[(t0 + kk) * p.words_per_row + widx] = word;
        }
      }
    }
  };

  // ---- which tiles this warp scans. An ordinary launch: all of them, once. A time-split launch
  // (few columns: spare SMs take later parts of the time axis): segment blockIdx.y, entered
  // warm_tiles early from V = 0 with its outputs held back until its own first tile - PLIF
  // trajectories driven by the same input become bit-identical after a few hundred steps, whatever
  // state they started from. The fix-up launch then walks the segments in order with the exact
  // state in hand, and rescans only those whose warmed-up state does not equal it bit for bit.
  // SPLIT is a template parameter: the kernels of ordinary launches carry none of this (with the
  // choice made at run time the packed row-parameter scan took 16 instead of 13 instructions per
  // step and half as long again).
  static_assert(!SPLIT || !MT::kStats, "no time split for the kernels that accumulate moments");
  constexpr bool split = SPLIT;
  const int seg_lo = split ? (p.fixup ? 1 : (int)blockIdx.y) : 0;
  const int seg_hi = split ? (p.fixup ? p.nseg : (int)blockIdx.y + 1) : 1;
  float carry[V], carryw[V];
  if (split && p.fixup) {
#pragma unroll
    for (int j = 0; j < V; ++j) {
      carry[j] = valid[j] ? p.vend[colj[j]] : 0.0f;
      carryw[j] = (MT::kSecond && valid[j]) ? p.wend[colj[j]] : 0.0f;
    }
  }
  unsigned int rescans = 0;
  for (int seg = seg_lo; seg < seg_hi && !failed; ++seg) {
    int tile_begin = 0, tile_emit = 0, tile_end = ntiles_total;
    if (split) {
      tile_emit = seg * p.seg_tiles;
      tile_end = tile_emit + p.seg_tiles < ntiles_total ? tile_emit + p.seg_tiles : ntiles_total;
      if (p.fixup) {
        bool differs = false;
#pragma unroll
        for (int j = 0; j < V; ++j)
          if (valid[j]) {
            differs |= __float_as_uint(p.vspec[(long long)seg * row_elems + colj[j]]) != __float_as_uint(carry[j]);
            if (MT::kSecond)
              differs |= __float_as_uint(p.wspec[(long long)seg * row_elems + colj[j]]) != __float_as_uint(carryw[j]);
          }
        if (!__any_sync(0xffffffffu, differs)) {  // the speculation held: this segment's results stand
#pragma unroll
          for (int j = 0; j < V; ++j) {
            carry[j] = valid[j] ? p.vend[(long long)seg * row_elems + colj[j]] : 0.0f;
            carryw[j] = (MT::kSecond && valid[j]) ? p.wend[(long long)seg * row_elems + colj[j]] : 0.0f;
          }
          continue;
        }
        if (lane == 0 && p.fix_count) {
          atomicAdd(p.fix_count, 1u);
          atomicMax(p.fix_count + 1, ++rescans);  // the warp with the most rescans sets the second launch's time
        }
        tile_begin = tile_emit;
#pragma unroll
        for (int j = 0; j < V; ++j) {
          v[j] = carry[j];
          w[j] = carryw[j];
        }
      } else {
        tile_begin = seg == 0 ? 0 : tile_emit - p.warm_tiles;
        if (seg > 0) {
#pragma unroll
          for (int j = 0; j < V; ++j) v[j] = w[j] = 0.0f;
        }
      }
    }
    // (rotation: this warp's tiles are rw, rw + R, ...)
    const int nt = ROT ? (tile_end - tile_begin > rw ? (tile_end - tile_begin - rw + R - 1) / R : 0) : tile_end - tile_begin;
    auto abs_tile = [&](int i) { return ROT ? tile_begin + rw + i * R : tile_begin + i; };
    if constexpr (TMA) {
      if (lane == 0) {  // prime the ring from the stage that is consumed next
        const int pre = nt < stages ? nt : stages;
        for (int q = 0; q < pre; ++q) issue(abs_tile(q), (s_idx + q) % stages);
      }
    }
    if constexpr (MODE == MODE_ROWPAT) {
      if (p.pat_in) load_patterns(tile_begin, pin_cur);
    }
    for (int i = 0; i < nt; ++i) {
      const int ia = abs_tile(i);  // absolute tile index
      cur_tile = ia;
      t0 = (long long)ia * C;
      const bool emit = !split || ia >= tile_emit;
      const int nsteps = (p.T - t0) < C ? (int)(p.T - t0) : C;
      if (split && !p.fixup && seg > 0 && ia == tile_emit) {  // warmed up: what this segment assumes it starts from
#pragma unroll
        for (int j = 0; j < V; ++j)
          if (valid[j]) {
            p.vspec[(long long)seg * row_elems + colj[j]] = v[j];
            if (MT::kSecond) p.wspec[(long long)seg * row_elems + colj[j]] = w[j];
          }
      }
      if constexpr (MODE == MODE_ROWPAT) {
        if (p.pat_in && i + 1 < nt) load_patterns(ia + 1, pin_nxt);
      }
      if constexpr (TMA) {
        const bool ok = mbar_wait_bounded(bar0 + 8u * s_idx, phase, p.err, 1u, p.wait_ns);
        if (!__all_sync(0xffffffffu, ok)) {  // a lane that ran out of time takes the whole warp out
          failed = true;
          break;
        }
        sp = reinterpret_cast<const ST*>(data_ptr + (size_t)s_idx * STAGE_BYTES) + V * lane;
      }
      if (p.ckpt && emit && !ROT) {  // (rotation: written once the tile's starting state has arrived)
        if constexpr (VEC) {
          if (valid[0]) VecIO<float, V>::store(p.ckpt + (long long)ia * row_elems + colj[0], v);
          if (MT::kSecond && valid[0]) VecIO<float, V>::store(p.ckpt_w + (long long)ia * row_elems + colj[0], w);
        } else {
#pragma unroll
          for (int j = 0; j < V; ++j)
            if (valid[j]) {
              p.ckpt[(long long)ia * row_elems + colj[j]] = v[j];
              if (MT::kSecond) p.ckpt_w[(long long)ia * row_elems + colj[j]] = w[j];
            }
        }
      }
      bool warm_tile = false;
      if constexpr (SPLIT) warm_tile = !emit;
      if (warm_tile) {  // always a full tile: warm-up ends before the segment's own first step
        if constexpr (SPLIT) tile(std::true_type{}, std::false_type{}, std::false_type{}, C);
      } else if (nsteps == C) {
        if (any_direct)
          tile(std::true_type{}, std::true_type{}, std::true_type{}, C);
        else
          tile(std::true_type{}, std::false_type{}, std::true_type{}, C);
      } else {
        tile(std::false_type{}, std::true_type{}, std::true_type{}, nsteps);
      }
      if constexpr (ROT) {
        if (rot_failed) {
          failed = true;
          break;
        }
        state_out(false);
      }
      if constexpr (MODE == MODE_ROWPAT) {
#pragma unroll
        for (int q = 0; q < TOK; ++q) pin_cur[q] = pin_nxt[q];
      }

      if constexpr (TMA) {
        const bool store_spikes = DENSE_TMA && p.spike != nullptr && emit;
        if (store_spikes) proxy_async_fence();  // make this lane's shared-memory writes visible to TMA
        __syncwarp();
        if (lane == 0) {
          if (store_spikes) {
            tma_store_2d(&tm_spike, data0 + (uint32_t)s_idx * STAGE_BYTES + MT::kDrive * TILE_BYTES, (int)col0,
                         ia * C);
            bulk_commit_group();
          }
          if (store_spikes && p.defer) {
            // Refill the stage of the PREVIOUS tile: its store has had a whole tile of
            // compute to read shared memory, so this wait returns at once and the warp
            // never stands still behind its own store.
            bulk_wait_read_keep1();
            const int sp_idx = s_idx == 0 ? stages - 1 : s_idx - 1;
            if (i >= 1 && i - 1 + stages < nt) issue(abs_tile(i - 1 + stages), sp_idx);
          } else if (p.defer && DENSE_TMA && p.spike != nullptr) {
            // (a warm-up tile of a deferring launch: nothing was stored, keep the refill order)
            const int sp_idx = s_idx == 0 ? stages - 1 : s_idx - 1;
            if (i >= 1 && i - 1 + stages < nt) issue(abs_tile(i - 1 + stages), sp_idx);
          } else {
            if (store_spikes) bulk_wait_read_all();  // the stage is refilled next
            if (i + stages < nt) issue(abs_tile(i + stages), s_idx);
          }
        }
        if (++s_idx == stages) {
          s_idx = 0;
          phase ^= 1u;
        }
      }
    }
    if constexpr (TMA) {
      if (lane == 0) bulk_wait_all();  // every store of this range has left shared memory
      __syncwarp();
    }
    if (split && !failed) {
#pragma unroll
      for (int j = 0; j < V; ++j) {
        if (p.fixup) {
          carry[j] = v[j];
          carryw[j] = w[j];
        }
        if (valid[j]) {
          p.vend[(long long)seg * row_elems + colj[j]] = v[j];
          if (MT::kSecond) p.wend[(long long)seg * row_elems + colj[j]] = w[j];
        }
      }
    }
  }

  if constexpr (TMA) {
    if (failed) {
      state_out(true);  // (rotation: the warps waiting for this one's state give up at once)
      // Give every load that may still be in flight a bounded chance to land before the CTA's
      // shared memory is released, and leave NaN in the per-column outputs: the error word says
      // why, and nothing downstream can mistake unwritten memory for a result.
      mbar_drain(bar0, stages, s_idx, phase, p.wait_ns);
#pragma unroll
      for (int j = 0; j < V; ++j)
        if (valid[j]) {
          p.vlast[colj[j]] = __int_as_float(0x7fc00000);
          if (MT::kSecond) p.wlast[colj[j]] = __int_as_float(0x7fc00000);
        }
      return;
    }
  }
  if (split && p.fixup) {
#pragma unroll
    for (int j = 0; j < V; ++j) {
      v[j] = carry[j];
      w[j] = carryw[j];
    }
  }
  // (rotation: the final state is the one of the warp that ran the last tile)
  if ((!split || p.fixup) && (!ROT || (ntiles_total > 0 ? (ntiles_total - 1) % R == rw : rw == 0))) {
#pragma unroll
    for (int j = 0; j < V; ++j)
      if (valid[j]) {
        p.vlast[colj[j]] = v[j];
        if (MT::kSecond) p.wlast[colj[j]] = w[j];
      }
  }
  if constexpr (MT::kStats) {
    if (p.u_stats) {  // one (sum, sum of squares) pair per warp, lanes added in a fixed order
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        st_s += __shfl_down_sync(0xffffffffu, st_s, o);
        st_q += __shfl_down_sync(0xffffffffu, st_q, o);
      }
      if (lane == 0) {
        const long long gw = (long long)blockIdx.x * wpc + warp;
        p.u_stats[2 * gw] = st_s;
        p.u_stats[2 * gw + 1] = st_q;
      }
    }
  }
}

template <typename ST, int MODE, bool PACKED, int V, int C, bool TMA>
__global__ void plif_fwd_kernel(const FwdParams p, const __grid_constant__ CUtensorMap tm0,
                                const __grid_constant__ CUtensorMap tm1,
                                const __grid_constant__ CUtensorMap tm2,
                                const __grid_constant__ CUtensorMap tm3,
                                const __grid_constant__ CUtensorMap tm4,
                                const __grid_constant__ CUtensorMap tm_spike) {
  plif_fwd_body<ST, MODE, PACKED, V, C, TMA>(p, tm0, tm1, tm2, tm3, tm4, tm_spike);
}

// The same scan with the tiles of a column group taken in turn by several warps (see plif_fwd_body).
template <typename ST, int MODE, bool PACKED, int V, int C, bool TMA>
__global__ void __maxnreg__(80) plif_fwd_rot_kernel(const FwdParams p, const __grid_constant__ CUtensorMap tm0,
                                    const __grid_constant__ CUtensorMap tm1,
                                    const __grid_constant__ CUtensorMap tm2,
                                    const __grid_constant__ CUtensorMap tm3,
                                    const __grid_constant__ CUtensorMap tm4,
                                    const __grid_constant__ CUtensorMap tm_spike) {
  plif_fwd_body<ST, MODE, PACKED, V, C, TMA, false, true>(p, tm0, tm1, tm2, tm3, tm4, tm_spike);
}

// The same scan cut along time (few columns): grid.y = segment in the first launch, and the checking
// launch (p.fixup) afterwards. Built with one lane per thread only (see kSplitBuilt in launch_fwd_one).
template <typename ST, int MODE, bool PACKED, int V, int C, bool TMA>
__global__ void plif_fwd_split_kernel(const FwdParams p, const __grid_constant__ CUtensorMap tm0,
                                      const __grid_constant__ CUtensorMap tm1,
                                      const __grid_constant__ CUtensorMap tm2,
                                      const __grid_constant__ CUtensorMap tm3,
                                      const __grid_constant__ CUtensorMap tm4,
                                      const __grid_constant__ CUtensorMap tm_spike) {
  // the checking launch is a dependent launch: its CTAs take their places while the segments still run
  if (p.fixup) grid_dependency_wait(); else grid_dependents_may_launch();
  plif_fwd_body<ST, MODE, PACKED, V, C, TMA, true>(p, tm0, tm1, tm2, tm3, tm4, tm_spike);
}

// Same, held to 160 registers: for the 4-lane resonate-and-fire kernel with the modulation fused in
// that also accumulates the moments of u, so that 3 warps fit each SM sub-partition (12 per SM; at its
// natural 180 it is 8, and that kernel lives on resident warps: measured 4.8 ms at 11 warps per SM,
// 6.7-7.9 ms at 6).
template <typename ST, int MODE, bool PACKED, int V, int C, bool TMA>
__global__ void __maxnreg__(160) plif_fwd_kernel_r160(const FwdParams p, const __grid_constant__ CUtensorMap tm0,
                                                      const __grid_constant__ CUtensorMap tm1,
                                                      const __grid_constant__ CUtensorMap tm2,
                                                      const __grid_constant__ CUtensorMap tm3,
                                                      const __grid_constant__ CUtensorMap tm4,
                                                      const __grid_constant__ CUtensorMap tm_spike) {
  plif_fwd_body<ST, MODE, PACKED, V, C, TMA>(p, tm0, tm1, tm2, tm3, tm4, tm_spike);
}

// ------------------------------------------------------------------ backward

// 96 registers per thread keep the 21 warps per SM of the headline shape
// (196 608 columns, 2 per thread, 148 SMs) resident in a single wave.
constexpr int kBwdMaxRegs = 96;
// The 4-lane backward is left uncapped (~230 registers, 8 warps per SM). Capping it so that
// 11-12 warps fit an SM (the headline shape would then run in one wave) was measured: at 184
// registers an 11-warp CTA does not launch (3 warps land on one 16 K-register sub-partition), at
// 168 the spills cost 15-40 %.
constexpr int kBwdMaxRegsV4 = 255;
constexpr int kBwdMaxThreads = 256;

struct BwdParams {
  const void* s[7];  // stream base pointers (direct path), smem order
  const float* bias[4];  // modulated modes: b_beta, b_alpha, b_th, b_omega
  long long channels;
  float v_th_min;
  void* g_extra;     // MODE_RFMOD: grad raw_omega
  float* g_bias[4];  // modulated modes: per-column sums over time of the raw gradients
  const float* beta_row;
  const float* vth_row;
  const float* ckpt;
  const float* ckpt_w;
  float* g_winit;
  void* g_beta;
  void* g_drive;
  void* g_gain;
  void* g_vth;
  float* g_beta_row;
  float* g_vth_row;
  float* g_vinit;
  long long T, cols;
  int ntiles, stages, has_gv, nstreams;
  int defer;  // 1: a stage is refilled one tile after its outputs were handed to TMA
  float alpha;
  const float* alpha_dev;
  uint32_t* err;
  unsigned long long wait_ns;  // limit of the bounded barrier waits
  // Time split (few columns, row-parameter scan), as in the forward: nseg segments of seg_tiles
  // tiles run side by side, here from their last tile to their first. A segment other than the
  // last one starts warm_tiles later in time with a zero adjoint and keeps only what it computes
  // from its own last tile on. [nseg, cols] arrays: aspec = the adjoint a segment assumed on
  // entering its own part, aend = the adjoint it handed on, partb / partt = its share of the sums
  // over time of the row gradients. fixup = 1: the checking launch.
  int nseg, seg_tiles, warm_tiles, fixup;
  float* aspec;
  float* aend;
  float* partb;
  float* partt;
  unsigned int* fix_count;
  // Chained chunks (more CTAs than fit on the GPU at once): the time axis in chain_q chunks of
  // chain_tiles tiles; a CTA takes a ticket, tickets walk the chunks from the last to the first
  // and, within a chunk, the column blocks. The CTA of a chunk waits until the one of the next
  // chunk of its columns has finished, takes the adjoint (and the running sums over time) from the
  // per-column outputs, where that CTA left them, and leaves its own there. Same operations in the
  // same order as one CTA walking all of T: the results are bit-identical. What it buys: a column
  // block is no longer one indivisible piece of work, so the GPU stays full until the end of the
  // launch, and all resident CTAs read and write the same few rows of every tensor at a time.
  // chain_sync[0] = ticket counter, chain_sync[1 + w] = chunks finished by global warp w.
  int chain_q, chain_tiles;
  unsigned int* chain_sync;
};

// Warps that share one TMA box in the backward kernel. DRAM efficiency of the tiled copies
// depends on the length of a row segment, not on the bytes per box (measured on the selective
// backward, 9 streams: 8 x 128 B and 16 x 128 B boxes both stop at ~5.85 ms, 8 x 256 B reaches
// 5.03 ms), while the modulated backward only fits 2 columns per lane in registers (128-byte
// segments in bf16). There two neighbouring warps share boxes with 256-byte rows: the first one's
// lane 0 issues the copies, both wait on the same mbarrier, and a named barrier of 64 threads
// joins them before the box is stored. The plain resonate-and-fire backward gains a little the same
// way over its 4-lane form (timed alone 5.07 against 5.22 ms at B=32, T=8192, D=6144; alternating
// with its forward 5.27 against 5.30 ms); the first-order selective backward does not (5.37 against
// 5.06 ms) and keeps one warp per box.
// Whether the backward keeps two of the five modulation intermediates of the resonate-and-fire scan in
// dead input slots of the staged tile (see the kernel): 2 lanes of 16-bit elements only.
template <int MODE, int V, int C, bool TMA, size_t ELEM>
inline constexpr bool kBwdSlotStash = TMA && MODE == MODE_RFMOD && V == 2 && ELEM == 2;

template <int MODE, int V, int C, bool TMA>
struct BwdBox {
  static constexpr int kWarps = (TMA && (ModeTraits<MODE>::kMod || MODE == MODE_RF) && V == 2 && C == 8) ? 2 : 1;
};

// Named-barrier primitives for such a pair (id 1..15; all 64 threads must arrive). At the end of a
// tile only the first warp of a pair waits (it hands the box to TMA); the second one arrives and goes
// on to the next tile, whose stage it can enter as soon as its data has landed. It can therefore be
// up to one ring of tiles ahead, so every stage of a box has a barrier id of its own: a second
// arrival on an id comes only after the stage was refilled, i.e. after the first warp consumed the
// first one. Writes made before the arrival are visible to the waiting warp (producer/consumer form).
__device__ __forceinline__ void pair_sync(int id) { asm volatile("bar.sync %0, 64;" ::"r"(id) : "memory"); }
__device__ __forceinline__ void pair_arrive(int id) { asm volatile("bar.arrive %0, 64;" ::"r"(id) : "memory"); }

// Surrogate derivative on the V lanes of a thread.
//   arctangent: (alpha/2) / (1 + (pi/2*alpha*x)^2)      c1 = pi/2*alpha, c2 = alpha/2
//   sigmoid:    alpha*sig*(1-sig) = alpha*e/(1+e)^2 with e = exp(-alpha*|x|) in (0,1]
//               (even in x, so it cannot overflow and needs no clamp)  c1 = -alpha*log2(e)
// PAIRS: two lanes at a time on the packed fp32x2 instructions (the modulated scans, which are bound
// by instruction issue; the results differ from the scalar form in the last place at most).
template <int SURR, int V, bool PAIRS = false>
__device__ __forceinline__ void surrogate_grad(float (&sg)[V], const float (&x)[V], float alpha, float c1,
                                               float c2) {
  if constexpr (PAIRS && V % 2 == 0) {
    using P = mod::Pack<2>;
#pragma unroll
    for (int j = 0; j < V; j += 2) {
      if constexpr (SURR == NSB_SURR_ATAN) {
        const P z = mul(P::load(&x[j]), P::splat(c1));
        const P r = fma(z, z, P::splat(1.0f)).map([](float d) { return mod::rcp_approx(d); });
        mul(P::splat(c2), r).store(&sg[j]);
      } else {
        const P e = P::load(&x[j]).map([c1](float xx) { return mod::ex2_approx(c1 * fabsf(xx)); });
        const P r = add(P::splat(1.0f), e).map([](float d) { return mod::rcp_approx(d); });
        mul(mul(P::splat(alpha), e), mul(r, r)).store(&sg[j]);
      }
    }
  } else if constexpr (SURR == NSB_SURR_ATAN) {
    float z[V], d[V], one[V];
#pragma unroll
    for (int j = 0; j < V; ++j) one[j] = 1.0f;
    vmuls<V>(z, x, c1);
    vfma<V>(d, z, z, one);
#pragma unroll
    for (int j = 0; j < V; ++j) sg[j] = __fdividef(c2, d[j]);
  } else {
#pragma unroll
    for (int j = 0; j < V; ++j) {
      // the argument is <= 0, so the result is in [0, 1]: the hardware exponential
      // (relative error 2^-22, tiny results flushed to zero) needs no range handling
      float e, r;
      asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(c1 * fabsf(x[j])));
      asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
      sg[j] = (alpha * e) * (r * r);
    }
  }
}

template <typename ST, int MODE, int SURR, int V, int C, bool TMA, bool HAS_GV, bool SPLIT = false>
__global__ void __maxnreg__((TMA && C * V <= 16) ? ((MODE == MODE_RF || MODE == MODE_MOD) ? 128 : (MODE == MODE_RFMOD ? 168 : kBwdMaxRegs)) : ((TMA && C * V == 32 && MODE != MODE_RF && MODE != MODE_RFMOD) ? kBwdMaxRegsV4 : 255)) plif_bwd_kernel(const BwdParams p, const __grid_constant__ CUtensorMap tm0,
                                const __grid_constant__ CUtensorMap tm1,
                                const __grid_constant__ CUtensorMap tm2,
                                const __grid_constant__ CUtensorMap tm3,
                                const __grid_constant__ CUtensorMap tm4,
                                const __grid_constant__ CUtensorMap tm5,
                                const __grid_constant__ CUtensorMap tm6,
                                const __grid_constant__ CUtensorMap tmo_beta,
                                const __grid_constant__ CUtensorMap tmo_drive,
                                const __grid_constant__ CUtensorMap tmo_gain,
                                const __grid_constant__ CUtensorMap tmo_vth,
                                const __grid_constant__ CUtensorMap tmo_omega) {
  using MT = ModeTraits<MODE>;
  using E = Elem<ST>;
  using IO = VecIO<ST, V>;
  if constexpr (SPLIT) {  // the checking launch is a dependent launch (see plif_fwd_split_kernel)
    if (p.fixup) grid_dependency_wait(); else grid_dependents_may_launch();
  }
  constexpr int NF = MT::kFwdStreams;  // forward inputs; then g_spike, then optional g_vpost
  constexpr int kGS = NF, kGV = NF + 1;
  constexpr int G = BwdBox<MODE, V, C, TMA>::kWarps;  // warps per TMA box
  constexpr int ROW = 32 * V * G;                      // elements per shared-memory row of a box
  constexpr int TILE_ELEMS = C * 32 * V;               // one warp's share of a box
  constexpr int BOX_ELEMS = C * ROW;
  constexpr uint32_t TILE_BYTES = BOX_ELEMS * sizeof(ST);
  extern __shared__ __align__(128) uint8_t smem_raw[];

  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int wpc = blockDim.x >> 5;
  const int box = warp / G, half = warp % G;
  const int nbox = wpc / G;
  const int pair_id = 1 + box * p.stages;  // + the stage index (the host keeps boxes x stages <= 15)
  const bool leader = half == 0 && lane == 0;
  int vblock = blockIdx.x, chunk = 0;
  const bool chained = !SPLIT && p.chain_q > 1;
  if (chained) {
    __shared__ unsigned int s_ticket;
    if (threadIdx.x == 0) s_ticket = atomicAdd(p.chain_sync, 1u);
    __syncthreads();
    const unsigned int nb = gridDim.x / (unsigned int)p.chain_q;  // column blocks
    chunk = p.chain_q - 1 - (int)(s_ticket / nb);
    vblock = (int)(s_ticket % nb);
  }
  const long long boxcol0 = ((long long)vblock * nbox + box) * ROW;
  if (boxcol0 >= p.cols) return;  // the same for every warp of a box
  const long long col0 = boxcol0 + (long long)half * (32 * V);

  constexpr int nstreams = NF + 1 + (HAS_GV ? 1 : 0);
  constexpr bool has_gv = HAS_GV;
  constexpr uint32_t stage_bytes = (uint32_t)nstreams * TILE_BYTES;
  // Modulated modes: the recompute pass leaves what the adjoint pass needs of the modulation
  // (unscaled beta, alpha, sigmoid(z_alpha) [, unscaled omega, sigmoid(z_omega)]) in a private
  // fp32 region of shared memory, so that the transcendental work is done once per element.
  constexpr int NQ = ModeTraits<MODE>::kMod ? (ModeTraits<MODE>::kSecond ? 5 : 3) : 0;
  constexpr bool STASH = TMA && NQ > 0;
  // Resonate-and-fire, 2 lanes of 16-bit elements: two of the five go into staged input slots that are
  // dead between the two passes (a thread's 2 elements of a stream are one 32-bit word: raw_alpha's and
  // I's take the two lanes of I*sigmoid(z_alpha), raw_beta's and raw_omega's those of sigmoid(z_omega)).
  // The private region shrinks from 10 to 6 KB per warp, which lets a third CTA of 4 warps onto an SM:
  // 196 608 columns are 3 072 warps, i.e. 2.6 rounds of 8 resident warps per SM but 1.7 rounds of 12.
  constexpr bool SLOT = STASH && kBwdSlotStash<MODE, V, C, TMA, sizeof(ST)>;
  constexpr int NQS = SLOT ? 3 : NQ;  // arrays in the private region

  long long colj[V];
  bool valid[V];
  float brow[V], trow[V], acc[V], accw[V], accb[V], acct[V];
#pragma unroll
  for (int j = 0; j < V; ++j) {
    colj[j] = col0 + V * lane + j;
    valid[j] = colj[j] < p.cols;
    acc[j] = accw[j] = accb[j] = acct[j] = 0.0f;
    brow[j] = trow[j] = 0.0f;
    if (MODE == MODE_ROW && valid[j]) {
      brow[j] = p.beta_row[colj[j]];
      trow[j] = p.vth_row[colj[j]];
    }
  }
  // modulated modes: biases of this thread's channels, and the sums over time of the raw
  // gradients (= bias gradients per column; accb / acct take those of beta and v_th)
  mod::Bias<V> bias = {};
  float acca[V], acco[V];
#pragma unroll
  for (int j = 0; j < V; ++j) acca[j] = acco[j] = 0.0f;
  if constexpr (MT::kMod) {
#pragma unroll
    for (int j = 0; j < V; ++j) {
      if (valid[j]) {
        const long long ch = colj[j] % p.channels;
        bias.beta[j] = p.bias[0][ch];
        bias.alpha[j] = p.bias[1][ch];
        bias.th[j] = p.bias[2][ch];
        if (MT::kSecond) bias.omega[j] = p.bias[3][ch];
      }
    }
  }

  const int stages = p.stages;
  uint32_t bar0 = 0, data0 = 0;
  const uint8_t* data_ptr = nullptr;
  float* stash = nullptr;
  volatile uint32_t* box_fail = nullptr;
  if constexpr (TMA) {
    const uint32_t base = smem_u32(smem_raw);
    bar0 = base + (uint32_t)(box * stages) * 8u;
    const uint32_t data_base = (base + (uint32_t)(wpc * stages) * 8u + 127u) & ~127u;
    data0 = data_base + (uint32_t)(box * stages) * stage_bytes;
    data_ptr = smem_raw + (data0 - base);
    if constexpr (STASH)
      stash = reinterpret_cast<float*>(smem_raw + (data_base - base) + (size_t)(nbox * stages) * stage_bytes) +
              (size_t)warp * (NQS * TILE_ELEMS) + V * lane;
    if constexpr (G > 1)  // set by the second warp of a pair when it gives up a wait; read by the first
      box_fail = reinterpret_cast<volatile uint32_t*>(smem_raw + (size_t)(nbox * stages) * 8u + (size_t)box * 4u);
    if (leader) {
      for (int s = 0; s < stages; ++s) mbar_init(bar0 + 8u * s, 1);
      if constexpr (G > 1) *box_fail = 0u;
      mbar_init_fence();
      proxy_async_fence();
    }
    __syncwarp();
    if constexpr (G > 1) pair_sync(pair_id);
  }

  auto issue = [&](int tile, int s) {
    if constexpr (TMA) {
      const uint32_t bar = bar0 + 8u * s;
      const uint32_t dst = data0 + (uint32_t)s * stage_bytes;
      mbar_arrive_expect_tx(bar, stage_bytes);
      const int x = (int)boxcol0, y = tile * C;
      tma_load_2d(dst, &tm0, x, y, bar);
      tma_load_2d(dst + TILE_BYTES, &tm1, x, y, bar);
      if (nstreams > 2) tma_load_2d(dst + 2 * TILE_BYTES, &tm2, x, y, bar);
      if (nstreams > 3) tma_load_2d(dst + 3 * TILE_BYTES, &tm3, x, y, bar);
      if (nstreams > 4) tma_load_2d(dst + 4 * TILE_BYTES, &tm4, x, y, bar);
      if (nstreams > 5) tma_load_2d(dst + 5 * TILE_BYTES, &tm5, x, y, bar);
      if (nstreams > 6) tma_load_2d(dst + 6 * TILE_BYTES, &tm6, x, y, bar);
    }
  };

  const int ntiles = p.ntiles;

  const ST* sp = nullptr;  // this thread's first element inside the current stage
  ST regs[TMA ? 1 : (NF + 2) * C * V] = {};
  auto fetch = [&](int stream, int k, float (&out)[V]) {
    if constexpr (TMA) {
      IO::load(sp + stream * BOX_ELEMS + k * ROW, out);
    } else {
#pragma unroll
      for (int j = 0; j < V; ++j) out[j] = E::to_f32(regs[(stream * C + k) * V + j]);
    }
  };

  const float alpha = p.alpha_dev ? __ldg(p.alpha_dev) : p.alpha;
  const float c1 = SURR == NSB_SURR_ATAN ? 1.5707963267948966f * alpha : -alpha * 1.4426950408889634f;
  const float c2 = 0.5f * alpha;
  const long long row_elems = p.cols;

  long long t0 = 0;
  float v[V];
  // The checkpoint of a tile (membrane state before its first step) is read
  // straight from global memory one tile ahead of its use.
  float vnext[V], w[V], wnext[V];
#pragma unroll
  for (int j = 0; j < V; ++j) vnext[j] = w[j] = wnext[j] = 0.0f;
  // emit_tag = false: a warm-up tile of a time-split scan; the adjoint advances, nothing is written or summed
  auto tile = [&](auto full_tag, auto emit_tag, int nsteps) {
    constexpr bool FULL = decltype(full_tag)::value;
    constexpr bool EMIT = decltype(emit_tag)::value;
    // recompute the tile forward, keeping V[k-1] and x[k] = V_pre[k] - V_th[k]
    float vprev[C][V], xs[C][V], wprev[MT::kSecond ? C : 1][V];
    // Modulated modes: steps whose modulation is evaluated together. 1 here: evaluating several
    // steps ahead, which pays in the forward kernel, costs the backward more in registers (and so
    // in resident warps) than it gains (measured: 6.3 -> 6.5 ms first order, 10.3 -> 11.3 ms RF; with 1 lane
    // per thread, where registers are plentiful, 4 steps at once change nothing: 2.97 against 3.00 ms).
    constexpr int CH = 1;
    float mb[CH][V], mu[CH][V], mth[CH][V], mom[CH][V];
#pragma unroll
    for (int k = 0; k < C; ++k) {
#pragma unroll
      for (int j = 0; j < V; ++j) {
        vprev[k][j] = v[j];
        if (MT::kSecond) wprev[MT::kSecond ? k : 0][j] = w[j];
        xs[k][j] = 0.0f;
      }
      if (FULL || k < nsteps) {
        float b[V], th[V], dr[V], om[V];
        bool s_[V];
        fetch(MT::kDrive, k, dr);
        if constexpr (MODE == MODE_ROW) {
#pragma unroll
          for (int j = 0; j < V; ++j) {
            b[j] = brow[j];
            th[j] = trow[j];
          }
        } else if constexpr (MODE == MODE_LIN) {
          fetch(MT::kBeta, k, b);
#pragma unroll
          for (int j = 0; j < V; ++j) th[j] = __int_as_float(0x7f800000);
        } else {
          fetch(MT::kBeta, k, b);
          fetch(MT::kVth, k, th);
        }
        if constexpr (MODE == MODE_AI) {
          float gn[V];
          fetch(MT::kGain, k, gn);
          vmul<V>(dr, gn, dr);
        }
        if constexpr (MT::kSecond) fetch(MT::kOmega, k, om);
        if constexpr (MT::kMod) {
          if (k % CH == 0) {
#pragma unroll
            for (int kk = 0; kk < CH; ++kk) {
              if (k + kk < C && (FULL || k + kk < nsteps)) {
                float ra[V], q0[V], q1[V], q2[V], q3[V], q4[V];
                fetch(MT::kBeta, k + kk, mb[kk]);
                fetch(MT::kVth, k + kk, mth[kk]);
                fetch(MT::kDrive, k + kk, mu[kk]);
                fetch(MT::kGain, k + kk, ra);
                if constexpr (MT::kSecond) fetch(MT::kOmega, k + kk, mom[kk]);
                float cin[V];
#pragma unroll
                for (int j = 0; j < V; ++j) cin[j] = mu[kk][j];
                mod::forward_lanes<MT::kSecond, V>(mb[kk], ra, mth[kk], mom[kk], mu[kk], bias, p.v_th_min, q0, q1,
                                                   q2, q3, q4);
                if constexpr (STASH) {
                  // q2 := I * sigmoid(z_alpha), the factor of grad raw_alpha (the adjoint pass then needs no I)
#pragma unroll
                  for (int j = 0; j < V; ++j) q2[j] = __fmul_rn(cin[j], q2[j]);
                  VecIO<float, V>::store(stash + (0 * C + k + kk) * (32 * V), q0);
                  VecIO<float, V>::store(stash + (1 * C + k + kk) * (32 * V), q1);
                  if constexpr (SLOT) {
                    ST* slot = const_cast<ST*>(sp) + (k + kk) * ROW;
                    VecIO<float, V>::store(stash + (2 * C + k + kk) * (32 * V), q3);
                    slot_put(slot + MT::kGain * BOX_ELEMS, q2[0]);
                    slot_put(slot + MT::kDrive * BOX_ELEMS, q2[V - 1]);
                    slot_put(slot + MT::kBeta * BOX_ELEMS, q4[0]);
                    slot_put(slot + MT::kOmega * BOX_ELEMS, q4[V - 1]);
                  } else {
                    VecIO<float, V>::store(stash + (2 * C + k + kk) * (32 * V), q2);
                    if constexpr (MT::kSecond) {
                      VecIO<float, V>::store(stash + (3 * C + k + kk) * (32 * V), q3);
                      VecIO<float, V>::store(stash + (4 * C + k + kk) * (32 * V), q4);
                    }
                  }
                }
              }
            }
          }
#pragma unroll
          for (int j = 0; j < V; ++j) {
            b[j] = mb[k % CH][j];
            th[j] = mth[k % CH][j];
            dr[j] = mu[k % CH][j];
            om[j] = mom[k % CH][j];
          }
        }
        if constexpr (MT::kSecond) {
          rf_step<V>(v, w, b, om, dr, th, xs[k], s_);
        } else {
          plif_step<V>(v, b, dr, th, xs[k], s_);
        }
      }
    }

    // adjoint recurrence, last step of the tile first. On the TMA path each
    // gradient of step k is written over the input it corresponds to in shared
    // memory (grad beta over beta[k], grad drive over drive[k], ...): that slot
    // is dead once step k has read it, and the finished tiles leave through one
    // TMA store each, which also clips the ragged edges.
    const size_t tile_off = (size_t)(t0 * row_elems + colj[0]);
    ST* o_beta = (!TMA && MODE != MODE_ROW && p.g_beta) ? static_cast<ST*>(p.g_beta) + tile_off : nullptr;
    ST* o_vth = (!TMA && MODE != MODE_ROW && p.g_vth) ? static_cast<ST*>(p.g_vth) + tile_off : nullptr;
    ST* o_drive = (!TMA && p.g_drive) ? static_cast<ST*>(p.g_drive) + tile_off : nullptr;
    ST* o_gain = (!TMA && MT::kFwdStreams >= 4 && p.g_gain) ? static_cast<ST*>(p.g_gain) + tile_off : nullptr;
    ST* o_omega = (!TMA && MODE == MODE_RFMOD && p.g_extra) ? static_cast<ST*>(p.g_extra) + tile_off : nullptr;
    ST* wsp = const_cast<ST*>(sp);
#pragma unroll
    for (int kk = 0; kk < C; ++kk) {
      const int k = C - 1 - kk;
      if (FULL || k < nsteps) {
        float sg[V], gs[V], tot[V], gssg[V], gpre[V], b[V], gb[V], gth[V], gd[V], gg[V], go[V];
        if constexpr (MODE != MODE_LIN) surrogate_grad<SURR, V, MT::kMod>(sg, xs[k], alpha, c1, c2);
        fetch(kGS, k, gs);
        if (has_gv) {
          float gv[V];
          fetch(kGV, k, gv);
          vadd<V>(tot, acc, gv);
        } else {
#pragma unroll
          for (int j = 0; j < V; ++j) tot[j] = acc[j];
        }
        if constexpr (MODE == MODE_LIN) {
          // the incoming stream is dL/dV[k]: g = acc + dV[k]; grad u = g; grad beta = g*V[k-1]; acc = g*beta
#pragma unroll
          for (int j = 0; j < V; ++j) gssg[j] = gs[j];
        } else {
          if constexpr (MT::kMod && V % 2 == 0) {
            using P2 = mod::Pack<2>;
#pragma unroll
            for (int j = 0; j < V; j += 2) mul(P2::load(&gs[j]), P2::load(&sg[j])).store(&gssg[j]);
          } else {
            vmul<V>(gssg, gs, sg);
          }
        }
        if constexpr (MT::kMod && V % 2 == 0) {
          using P2 = mod::Pack<2>;
#pragma unroll
          for (int j = 0; j < V; j += 2) {
            const P2 g = add(P2::load(&gssg[j]), P2::load(&tot[j]));
            g.store(&gpre[j]);
            mul(g, P2::load(&vprev[k][j])).store(&gb[j]);
          }
        } else {
          vadd<V>(gpre, gssg, tot);
          vmul<V>(gb, gpre, vprev[k]);
        }
        // grad v_th = -gS*sg - tot*spike = -(spike ? gpre : gS*sg)
#pragma unroll
        for (int j = 0; j < V; ++j) gth[j] = -(xs[k][j] >= 0.0f ? gpre[j] : gssg[j]);
        if constexpr (MODE == MODE_RF) {
          // coupled V/W adjoints: grad_beta = gpre*V[k-1] + aw*W[k-1], grad_omega = aw*V[k-1] - gpre*W[k-1],
          // acc_v = gpre*beta + aw*omega, acc_w = aw*beta - gpre*omega  (aw = adjoint of W arriving at step k)
          float om[V];
          fetch(MT::kBeta, k, b);
          fetch(MT::kOmega, k, om);
#pragma unroll
          for (int j = 0; j < V; ++j) {
            const float vp_ = vprev[k][j], wp_ = wprev[MT::kSecond ? k : 0][j], aw = accw[j];
            gb[j] = fmaf(aw, wp_, gb[j]);
            gg[j] = aw * vp_ - gpre[j] * wp_;
            gd[j] = gpre[j];
            acc[j] = gpre[j] * b[j] + aw * om[j];
            accw[j] = aw * b[j] - gpre[j] * om[j];
          }
        }
        if constexpr (MT::kMod) {
          // Modulated modes: recompute the modulation of step k together with its derivative
          // factors, push the scan's adjoints (w.r.t. beta, omega, u, v_th) through it and leave
          // the gradients of the raw projections and of I in gb / go / gg / gth / gd.
          //   d sigmoid = s(1-s); d softplus(z) = sigmoid(z); d|z| = sign(z);
          //   rescale active (beta, omega) = scale*(b0, o0), scale = 0.999/r:
          //     G_b0 = scale*(G_beta - dot*b0), G_o0 = scale*(G_omega - dot*o0), dot = (G_beta*b0 + G_omega*o0)/r2
          // sav: I * sigmoid(z_alpha)
          float rt[V], b0v[V], alv[V], sav[V], o0v[V], sov[V];
          fetch(MT::kVth, k, rt);
          if constexpr (SLOT) {
            const ST* slot = sp + k * ROW;
            VecIO<float, V>::load(stash + (0 * C + k) * (32 * V), b0v);
            VecIO<float, V>::load(stash + (1 * C + k) * (32 * V), alv);
            VecIO<float, V>::load(stash + (2 * C + k) * (32 * V), o0v);
            sav[0] = slot_get(slot + MT::kGain * BOX_ELEMS);
            sav[V - 1] = slot_get(slot + MT::kDrive * BOX_ELEMS);
            sov[0] = slot_get(slot + MT::kBeta * BOX_ELEMS);
            sov[V - 1] = slot_get(slot + MT::kOmega * BOX_ELEMS);
          } else if constexpr (STASH) {
            VecIO<float, V>::load(stash + (0 * C + k) * (32 * V), b0v);
            VecIO<float, V>::load(stash + (1 * C + k) * (32 * V), alv);
            VecIO<float, V>::load(stash + (2 * C + k) * (32 * V), sav);
            if constexpr (MT::kSecond) {
              VecIO<float, V>::load(stash + (3 * C + k) * (32 * V), o0v);
              VecIO<float, V>::load(stash + (4 * C + k) * (32 * V), sov);
            }
          } else {
            float rb[V], ra[V], ro[V], th_[V], u_[V], ci[V];
            fetch(MT::kDrive, k, ci);
            fetch(MT::kBeta, k, rb);
            fetch(MT::kGain, k, ra);
            if constexpr (MT::kSecond) fetch(MT::kOmega, k, ro);
#pragma unroll
            for (int j = 0; j < V; ++j) {
              th_[j] = rt[j];
              u_[j] = ci[j];
            }
            mod::forward_lanes<MT::kSecond, V>(rb, ra, th_, ro, u_, bias, p.v_th_min, b0v, alv, sav, o0v, sov);
#pragma unroll
            for (int j = 0; j < V; ++j) sav[j] = __fmul_rn(ci[j], sav[j]);
          }
          // pairs of lanes on the packed fp32x2 instructions where V is even (no rounding
          // contract here: gradients are compared to a tolerance)
          constexpr int N = V % 2 == 0 ? 2 : 1;
          using P = mod::Pack<N>;
          const P minus1 = P::splat(-1.0f);
#pragma unroll
          for (int j = 0; j < V; j += N) {
            const P B0 = P::load(&b0v[j]), Gpre = P::load(&gpre[j]);
            P Gb = P::load(&gb[j]);
            if constexpr (MT::kSecond) {
              const P O0 = P::load(&o0v[j]);
              // the rescale as in the forward (same operations, so the same beta and omega), and for its
              // adjoint nc = -1/r2 where it is active (r2 = (0.999/scale)^2 there), 0 where it is not
              const P r2 = fma(B0, B0, mul(O0, O0));
              const P scale = r2.map([](float x) { return x > mod::kRmaxSq ? __fmul_rn(mod::kRmax, mod::rsqrt_approx(x)) : 1.0f; });
              const P nc = r2.map([](float x) { return x > mod::kRmaxSq ? (float)(-1.0 / (0.999 * 0.999)) : 0.0f; });
              const P be = mul(B0, scale), om_ = mul(O0, scale);
              const P VP = P::load(&vprev[k][j]), WP = P::load(&wprev[MT::kSecond ? k : 0][j]);
              const P AW = P::load(&accw[j]), NG = mul(Gpre, minus1);
              Gb = fma(AW, WP, Gb);
              P Go = fma(NG, WP, mul(AW, VP));
              fma(Gpre, be, mul(AW, om_)).store(&acc[j]);
              fma(NG, om_, mul(AW, be)).store(&accw[j]);
              // through the rescale: where it is inactive scale = 1 and ndot = 0, which leave Gb and Go as they are
              const P ndot = mul(mul(fma(Gb, B0, mul(Go, O0)), mul(scale, scale)), nc);
              Gb = mul(scale, fma(ndot, B0, Gb));
              Go = mul(scale, fma(ndot, O0, Go));
              const P g = mul(Go, P::load(&sov[j]));
              g.store(&go[j]);
              add(P::load(&acco[j]), g).store(&acco[j]);
            } else {
              mul(Gpre, B0).store(&acc[j]);
            }
            const P gB = mul(Gb, mul(B0, fma(B0, minus1, P::splat(1.0f))));
            const P gA = mul(Gpre, P::load(&sav[j]));
            gB.store(&gb[j]);
            gA.store(&gg[j]);
            mul(Gpre, P::load(&alv[j])).store(&gd[j]);
            // grad raw_th = grad v_th * sign(z_th) (0 at z_th = 0): flip the sign bit, no branch
            const P gT = zip(add(P::load(&rt[j]), P::load(&bias.th[j])), P::load(&gth[j]), P::splat(0.0f),
                             [](float zt, float g_, float) {
                               return zt == 0.0f ? 0.0f
                                                 : __uint_as_float(__float_as_uint(g_) ^
                                                                   (__float_as_uint(zt) & 0x80000000u));
                             });
            gT.store(&gth[j]);
            add(P::load(&accb[j]), gB).store(&accb[j]);
            add(P::load(&acca[j]), gA).store(&acca[j]);
            add(P::load(&acct[j]), gT).store(&acct[j]);
          }
        } else if constexpr (MODE == MODE_ROW) {
#pragma unroll
          for (int j = 0; j < V; ++j) b[j] = brow[j];
          if constexpr (EMIT) {
            vadd<V>(accb, accb, gb);
            vadd<V>(acct, acct, gth);
          }
        } else if constexpr (MODE != MODE_RF) {
          fetch(MT::kBeta, k, b);
        }
        if constexpr (MODE == MODE_AI) {
          float gn[V], dr[V];
          fetch(MT::kGain, k, gn);
          fetch(MT::kDrive, k, dr);
          vmul<V>(gd, gpre, gn);
          vmul<V>(gg, gpre, dr);
        }
        if constexpr (MODE != MODE_RF && !MT::kMod) vmul<V>(acc, gpre, b);

        if constexpr (TMA && EMIT) {
          if constexpr (MODE != MODE_ROW) IO::store(wsp + MT::kBeta * BOX_ELEMS + k * ROW, gb);
          if constexpr (MODE != MODE_ROW && MODE != MODE_LIN)
            IO::store(wsp + MT::kVth * BOX_ELEMS + k * ROW, gth);
          if constexpr (MODE == MODE_RFMOD) IO::store(wsp + MT::kOmega * BOX_ELEMS + k * ROW, go);
          if constexpr (MT::kFwdStreams >= 4) {
            IO::store(wsp + MT::kDrive * BOX_ELEMS + k * ROW, gd);
            IO::store(wsp + MT::kGain * BOX_ELEMS + k * ROW, gg);
          } else {
            IO::store(wsp + MT::kDrive * BOX_ELEMS + k * ROW, gpre);
          }
        } else if constexpr (!TMA) {
          const size_t ro = (size_t)k * row_elems;
          auto put = [&](ST* dst, const float (&val)[V]) {
            if (!dst) return;
#pragma unroll
            for (int j = 0; j < V; ++j)
              if (valid[j]) dst[ro + j] = E::from_f32(val[j]);
          };
          if constexpr (MODE != MODE_ROW) put(o_beta, gb);
          if constexpr (MODE != MODE_ROW && MODE != MODE_LIN) put(o_vth, gth);
          if constexpr (MODE == MODE_RFMOD) put(o_omega, go);
          if constexpr (MT::kFwdStreams >= 4) {
            put(o_drive, gd);
            put(o_gain, gg);
          } else {
            put(o_drive, gpre);
          }
        }
      }
    }
  };

  int s_idx = 0;
  uint32_t phase = 0;
  bool failed = false;
  // ---- which tiles this warp walks (from the last to the first). An ordinary launch: all of them.
  // A time-split launch: segment blockIdx.y, entered warm_tiles later in time with a zero adjoint
  // (the adjoint recurrence acc' = beta*(acc + ...) forgets its starting value just as the forward
  // forgets its state) and silent until it reaches its own last tile. The checking launch walks
  // the segments from the last one (exact: the adjoint is zero beyond T) to the first, compares
  // the adjoint each one assumed with the exact one bit for bit and redoes those that differ.
  static_assert(!SPLIT || (MODE == MODE_ROW && TMA && !HAS_GV && G == 1), "time split: row-parameter scan only");
  constexpr bool split = SPLIT;
  float carry[V], sumb[V], sumt[V];
  int seg_first = 0, seg_last = 0;  // inclusive, walked downwards
  if constexpr (SPLIT) {
    if (p.fixup) {
      seg_first = p.nseg - 2;
#pragma unroll
      for (int j = 0; j < V; ++j) {
        const long long o = (long long)(p.nseg - 1) * row_elems + colj[j];
        carry[j] = valid[j] ? p.aend[o] : 0.0f;
        sumb[j] = valid[j] ? p.partb[o] : 0.0f;
        sumt[j] = valid[j] ? p.partt[o] : 0.0f;
      }
    } else {
      seg_first = seg_last = (int)blockIdx.y;
    }
  }
  unsigned int* const chain_flag = chained ? p.chain_sync + 1 + ((long long)vblock * wpc + warp) : nullptr;
  if (chained && chunk < p.chain_q - 1) {
    // the later chunk of these columns must be finished: its CTA holds an earlier ticket, so it is running or done
    bool ok = true;
    if (lane == 0) ok = counter_wait_bounded(chain_flag, (unsigned int)(p.chain_q - 1 - chunk), p.err, 2u, p.wait_ns);
    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
    __syncwarp();  // the other lanes' loads below are ordered after lane 0's acquire
    if constexpr (G > 1) {
      // Both warps of a box take the same way: one that went on alone would wait at the box's named
      // barrier, which has no limit, for a partner that has left. Neither has entered the tile loop yet.
      if (!ok && lane == 0) *box_fail = 1u;
      __syncwarp();
      pair_sync(pair_id);
      ok = *box_fail == 0u;
    }
    if (!ok) {
      failed = true;
    } else {
#pragma unroll
      for (int j = 0; j < V; ++j) {
        if (!valid[j]) continue;
        acc[j] = __ldcg(p.g_vinit + colj[j]);
        if constexpr (MT::kSecond) accw[j] = __ldcg(p.g_winit + colj[j]);
        if constexpr (MT::kMod) {
          accb[j] = __ldcg(p.g_bias[0] + colj[j]);
          acca[j] = __ldcg(p.g_bias[1] + colj[j]);
          acct[j] = __ldcg(p.g_bias[2] + colj[j]);
          if constexpr (MT::kSecond) acco[j] = __ldcg(p.g_bias[3] + colj[j]);
        }
        if constexpr (MODE == MODE_ROW) {
          accb[j] = __ldcg(p.g_beta_row + colj[j]);
          acct[j] = __ldcg(p.g_vth_row + colj[j]);
        }
      }
    }
  }
  bool primed = false;  // whether any copy was issued (a CTA that gives up before has nothing in flight)
  [[maybe_unused]] unsigned int rescans = 0;
  for (int seg = seg_first; seg >= seg_last && !failed; --seg) {
    primed = true;
    int tile_lo = 0, tile_top = ntiles, tile_emit_top = ntiles;  // walk tiles tile_top-1 .. tile_lo; emit below tile_emit_top
    if (chained) {
      tile_lo = chunk * p.chain_tiles;
      tile_top = tile_emit_top = tile_lo + p.chain_tiles < ntiles ? tile_lo + p.chain_tiles : ntiles;
    }
    if constexpr (SPLIT) {
      tile_lo = seg * p.seg_tiles;
      tile_emit_top = tile_lo + p.seg_tiles < ntiles ? tile_lo + p.seg_tiles : ntiles;
      if (p.fixup) {
        bool differs = false;
#pragma unroll
        for (int j = 0; j < V; ++j)
          if (valid[j])
            differs |= __float_as_uint(p.aspec[(long long)seg * row_elems + colj[j]]) != __float_as_uint(carry[j]);
        if (!__any_sync(0xffffffffu, differs)) {  // the speculation held: this segment's results stand
#pragma unroll
          for (int j = 0; j < V; ++j) {
            const long long o = (long long)seg * row_elems + colj[j];
            carry[j] = valid[j] ? p.aend[o] : 0.0f;
            sumb[j] += valid[j] ? p.partb[o] : 0.0f;
            sumt[j] += valid[j] ? p.partt[o] : 0.0f;
          }
          continue;
        }
        if (lane == 0 && p.fix_count) {
          atomicAdd(p.fix_count, 1u);
          atomicMax(p.fix_count + 1, ++rescans);
        }
        tile_top = tile_emit_top;
#pragma unroll
        for (int j = 0; j < V; ++j) acc[j] = carry[j];
      } else {
        tile_top = tile_emit_top + p.warm_tiles < ntiles ? tile_emit_top + p.warm_tiles : ntiles;
      }
#pragma unroll
      for (int j = 0; j < V; ++j) accb[j] = acct[j] = 0.0f;
    }
    const int nt = tile_top - tile_lo;
    if constexpr (TMA) {
      if (leader) {  // prime the ring from the stage that is consumed next
        const int pre = nt < stages ? nt : stages;
        for (int q = 0; q < pre; ++q) issue(tile_top - 1 - q, (s_idx + q) % stages);
      }
      if (nt > 0 && valid[0]) {  // the checkpoint of the first tile walked; the others are fetched one tile ahead
        VecIO<float, V>::load(p.ckpt + (long long)(tile_top - 1) * row_elems + colj[0], vnext);
        if (MT::kSecond) VecIO<float, V>::load(p.ckpt_w + (long long)(tile_top - 1) * row_elems + colj[0], wnext);
      }
    }
    for (int n = 0; n < nt; ++n) {
      const int i = tile_top - 1 - n;
      t0 = (long long)i * C;
      const bool emit = !split || i < tile_emit_top;
      const int nsteps = (p.T - t0) < C ? (int)(p.T - t0) : C;
      if constexpr (SPLIT) {
        if (!p.fixup && i == tile_emit_top - 1 && tile_emit_top < ntiles) {  // warmed up: the adjoint this segment assumes
#pragma unroll
          for (int j = 0; j < V; ++j)
            if (valid[j]) p.aspec[(long long)seg * row_elems + colj[j]] = acc[j];
        }
      }
      if constexpr (TMA) {
        const bool ok = mbar_wait_bounded(bar0 + 8u * s_idx, phase, p.err, 2u, p.wait_ns);
        const bool gave_up = !__all_sync(0xffffffffu, ok);
        if (gave_up) {
          if constexpr (G > 1) {
            if (half != 0) {  // the first warp waits for this one at the end of the tile: tell it, and arrive
              if (lane == 0) *box_fail = 1u;
              __syncwarp();
              pair_arrive(pair_id + s_idx);
            }
          }
          failed = true;
          break;
        }
        const uint8_t* sp8 = data_ptr + (size_t)s_idx * stage_bytes;
        sp = reinterpret_cast<const ST*>(sp8) + half * (32 * V) + V * lane;
#pragma unroll
        for (int j = 0; j < V; ++j) {
          v[j] = vnext[j];
          w[j] = wnext[j];
        }
        if (i > tile_lo && valid[0]) {
          VecIO<float, V>::load(p.ckpt + (long long)(i - 1) * row_elems + colj[0], vnext);
          if (MT::kSecond) VecIO<float, V>::load(p.ckpt_w + (long long)(i - 1) * row_elems + colj[0], wnext);
        }
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
                  (present && k < nsteps && valid[j]) ? g[(t0 + k) * row_elems + colj[j]] : E::zero();
        }
#pragma unroll
        for (int j = 0; j < V; ++j) {
          v[j] = valid[j] ? p.ckpt[(long long)i * row_elems + colj[j]] : 0.0f;
          w[j] = (MT::kSecond && valid[j]) ? p.ckpt_w[(long long)i * row_elems + colj[j]] : 0.0f;
        }
      }

      bool warm_tile = false;
      if constexpr (SPLIT) warm_tile = !emit;
      if (warm_tile) {  // (a warm-up tile lies before the end of time only if it is a full one or the very last)
        if constexpr (SPLIT) {
          if (nsteps == C)
            tile(std::true_type{}, std::false_type{}, C);
          else
            tile(std::false_type{}, std::false_type{}, nsteps);
        }
      } else if (nsteps == C) {
        tile(std::true_type{}, std::true_type{}, C);
      } else {
        tile(std::false_type{}, std::true_type{}, nsteps);
      }

      if constexpr (TMA) {
        proxy_async_fence();  // make this lane's shared-memory writes visible to TMA
        __syncwarp();
        if constexpr (G > 1) {
          if (half != 0) {
            pair_arrive(pair_id + s_idx);
          } else {
            pair_sync(pair_id + s_idx);
            if (*box_fail != 0u) {  // the other warp gave up: this box is lost
              failed = true;
              break;
            }
          }
        }
        if (leader) {
          const uint32_t src = data0 + (uint32_t)s_idx * stage_bytes;
          const int x = (int)boxcol0, y = i * C;
          if (emit) {
            if (MODE != MODE_ROW && p.g_beta) tma_store_2d(&tmo_beta, src + MT::kBeta * TILE_BYTES, x, y);
            if (MODE != MODE_ROW && MODE != MODE_LIN && p.g_vth) tma_store_2d(&tmo_vth, src + MT::kVth * TILE_BYTES, x, y);
            if (p.g_drive) tma_store_2d(&tmo_drive, src + MT::kDrive * TILE_BYTES, x, y);
            if (MT::kFwdStreams >= 4 && p.g_gain) tma_store_2d(&tmo_gain, src + MT::kGain * TILE_BYTES, x, y);
            if (MODE == MODE_RFMOD && p.g_extra) tma_store_2d(&tmo_omega, src + MT::kOmega * TILE_BYTES, x, y);
          }
          bulk_commit_group();
          if (p.defer) {
            // see the forward kernel: refill the stage of the previous tile
            bulk_wait_read_keep1();
            const int sp_idx = s_idx == 0 ? stages - 1 : s_idx - 1;
            if (i + 1 <= tile_top - 1 && i + 1 - stages >= tile_lo) issue(i + 1 - stages, sp_idx);
          } else {
            bulk_wait_read_all();  // the stage is refilled next
            if (i - stages >= tile_lo) issue(i - stages, s_idx);
          }
        }
        if (++s_idx == stages) {
          s_idx = 0;
          phase ^= 1u;
        }
      }
    }
    if constexpr (TMA) {
      if (leader) bulk_wait_all();  // every store of this range has left shared memory
      __syncwarp();
    }
    if constexpr (SPLIT) {
      if (!failed) {
#pragma unroll
        for (int j = 0; j < V; ++j) {
          const long long o = (long long)seg * row_elems + colj[j];
          if (valid[j]) {
            p.aend[o] = acc[j];
            p.partb[o] = accb[j];
            p.partt[o] = acct[j];
          }
          if (p.fixup) {
            carry[j] = acc[j];
            sumb[j] += accb[j];
            sumt[j] += acct[j];
          }
        }
      }
    }
  }

  if constexpr (TMA) {
    if (failed) {
      // a chained launch: the CTAs that wait for this chunk give up at once instead of running out their own limit
      if (chained && chunk > 0 && lane == 0) counter_publish(chain_flag, kCounterPoisoned);
      if (primed) mbar_drain(bar0, stages, s_idx, phase, p.wait_ns);
#pragma unroll
      for (int j = 0; j < V; ++j)
        if (valid[j] && p.g_vinit) p.g_vinit[colj[j]] = __int_as_float(0x7fc00000);
      return;
    }
  }
  if constexpr (SPLIT) {
    if (!p.fixup) return;  // the checking launch writes the per-column results
#pragma unroll
    for (int j = 0; j < V; ++j) {
      acc[j] = carry[j];
      accb[j] = sumb[j];
      acct[j] = sumt[j];
    }
  }
#pragma unroll
  for (int j = 0; j < V; ++j) {
    if (valid[j]) {
      if (p.g_vinit) p.g_vinit[colj[j]] = acc[j];
      if (MT::kSecond && p.g_winit) p.g_winit[colj[j]] = accw[j];
      if (MT::kMod) {
        if (p.g_bias[0]) p.g_bias[0][colj[j]] = accb[j];
        if (p.g_bias[1]) p.g_bias[1][colj[j]] = acca[j];
        if (p.g_bias[2]) p.g_bias[2][colj[j]] = acct[j];
        if (MT::kSecond && p.g_bias[3]) p.g_bias[3][colj[j]] = acco[j];
      }
      if (MODE == MODE_ROW) {
        if (p.g_beta_row) p.g_beta_row[colj[j]] = accb[j];
        if (p.g_vth_row) p.g_vth_row[colj[j]] = acct[j];
      }
    }
  }
  if (chained && chunk > 0) {  // hand over to the CTA of the chunk before this one
    // (the fence costs each warp a few microseconds at the end of a chunk, which the other resident warps
    // cover: publishing without it - a timing experiment only - ran no faster)
    __threadfence();
    __syncwarp();
    if (lane == 0) counter_publish(chain_flag, (unsigned int)(p.chain_q - chunk));
  }
}

// -------------------------------------------------------------- host launchers

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Whether a ring stage is refilled one tile late (so that the producer lane never
// waits for its own TMA store to finish reading shared memory). It costs one stage
// of prefetch depth, so it is for launches with few warps per SM, where that wait
// is exposed; with many resident warps the other warps cover it.
inline int defer_refill(const Tuning& tune, const Plan& plan, const DeviceInfo& dev) {
  if (plan.stages < 3) return 0;
  if (tune.force_direct == 2) return 1;
  if (tune.force_direct == 3) return 0;
  return (long long)plan.grid * plan.wpc <= 8LL * std::max(1, dev.sm_count);
}

// The planner works from register estimates. If the CTA it chose does not fit an SM with the
// registers the kernel really has, halve the warps per CTA (shared memory is per warp, so it
// shrinks in proportion) until it does.
// `group` = warps that must stay together in a CTA (those sharing a TMA box).
template <typename K>
int shrink_to_fit(K kern, Plan& plan, long long nwarps, int group = 1) {
  for (;;) {
    int blocks = 0;
    NSB_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, kern, plan.wpc * 32, plan.smem),
                 "cudaOccupancyMaxActiveBlocksPerMultiprocessor");
    if (blocks > 0) return NSB_OK;
    if (plan.wpc <= group) return NSB_ERR_UNSUPPORTED;
    const size_t per_warp = (plan.smem - 256) / plan.wpc;
    plan.wpc = group * ((plan.wpc / group + 1) / 2);
    plan.smem = per_warp * plan.wpc + 256;
    plan.grid = (int)((nwarps + plan.wpc - 1) / plan.wpc);
  }
}

template <typename ST, int MODE, bool PACKED, int V, int C, bool TMA>
int launch_fwd_one(const FwdArgs& a, const DeviceInfo& dev, const Tuning& tune, const Plan& planned) {
  if (int r = sticky_device_error(); r != NSB_OK) return r;  // an earlier kernel gave up: say so, launch nothing
  using MT = ModeTraits<MODE>;
  constexpr int NS = MT::kFwdStreams;
  // only the moment-accumulating 4-lane resonate-and-fire kernel needs the limit (natural count 180)
  constexpr bool kCap160 = MODE == MODE_RFMODS && V == 4 && TMA;
  auto kern = [] {
    if constexpr (kCap160)
      return plif_fwd_kernel_r160<ST, MODE, PACKED, V, C, TMA>;
    else
      return plif_fwd_kernel<ST, MODE, PACKED, V, C, TMA>;
  }();
  FwdParams p = {};
  const void* streams[5] = {nullptr, nullptr, nullptr, nullptr, nullptr};
  if (MT::kRow) {
    streams[0] = a.drive; streams[1] = a.extra;  // MODE_ROWRES: the frames to add
  } else if (NS >= 4) {
    streams[0] = a.beta; streams[1] = a.drive; streams[2] = a.gain; streams[3] = a.vth; streams[4] = a.extra;
  } else {
    streams[0] = a.beta; streams[1] = a.drive; streams[2] = a.vth;  // (MODE_LIN: no v_th stream)
  }
  for (int i = 0; i < 5; ++i) p.s[i] = streams[i];
  for (int i = 0; i < 4; ++i) p.bias[i] = a.bias[i];
  p.channels = a.channels > 0 ? a.channels : 1; p.v_th_min = a.v_th_min;
  p.u_stats = MT::kStats ? a.u_stats : nullptr;
  p.beta_row = a.beta_row; p.vth_row = a.vth_row; p.v_init = a.v_init; p.w_init = a.w_init;
  p.spike = a.spike; p.packed = a.packed; p.vpost = a.vpost; p.w_out = a.w_out; p.ckpt = a.ckpt;
  p.ckpt_w = a.ckpt_w; p.vlast = a.vlast; p.wlast = a.wlast;
  p.T = a.T; p.cols = a.cols; p.words_per_row = (a.cols + 31) / 32;
  p.residual_compiled = a.residual_compiled;
  p.pat_in = a.pat_in; p.pat_out = a.pat_out; p.frame_dtype = a.frame_dtype;
  p.ntiles = (int)((a.T + C - 1) / C);
  p.err = device_error_word_ptr();
  p.wait_ns = get_wait_limit_ns();

  const long long nwarps = (a.cols + 32 * V - 1) / (32 * V);
  CUtensorMap tm[6];
  memset(tm, 0, sizeof tm);
  Plan plan;
  LaunchInfo& li = last_launch();
  if (TMA) {
    for (int i = 0; i < NS; ++i) {
      int r = make_tensor_map_2d(&tm[i], streams[i], Elem<ST>::kDtype, (uint64_t)a.T, (uint64_t)a.cols, C,
                                 32 * V);
      if (r != NSB_OK) return r;
    }
    if (!PACKED && a.spike) {
      int r = make_tensor_map_2d(&tm[5], a.spike, Elem<ST>::kDtype, (uint64_t)a.T, (uint64_t)a.cols, C, 32 * V);
      if (r != NSB_OK) return r;
    }
    plan = planned;
    if (plan.grid == 0) return NSB_ERR_UNSUPPORTED;
    NSB_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)plan.smem),
                 "cudaFuncSetAttribute(fwd)");
    if (int r = shrink_to_fit(kern, plan, nwarps); r != NSB_OK) return r;
  } else {
    plan.wpc = tune.warps_per_cta > 0 ? tune.warps_per_cta : 4;
    plan.stages = 1;
    plan.grid = (int)((nwarps + plan.wpc - 1) / plan.wpc);
    plan.smem = 0;
  }
  p.stages = plan.stages;
  p.defer = defer_refill(tune, plan, dev);
  // Few columns: cut the time axis into segments that run side by side (see the kernel); needs the
  // caller's scratch for the segment boundary states.
  TimeSplit ts;
  // built for: the row-parameter family, and the selective, resonate-and-fire and modulated scans of the
  // layers' hidden neurons (a single sequence is 6 144 columns there); tiled copies, one lane per thread,
  // tiles of 16 or 32 steps
  constexpr bool kSplitBuilt = (MODE == MODE_ROW || MODE == MODE_ROWRES || MODE == MODE_ROWPAT || MODE == MODE_U ||
                                MODE == MODE_RF || MODE == MODE_MOD || MODE == MODE_RFMOD) &&
                               TMA && V == 1 && (C == 16 || C == 32);
  if (kSplitBuilt && a.split_scratch)
    ts = plan_time_split(dev, a.T, a.cols, C, V, plan.wpc, false, MT::kMod ? 2 : (MT::kRow ? 0 : 1));
  const bool feedback = ts.nseg > 1 && time_split_automatic();
  if (feedback && !split_feedback_allows(a.beta_row, a.T, a.cols, false)) ts = TimeSplit();
  last_time_split() = ts;
  if (ts.nseg > 1) {
    if constexpr (kSplitBuilt) {
      auto skern = plif_fwd_split_kernel<ST, MODE, PACKED, V, C, TMA>;
      NSB_CUDA_TRY(cudaFuncSetAttribute(skern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)plan.smem),
                   "cudaFuncSetAttribute(fwd split)");
      p.nseg = ts.nseg; p.seg_tiles = ts.seg_tiles; p.warm_tiles = ts.warm_tiles;
      const size_t plane = (size_t)ts.nseg * a.cols;
      p.vspec = a.split_scratch;
      p.vend = a.split_scratch + plane;
      p.wspec = a.split_scratch + 2 * plane;
      p.wend = a.split_scratch + 3 * plane;
      p.fix_count = reinterpret_cast<unsigned int*>(a.split_scratch + (MT::kSecond ? 4 : 2) * plane);
      NSB_CUDA_TRY(cudaMemsetAsync(p.fix_count, 0, 2 * sizeof(unsigned int), a.stream), "clear the rescan counters");
      p.fixup = 0;
      skern<<<dim3(plan.grid, ts.nseg), plan.wpc * 32, plan.smem, a.stream>>>(p, tm[0], tm[1], tm[2], tm[3], tm[4], tm[5]);
      NSB_CUDA_TRY(cudaGetLastError(), "launch plif_fwd_split_kernel");
      p.fixup = 1;
      NSB_CUDA_TRY(launch_dependent(skern, dim3(plan.grid), dim3(plan.wpc * 32), plan.smem, a.stream, p, tm[0], tm[1], tm[2],
                                    tm[3], tm[4], tm[5]),
                   "launch plif_fwd_split_kernel (check)");
      if (feedback) split_feedback_record(a.beta_row, a.T, a.cols, false, p.fix_count, ts.allow_rescans, a.stream);
    }
  } else {
    // Few columns and the modulation fused in: several warps take the tiles of a column group in turn
    // (see plif_fwd_body). Built for one lane per thread, tiled copies, tiles of 8 steps.
    constexpr bool kRotBuilt = (MODE == MODE_MOD || MODE == MODE_RFMOD) && TMA && V == 1 && C == 8;
    int rot = 1;
    if constexpr (kRotBuilt) rot = plan_rotation(dev, nwarps, p.ntiles);
    [[maybe_unused]] const size_t per_warp = (plan.smem - 256) / plan.wpc;  // a warp's ring at the planned depth
    if constexpr (kRotBuilt) {
      // One CTA per column group, and all of them resident at once: a CTA walks all of T, so a second
      // round of CTAs would cost as much as the first (measured at 49 152 columns with 768 CTAs for 740
      // places: 1.42 -> 1.80 ms). Fewer warps per group until they fit.
      auto rkern = plif_fwd_rot_kernel<ST, MODE, PACKED, V, C, TMA>;
      for (; rot > 1; --rot) {
        const size_t smem = per_warp * rot + 256 + 48 + 8 * 32 * V;
        if (cudaFuncSetAttribute(rkern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
          cudaGetLastError();
          continue;
        }
        int blocks = 0;
        NSB_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, rkern, rot * 32, smem),
                     "cudaOccupancyMaxActiveBlocksPerMultiprocessor(fwd rotation)");
        if ((long long)blocks * std::max(1, dev.sm_count) >= nwarps || get_rotation_forced()) break;
      }
    }
    last_rotation() = rot;
    if (rot > 1) {
      if constexpr (kRotBuilt) {
        auto rkern = plif_fwd_rot_kernel<ST, MODE, PACKED, V, C, TMA>;
        plan.wpc = rot;
        plan.smem = per_warp * rot + 256 + 48 + 8 * 32 * V;
        plan.grid = (int)nwarps;
        p.rot = rot;
        rkern<<<plan.grid, plan.wpc * 32, plan.smem, a.stream>>>(p, tm[0], tm[1], tm[2], tm[3], tm[4], tm[5]);
        NSB_CUDA_TRY(cudaGetLastError(), "launch plif_fwd_rot_kernel");
      }
    } else {
      kern<<<plan.grid, plan.wpc * 32, plan.smem, a.stream>>>(p, tm[0], tm[1], tm[2], tm[3], tm[4], tm[5]);
      NSB_CUDA_TRY(cudaGetLastError(), "launch plif_fwd_kernel");
    }
  }
  if (MT::kStats && a.u_stats && a.alpha_out) {
    // u is never stored, so its standard deviation is taken at fp32 (no rounding to a storage dtype)
    int r = launch_alpha_finalize(a.u_stats, (int)nwarps, a.T * a.cols, NSB_F32, a.alpha0, a.sigma0, a.alpha_out,
                                  a.stream);
    if (r != NSB_OK) return r;
  }
  li.used_tma = TMA; li.warps_per_cta = plan.wpc; li.stages = plan.stages; li.lanes_per_thread = V;
  li.grid = plan.grid; li.smem_bytes = (int)plan.smem; li.tile_steps = C; li.launches = ts.nseg > 1 ? 2 : 1;
  return NSB_OK;
}

template <typename ST, int MODE, int SURR, int V, int C, bool TMA, bool HAS_GV>
int launch_bwd_impl(const BwdArgs& a, const DeviceInfo& dev, const Tuning& tune, const Plan& planned) {
  if (int r = sticky_device_error(); r != NSB_OK) return r;
  using MT = ModeTraits<MODE>;
  constexpr int NF = MT::kFwdStreams;
  auto kern = plif_bwd_kernel<ST, MODE, SURR, V, C, TMA, HAS_GV>;
  BwdParams p = {};
  const void* streams[7] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  if (MODE == MODE_ROW) {
    streams[0] = a.drive;
  } else if (NF >= 4) {
    streams[0] = a.beta; streams[1] = a.drive; streams[2] = a.gain; streams[3] = a.vth; streams[4] = a.extra;
  } else {
    streams[0] = a.beta; streams[1] = a.drive; streams[2] = a.vth;
  }
  streams[NF] = a.g_spike;
  streams[NF + 1] = a.g_vpost;
  const int has_gv = a.g_vpost != nullptr;
  const int nstreams = NF + 1 + has_gv;
  for (int i = 0; i < 7; ++i) p.s[i] = streams[i];
  for (int i = 0; i < 4; ++i) {
    p.bias[i] = a.bias[i];
    p.g_bias[i] = a.g_bias[i];
  }
  p.channels = a.channels > 0 ? a.channels : 1; p.v_th_min = a.v_th_min; p.g_extra = a.g_extra;
  p.beta_row = a.beta_row; p.vth_row = a.vth_row; p.ckpt = a.ckpt; p.ckpt_w = a.ckpt_w; p.g_winit = a.g_winit;
  p.g_beta = a.g_beta; p.g_drive = a.g_drive; p.g_gain = a.g_gain; p.g_vth = a.g_vth;
  p.g_beta_row = a.g_beta_row; p.g_vth_row = a.g_vth_row; p.g_vinit = a.g_vinit;
  p.T = a.T; p.cols = a.cols;
  p.ntiles = (int)((a.T + C - 1) / C);
  p.has_gv = has_gv; p.nstreams = nstreams; p.alpha = a.alpha; p.alpha_dev = a.alpha_dev;
  p.err = device_error_word_ptr();
  p.wait_ns = get_wait_limit_ns();

  // warps sharing one TMA box (and its shared-memory rows); the grid is counted in whole boxes
  constexpr int G = BwdBox<MODE, V, C, TMA>::kWarps;
  const long long nwarps = G * ((a.cols + 32 * V * G - 1) / (32 * V * G));
  CUtensorMap tm[12];
  memset(tm, 0, sizeof tm);
  Plan plan;
  if (TMA) {
    for (int i = 0; i < nstreams; ++i) {
      int r = make_tensor_map_2d(&tm[i], streams[i], Elem<ST>::kDtype, (uint64_t)a.T, (uint64_t)a.cols, C,
                                 32 * V * G);
      if (r != NSB_OK) return r;
    }
    const void* outs[5] = {a.g_beta, a.g_drive, a.g_gain, a.g_vth, a.g_extra};
    for (int i = 0; i < 5; ++i) {
      if (!outs[i]) continue;
      int r = make_tensor_map_2d(&tm[7 + i], outs[i], Elem<ST>::kDtype, (uint64_t)a.T, (uint64_t)a.cols, C,
                                 32 * V * G);
      if (r != NSB_OK) return r;
    }
    plan = planned;
    if (plan.grid == 0) return NSB_ERR_UNSUPPORTED;
    if (G > 1) {  // whole boxes per CTA; shared memory is per warp, so it scales with the warp count
      const size_t per_warp = (plan.smem - 256) / plan.wpc;
      // one named barrier (ids 1..15) per box and stage
      plan.wpc = std::min(G * ((plan.wpc + G - 1) / G), G * std::max(1, 15 / std::max(1, plan.stages)));
      plan.smem = per_warp * plan.wpc + 256;
      if (plan.smem > (size_t)dev.max_smem_optin) {
        plan.wpc = G;
        plan.smem = per_warp * plan.wpc + 256;
      }
      plan.grid = (int)((nwarps + plan.wpc - 1) / plan.wpc);
    }
    NSB_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)plan.smem),
                 "cudaFuncSetAttribute(bwd)");
    if (int r = shrink_to_fit(kern, plan, nwarps, G); r != NSB_OK) return r;
  } else {
    plan.wpc = tune.warps_per_cta > 0 ? std::min(tune.warps_per_cta, kBwdMaxThreads / 32) : 4;
    plan.stages = 1;
    plan.grid = (int)((nwarps + plan.wpc - 1) / plan.wpc);
    plan.smem = 0;
  }
  p.stages = plan.stages;
  p.defer = defer_refill(tune, plan, dev);
  // Few columns: the time axis cut into segments that run side by side (see the kernel)
  TimeSplit ts;
  constexpr bool kSplitBuilt = MODE == MODE_ROW && TMA && !HAS_GV && V == 1 && (C == 16 || C == 32);
  if (kSplitBuilt && a.split_scratch) ts = plan_time_split(dev, a.T, a.cols, C, V, plan.wpc, true, 0);
  const bool feedback = ts.nseg > 1 && time_split_automatic();
  if (feedback && !split_feedback_allows(a.beta_row, a.T, a.cols, true)) ts = TimeSplit();
  last_time_split() = ts;
  set_last_chain_chunks(1);
  int launched_grid = plan.grid;
  if (ts.nseg > 1) {
    if constexpr (kSplitBuilt) {
      auto skern = plif_bwd_kernel<ST, MODE, SURR, V, C, TMA, HAS_GV, true>;
      NSB_CUDA_TRY(cudaFuncSetAttribute(skern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)plan.smem),
                   "cudaFuncSetAttribute(bwd split)");
      const size_t n = (size_t)ts.nseg * a.cols;
      p.nseg = ts.nseg; p.seg_tiles = ts.seg_tiles; p.warm_tiles = ts.warm_tiles;
      p.aspec = a.split_scratch; p.aend = a.split_scratch + n;
      p.partb = a.split_scratch + 2 * n; p.partt = a.split_scratch + 3 * n;
      p.fix_count = reinterpret_cast<unsigned int*>(a.split_scratch + 4 * n);
      NSB_CUDA_TRY(cudaMemsetAsync(p.fix_count, 0, 2 * sizeof(unsigned int), a.stream), "clear the rescan counters");
      p.fixup = 0;
      skern<<<dim3(plan.grid, ts.nseg), plan.wpc * 32, plan.smem, a.stream>>>(p, tm[0], tm[1], tm[2], tm[3], tm[4], tm[5], tm[6],
                                                                                tm[7], tm[8], tm[9], tm[10], tm[11]);
      NSB_CUDA_TRY(cudaGetLastError(), "launch plif_bwd_kernel (time-split)");
      p.fixup = 1;
      NSB_CUDA_TRY(launch_dependent(skern, dim3(plan.grid), dim3(plan.wpc * 32), plan.smem, a.stream, p, tm[0], tm[1], tm[2],
                                    tm[3], tm[4], tm[5], tm[6], tm[7], tm[8], tm[9], tm[10], tm[11]),
                   "launch plif_bwd_kernel (time-split check)");
      if (feedback) split_feedback_record(a.beta_row, a.T, a.cols, true, p.fix_count, ts.allow_rescans, a.stream);
    }
  } else {
    // More CTAs than fit on the GPU at once: chunks of the time axis chained through the per-column
    // outputs (see BwdParams), so that the last round of resident CTAs is a full one.
    int chunks = 1;
    // (a row-parameter scan too wide for the time split uses its scratch for the chain)
    unsigned int* chain_sync = a.chain_sync;
    if (MODE == MODE_ROW && !chain_sync) chain_sync = reinterpret_cast<unsigned int*>(a.split_scratch);
    if constexpr (TMA) {
      const bool outputs = a.g_vinit && (!MT::kSecond || a.g_winit) &&
                           (!MT::kMod || (a.g_bias[0] && a.g_bias[1] && a.g_bias[2] && (!MT::kSecond || a.g_bias[3]))) &&
                           (MODE != MODE_ROW || (a.g_beta_row && a.g_vth_row));
      if (chain_sync && outputs) {
        bool eligible = false;  // measured, see plan_chain_chunks
        int target_steps = 128;
        if constexpr (MT::kMod) {
          int blocks = 0;
          NSB_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, kern, plan.wpc * 32, plan.smem),
                       "cudaOccupancyMaxActiveBlocksPerMultiprocessor");
          eligible = plan.grid > (long long)blocks * std::max(1, dev.sm_count);
          target_steps = 1024;
        } else if constexpr (MODE != MODE_ROW) {
          eligible = a.cols >= 49152;
          target_steps = a.cols >= 98304 ? 128 : 512;
        }
        chunks = plan_chain_chunks(eligible, p.ntiles, target_steps / C);
      }
    }
    int grid = plan.grid;
    if (chunks > 1) {
      p.chain_tiles = (p.ntiles + chunks - 1) / chunks;
      p.chain_q = (p.ntiles + p.chain_tiles - 1) / p.chain_tiles;  // no empty chunk
      p.chain_sync = chain_sync;
      NSB_CUDA_TRY(cudaMemsetAsync(chain_sync, 0, sizeof(unsigned int) * (1 + (size_t)plan.grid * plan.wpc), a.stream),
                   "clear the chain counters");
      grid = plan.grid * p.chain_q;
      set_last_chain_chunks(p.chain_q);
    }
    launched_grid = grid;
    kern<<<grid, plan.wpc * 32, plan.smem, a.stream>>>(p, tm[0], tm[1], tm[2], tm[3], tm[4], tm[5], tm[6], tm[7], tm[8],
                                                       tm[9], tm[10], tm[11]);
    NSB_CUDA_TRY(cudaGetLastError(), "launch plif_bwd_kernel");
  }
  LaunchInfo& li = last_launch();
  li.used_tma = TMA; li.warps_per_cta = plan.wpc; li.stages = plan.stages; li.lanes_per_thread = V;
  li.grid = launched_grid; li.smem_bytes = (int)plan.smem; li.tile_steps = C; li.launches = ts.nseg > 1 ? 2 : 1;
  return NSB_OK;
}

template <typename ST, int MODE, int SURR, int V, int C, bool TMA>
int launch_bwd_one(const BwdArgs& a, const DeviceInfo& dev, const Tuning& tune, const Plan& planned) {
  return a.g_vpost ? launch_bwd_impl<ST, MODE, SURR, V, C, TMA, true>(a, dev, tune, planned)
                   : launch_bwd_impl<ST, MODE, SURR, V, C, TMA, false>(a, dev, tune, planned);
}

// The TMA path needs 16-byte aligned bases and row pitch, int32 coordinates and
// an sm_100 device; anything else takes the direct-load kernel.
template <typename ST>
inline bool tma_ok_common(const DeviceInfo& dev, long long T, long long cols, const Tuning& tune) {
  if (tune.force_direct == 1) return false;
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
  const void* ptrs[] = {a.beta, a.drive, a.gain, a.vth, a.spike, a.vpost, a.ckpt, a.w_out, a.ckpt_w};
  for (const void* q : ptrs) tma = tma && aligned16(q);
  const bool packed = a.packed != nullptr;
  const int C = a.tile;
  Plan plan;
  if (tma) {
    PlanQuery q;
    q.T = a.T; q.cols = a.cols; q.elem_size = (int)sizeof(ST);
    q.nstreams = a.mode == MODE_ROW ? 1 : ((a.mode == MODE_AI || a.mode == MODE_RF) ? 4 : 3);
    q.tile = C; q.backward = false; q.max_lanes = C == 32 ? 1 : 4;  // 32-step tiles: 1 lane per thread only
    plan = plan_scan(dev, q, tune);
    if (plan.grid == 0) return NSB_ERR_UNSUPPORTED;  // the tuning override admits no launch shape
  }
  const int V = plan.lanes;

#define NSB_FWD_CASE(MODE_, PACKED_, V_, C_)                                           \
  if (a.mode == MODE_ && packed == PACKED_ && V == V_ && C == C_)                      \
    return launch_fwd_one<ST, MODE_, PACKED_, V_, C_, true>(a, dev, tune, plan);
#define NSB_FWD_CASES_V(MODE_, PACKED_)                                                \
  NSB_FWD_CASE(MODE_, PACKED_, 1, 8) NSB_FWD_CASE(MODE_, PACKED_, 2, 8)                \
  NSB_FWD_CASE(MODE_, PACKED_, 4, 8) NSB_FWD_CASE(MODE_, PACKED_, 1, 16)               \
  NSB_FWD_CASE(MODE_, PACKED_, 2, 16) NSB_FWD_CASE(MODE_, PACKED_, 4, 16)              \
  NSB_FWD_CASE(MODE_, PACKED_, 1, 32)
  if (tma) {
    NSB_FWD_CASES_V(MODE_U, false) NSB_FWD_CASES_V(MODE_U, true)
    NSB_FWD_CASES_V(MODE_AI, false) NSB_FWD_CASES_V(MODE_AI, true)
    NSB_FWD_CASES_V(MODE_ROW, false) NSB_FWD_CASES_V(MODE_ROW, true)
    NSB_FWD_CASES_V(MODE_RF, false) NSB_FWD_CASES_V(MODE_RF, true)
    return NSB_ERR_INVALID_ARG;
  }
#undef NSB_FWD_CASES_V
#undef NSB_FWD_CASE
#define NSB_FWD_DIRECT(MODE_, C_)                                                      \
  if (a.mode == MODE_ && C == C_)                                                      \
    return packed ? launch_fwd_one<ST, MODE_, true, 1, C_, false>(a, dev, tune, plan)  \
                  : launch_fwd_one<ST, MODE_, false, 1, C_, false>(a, dev, tune, plan);
  NSB_FWD_DIRECT(MODE_U, 8) NSB_FWD_DIRECT(MODE_U, 16)
  NSB_FWD_DIRECT(MODE_AI, 8) NSB_FWD_DIRECT(MODE_AI, 16)
  NSB_FWD_DIRECT(MODE_ROW, 8) NSB_FWD_DIRECT(MODE_ROW, 16)
  NSB_FWD_DIRECT(MODE_RF, 8) NSB_FWD_DIRECT(MODE_RF, 16)
  NSB_FWD_DIRECT(MODE_U, 32) NSB_FWD_DIRECT(MODE_AI, 32) NSB_FWD_DIRECT(MODE_ROW, 32) NSB_FWD_DIRECT(MODE_RF, 32)
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
  const void* ptrs[] = {a.beta, a.drive, a.gain, a.vth, a.ckpt, a.ckpt_w, a.g_spike, a.g_vpost,
                        a.g_beta, a.g_drive, a.g_gain, a.g_vth};
  for (const void* q : ptrs) tma = tma && aligned16(q);
  const int C = a.tile;
  Plan plan;
  if (tma) {
    // resonate-and-fire with enough columns to fill the GPU: 2 lanes per thread as pairs of warps
    // per TMA box, two boxes per CTA, 3-deep ring (measured best, see BwdBox)
    Tuning tune_rf = tune;
    if (a.mode == MODE_RF && C == 8 && !a.g_vpost && tune.lanes_per_thread <= 0 &&
        a.cols >= 64LL * 8 * std::max(1, dev.sm_count)) {
      tune_rf.lanes_per_thread = 2;
      if (tune_rf.warps_per_cta <= 0) tune_rf.warps_per_cta = 4;
      if (tune_rf.stages <= 0) tune_rf.stages = 3;
    }
    PlanQuery q;
    q.T = a.T; q.cols = a.cols; q.elem_size = (int)sizeof(ST);
    q.nstreams = (a.mode == MODE_ROW ? 1 : ((a.mode == MODE_AI || a.mode == MODE_RF) ? 4 : 3)) + 1 + (a.g_vpost ? 1 : 0);
    q.tile = C; q.backward = true; q.max_lanes = C == 8 ? 4 : (C == 16 ? 2 : 1);
    plan = plan_scan(dev, q, tune_rf);
    if (plan.grid == 0) return NSB_ERR_UNSUPPORTED;  // the tuning override admits no launch shape
  }
  const int V = plan.lanes;

#define NSB_BWD_CASE(MODE_, SURR_, V_, C_)                                             \
  if (a.mode == MODE_ && a.surrogate == SURR_ && V == V_ && C == C_)                   \
    return launch_bwd_one<ST, MODE_, SURR_, V_, C_, true>(a, dev, tune, plan);
#define NSB_BWD_CASES_V(MODE_, SURR_)                                                  \
  NSB_BWD_CASE(MODE_, SURR_, 1, 8) NSB_BWD_CASE(MODE_, SURR_, 2, 8)                    \
  NSB_BWD_CASE(MODE_, SURR_, 4, 8) NSB_BWD_CASE(MODE_, SURR_, 1, 16)                   \
  NSB_BWD_CASE(MODE_, SURR_, 2, 16) NSB_BWD_CASE(MODE_, SURR_, 1, 32)
#define NSB_BWD_CASES_RF(SURR_)                                                         \
  NSB_BWD_CASE(MODE_RF, SURR_, 1, 8) NSB_BWD_CASE(MODE_RF, SURR_, 2, 8)                \
  NSB_BWD_CASE(MODE_RF, SURR_, 4, 8) NSB_BWD_CASE(MODE_RF, SURR_, 1, 16)               \
  NSB_BWD_CASE(MODE_RF, SURR_, 2, 16) NSB_BWD_CASE(MODE_RF, SURR_, 1, 32)
  if (tma) {
    NSB_BWD_CASES_V(MODE_U, NSB_SURR_SIGMOID) NSB_BWD_CASES_V(MODE_U, NSB_SURR_ATAN)
    NSB_BWD_CASES_V(MODE_AI, NSB_SURR_SIGMOID) NSB_BWD_CASES_V(MODE_AI, NSB_SURR_ATAN)
    NSB_BWD_CASES_V(MODE_ROW, NSB_SURR_SIGMOID) NSB_BWD_CASES_V(MODE_ROW, NSB_SURR_ATAN)
    NSB_BWD_CASES_RF(NSB_SURR_SIGMOID) NSB_BWD_CASES_RF(NSB_SURR_ATAN)
    return NSB_ERR_INVALID_ARG;
  }
#undef NSB_BWD_CASES_V
#undef NSB_BWD_CASES_RF
#undef NSB_BWD_CASE
#define NSB_BWD_DIRECT(MODE_, SURR_, C_)                                               \
  if (a.mode == MODE_ && a.surrogate == SURR_ && C == C_)                              \
    return launch_bwd_one<ST, MODE_, SURR_, 1, C_, false>(a, dev, tune, plan);
#define NSB_BWD_DIRECT_S(MODE_)                                                        \
  NSB_BWD_DIRECT(MODE_, NSB_SURR_SIGMOID, 8) NSB_BWD_DIRECT(MODE_, NSB_SURR_SIGMOID, 16) \
  NSB_BWD_DIRECT(MODE_, NSB_SURR_ATAN, 8) NSB_BWD_DIRECT(MODE_, NSB_SURR_ATAN, 16)       \
  NSB_BWD_DIRECT(MODE_, NSB_SURR_SIGMOID, 32) NSB_BWD_DIRECT(MODE_, NSB_SURR_ATAN, 32)
  NSB_BWD_DIRECT_S(MODE_U) NSB_BWD_DIRECT_S(MODE_AI) NSB_BWD_DIRECT_S(MODE_ROW) NSB_BWD_DIRECT_S(MODE_RF)
#undef NSB_BWD_DIRECT_S
#undef NSB_BWD_DIRECT
  return NSB_ERR_INVALID_ARG;
}

// Modulated modes: tiles of 8 steps (1, 2 or 4 lanes per thread) or 32 steps (1 lane); the
// fused scan returns spikes only, so there is no V_post gradient stream.
template <typename ST>
int scan_mod_fwd_dispatch(const FwdArgs& a) {
  DeviceInfo dev;
  int r = get_device_info(&dev);
  if (r != NSB_OK) return r;
  if (dev.cc_major != 10) return NSB_ERR_UNSUPPORTED;
  Tuning tune = get_tuning();
  // Measured launch shapes between the few-column regime and a full GPU (B200, bf16, T = 8192, 8-step tiles).
  // 49 152 columns (the hidden layer of the 768-wide model at batch 8): 1 lane, 4 warps per CTA, 3 stages:
  // resonate-and-fire 1.42 ms against 2.01 for the 2-lane single-warp CTAs the cost model picks, first
  // order 0.93 against 1.16. 98 304 columns: 2 lanes, 4 warps: 2.43 against 3.15 ms (4 lanes, 1 warp) and
  // 1.45 against 1.62.
  if (a.tile == 8 && tune.lanes_per_thread <= 0 && tune.warps_per_cta <= 0 && tune.stages <= 0 && a.cols > 32768) {
    const long long sms = std::max(1, dev.sm_count);
    if (a.cols < 512 * sms) {
      tune.lanes_per_thread = 1; tune.warps_per_cta = 4; tune.stages = 3;
    } else if (a.cols < 1328 * sms) {
      tune.lanes_per_thread = 2; tune.warps_per_cta = 4; tune.stages = a.mode == MODE_RFMOD ? 2 : 3;
    }
  }
  // Fewer columns, 8-step tiles, no moments of u: one lane per thread, which is what the rotation among
  // warps is built for (see plif_fwd_body).
  if (a.tile == 8 && tune.lanes_per_thread <= 0 && a.cols <= 32768 && !a.u_stats) tune.lanes_per_thread = 1;
  bool tma = tma_ok_common<ST>(dev, a.T, a.cols, tune);
  const void* ptrs[] = {a.beta, a.drive, a.gain, a.vth, a.extra, a.spike, a.ckpt, a.ckpt_w};
  for (const void* q : ptrs) tma = tma && aligned16(q);
  const bool packed = a.packed != nullptr;
  const int C = a.tile;
  Plan plan;
  if (tma) {
    PlanQuery q;
    q.T = a.T; q.cols = a.cols; q.elem_size = (int)sizeof(ST);
    q.nstreams = a.mode == MODE_RFMOD ? 5 : 4;
    q.modulated = a.mode == MODE_RFMOD ? 2 : 1;
    q.tile = C; q.backward = false; q.max_lanes = C == 32 ? 1 : 4;
    plan = plan_scan(dev, q, tune);
    if (plan.grid == 0) return NSB_ERR_UNSUPPORTED;  // the tuning override admits no launch shape
  }
  const int V = plan.lanes;
#define NSB_MFWD_CASE(MODE_, PACKED_, V_, C_)                                          \
  if (a.mode == MODE_ && packed == PACKED_ && V == V_ && C == C_)                      \
    return launch_fwd_one<ST, MODE_, PACKED_, V_, C_, true>(a, dev, tune, plan);
#define NSB_MFWD_CASES(MODE_, PACKED_)                                                 \
  NSB_MFWD_CASE(MODE_, PACKED_, 1, 8) NSB_MFWD_CASE(MODE_, PACKED_, 2, 8)              \
  NSB_MFWD_CASE(MODE_, PACKED_, 4, 8) NSB_MFWD_CASE(MODE_, PACKED_, 1, 32)
#define NSB_MFWD_STATS(MODE_, SMODE_, V_, C_)                                          \
  if (a.mode == MODE_ && V == V_ && C == C_)                                           \
    return launch_fwd_one<ST, SMODE_, false, V_, C_, true>(a, dev, tune, plan);
#define NSB_MFWD_STATS_V(MODE_, SMODE_)                                                \
  NSB_MFWD_STATS(MODE_, SMODE_, 1, 8) NSB_MFWD_STATS(MODE_, SMODE_, 2, 8)              \
  NSB_MFWD_STATS(MODE_, SMODE_, 4, 8) NSB_MFWD_STATS(MODE_, SMODE_, 1, 32)
  if (tma && a.u_stats) {  // also accumulate the moments of u (dense spikes only)
    if (packed) return NSB_ERR_INVALID_ARG;
    NSB_MFWD_STATS_V(MODE_MOD, MODE_MODS) NSB_MFWD_STATS_V(MODE_RFMOD, MODE_RFMODS)
    return NSB_ERR_INVALID_ARG;
  }
#undef NSB_MFWD_STATS_V
#undef NSB_MFWD_STATS
  if (tma) {
    NSB_MFWD_CASES(MODE_MOD, false) NSB_MFWD_CASES(MODE_MOD, true)
    NSB_MFWD_CASES(MODE_RFMOD, false) NSB_MFWD_CASES(MODE_RFMOD, true)
    return NSB_ERR_INVALID_ARG;
  }
#undef NSB_MFWD_CASES
#undef NSB_MFWD_CASE
#define NSB_MFWD_DIRECT(MODE_, C_)                                                     \
  if (a.mode == MODE_ && C == C_)                                                      \
    return packed ? launch_fwd_one<ST, MODE_, true, 1, C_, false>(a, dev, tune, plan)  \
                  : launch_fwd_one<ST, MODE_, false, 1, C_, false>(a, dev, tune, plan);
  if (a.u_stats) {
    if (packed) return NSB_ERR_INVALID_ARG;
    if (a.mode == MODE_MOD && C == 8) return launch_fwd_one<ST, MODE_MODS, false, 1, 8, false>(a, dev, tune, plan);
    if (a.mode == MODE_MOD && C == 32) return launch_fwd_one<ST, MODE_MODS, false, 1, 32, false>(a, dev, tune, plan);
    if (a.mode == MODE_RFMOD && C == 8) return launch_fwd_one<ST, MODE_RFMODS, false, 1, 8, false>(a, dev, tune, plan);
    if (a.mode == MODE_RFMOD && C == 32) return launch_fwd_one<ST, MODE_RFMODS, false, 1, 32, false>(a, dev, tune, plan);
    return NSB_ERR_INVALID_ARG;
  }
  NSB_MFWD_DIRECT(MODE_MOD, 8) NSB_MFWD_DIRECT(MODE_MOD, 32)
  NSB_MFWD_DIRECT(MODE_RFMOD, 8) NSB_MFWD_DIRECT(MODE_RFMOD, 32)
#undef NSB_MFWD_DIRECT
  return NSB_ERR_INVALID_ARG;
}

// Row-parameter scan + binary residual (MODE_ROWRES): tiles of 16 steps (one token; 1, 2 or 4
// lanes per thread) or 32 steps (1 lane).
template <typename ST>
int scan_res_fwd_dispatch(const FwdArgs& a) {
  DeviceInfo dev;
  int r = get_device_info(&dev);
  if (r != NSB_OK) return r;
  if (dev.cc_major != 10) return NSB_ERR_UNSUPPORTED;
  const Tuning tune = get_tuning();
  bool tma = tma_ok_common<ST>(dev, a.T, a.cols, tune);
  const void* ptrs[] = {a.drive, a.extra, a.spike, a.ckpt};
  for (const void* q : ptrs) tma = tma && aligned16(q);
  const int C = a.tile;
  Plan plan;
  if (tma) {
    PlanQuery q;
    q.T = a.T; q.cols = a.cols; q.elem_size = (int)sizeof(ST);
    q.nstreams = 2;
    q.tile = C; q.backward = false; q.max_lanes = C == 32 ? 1 : 4;
    plan = plan_scan(dev, q, tune);
    if (plan.grid == 0) return NSB_ERR_UNSUPPORTED;  // the tuning override admits no launch shape
  }
  const int V = plan.lanes;
#define NSB_RFWD_CASE(V_, C_)                                                          \
  if (V == V_ && C == C_) return launch_fwd_one<ST, MODE_ROWRES, false, V_, C_, true>(a, dev, tune, plan);
  if (tma) {
    NSB_RFWD_CASE(1, 16) NSB_RFWD_CASE(2, 16) NSB_RFWD_CASE(4, 16) NSB_RFWD_CASE(1, 32)
    return NSB_ERR_INVALID_ARG;
  }
#undef NSB_RFWD_CASE
  if (C == 16) return launch_fwd_one<ST, MODE_ROWRES, false, 1, 16, false>(a, dev, tune, plan);
  if (C == 32) return launch_fwd_one<ST, MODE_ROWRES, false, 1, 32, false>(a, dev, tune, plan);
  return NSB_ERR_INVALID_ARG;
}

// Row-parameter scan with spikes packed in time (MODE_ROWPAT): as the residual scan, one streamed input.
template <typename ST>
int scan_pat_fwd_dispatch(const FwdArgs& a) {
  DeviceInfo dev;
  int r = get_device_info(&dev);
  if (r != NSB_OK) return r;
  if (dev.cc_major != 10) return NSB_ERR_UNSUPPORTED;
  const Tuning tune = get_tuning();
  bool tma = tma_ok_common<ST>(dev, a.T, a.cols, tune);
  // a thread moves its V patterns with one access: the pattern rows must keep V*2-byte alignment
  tma = tma && aligned16(a.drive) && aligned16(a.ckpt) && a.cols % 8 == 0 &&
        (reinterpret_cast<uintptr_t>(a.pat_out) % 8 == 0) && (reinterpret_cast<uintptr_t>(a.pat_in) % 8 == 0);
  const int C = a.tile;
  Plan plan;
  if (tma) {
    PlanQuery q;
    q.T = a.T; q.cols = a.cols; q.elem_size = (int)sizeof(ST);
    q.nstreams = 1;
    q.tile = C; q.backward = false; q.max_lanes = C == 32 ? 1 : 4;
    plan = plan_scan(dev, q, tune);
    if (plan.grid == 0) return NSB_ERR_UNSUPPORTED;  // the tuning override admits no launch shape
  }
  const int V = plan.lanes;
#define NSB_PFWD_CASE(V_, C_)                                                          \
  if (V == V_ && C == C_) return launch_fwd_one<ST, MODE_ROWPAT, true, V_, C_, true>(a, dev, tune, plan);
  if (tma) {
    NSB_PFWD_CASE(1, 16) NSB_PFWD_CASE(2, 16) NSB_PFWD_CASE(4, 16) NSB_PFWD_CASE(1, 32)
    return NSB_ERR_INVALID_ARG;
  }
#undef NSB_PFWD_CASE
  if (C == 16) return launch_fwd_one<ST, MODE_ROWPAT, true, 1, 16, false>(a, dev, tune, plan);
  if (C == 32) return launch_fwd_one<ST, MODE_ROWPAT, true, 1, 32, false>(a, dev, tune, plan);
  return NSB_ERR_INVALID_ARG;
}

// Linear recurrence (MODE_LIN): tiles of 8 steps (1, 2 or 4 lanes per thread) or 32 steps (1 lane).
template <typename ST>
int scan_lin_fwd_dispatch(const FwdArgs& a) {
  DeviceInfo dev;
  int r = get_device_info(&dev);
  if (r != NSB_OK) return r;
  if (dev.cc_major != 10) return NSB_ERR_UNSUPPORTED;
  const Tuning tune = get_tuning();
  bool tma = tma_ok_common<ST>(dev, a.T, a.cols, tune);
  const void* ptrs[] = {a.beta, a.drive, a.spike, a.vpost, a.ckpt};
  for (const void* q : ptrs) tma = tma && aligned16(q);
  const int C = a.tile;
  Plan plan;
  if (tma) {
    PlanQuery q;
    q.T = a.T; q.cols = a.cols; q.elem_size = (int)sizeof(ST);
    q.nstreams = 2;
    q.tile = C; q.backward = false; q.max_lanes = C == 32 ? 1 : 4;
    plan = plan_scan(dev, q, tune);
    if (plan.grid == 0) return NSB_ERR_UNSUPPORTED;  // the tuning override admits no launch shape
  }
  const int V = plan.lanes;
#define NSB_LFWD_CASE(V_, C_)                                                          \
  if (V == V_ && C == C_) return launch_fwd_one<ST, MODE_LIN, false, V_, C_, true>(a, dev, tune, plan);
  if (tma) {
    NSB_LFWD_CASE(1, 8) NSB_LFWD_CASE(2, 8) NSB_LFWD_CASE(4, 8) NSB_LFWD_CASE(1, 32)
    return NSB_ERR_INVALID_ARG;
  }
#undef NSB_LFWD_CASE
  if (C == 8) return launch_fwd_one<ST, MODE_LIN, false, 1, 8, false>(a, dev, tune, plan);
  if (C == 32) return launch_fwd_one<ST, MODE_LIN, false, 1, 32, false>(a, dev, tune, plan);
  return NSB_ERR_INVALID_ARG;
}

template <typename ST>
int scan_lin_bwd_dispatch(const BwdArgs& a) {
  DeviceInfo dev;
  int r = get_device_info(&dev);
  if (r != NSB_OK) return r;
  if (dev.cc_major != 10) return NSB_ERR_UNSUPPORTED;
  if (a.g_vpost) return NSB_ERR_INVALID_ARG;
  const Tuning tune = get_tuning();
  bool tma = tma_ok_common<ST>(dev, a.T, a.cols, tune);
  const void* ptrs[] = {a.beta, a.drive, a.ckpt, a.g_spike, a.g_beta, a.g_drive};
  for (const void* q : ptrs) tma = tma && aligned16(q);
  const int C = a.tile;
  Plan plan;
  if (tma) {
    PlanQuery q;
    q.T = a.T; q.cols = a.cols; q.elem_size = (int)sizeof(ST);
    q.nstreams = 3;
    q.tile = C; q.backward = true; q.max_lanes = C == 8 ? 4 : 1;
    plan = plan_scan(dev, q, tune);
    if (plan.grid == 0) return NSB_ERR_UNSUPPORTED;  // the tuning override admits no launch shape
  }
  const int V = plan.lanes;
#define NSB_LBWD_CASE(V_, C_)                                                          \
  if (V == V_ && C == C_)                                                              \
    return launch_bwd_impl<ST, MODE_LIN, NSB_SURR_SIGMOID, V_, C_, true, false>(a, dev, tune, plan);
  if (tma) {
    NSB_LBWD_CASE(1, 8) NSB_LBWD_CASE(2, 8) NSB_LBWD_CASE(4, 8) NSB_LBWD_CASE(1, 32)
    return NSB_ERR_INVALID_ARG;
  }
#undef NSB_LBWD_CASE
  if (C == 8) return launch_bwd_impl<ST, MODE_LIN, NSB_SURR_SIGMOID, 1, 8, false, false>(a, dev, tune, plan);
  if (C == 32) return launch_bwd_impl<ST, MODE_LIN, NSB_SURR_SIGMOID, 1, 32, false, false>(a, dev, tune, plan);
  return NSB_ERR_INVALID_ARG;
}

template <typename ST>
int scan_mod_bwd_dispatch(const BwdArgs& a) {
  DeviceInfo dev;
  int r = get_device_info(&dev);
  if (r != NSB_OK) return r;
  if (dev.cc_major != 10) return NSB_ERR_UNSUPPORTED;
  if (a.g_vpost) return NSB_ERR_INVALID_ARG;
  Tuning tune = get_tuning();
  // built for at most 2 lanes per thread (8-step tiles) / 1 lane (32-step tiles)
  tune.lanes_per_thread = std::min(tune.lanes_per_thread, a.tile == 8 ? 2 : 1);
  bool tma = tma_ok_common<ST>(dev, a.T, a.cols, tune);
  const void* ptrs[] = {a.beta, a.drive, a.gain, a.vth, a.extra, a.ckpt, a.ckpt_w, a.g_spike,
                        a.g_beta, a.g_drive, a.g_gain, a.g_vth, a.g_extra};
  for (const void* q : ptrs) tma = tma && aligned16(q);
  const int C = a.tile;
  Plan plan;
  if (tma) {
    PlanQuery q;
    q.T = a.T; q.cols = a.cols; q.elem_size = (int)sizeof(ST);
    q.nstreams = (a.mode == MODE_RFMOD ? 5 : 4) + 1;
    q.stash = a.mode == MODE_RFMOD ? 5 : 3;
    if (a.mode == MODE_RFMOD && sizeof(ST) == 2) q.stash_2lanes = 3;  // two of the five live in dead input slots
    q.modulated = a.mode == MODE_RFMOD ? 2 : 1;
    // 4 lanes per thread spill heavily with the modulation's extra live values (measured 3x slower)
    q.tile = C; q.backward = true; q.max_lanes = C == 8 ? 2 : 1;
    // The 2-lane kernels work in pairs of warps per TMA box. With enough columns to fill the GPU,
    // two boxes per CTA and a 2-deep ring measured best (B=32, T=8192, D=6144, bf16: first order
    // 5.58 ms against 6.2 ms for 1 or 4 boxes per CTA or a 3-deep ring; resonate-and-fire 9.7 ms
    // against 9.8-11.5 ms).
    if (C == 8 && tune.lanes_per_thread != 1 && a.cols >= 64LL * 8 * std::max(1, dev.sm_count)) {
      if (tune.warps_per_cta <= 0) tune.warps_per_cta = 4;
      if (tune.stages <= 0) tune.stages = 2;
    } else if (C == 8 && tune.lanes_per_thread <= 0 && tune.warps_per_cta <= 0 && tune.stages <= 0 && a.cols > 32768) {
      // fewer columns (49 152, same sizes): 1 lane, 4 warps per CTA: 3.00 ms against 3.23 (resonate-and-fire),
      // 2.05 against 2.11 (first order) for the cost model's 2 lanes in 2-warp CTAs
      tune.lanes_per_thread = 1; tune.warps_per_cta = 4; tune.stages = 2;
    }
    plan = plan_scan(dev, q, tune);
    if (plan.grid == 0) return NSB_ERR_UNSUPPORTED;  // the tuning override admits no launch shape
  }
  const int V = plan.lanes;
#define NSB_MBWD_CASE(MODE_, SURR_, V_, C_)                                            \
  if (a.mode == MODE_ && a.surrogate == SURR_ && V == V_ && C == C_)                   \
    return launch_bwd_impl<ST, MODE_, SURR_, V_, C_, true, false>(a, dev, tune, plan);
#define NSB_MBWD_CASES(MODE_, SURR_)                                                   \
  NSB_MBWD_CASE(MODE_, SURR_, 1, 8) NSB_MBWD_CASE(MODE_, SURR_, 2, 8)                  \
  NSB_MBWD_CASE(MODE_, SURR_, 1, 32)
  if (tma) {
    NSB_MBWD_CASES(MODE_MOD, NSB_SURR_SIGMOID) NSB_MBWD_CASES(MODE_MOD, NSB_SURR_ATAN)
    NSB_MBWD_CASES(MODE_RFMOD, NSB_SURR_SIGMOID) NSB_MBWD_CASES(MODE_RFMOD, NSB_SURR_ATAN)
    return NSB_ERR_INVALID_ARG;
  }
#undef NSB_MBWD_CASES
#undef NSB_MBWD_CASE
#define NSB_MBWD_DIRECT(MODE_, SURR_, C_)                                              \
  if (a.mode == MODE_ && a.surrogate == SURR_ && C == C_)                              \
    return launch_bwd_impl<ST, MODE_, SURR_, 1, C_, false, false>(a, dev, tune, plan);
  NSB_MBWD_DIRECT(MODE_MOD, NSB_SURR_SIGMOID, 8) NSB_MBWD_DIRECT(MODE_MOD, NSB_SURR_ATAN, 8)
  NSB_MBWD_DIRECT(MODE_MOD, NSB_SURR_SIGMOID, 32) NSB_MBWD_DIRECT(MODE_MOD, NSB_SURR_ATAN, 32)
  NSB_MBWD_DIRECT(MODE_RFMOD, NSB_SURR_SIGMOID, 8) NSB_MBWD_DIRECT(MODE_RFMOD, NSB_SURR_ATAN, 8)
  NSB_MBWD_DIRECT(MODE_RFMOD, NSB_SURR_SIGMOID, 32) NSB_MBWD_DIRECT(MODE_RFMOD, NSB_SURR_ATAN, 32)
#undef NSB_MBWD_DIRECT
  return NSB_ERR_INVALID_ARG;
}

#endif  // __CUDACC__

}  // namespace nsb
