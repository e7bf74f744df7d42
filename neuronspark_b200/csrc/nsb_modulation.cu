// Stand-alone modulation kernel: raw projections + per-channel biases -> beta, u, v_th
// (, omega), written out. The fused scans (nsb_plif_modulated_fwd / _bwd) never materialise
// these tensors; this entry exists for callers that want them (inference code that keeps the
// unfused scan, tests that compare the fused scan against modulation + plain scan).
//
// One thread owns VE consecutive channels of one row; pure streaming.
#include <initializer_list>

#include "nsb_common.cuh"
#include "nsb_modulation.cuh"

namespace nsb {
namespace {

template <typename TI, typename TO, int VE, bool RF>
__global__ void modulation_fwd_kernel(const TI* __restrict__ raw_beta, const TI* __restrict__ raw_alpha,
                                      const TI* __restrict__ raw_th, const TI* __restrict__ raw_omega,
                                      const TI* __restrict__ cur, const float* __restrict__ b_beta,
                                      const float* __restrict__ b_alpha, const float* __restrict__ b_th,
                                      const float* __restrict__ b_omega, float v_th_min, long long rows,
                                      long long ch, TO* __restrict__ beta, TO* __restrict__ u,
                                      TO* __restrict__ vth, TO* __restrict__ omega) {
  const long long cv = ch / VE;
  const long long total = rows * cv;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long c = (idx % cv) * VE;
    const long long off = (idx / cv) * ch + c;
    const Vec<TI, VE> rb = *reinterpret_cast<const Vec<TI, VE>*>(raw_beta + off);
    const Vec<TI, VE> ra = *reinterpret_cast<const Vec<TI, VE>*>(raw_alpha + off);
    const Vec<TI, VE> rt = *reinterpret_cast<const Vec<TI, VE>*>(raw_th + off);
    const Vec<TI, VE> ci = *reinterpret_cast<const Vec<TI, VE>*>(cur + off);
    Vec<TI, VE> ro;
    if constexpr (RF) ro = *reinterpret_cast<const Vec<TI, VE>*>(raw_omega + off);
    Vec<TO, VE> ob, ou, ot, oo;
    float b[VE], a[VE], th[VE], om[VE], dr[VE], q0[VE], q1[VE], q2[VE], q3[VE], q4[VE];
    mod::Bias<VE> bias;
#pragma unroll
    for (int j = 0; j < VE; ++j) {
      b[j] = Elem<TI>::to_f32(rb.v[j]);
      a[j] = Elem<TI>::to_f32(ra.v[j]);
      th[j] = Elem<TI>::to_f32(rt.v[j]);
      om[j] = RF ? Elem<TI>::to_f32(ro.v[j]) : 0.0f;
      dr[j] = Elem<TI>::to_f32(ci.v[j]);
      bias.beta[j] = b_beta[c + j];
      bias.alpha[j] = b_alpha[c + j];
      bias.th[j] = b_th[c + j];
      bias.omega[j] = RF ? b_omega[c + j] : 0.0f;
    }
    mod::forward_lanes<RF, VE>(b, a, th, om, dr, bias, v_th_min, q0, q1, q2, q3, q4);
#pragma unroll
    for (int j = 0; j < VE; ++j) {
      ob.v[j] = Elem<TO>::from_f32(b[j]);
      ou.v[j] = Elem<TO>::from_f32(dr[j]);
      ot.v[j] = Elem<TO>::from_f32(th[j]);
      if constexpr (RF) oo.v[j] = Elem<TO>::from_f32(om[j]);
    }
    *reinterpret_cast<Vec<TO, VE>*>(beta + off) = ob;
    *reinterpret_cast<Vec<TO, VE>*>(u + off) = ou;
    *reinterpret_cast<Vec<TO, VE>*>(vth + off) = ot;
    if constexpr (RF) *reinterpret_cast<Vec<TO, VE>*>(omega + off) = oo;
  }
}

template <typename TI, typename TO>
int launch_modulation(const void* raw_beta, const void* raw_alpha, const void* raw_th, const void* raw_omega,
                      const void* cur, const float* b_beta, const float* b_alpha, const float* b_th,
                      const float* b_omega, float v_th_min, long long rows, long long ch, void* beta, void* u,
                      void* vth, void* omega, cudaStream_t st) {
  DeviceInfo dev;
  int r = get_device_info(&dev);
  if (r != NSB_OK) return r;
  const bool rf = raw_omega != nullptr;
  // 4 channels per thread when the channel count and every pointer allow 4-wide vectors
  bool v4 = ch % 4 == 0;
  for (const void* p : {raw_beta, raw_alpha, raw_th, raw_omega, cur})
    v4 = v4 && reinterpret_cast<uintptr_t>(p) % (4 * sizeof(TI)) == 0;
  for (const void* p : {(const void*)beta, (const void*)u, (const void*)vth, (const void*)omega})
    v4 = v4 && reinterpret_cast<uintptr_t>(p) % (4 * sizeof(TO)) == 0;
  const long long items = rows * (ch / (v4 ? 4 : 1));
  const int threads = 256;
  long long blocks = (items + threads - 1) / threads;
  blocks = std::max<long long>(1, std::min<long long>(blocks, (long long)dev.sm_count * 16));
#define NSB_MOD_LAUNCH(VE_, RF_)                                                                         \
  modulation_fwd_kernel<TI, TO, VE_, RF_><<<(int)blocks, threads, 0, st>>>(                              \
      static_cast<const TI*>(raw_beta), static_cast<const TI*>(raw_alpha), static_cast<const TI*>(raw_th), \
      static_cast<const TI*>(raw_omega), static_cast<const TI*>(cur), b_beta, b_alpha, b_th, b_omega,    \
      v_th_min, rows, ch, static_cast<TO*>(beta), static_cast<TO*>(u), static_cast<TO*>(vth),            \
      static_cast<TO*>(omega))
  if (v4) {
    if (rf) NSB_MOD_LAUNCH(4, true); else NSB_MOD_LAUNCH(4, false);
  } else {
    if (rf) NSB_MOD_LAUNCH(1, true); else NSB_MOD_LAUNCH(1, false);
  }
#undef NSB_MOD_LAUNCH
  NSB_CUDA_TRY(cudaGetLastError(), "launch modulation_fwd_kernel");
  return NSB_OK;
}

}  // namespace
}  // namespace nsb

using namespace nsb;

extern "C" int nsb_modulation_fwd(const void* raw_beta, const void* raw_alpha, const void* raw_th,
                                  const void* raw_omega, const void* cur, const float* b_beta,
                                  const float* b_alpha, const float* b_th, const float* b_omega,
                                  float v_th_min, int64_t rows, int64_t channels, void* beta, void* u,
                                  void* v_th, void* omega, int dtype_in, int dtype_out, void* stream) {
  auto ok = [](int d) { return d == NSB_F32 || d == NSB_BF16 || d == NSB_F16; };
  if (rows < 0 || channels <= 0 || !ok(dtype_in) || !ok(dtype_out)) return NSB_ERR_INVALID_ARG;
  if (rows == 0) return NSB_OK;
  if (!raw_beta || !raw_alpha || !raw_th || !cur || !b_beta || !b_alpha || !b_th || !beta || !u || !v_th)
    return NSB_ERR_INVALID_ARG;
  if ((raw_omega != nullptr) != (b_omega != nullptr) || (raw_omega != nullptr) != (omega != nullptr))
    return NSB_ERR_INVALID_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
#define NSB_MOD_GO(TI, TO)                                                                              \
  return launch_modulation<TI, TO>(raw_beta, raw_alpha, raw_th, raw_omega, cur, b_beta, b_alpha, b_th,  \
                                   b_omega, v_th_min, rows, channels, beta, u, v_th, omega, st)
  if (dtype_out == NSB_F32) {
    if (dtype_in == NSB_F32) NSB_MOD_GO(float, float);
    if (dtype_in == NSB_BF16) NSB_MOD_GO(__nv_bfloat16, float);
    NSB_MOD_GO(__half, float);
  }
  if (dtype_out != dtype_in) return NSB_ERR_INVALID_ARG;  // low-precision outputs: same dtype as the inputs
  if (dtype_in == NSB_BF16) NSB_MOD_GO(__nv_bfloat16, __nv_bfloat16);
  NSB_MOD_GO(__half, __half);
#undef NSB_MOD_GO
}
