// extern "C" entry points of the PLIF scan family: argument checks and dispatch.
#include "nsb_scan.cuh"

namespace {

bool tile_ok(int c) { return c == 8 || c == 16 || c == 32; }
bool dtype_ok(int d) { return d == NSB_F32 || d == NSB_BF16 || d == NSB_F16; }
bool elem_aligned(const void* p, int dtype) {
  return (reinterpret_cast<uintptr_t>(p) % nsb::dtype_size(dtype)) == 0;
}
bool f32_aligned(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 3u) == 0; }

int run_fwd(const nsb::FwdArgs& a, int dtype) {
  switch (dtype) {
    case NSB_F32: return nsb::scan_fwd_f32(a);
    case NSB_BF16: return nsb::scan_fwd_bf16(a);
    default: return nsb::scan_fwd_f16(a);
  }
}
int run_bwd(const nsb::BwdArgs& a, int dtype) {
  switch (dtype) {
    case NSB_F32: return nsb::scan_bwd_f32(a);
    case NSB_BF16: return nsb::scan_bwd_bf16(a);
    default: return nsb::scan_bwd_f16(a);
  }
}

}  // namespace

extern "C" {

int nsb_plif_selective_fwd(const void* beta, const void* u_or_cur, const void* gain, const void* v_th,
                           const float* v_init, void* spike_dense, uint32_t* spike_packed, void* v_post,
                           float* v_ckpt, float* v_last, int64_t T, int64_t cols, int dtype,
                           int ckpt_interval, void* stream) {
  if (T < 0 || cols < 0 || !dtype_ok(dtype) || !tile_ok(ckpt_interval)) return NSB_ERR_INVALID_ARG;
  if (cols == 0) return NSB_OK;
  if (!v_init || !v_last || !f32_aligned(v_init) || !f32_aligned(v_last) || !f32_aligned(v_ckpt) ||
      !f32_aligned(spike_packed))
    return NSB_ERR_INVALID_ARG;
  if (T == 0) {  // nothing to scan: the final state is the initial state
    NSB_CUDA_TRY(cudaMemcpyAsync(v_last, v_init, sizeof(float) * cols, cudaMemcpyDeviceToDevice,
                                 static_cast<cudaStream_t>(stream)), "copy v_init");
    return NSB_OK;
  }
  if (!beta || !u_or_cur || !v_th) return NSB_ERR_INVALID_ARG;
  const void* ep[] = {beta, u_or_cur, gain, v_th, spike_dense, v_post};
  for (const void* p : ep)
    if (!elem_aligned(p, dtype)) return NSB_ERR_INVALID_ARG;
  nsb::FwdArgs a;
  a.beta = beta; a.drive = u_or_cur; a.gain = gain; a.vth = v_th; a.v_init = v_init;
  a.spike = spike_dense; a.packed = spike_packed; a.vpost = v_post; a.ckpt = v_ckpt; a.vlast = v_last;
  a.T = T; a.cols = cols; a.mode = gain ? nsb::MODE_AI : nsb::MODE_U; a.tile = ckpt_interval;
  a.stream = static_cast<cudaStream_t>(stream);
  return run_fwd(a, dtype);
}

int nsb_plif_rowparam_fwd(const float* beta_row, const void* u, const float* vth_row, const float* v_init,
                          void* spike_dense, uint32_t* spike_packed, void* v_post, float* v_ckpt,
                          float* v_last, int64_t T, int64_t cols, int dtype, int ckpt_interval,
                          void* stream) {
  if (T < 0 || cols < 0 || !dtype_ok(dtype) || !tile_ok(ckpt_interval)) return NSB_ERR_INVALID_ARG;
  if (cols == 0) return NSB_OK;
  if (!beta_row || !vth_row || !v_init || !v_last) return NSB_ERR_INVALID_ARG;
  const void* fp[] = {beta_row, vth_row, v_init, v_last, v_ckpt, spike_packed};
  for (const void* p : fp)
    if (!f32_aligned(p)) return NSB_ERR_INVALID_ARG;
  if (T == 0) {
    NSB_CUDA_TRY(cudaMemcpyAsync(v_last, v_init, sizeof(float) * cols, cudaMemcpyDeviceToDevice,
                                 static_cast<cudaStream_t>(stream)), "copy v_init");
    return NSB_OK;
  }
  if (!u) return NSB_ERR_INVALID_ARG;
  const void* ep[] = {u, spike_dense, v_post};
  for (const void* p : ep)
    if (!elem_aligned(p, dtype)) return NSB_ERR_INVALID_ARG;
  nsb::FwdArgs a;
  a.drive = u; a.beta_row = beta_row; a.vth_row = vth_row; a.v_init = v_init;
  a.spike = spike_dense; a.packed = spike_packed; a.vpost = v_post; a.ckpt = v_ckpt; a.vlast = v_last;
  a.T = T; a.cols = cols; a.mode = nsb::MODE_ROW; a.tile = ckpt_interval;
  a.stream = static_cast<cudaStream_t>(stream);
  return run_fwd(a, dtype);
}

int nsb_plif_selective_bwd(const void* beta, const void* u_or_cur, const void* gain, const void* v_th,
                           const float* v_ckpt, const void* g_spike, const void* g_vpost, void* g_beta,
                           void* g_u_or_cur, void* g_gain, void* g_vth, float* g_vinit, int64_t T,
                           int64_t cols, int dtype, int ckpt_interval, int surrogate, float alpha,
                           void* stream) {
  if (T < 0 || cols < 0 || !dtype_ok(dtype) || !tile_ok(ckpt_interval)) return NSB_ERR_INVALID_ARG;
  if (surrogate != NSB_SURR_SIGMOID && surrogate != NSB_SURR_ATAN) return NSB_ERR_INVALID_ARG;
  if (cols == 0) return NSB_OK;
  if (T == 0) {
    if (g_vinit) {
      NSB_CUDA_TRY(cudaMemsetAsync(g_vinit, 0, sizeof(float) * cols, static_cast<cudaStream_t>(stream)),
                   "memset g_vinit");
    }
    return NSB_OK;
  }
  if (!beta || !u_or_cur || !v_th || !v_ckpt || !g_spike) return NSB_ERR_INVALID_ARG;
  if (!f32_aligned(v_ckpt) || !f32_aligned(g_vinit)) return NSB_ERR_INVALID_ARG;
  const void* ep[] = {beta, u_or_cur, gain, v_th, g_spike, g_vpost, g_beta, g_u_or_cur, g_gain, g_vth};
  for (const void* p : ep)
    if (!elem_aligned(p, dtype)) return NSB_ERR_INVALID_ARG;
  nsb::BwdArgs a;
  a.beta = beta; a.drive = u_or_cur; a.gain = gain; a.vth = v_th; a.ckpt = v_ckpt;
  a.g_spike = g_spike; a.g_vpost = g_vpost; a.g_beta = g_beta; a.g_drive = g_u_or_cur;
  a.g_gain = gain ? g_gain : nullptr; a.g_vth = g_vth; a.g_vinit = g_vinit;
  a.T = T; a.cols = cols; a.mode = gain ? nsb::MODE_AI : nsb::MODE_U; a.tile = ckpt_interval;
  a.surrogate = surrogate; a.alpha = alpha; a.stream = static_cast<cudaStream_t>(stream);
  return run_bwd(a, dtype);
}

int nsb_plif_rowparam_bwd(const float* beta_row, const void* u, const float* vth_row, const float* v_ckpt,
                          const void* g_spike, const void* g_vpost, float* g_beta_row, void* g_u,
                          float* g_vth_row, float* g_vinit, int64_t T, int64_t cols, int dtype,
                          int ckpt_interval, int surrogate, float alpha, void* stream) {
  if (T < 0 || cols < 0 || !dtype_ok(dtype) || !tile_ok(ckpt_interval)) return NSB_ERR_INVALID_ARG;
  if (surrogate != NSB_SURR_SIGMOID && surrogate != NSB_SURR_ATAN) return NSB_ERR_INVALID_ARG;
  if (cols == 0) return NSB_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (T == 0) {
    float* z[] = {g_beta_row, g_vth_row, g_vinit};
    for (float* q : z)
      if (q) NSB_CUDA_TRY(cudaMemsetAsync(q, 0, sizeof(float) * cols, st), "memset row grads");
    return NSB_OK;
  }
  if (!beta_row || !u || !vth_row || !v_ckpt || !g_spike) return NSB_ERR_INVALID_ARG;
  const void* fp[] = {beta_row, vth_row, v_ckpt, g_beta_row, g_vth_row, g_vinit};
  for (const void* p : fp)
    if (!f32_aligned(p)) return NSB_ERR_INVALID_ARG;
  const void* ep[] = {u, g_spike, g_vpost, g_u};
  for (const void* p : ep)
    if (!elem_aligned(p, dtype)) return NSB_ERR_INVALID_ARG;
  nsb::BwdArgs a;
  a.drive = u; a.beta_row = beta_row; a.vth_row = vth_row; a.ckpt = v_ckpt;
  a.g_spike = g_spike; a.g_vpost = g_vpost; a.g_drive = g_u;
  a.g_beta_row = g_beta_row; a.g_vth_row = g_vth_row; a.g_vinit = g_vinit;
  a.T = T; a.cols = cols; a.mode = nsb::MODE_ROW; a.tile = ckpt_interval;
  a.surrogate = surrogate; a.alpha = alpha; a.stream = st;
  return run_bwd(a, dtype);
}

int nsb_plif_rf_fwd(const void* beta, const void* omega, const void* u, const void* v_th,
                    const float* v_init, const float* w_init, void* spike_dense, uint32_t* spike_packed,
                    void* v_post, void* w_out, float* v_ckpt, float* w_ckpt, float* v_last, float* w_last,
                    int64_t T, int64_t cols, int dtype, int ckpt_interval, void* stream) {
  if (T < 0 || cols < 0 || !dtype_ok(dtype) || !tile_ok(ckpt_interval)) return NSB_ERR_INVALID_ARG;
  if (cols == 0) return NSB_OK;
  if (!v_init || !w_init || !v_last || !w_last) return NSB_ERR_INVALID_ARG;
  if ((v_ckpt == nullptr) != (w_ckpt == nullptr)) return NSB_ERR_INVALID_ARG;
  const void* fp[] = {v_init, w_init, v_last, w_last, v_ckpt, w_ckpt, spike_packed};
  for (const void* p : fp)
    if (!f32_aligned(p)) return NSB_ERR_INVALID_ARG;
  if (T == 0) {
    cudaStream_t st0 = static_cast<cudaStream_t>(stream);
    NSB_CUDA_TRY(cudaMemcpyAsync(v_last, v_init, sizeof(float) * cols, cudaMemcpyDeviceToDevice, st0),
                 "copy v_init");
    NSB_CUDA_TRY(cudaMemcpyAsync(w_last, w_init, sizeof(float) * cols, cudaMemcpyDeviceToDevice, st0),
                 "copy w_init");
    return NSB_OK;
  }
  if (!beta || !omega || !u || !v_th) return NSB_ERR_INVALID_ARG;
  const void* ep[] = {beta, omega, u, v_th, spike_dense, v_post, w_out};
  for (const void* p : ep)
    if (!elem_aligned(p, dtype)) return NSB_ERR_INVALID_ARG;
  nsb::FwdArgs a;
  a.beta = beta; a.drive = u; a.gain = omega; a.vth = v_th; a.v_init = v_init; a.w_init = w_init;
  a.spike = spike_dense; a.packed = spike_packed; a.vpost = v_post; a.w_out = w_out;
  a.ckpt = v_ckpt; a.ckpt_w = w_ckpt; a.vlast = v_last; a.wlast = w_last;
  a.T = T; a.cols = cols; a.mode = nsb::MODE_RF; a.tile = ckpt_interval;
  a.stream = static_cast<cudaStream_t>(stream);
  return run_fwd(a, dtype);
}

int nsb_plif_rf_bwd(const void* beta, const void* omega, const void* u, const void* v_th,
                    const float* v_ckpt, const float* w_ckpt, const void* g_spike, const void* g_vpost,
                    void* g_beta, void* g_omega, void* g_u, void* g_vth, float* g_vinit, float* g_winit,
                    int64_t T, int64_t cols, int dtype, int ckpt_interval, int surrogate, float alpha,
                    void* stream) {
  if (T < 0 || cols < 0 || !dtype_ok(dtype) || !tile_ok(ckpt_interval)) return NSB_ERR_INVALID_ARG;
  if (surrogate != NSB_SURR_SIGMOID && surrogate != NSB_SURR_ATAN) return NSB_ERR_INVALID_ARG;
  if (cols == 0) return NSB_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (T == 0) {
    float* z[] = {g_vinit, g_winit};
    for (float* q : z)
      if (q) NSB_CUDA_TRY(cudaMemsetAsync(q, 0, sizeof(float) * cols, st), "memset state grads");
    return NSB_OK;
  }
  if (!beta || !omega || !u || !v_th || !v_ckpt || !w_ckpt || !g_spike) return NSB_ERR_INVALID_ARG;
  const void* fp[] = {v_ckpt, w_ckpt, g_vinit, g_winit};
  for (const void* p : fp)
    if (!f32_aligned(p)) return NSB_ERR_INVALID_ARG;
  const void* ep[] = {beta, omega, u, v_th, g_spike, g_vpost, g_beta, g_omega, g_u, g_vth};
  for (const void* p : ep)
    if (!elem_aligned(p, dtype)) return NSB_ERR_INVALID_ARG;
  nsb::BwdArgs a;
  a.beta = beta; a.drive = u; a.gain = omega; a.vth = v_th; a.ckpt = v_ckpt; a.ckpt_w = w_ckpt;
  a.g_spike = g_spike; a.g_vpost = g_vpost; a.g_beta = g_beta; a.g_drive = g_u; a.g_gain = g_omega;
  a.g_vth = g_vth; a.g_vinit = g_vinit; a.g_winit = g_winit;
  a.T = T; a.cols = cols; a.mode = nsb::MODE_RF; a.tile = ckpt_interval;
  a.surrogate = surrogate; a.alpha = alpha; a.stream = st;
  return run_bwd(a, dtype);
}

}  // extern "C"
