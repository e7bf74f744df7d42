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

int run_mod_fwd(const nsb::FwdArgs& a, int dtype) {
  switch (dtype) {
    case NSB_F32: return nsb::scan_mod_fwd_f32(a);
    case NSB_BF16: return nsb::scan_mod_fwd_bf16(a);
    default: return nsb::scan_mod_fwd_f16(a);
  }
}
int run_res_fwd(const nsb::FwdArgs& a, int dtype) {
  switch (dtype) {
    case NSB_F32: return nsb::scan_res_fwd_f32(a);
    case NSB_BF16: return nsb::scan_res_fwd_bf16(a);
    default: return nsb::scan_res_fwd_f16(a);
  }
}
int run_pat_fwd(const nsb::FwdArgs& a, int dtype) {
  switch (dtype) {
    case NSB_F32: return nsb::scan_pat_fwd_f32(a);
    case NSB_BF16: return nsb::scan_pat_fwd_bf16(a);
    default: return nsb::scan_pat_fwd_f16(a);
  }
}
int run_lin_fwd(const nsb::FwdArgs& a, int dtype) {
  switch (dtype) {
    case NSB_F32: return nsb::scan_lin_fwd_f32(a);
    case NSB_BF16: return nsb::scan_lin_fwd_bf16(a);
    default: return nsb::scan_lin_fwd_f16(a);
  }
}
int run_lin_bwd(const nsb::BwdArgs& a, int dtype) {
  switch (dtype) {
    case NSB_F32: return nsb::scan_lin_bwd_f32(a);
    case NSB_BF16: return nsb::scan_lin_bwd_bf16(a);
    default: return nsb::scan_lin_bwd_f16(a);
  }
}
int run_mod_bwd(const nsb::BwdArgs& a, int dtype) {
  switch (dtype) {
    case NSB_F32: return nsb::scan_mod_bwd_f32(a);
    case NSB_BF16: return nsb::scan_mod_bwd_bf16(a);
    default: return nsb::scan_mod_bwd_f16(a);
  }
}

// out[n][c] = sum over b of in[n][b*ch + c], b ascending (deterministic).
__global__ void sum_over_batch_kernel(const float* __restrict__ in, float* __restrict__ out0,
                                      float* __restrict__ out1, float* __restrict__ out2,
                                      float* __restrict__ out3, long long batch, long long ch, int n) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)n * ch) return;
  const int which = (int)(idx / ch);
  const long long c = idx % ch;
  const float* src = in + (long long)which * batch * ch + c;
  float acc = 0.0f;
  for (long long b = 0; b < batch; ++b) acc += src[b * ch];
  float* out = which == 0 ? out0 : (which == 1 ? out1 : (which == 2 ? out2 : out3));
  if (out) out[c] = acc;
}

}  // namespace

extern "C" {

int nsb_plif_selective_fwd(const void* beta, const void* u_or_cur, const void* gain, const void* v_th,
                           const float* v_init, void* spike_dense, uint32_t* spike_packed, void* v_post,
                           float* v_ckpt, float* v_last, int64_t T, int64_t cols, int dtype,
                           int ckpt_interval, float* split_scratch, void* stream) {
  if (T < 0 || cols < 0 || !dtype_ok(dtype) || !tile_ok(ckpt_interval)) return NSB_ERR_INVALID_ARG;
  if (cols == 0) return NSB_OK;
  if (!v_init || !v_last || !f32_aligned(v_init) || !f32_aligned(v_last) || !f32_aligned(v_ckpt) ||
      !f32_aligned(spike_packed) || !f32_aligned(split_scratch))
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
  a.split_scratch = split_scratch;
  a.stream = static_cast<cudaStream_t>(stream);
  return run_fwd(a, dtype);
}

int nsb_plif_rowparam_fwd(const float* beta_row, const void* u, const float* vth_row, const float* v_init,
                          void* spike_dense, uint32_t* spike_packed, void* v_post, float* v_ckpt,
                          float* v_last, int64_t T, int64_t cols, int dtype, int ckpt_interval,
                          float* split_scratch, void* stream) {
  if (T < 0 || cols < 0 || !dtype_ok(dtype) || !tile_ok(ckpt_interval)) return NSB_ERR_INVALID_ARG;
  if (cols == 0) return NSB_OK;
  if (!beta_row || !vth_row || !v_init || !v_last) return NSB_ERR_INVALID_ARG;
  const void* fp[] = {beta_row, vth_row, v_init, v_last, v_ckpt, spike_packed, split_scratch};
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
  a.split_scratch = split_scratch;
  a.stream = static_cast<cudaStream_t>(stream);
  return run_fwd(a, dtype);
}

int nsb_plif_selective_bwd(const void* beta, const void* u_or_cur, const void* gain, const void* v_th,
                           const float* v_ckpt, const void* g_spike, const void* g_vpost, void* g_beta,
                           void* g_u_or_cur, void* g_gain, void* g_vth, float* g_vinit, int64_t T,
                           int64_t cols, int dtype, int ckpt_interval, int surrogate, float alpha,
                           uint32_t* chain_scratch, void* stream) {
  if (T < 0 || cols < 0 || !dtype_ok(dtype) || !tile_ok(ckpt_interval)) return NSB_ERR_INVALID_ARG;
  if (surrogate != NSB_SURR_SIGMOID && surrogate != NSB_SURR_ATAN) return NSB_ERR_INVALID_ARG;
  if (!f32_aligned(chain_scratch)) return NSB_ERR_INVALID_ARG;
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
  a.chain_sync = chain_scratch;
  return run_bwd(a, dtype);
}

static int rowparam_bwd_impl(const float* beta_row, const void* u, const float* vth_row, const float* v_ckpt,
                             const void* g_spike, const void* g_vpost, float* g_beta_row, void* g_u,
                             float* g_vth_row, float* g_vinit, int64_t T, int64_t cols, int dtype,
                             int ckpt_interval, int surrogate, float alpha, const float* alpha_dev,
                             float* split_scratch, void* stream) {
  if (T < 0 || cols < 0 || !dtype_ok(dtype) || !tile_ok(ckpt_interval)) return NSB_ERR_INVALID_ARG;
  if (surrogate != NSB_SURR_SIGMOID && surrogate != NSB_SURR_ATAN) return NSB_ERR_INVALID_ARG;
  if (!f32_aligned(split_scratch)) return NSB_ERR_INVALID_ARG;
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
  a.surrogate = surrogate; a.alpha = alpha; a.alpha_dev = alpha_dev; a.stream = st;
  a.split_scratch = split_scratch;
  return run_bwd(a, dtype);
}

int nsb_plif_rowparam_bwd(const float* beta_row, const void* u, const float* vth_row, const float* v_ckpt,
                          const void* g_spike, const void* g_vpost, float* g_beta_row, void* g_u,
                          float* g_vth_row, float* g_vinit, int64_t T, int64_t cols, int dtype,
                          int ckpt_interval, int surrogate, float alpha, float* split_scratch, void* stream) {
  return rowparam_bwd_impl(beta_row, u, vth_row, v_ckpt, g_spike, g_vpost, g_beta_row, g_u, g_vth_row, g_vinit,
                           T, cols, dtype, ckpt_interval, surrogate, alpha, nullptr, split_scratch, stream);
}

int nsb_plif_rowparam_bwd_dalpha(const float* beta_row, const void* u, const float* vth_row,
                                 const float* v_ckpt, const void* g_spike, const void* g_vpost,
                                 float* g_beta_row, void* g_u, float* g_vth_row, float* g_vinit, int64_t T,
                                 int64_t cols, int dtype, int ckpt_interval, int surrogate,
                                 const float* alpha_dev, float* split_scratch, void* stream) {
  if (!alpha_dev || !f32_aligned(alpha_dev)) return NSB_ERR_INVALID_ARG;
  return rowparam_bwd_impl(beta_row, u, vth_row, v_ckpt, g_spike, g_vpost, g_beta_row, g_u, g_vth_row, g_vinit,
                           T, cols, dtype, ckpt_interval, surrogate, 0.0f, alpha_dev, split_scratch, stream);
}

int nsb_plif_rf_fwd(const void* beta, const void* omega, const void* u, const void* v_th,
                    const float* v_init, const float* w_init, void* spike_dense, uint32_t* spike_packed,
                    void* v_post, void* w_out, float* v_ckpt, float* w_ckpt, float* v_last, float* w_last,
                    int64_t T, int64_t cols, int dtype, int ckpt_interval, float* split_scratch,
                    void* stream) {
  if (T < 0 || cols < 0 || !dtype_ok(dtype) || !tile_ok(ckpt_interval)) return NSB_ERR_INVALID_ARG;
  if (cols == 0) return NSB_OK;
  if (!v_init || !w_init || !v_last || !w_last) return NSB_ERR_INVALID_ARG;
  if ((v_ckpt == nullptr) != (w_ckpt == nullptr)) return NSB_ERR_INVALID_ARG;
  const void* fp[] = {v_init, w_init, v_last, w_last, v_ckpt, w_ckpt, spike_packed, split_scratch};
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
  a.split_scratch = split_scratch;
  a.stream = static_cast<cudaStream_t>(stream);
  return run_fwd(a, dtype);
}

static int rf_bwd_impl(const void* beta, const void* omega, const void* u, const void* v_th,
                       const float* v_ckpt, const float* w_ckpt, const void* g_spike, const void* g_vpost,
                       void* g_beta, void* g_omega, void* g_u, void* g_vth, float* g_vinit, float* g_winit,
                       int64_t T, int64_t cols, int dtype, int ckpt_interval, int surrogate, float alpha,
                       const float* alpha_dev, uint32_t* chain_scratch, void* stream) {
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
  a.surrogate = surrogate; a.alpha = alpha; a.alpha_dev = alpha_dev; a.stream = st;
  if (!f32_aligned(chain_scratch)) return NSB_ERR_INVALID_ARG;
  a.chain_sync = chain_scratch;
  return run_bwd(a, dtype);
}

int nsb_plif_rf_bwd(const void* beta, const void* omega, const void* u, const void* v_th,
                    const float* v_ckpt, const float* w_ckpt, const void* g_spike, const void* g_vpost,
                    void* g_beta, void* g_omega, void* g_u, void* g_vth, float* g_vinit, float* g_winit,
                    int64_t T, int64_t cols, int dtype, int ckpt_interval, int surrogate, float alpha,
                    uint32_t* chain_scratch, void* stream) {
  return rf_bwd_impl(beta, omega, u, v_th, v_ckpt, w_ckpt, g_spike, g_vpost, g_beta, g_omega, g_u, g_vth,
                     g_vinit, g_winit, T, cols, dtype, ckpt_interval, surrogate, alpha, nullptr, chain_scratch,
                     stream);
}

int nsb_plif_rf_bwd_dalpha(const void* beta, const void* omega, const void* u, const void* v_th,
                           const float* v_ckpt, const float* w_ckpt, const void* g_spike,
                           const void* g_vpost, void* g_beta, void* g_omega, void* g_u, void* g_vth,
                           float* g_vinit, float* g_winit, int64_t T, int64_t cols, int dtype,
                           int ckpt_interval, int surrogate, const float* alpha_dev, uint32_t* chain_scratch,
                           void* stream) {
  if (!alpha_dev || !f32_aligned(alpha_dev)) return NSB_ERR_INVALID_ARG;
  return rf_bwd_impl(beta, omega, u, v_th, v_ckpt, w_ckpt, g_spike, g_vpost, g_beta, g_omega, g_u, g_vth,
                     g_vinit, g_winit, T, cols, dtype, ckpt_interval, surrogate, 0.0f, alpha_dev, chain_scratch,
                     stream);
}

int nsb_plif_modulated_fwd(const void* raw_beta, const void* raw_alpha, const void* raw_th,
                           const void* raw_omega, const void* cur, const float* b_beta,
                           const float* b_alpha, const float* b_th, const float* b_omega, float v_th_min,
                           int64_t channels, const float* v_init, const float* w_init, void* spike_dense,
                           uint32_t* spike_packed, float* v_ckpt, float* w_ckpt, float* v_last,
                           float* w_last, float alpha0, float sigma0, double* u_stats, float* alpha_out,
                           int64_t T, int64_t cols, int dtype, int ckpt_interval, float* split_scratch,
                           void* stream) {
  if (T < 0 || cols < 0 || !dtype_ok(dtype) || (ckpt_interval != 8 && ckpt_interval != 32))
    return NSB_ERR_INVALID_ARG;
  if (cols == 0) return NSB_OK;
  if (channels <= 0 || cols % channels != 0) return NSB_ERR_INVALID_ARG;
  const bool rf = raw_omega != nullptr || b_omega != nullptr;  // (an empty raw_omega may be NULL)
  if (!v_init || !v_last || !b_beta || !b_alpha || !b_th) return NSB_ERR_INVALID_ARG;
  if (rf && (!b_omega || !w_init || !w_last)) return NSB_ERR_INVALID_ARG;
  if (rf && (v_ckpt == nullptr) != (w_ckpt == nullptr)) return NSB_ERR_INVALID_ARG;
  const void* fp[] = {v_init, w_init, v_last, w_last, v_ckpt, w_ckpt, spike_packed, b_beta, b_alpha, b_th, b_omega,
                      alpha_out};
  for (const void* p : fp)
    if (!f32_aligned(p)) return NSB_ERR_INVALID_ARG;
  if ((u_stats == nullptr) != (alpha_out == nullptr) || (reinterpret_cast<uintptr_t>(u_stats) & 7u))
    return NSB_ERR_INVALID_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (T == 0) {
    NSB_CUDA_TRY(cudaMemcpyAsync(v_last, v_init, sizeof(float) * cols, cudaMemcpyDeviceToDevice, st), "copy v_init");
    if (rf)
      NSB_CUDA_TRY(cudaMemcpyAsync(w_last, w_init, sizeof(float) * cols, cudaMemcpyDeviceToDevice, st),
                   "copy w_init");
    if (alpha_out) return nsb::launch_alpha_finalize(u_stats, 0, 0, NSB_F32, alpha0, sigma0, alpha_out, st);
    return NSB_OK;
  }
  if (!raw_beta || !raw_alpha || !raw_th || !cur || (rf && !raw_omega)) return NSB_ERR_INVALID_ARG;
  const void* ep[] = {raw_beta, raw_alpha, raw_th, raw_omega, cur, spike_dense};
  for (const void* p : ep)
    if (!elem_aligned(p, dtype)) return NSB_ERR_INVALID_ARG;
  nsb::FwdArgs a;
  a.beta = raw_beta; a.drive = cur; a.gain = raw_alpha; a.vth = raw_th; a.extra = raw_omega;
  a.bias[0] = b_beta; a.bias[1] = b_alpha; a.bias[2] = b_th; a.bias[3] = b_omega;
  a.channels = channels; a.v_th_min = v_th_min;
  a.v_init = v_init; a.w_init = w_init; a.spike = spike_dense; a.packed = spike_packed;
  a.ckpt = v_ckpt; a.ckpt_w = w_ckpt; a.vlast = v_last; a.wlast = w_last;
  a.u_stats = u_stats; a.alpha_out = alpha_out; a.alpha0 = alpha0; a.sigma0 = sigma0;
  a.T = T; a.cols = cols; a.mode = rf ? nsb::MODE_RFMOD : nsb::MODE_MOD; a.tile = ckpt_interval;
  if (!f32_aligned(split_scratch)) return NSB_ERR_INVALID_ARG;
  a.split_scratch = u_stats ? nullptr : split_scratch;  // (the kernels that accumulate moments are not split)
  a.stream = st;
  return run_mod_fwd(a, dtype);
}

// 4 per-column rows of bias-gradient sums, then the counters of a chained launch
int64_t nsb_plif_modulated_bwd_scratch_floats(int64_t cols) {
  return cols > 0 ? 4 * cols + nsb::chain_scratch_words(cols) : 0;
}
int64_t nsb_plif_modulated_fwd_stats_doubles(int64_t cols) { return cols > 0 ? 2 * ((cols + 31) / 32) : 0; }

int nsb_plif_modulated_bwd(const void* raw_beta, const void* raw_alpha, const void* raw_th,
                           const void* raw_omega, const void* cur, const float* b_beta,
                           const float* b_alpha, const float* b_th, const float* b_omega, float v_th_min,
                           int64_t channels, const float* v_ckpt, const float* w_ckpt, const void* g_spike,
                           void* g_raw_beta, void* g_raw_alpha, void* g_raw_th, void* g_raw_omega,
                           void* g_cur, float* g_b_beta, float* g_b_alpha, float* g_b_th, float* g_b_omega,
                           float* scratch, float* g_vinit, float* g_winit, int64_t T, int64_t cols,
                           int dtype, int ckpt_interval, int surrogate, float alpha, const float* alpha_dev,
                           void* stream) {
  if (T < 0 || cols < 0 || !dtype_ok(dtype) || (ckpt_interval != 8 && ckpt_interval != 32))
    return NSB_ERR_INVALID_ARG;
  if (surrogate != NSB_SURR_SIGMOID && surrogate != NSB_SURR_ATAN) return NSB_ERR_INVALID_ARG;
  if (cols == 0) return NSB_OK;
  if (channels <= 0 || cols % channels != 0) return NSB_ERR_INVALID_ARG;
  const bool rf = raw_omega != nullptr || b_omega != nullptr;  // (an empty raw_omega may be NULL)
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const void* fp[] = {v_ckpt, w_ckpt, g_vinit, g_winit, b_beta, b_alpha, b_th, b_omega,
                      g_b_beta, g_b_alpha, g_b_th, g_b_omega, scratch};
  for (const void* p : fp)
    if (!f32_aligned(p)) return NSB_ERR_INVALID_ARG;
  if (T == 0) {
    float* zc[] = {g_vinit, rf ? g_winit : nullptr};
    for (float* q : zc)
      if (q) NSB_CUDA_TRY(cudaMemsetAsync(q, 0, sizeof(float) * cols, st), "memset state grads");
    float* zb[] = {g_b_beta, g_b_alpha, g_b_th, rf ? g_b_omega : nullptr};
    for (float* q : zb)
      if (q) NSB_CUDA_TRY(cudaMemsetAsync(q, 0, sizeof(float) * channels, st), "memset bias grads");
    return NSB_OK;
  }
  if (!raw_beta || !raw_alpha || !raw_th || !cur || !b_beta || !b_alpha || !b_th || !v_ckpt || !g_spike)
    return NSB_ERR_INVALID_ARG;
  if (rf && (!raw_omega || !b_omega || !w_ckpt)) return NSB_ERR_INVALID_ARG;
  const bool want_bias = g_b_beta || g_b_alpha || g_b_th || (rf && g_b_omega);
  if (want_bias && !scratch) return NSB_ERR_INVALID_ARG;
  const void* ep[] = {raw_beta, raw_alpha, raw_th, raw_omega, cur, g_spike,
                      g_raw_beta, g_raw_alpha, g_raw_th, g_raw_omega, g_cur};
  for (const void* p : ep)
    if (!elem_aligned(p, dtype)) return NSB_ERR_INVALID_ARG;
  nsb::BwdArgs a;
  a.beta = raw_beta; a.drive = cur; a.gain = raw_alpha; a.vth = raw_th; a.extra = raw_omega;
  a.bias[0] = b_beta; a.bias[1] = b_alpha; a.bias[2] = b_th; a.bias[3] = b_omega;
  a.channels = channels; a.v_th_min = v_th_min;
  a.ckpt = v_ckpt; a.ckpt_w = w_ckpt; a.g_spike = g_spike;
  a.g_beta = g_raw_beta; a.g_drive = g_cur; a.g_gain = g_raw_alpha; a.g_vth = g_raw_th; a.g_extra = g_raw_omega;
  const int nb = rf ? 4 : 3;
  if (want_bias)
    for (int i = 0; i < nb; ++i) a.g_bias[i] = scratch + (long long)i * cols;
  if (scratch) a.chain_sync = reinterpret_cast<unsigned int*>(scratch + 4LL * cols);
  a.g_vinit = g_vinit; a.g_winit = g_winit;
  a.T = T; a.cols = cols; a.mode = rf ? nsb::MODE_RFMOD : nsb::MODE_MOD; a.tile = ckpt_interval;
  a.surrogate = surrogate; a.alpha = alpha; a.alpha_dev = alpha_dev; a.stream = st;
  if (!f32_aligned(alpha_dev)) return NSB_ERR_INVALID_ARG;
  int r = run_mod_bwd(a, dtype);
  if (r != NSB_OK || !want_bias) return r;
  const long long items = (long long)nb * channels;
  const int threads = 128;
  sum_over_batch_kernel<<<(int)((items + threads - 1) / threads), threads, 0, st>>>(
      scratch, g_b_beta, g_b_alpha, g_b_th, rf ? g_b_omega : nullptr, cols / channels, channels, nb);
  NSB_CUDA_TRY(cudaGetLastError(), "launch sum_over_batch_kernel");
  return NSB_OK;
}

int nsb_plif_rowparam_residual_fwd(const float* beta_row, const void* u, const float* vth_row,
                                   const float* v_init, const void* frames_in, void* frames_out,
                                   float* v_ckpt, float* v_last, int64_t T, int64_t cols, int dtype,
                                   int ckpt_interval, int rounding, float* split_scratch, void* stream) {
  if (T < 0 || cols < 0 || T % 16 != 0 || !dtype_ok(dtype) || (ckpt_interval != 16 && ckpt_interval != 32) ||
      (rounding != NSB_RESIDUAL_EAGER && rounding != NSB_RESIDUAL_COMPILED))
    return NSB_ERR_INVALID_ARG;
  if (cols == 0) return NSB_OK;
  if (!beta_row || !vth_row || !v_init || !v_last) return NSB_ERR_INVALID_ARG;
  const void* fp[] = {beta_row, vth_row, v_init, v_last, v_ckpt, split_scratch};
  for (const void* p : fp)
    if (!f32_aligned(p)) return NSB_ERR_INVALID_ARG;
  if (T == 0) {
    NSB_CUDA_TRY(cudaMemcpyAsync(v_last, v_init, sizeof(float) * cols, cudaMemcpyDeviceToDevice,
                                 static_cast<cudaStream_t>(stream)), "copy v_init");
    return NSB_OK;
  }
  if (!u || !frames_in || !frames_out) return NSB_ERR_INVALID_ARG;
  if (!elem_aligned(u, dtype) || !elem_aligned(frames_in, dtype) || !elem_aligned(frames_out, dtype))
    return NSB_ERR_INVALID_ARG;
  nsb::FwdArgs a;
  a.drive = u; a.extra = frames_in; a.beta_row = beta_row; a.vth_row = vth_row; a.v_init = v_init;
  a.spike = frames_out; a.ckpt = v_ckpt; a.vlast = v_last;
  a.T = T; a.cols = cols; a.mode = nsb::MODE_ROWRES; a.tile = ckpt_interval;
  a.residual_compiled = rounding == NSB_RESIDUAL_COMPILED;
  a.split_scratch = split_scratch;
  a.stream = static_cast<cudaStream_t>(stream);
  return run_res_fwd(a, dtype);
}

int nsb_plif_rowparam_pattern_fwd(const float* beta_row, const void* u, const float* vth_row,
                                  const float* v_init, const uint16_t* patterns_in, uint16_t* patterns_out,
                                  float* v_ckpt, float* v_last, int64_t T, int64_t cols, int dtype,
                                  int ckpt_interval, int frame_dtype, int rounding, float* split_scratch,
                                  void* stream) {
  if (T < 0 || cols < 0 || T % 16 != 0 || !dtype_ok(dtype) || !dtype_ok(frame_dtype) ||
      (ckpt_interval != 16 && ckpt_interval != 32) ||
      (rounding != NSB_RESIDUAL_EAGER && rounding != NSB_RESIDUAL_COMPILED))
    return NSB_ERR_INVALID_ARG;
  if (cols == 0) return NSB_OK;
  if (!beta_row || !vth_row || !v_init || !v_last) return NSB_ERR_INVALID_ARG;
  const void* fp[] = {beta_row, vth_row, v_init, v_last, v_ckpt, split_scratch};
  for (const void* p : fp)
    if (!f32_aligned(p)) return NSB_ERR_INVALID_ARG;
  if (T == 0) {
    NSB_CUDA_TRY(cudaMemcpyAsync(v_last, v_init, sizeof(float) * cols, cudaMemcpyDeviceToDevice,
                                 static_cast<cudaStream_t>(stream)), "copy v_init");
    return NSB_OK;
  }
  if (!u || !patterns_out || !elem_aligned(u, dtype)) return NSB_ERR_INVALID_ARG;
  if (reinterpret_cast<uintptr_t>(patterns_out) % 2 || reinterpret_cast<uintptr_t>(patterns_in) % 2)
    return NSB_ERR_INVALID_ARG;
  nsb::FwdArgs a;
  a.drive = u; a.beta_row = beta_row; a.vth_row = vth_row; a.v_init = v_init;
  a.pat_in = patterns_in; a.pat_out = patterns_out; a.frame_dtype = frame_dtype;
  a.ckpt = v_ckpt; a.vlast = v_last;
  a.T = T; a.cols = cols; a.mode = nsb::MODE_ROWPAT; a.tile = ckpt_interval;
  a.residual_compiled = rounding == NSB_RESIDUAL_COMPILED;
  a.split_scratch = split_scratch;
  a.stream = static_cast<cudaStream_t>(stream);
  return run_pat_fwd(a, dtype);
}

int nsb_linear_recurrence_fwd(const void* beta, const void* u, const float* v_init, void* v_out,
                              float* v_ckpt, float* v_last, int64_t T, int64_t cols, int dtype,
                              int ckpt_interval, void* stream) {
  if (T < 0 || cols < 0 || !dtype_ok(dtype) || (ckpt_interval != 8 && ckpt_interval != 32))
    return NSB_ERR_INVALID_ARG;
  if (cols == 0) return NSB_OK;
  if (!v_init || !v_last || !f32_aligned(v_init) || !f32_aligned(v_last) || !f32_aligned(v_ckpt))
    return NSB_ERR_INVALID_ARG;
  if (T == 0) {
    NSB_CUDA_TRY(cudaMemcpyAsync(v_last, v_init, sizeof(float) * cols, cudaMemcpyDeviceToDevice,
                                 static_cast<cudaStream_t>(stream)), "copy v_init");
    return NSB_OK;
  }
  if (!beta || !u || !v_out) return NSB_ERR_INVALID_ARG;
  if (!elem_aligned(beta, dtype) || !elem_aligned(u, dtype) || !elem_aligned(v_out, dtype))
    return NSB_ERR_INVALID_ARG;
  nsb::FwdArgs a;
  a.beta = beta; a.drive = u; a.v_init = v_init; a.spike = v_out; a.ckpt = v_ckpt; a.vlast = v_last;
  a.T = T; a.cols = cols; a.mode = nsb::MODE_LIN; a.tile = ckpt_interval;
  a.stream = static_cast<cudaStream_t>(stream);
  return run_lin_fwd(a, dtype);
}

int nsb_linear_recurrence_bwd(const void* beta, const void* u, const float* v_ckpt, const void* g_v,
                              void* g_beta, void* g_u, float* g_vinit, int64_t T, int64_t cols, int dtype,
                              int ckpt_interval, uint32_t* chain_scratch, void* stream) {
  if (T < 0 || cols < 0 || !dtype_ok(dtype) || (ckpt_interval != 8 && ckpt_interval != 32))
    return NSB_ERR_INVALID_ARG;
  if (cols == 0) return NSB_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (!f32_aligned(v_ckpt) || !f32_aligned(g_vinit)) return NSB_ERR_INVALID_ARG;
  if (T == 0) {
    if (g_vinit) NSB_CUDA_TRY(cudaMemsetAsync(g_vinit, 0, sizeof(float) * cols, st), "memset grad v_init");
    return NSB_OK;
  }
  if (!beta || !u || !v_ckpt || !g_v) return NSB_ERR_INVALID_ARG;
  const void* ep[] = {beta, u, g_v, g_beta, g_u};
  for (const void* p : ep)
    if (!elem_aligned(p, dtype)) return NSB_ERR_INVALID_ARG;
  nsb::BwdArgs a;
  a.beta = beta; a.drive = u; a.ckpt = v_ckpt; a.g_spike = g_v; a.g_beta = g_beta; a.g_drive = g_u;
  a.g_vinit = g_vinit;
  a.T = T; a.cols = cols; a.mode = nsb::MODE_LIN; a.tile = ckpt_interval;
  a.surrogate = NSB_SURR_SIGMOID; a.alpha = 1.0f; a.stream = st;
  if (!f32_aligned(chain_scratch)) return NSB_ERR_INVALID_ARG;
  a.chain_sync = chain_scratch;
  return run_lin_bwd(a, dtype);
}

}  // extern "C"
