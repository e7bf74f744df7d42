/*
 * neuronspark_b200 — C ABI of the B200 (sm_100a) PLIF scan path.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream
 * (passed as void*, i.e. a cudaStream_t), returns an int status (0 = NSB_OK),
 * never throws and never exits. Nothing here allocates device memory unless
 * its comment says so. All kernels are asynchronous on the given stream.
 *
 * Layouts follow the reference project (Brain2nd/NeuronSpark):
 *   scan tensors   time-major [T, cols], cols = product of the trailing dims
 *                  (batch * channels), contiguous
 *                  (atomic_ops/parallel_scan.py:713-714)
 *   per-column     [cols] vectors, always fp32 on this ABI
 *   codec frames   [S*16, B, D]; codec values [B, S, D]
 *                  (atomic_ops/fp16_codec.py:17-46)
 *
 * "stream dtype" is the element type of the big [T, cols] tensors of one call
 * (all of them share it). The arithmetic is always fp32 with one rounded
 * multiply and one rounded add per state update (no fused multiply-add), so
 * spikes agree bit for bit with the reference's eager PyTorch time loop.
 */
#ifndef NEURONSPARK_B200_H_
#define NEURONSPARK_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ---- */
#define NSB_OK 0
#define NSB_ERR_INVALID_ARG 1   /* null/misaligned pointer, bad size or enum   */
#define NSB_ERR_UNSUPPORTED 2   /* device is not sm_100, or option unavailable */
#define NSB_ERR_CUDA 3          /* a CUDA runtime/driver call failed           */
#define NSB_ERR_DEVICE_TIMEOUT 4 /* a bounded device-side wait ran out         */
#define NSB_ERR_TOO_LARGE 5     /* size exceeds a documented fixed maximum     */

/* ---- element types of streamed tensors ---- */
#define NSB_F32 0
#define NSB_BF16 1
#define NSB_F16 2

/* ---- rounding of the binary residual on bf16 frames ----
 * fp32 and fp16 frames leave no choice (every intermediate of decode + add is
 * exact in them); for bf16 frames the reference behaves in two ways:
 *   EAGER     its ops run one by one (_binary_residual_naive, or
 *             _binary_residual_fwd called directly, atomic_ops/fp16_codec.py:103-164):
 *             mantissa sum, 1+m, both decoded values and their sum are each
 *             rounded to bf16;
 *   COMPILED  binary_residual() as it runs on a GPU, through
 *             torch.compile(_binary_residual_fwd) (:168-186): the decode stays in
 *             fp32 inside inductor's fused kernel and only the sum - a bf16 tensor
 *             between two kernels - is rounded to bf16 (observed bit for bit on a
 *             B200, torch 2.11, on the frames of the reference's own layers).   */
#define NSB_RESIDUAL_EAGER 0
#define NSB_RESIDUAL_COMPILED 1

/* ---- surrogate gradients ---- */
#define NSB_SURR_SIGMOID 0 /* a*sig(ax)*(1-sig(ax)), exp argument clamped at 88
                              (atomic_ops/parallel_scan.py:291-296)            */
#define NSB_SURR_ATAN 1    /* (a/2)/(1+(pi/2*a*x)^2), the derivative of
                              atan(pi/2*a*x)/pi + 1/2 (SpikingJelly's ATan); the
                              reference's fused kernels have sigmoid only, so
                              this one is checked against torch autograd
                              through that primitive                           */

/* Library version (major*10000 + minor*100 + patch). */
int nsb_version(void);

/* Human-readable text for a status code; never NULL. */
const char* nsb_status_string(int status);

/* Text of the last CUDA error this library saw on the calling thread. */
const char* nsb_last_cuda_error(void);

/* Reads and clears the device-side error word (set when a bounded wait inside
 * a kernel gave up). Synchronises nothing: the word lives in mapped host
 * memory; call after synchronising the stream you care about.
 *
 * The word is sticky: while it is non-zero every entry point of the scan family
 * (nsb_plif_*, nsb_linear_recurrence_*) returns NSB_ERR_DEVICE_TIMEOUT before it
 * launches anything, so a caller that never looks at the word still learns of a
 * timed-out scan at its next call; this function is what clears it. A warp that
 * gives up leaves NaN in its columns of V_last / W_last (forward) or grad_v_init
 * (backward) and does not write the rest of its outputs.
 * The first scan call of a process allocates the (64-byte, mapped, pinned) word:
 * make that call outside CUDA stream capture.
 * The reference has no counterpart: its Triton kernels have no waits to bound. */
int nsb_device_error_word(uint32_t* out);

/* Limit of every bounded device-side wait in nanoseconds; 0 restores the default
 * of 2 s. Process-global, read at each launch. */
int nsb_set_wait_limit_ns(uint64_t ns);

/* Self-test of the timeout path, for test suites: launches one warp that waits,
 * with the current limit, on a barrier that nothing will ever complete, and one
 * that waits for a counter in global memory that nothing advances (the wait of a
 * chained backward launch). Both give up, set bits 31 and 30 of the error word
 * and return; nothing faults and no memory operation is left in flight. Set a
 * short limit first (nsb_set_wait_limit_ns) unless a 2 s kernel is wanted. */
int nsb_selftest_wait_timeout(void* stream);

/*
 * One element type per call. Every [T, cols] tensor of a scan call ("stream") has the call's
 * `dtype`; per-column vectors are fp32. The reference widens each pointer from its own element
 * type (tl.load(...).to(tl.float32), atomic_ops/parallel_scan.py:223-225) and returns each
 * gradient in its input's type (:752-755), so a call with, say, fp32 beta and bf16 u is legal
 * there. Here such a caller first brings the streams to one type - fp32 if they differ, which
 * is exact - and converts outputs back where it needs to, with this kernel (widening exact,
 * narrowing round-to-nearest-even); the Python mirror does exactly that. A type per tensor
 * would multiply the scan kernels by 3^4 instantiations for a case the reference's own layers
 * do not produce (under autocast all modulation outputs are fp32, under bf16 parameters all
 * are bf16).
 */
int nsb_convert(const void* src, void* dst, int64_t n, int src_dtype, int dst_dtype, void* stream);

/*
 * Time split of scans over few columns: the row-parameter scans by default, and - forward only, and only
 * on request (nsb_set_time_split with max_segments above 1) - the selective u-form, resonate-and-fire and
 * modulated scans, whose `split_scratch` argument has the same meaning (a single sequence of the 768-wide
 * model is 6 144 columns of hidden neurons; those neurons' memory can be longer than any affordable warm-up,
 * see below, so the caller who knows their dynamics decides). A scan over a few thousand
 * columns occupies a few hundred warps while each warp is bound by its own serial chain over T;
 * the other SMs idle. Given scratch memory (`split_scratch` of nsb_plif_rowparam_fwd,
 * nsb_plif_rowparam_residual_fwd, nsb_plif_rowparam_pattern_fwd, nsb_plif_rowparam_bwd and
 * nsb_plif_rowparam_bwd_dalpha: NULL, or
 * nsb_time_split_scratch_floats(cols) floats of device memory that the call may overwrite - 64 per
 * column up to 37 888 columns, the widest scan that is ever split; beyond that only the few KB of
 * counters that let the two backward entry points chain chunks of the time axis, see
 * nsb_set_chain_chunks), such a scan is cut along time into up to 16 segments that run side by side: a later segment is entered
 * `warm_steps` early from V = 0 and keeps what it computes from its own first step on - PLIF
 * trajectories driven by the same input become bit-identical a few hundred steps after they
 * started apart - and a second launch compares every segment's assumed starting state with the
 * exact one, bit for bit, and rescans the segments where they differ. Results therefore equal the
 * unsplit scan's exactly for every input; only the time taken depends on how often a rescan is
 * needed. The backward is cut the same way, walking each segment from its last step to its first:
 * its adjoint recurrence acc' = beta*(acc + ...) forgets its starting value as the forward forgets
 * its state, grad_u and grad_v_init come out bit-identical to the serial launch, and the sums over
 * time of grad_beta_row / grad_v_th_row are added up segment by segment (same terms, another
 * association: equal to the serial sums to fp32 rounding, and deterministic). The reference has no counterpart (its kernels walk T serially, one program per 128
 * columns, atomic_ops/parallel_scan.py:496-530).
 *
 * A neuron whose beta has been trained close to 1 forgets more slowly than the warm-up is long; its
 * segments are rescanned and the two launches cost more than the plain scan. In automatic mode each
 * split launch therefore copies its rescan counters to pinned host memory (asynchronously, 8 bytes),
 * and the next launch with the same beta_row vector, T, cols and direction reads what has arrived:
 * when one warp had to rescan more segments than the split saved, that neuron's scans run unsplit for
 * the next 64 calls and then try again. The results do not depend on any of this. (The neuron is known
 * by the address of its beta_row vector: a caller that rebuilds the vector every step gets the feedback
 * where its allocator hands out the same address again, as a caching allocator does in a steady loop.
 * The first automatic split launch allocates 2 KB of pinned memory; inside a stream capture it skips that.)
 *
 * nsb_set_time_split      max_segments: 0 = automatic, 1 = never split, 2..16 = at most that many
 *                         (and split even where the planner expects little gain, without the
 *                         feedback above); warm_steps: 0 = default (1024). Process-global, read at
 *                         each launch; a call also forgets what earlier launches rescanned.
 * nsb_last_time_split     {segments, tiles per segment, warm-up tiles} of the calling thread's last
 *                         forward scan launch (segments = 1: it was not split). After a split
 *                         launch the number of rescanned (warp, segment) pairs is the uint32 at
 *                         split_scratch[k*segments*cols], k = 2 for a first-order forward, 4 for a
 *                         resonate-and-fire forward and for the backward; the uint32 after it is
 *                         the largest number of segments any one warp rescanned.
 */
int nsb_set_time_split(int max_segments, int warm_steps);
int64_t nsb_time_split_scratch_floats(int64_t cols);
int nsb_last_time_split(int32_t out[3]);

/*
 * Chained chunks of a backward scan over many columns. A backward launch gives every block of
 * columns to one CTA that walks all of T; with more CTAs than the GPU holds at once (768 for 444
 * places at 196 608 columns) the last round of CTAs is partly empty and lasts as long as a full
 * one, and at any moment the resident CTAs are spread over all of T, where walking the same few
 * rows of every [T, cols] tensor together suits DRAM better. Given scratch, the library cuts the time axis into q chunks, launches q times as many CTAs
 * and lets each take a ticket: tickets walk the chunks from the last to the first. The CTA of a
 * chunk waits (bounded, see nsb_set_wait_limit_ns) until the CTA of the next chunk of its columns -
 * an earlier ticket, so running or finished - has left the adjoint and the running sums over time
 * in the per-column outputs (g_vinit, g_winit, the row / bias gradient rows), continues from
 * them and leaves its own there. The operations and their order are those of one CTA walking all of
 * T, so every output is bit-identical to the unchained launch. Used by the backward entry points
 * that take chain_scratch (nsb_plif_selective_bwd, nsb_plif_rf_bwd[_dalpha],
 * nsb_linear_recurrence_bwd), by nsb_plif_modulated_bwd (inside its own scratch) and by
 * nsb_plif_rowparam_bwd[_dalpha] (inside split_scratch, for scans too wide for the time split), when g_vinit (and g_winit, and the bias
 * gradients, where the scan has them) are requested. The reference has no counterpart (one Triton
 * program per 128 columns walks T, atomic_ops/parallel_scan.py:234-307).
 *
 * nsb_chain_scratch_words  words (uint32) of scratch for a scan over `cols` columns.
 * nsb_set_chain_chunks     0 = automatic (selective, resonate-and-fire and linear scans over 49 152
 *                          columns and more: chunks of 512 steps, of 128 from 98 304 columns on; with the
 *                          modulation fused in: chunks of 1024 steps where the launch has more CTAs than
 *                          the GPU holds; row-parameter scans: never), 1 = never, 2..1024 = that many
 *                          chunks (at most one per tile) on every launch that is given the scratch.
 *                          Process-global.
 * nsb_last_chain_chunks    chunks of the last backward launch of the process (1 = not chained).
 */
int64_t nsb_chain_scratch_words(int64_t cols);
int nsb_set_chain_chunks(int chunks);
int nsb_last_chain_chunks(void);

/*
 * Rotation of forward scans with the modulation fused in (nsb_plif_modulated_fwd without the moments of
 * u) over few columns. Two thirds of such a scan's instructions - sigmoid, softplus, the stability
 * rescale - depend on the step's inputs only; the recurrence itself is a handful per step. Over few
 * columns (49 152 for one batch of 8 sequences of the 768-wide model: 2.5 warps per warp scheduler,
 * 56 % of the issue slots busy) the launch is bound by how few warps there are, so R = 2..4 warps of a
 * CTA share each group of 32 columns and take its tiles in turn: a warp evaluates its tile's modulation,
 * then waits (bounded, see nsb_set_wait_limit_ns) for the membrane state its predecessor left after the
 * tile before, runs the tile's steps and hands the state on through shared memory. Per column the
 * operations and their order are those of the one-warp scan: every output is bit-identical. The
 * reference has no counterpart (modulation and scan are separate passes there,
 * atomic_ops/snn_block.py:52-76 and atomic_ops/parallel_scan.py:1655-1715).
 *
 * Measured (B200, bf16, T = 8192, 6 144 channels, forward ms on 32-step tiles with one warp per group ->
 * rotating on 8-step tiles): resonate-and-fire, one sequence (6 144 columns) 0.89 -> 0.50, two 0.89 -> 0.57,
 * four 1.00 -> 0.88; first order, one sequence 0.62 -> 0.43. At 49 152 columns, where every scheduler has
 * 2.6 warps already, it is a loss (1.43 -> 1.80 ms) and is not used. Built for 8-step tiles (ckpt_interval
 * 8), one lane per thread (the library's choice for such calls up to 32 768 columns).
 *
 * nsb_set_scan_rotation   0 = automatic (up to 1.5 column warps per warp scheduler, i.e. 28 416 columns:
 *                         about five warps per scheduler, at most 4 per group, all CTAs resident),
 *                         1 = never, 2..4 = that many warps per column group. Process-global.
 * nsb_last_scan_rotation  warps per column group of the calling thread's last forward scan launch (1 = none).
 * nsb_scan_rotation_query what the current setting gives a scan of T steps over `cols` columns (one lane per
 *                         thread, `tile` steps per tile) on a B200, before the check that all CTAs are
 *                         resident; host arithmetic, needs no GPU. 0 for invalid arguments.
 */
int nsb_set_scan_rotation(int warps);
int nsb_last_scan_rotation(void);
int nsb_scan_rotation_query(int64_t T, int64_t cols, int tile);

/* Tuning override for the scan kernels, used by sweeps and tests. Any field
 * <= 0 keeps the built-in heuristic. warps_per_cta: warps of one CTA (each
 * warp owns 32*lanes_per_thread columns and its own TMA pipeline); stages:
 * depth of each warp's shared-memory ring; lanes_per_thread: 1, 2 or 4;
 * force_direct: 0 = automatic, 1 = never use the TMA path, 2 / 3 = TMA path with
 * the ring refilled one tile late always / never (automatic: late when the
 * launch has few warps per SM). Process-global. */
int nsb_set_tuning(int warps_per_cta, int stages, int lanes_per_thread, int force_direct);

/* How the last scan launch on this thread was configured (for benchmarks):
 * out[0]=used_tma, out[1]=warps_per_cta, out[2]=stages, out[3]=lanes_per_thread,
 * out[4]=grid, out[5]=dynamic smem bytes per CTA, out[6]=steps per tile,
 * out[7]=kernel launches issued by the call. */
int nsb_last_launch_info(int32_t out[8]);

/* The launch plan the scan kernels would use on a B200 for a problem, computed on
 * the host without touching CUDA: out[0]=lanes per thread, out[1]=warps per CTA,
 * out[2]=ring stages, out[3]=grid, out[4]=dynamic shared memory per CTA.
 * nstreams = number of streamed [T, cols] inputs (forward: 1 row-param, 3 u-form,
 * 4 gain*cur form; backward: those + 1 for g_spike + 1 if g_vpost). */
int nsb_scan_plan_query(int backward, int nstreams, int elem_size, int64_t T, int64_t cols,
                        int tile, int32_t out[5]);

/* How the time axis of a scan would be divided on a B200, computed on the host: out[0..2] = segments,
 * tiles per segment and warm-up tiles of the time split a row-parameter scan of this shape takes when it
 * is given scratch (1, 0, 0: none); out[3] = chained chunks of a backward launch over these columns
 * (1: none; the modulated kernels' rule is evaluated for CTAs of warps_per_cta warps, three per SM).
 * lanes / warps_per_cta: the launch shape (nsb_scan_plan_query). */
int nsb_time_plan_query(int backward, int modulated, int64_t T, int64_t cols, int tile, int lanes,
                        int warps_per_cta, int32_t out[4]);

/*
 * Selective PLIF forward scan. Replaces _TritonPLIFForward.forward /
 * _fused_plif_fwd_kernel (atomic_ops/parallel_scan.py:196-232, 706-735).
 *
 *   v = v_init; for k in [0,T):  v_pre = beta[k]*v + drive[k]
 *                                s = (v_pre >= v_th[k]);  v = v_pre - v_th[k]*s
 *   drive[k] = u[k]                    when gain == NULL  (reference signature)
 *            = gain[k]*cur[k]          otherwise (SelectivePLIFNode form,
 *                                       atomic_ops/selective_plif.py:127)
 *
 * beta, u_or_cur, gain, v_th : [T, cols] in `dtype`
 * v_init                     : [cols] fp32
 * spike_dense  (optional)    : [T, cols] in `dtype`, values {0,1}
 * spike_packed (optional)    : [T, ceil(cols/32)] uint32, bit i of word w is
 *                              column 32*w+i, tail bits zero
 * v_post       (optional)    : [T, cols] in `dtype`
 * v_ckpt       (optional)    : [ceil(T/ckpt_interval), cols] fp32; row j holds
 *                              the membrane state BEFORE step j*ckpt_interval
 *                              (row 0 = v_init). Needed by the backward.
 * v_last                     : [cols] fp32, state after the last step
 * ckpt_interval              : 8, 16 or 32 (also the time-tile of the pipeline; longer
 *                              tiles amortise per-tile overhead when there are few
 *                              columns, 8 gives the widest kernels for many columns)
 */
int nsb_plif_selective_fwd(const void* beta, const void* u_or_cur, const void* gain,
                           const void* v_th, const float* v_init, void* spike_dense,
                           uint32_t* spike_packed, void* v_post, float* v_ckpt,
                           float* v_last, int64_t T, int64_t cols, int dtype,
                           int ckpt_interval, float* split_scratch, void* stream);

/*
 * Reverse-time surrogate-gradient pass of the selective scan. Replaces
 * _TritonPLIFForward.backward / _fused_plif_bwd_kernel
 * (atomic_ops/parallel_scan.py:234-307, 737-768) with the same recurrence:
 *   tot = g_vpost[k] + acc;  gpre = g_spike[k]*sg(x_k) + tot
 *   g_beta[k] = gpre*V[k-1]; g_u[k] = gpre; g_vth[k] = -g_spike[k]*sg - tot*s[k]
 *   acc = gpre*beta[k];      g_vinit = acc after k = 0
 * and for the gain*cur form g_cur = gpre*gain, g_gain = gpre*cur.
 * Instead of reading a stored V_post it recomputes each time tile from v_ckpt
 * with the forward's exact arithmetic, so spikes and states are identical.
 *
 * g_vpost may be NULL (treated as zero). g_gain is ignored when gain == NULL.
 * Any of the gradient outputs may be NULL (not written).
 * chain_scratch: NULL, or nsb_chain_scratch_words(cols) words of device memory that let a
 * launch with more CTAs than the GPU holds at once cut the time axis into chained chunks
 * (see nsb_set_chain_chunks); results are bit-identical either way.
 */
int nsb_plif_selective_bwd(const void* beta, const void* u_or_cur, const void* gain,
                           const void* v_th, const float* v_ckpt, const void* g_spike,
                           const void* g_vpost, void* g_beta, void* g_u_or_cur,
                           void* g_gain, void* g_vth, float* g_vinit, int64_t T,
                           int64_t cols, int dtype, int ckpt_interval, int surrogate,
                           float alpha, uint32_t* chain_scratch, void* stream);

/*
 * Row-parameter PLIF forward scan (beta and v_th constant over time, one fp32
 * value per column). Replaces _fused_plif_fwd_rowparam_kernel and
 * _fused_plif_fwd_rowparam_noV_kernel (atomic_ops/parallel_scan.py:314-343,
 * 496-523) — pass v_post = NULL for the latter. Outputs as in
 * nsb_plif_selective_fwd.
 */
int nsb_plif_rowparam_fwd(const float* beta_row, const void* u, const float* vth_row,
                          const float* v_init, void* spike_dense, uint32_t* spike_packed,
                          void* v_post, float* v_ckpt, float* v_last, int64_t T,
                          int64_t cols, int dtype, int ckpt_interval, float* split_scratch, void* stream);

/*
 * Reverse pass of the row-parameter scan. Replaces
 * _fused_plif_bwd_rowparam_kernel and _fused_plif_bwd_rowparam_recomp_kernel
 * (atomic_ops/parallel_scan.py:345-413, 525-612): g_u per step, g_beta_row and
 * g_vth_row reduced over time per column (fp32 [cols]). g_vpost may be NULL.
 */
int nsb_plif_rowparam_bwd(const float* beta_row, const void* u, const float* vth_row,
                          const float* v_ckpt, const void* g_spike, const void* g_vpost,
                          float* g_beta_row, void* g_u, float* g_vth_row, float* g_vinit,
                          int64_t T, int64_t cols, int dtype, int ckpt_interval,
                          int surrogate, float alpha, float* split_scratch,
                          void* stream);

/*
 * Resonate-and-fire (second-order) PLIF scan, forward. Replaces
 * _fused_rf_plif_fwd_kernel and _fused_rf_plif_fwd_recompute_kernel
 * (atomic_ops/parallel_scan.py:777-818, 924-956; callers :1610-1726,
 * atomic_ops/snn_block.py:252-256):
 *   v_pre = (beta[k]*v - omega[k]*w) + u[k];   w' = omega[k]*v + beta[k]*w
 *   s = (v_pre >= v_th[k]);  v = v_pre - v_th[k]*s;  w = w'      (W is never reset)
 * beta, omega, u, v_th [T, cols] in `dtype`; v_init, w_init [cols] fp32.
 * Optional outputs: spike_dense, spike_packed, v_post, w_out ([T, cols]); the
 * checkpoints v_ckpt and w_ckpt ([ceil(T/ckpt_interval), cols] fp32, both or
 * neither) are what the backward needs. v_last, w_last [cols] fp32 are required.
 */
int nsb_plif_rf_fwd(const void* beta, const void* omega, const void* u, const void* v_th,
                    const float* v_init, const float* w_init, void* spike_dense,
                    uint32_t* spike_packed, void* v_post, void* w_out, float* v_ckpt,
                    float* w_ckpt, float* v_last, float* w_last, int64_t T, int64_t cols,
                    int dtype, int ckpt_interval, float* split_scratch, void* stream);

/*
 * Reverse pass of the resonate-and-fire scan. Replaces _fused_rf_plif_bwd_kernel and
 * _fused_rf_plif_bwd_recompute_kernel (atomic_ops/parallel_scan.py:820-916, 958-1069)
 * with the same coupled V/W adjoint recurrence (:835-848):
 *   gpre = g_spike*sg + (g_vpost + acc_v);   g_u = gpre
 *   g_beta  = gpre*V[k-1] + acc_w*W[k-1];    g_omega = acc_w*V[k-1] - gpre*W[k-1]
 *   g_vth   = -g_spike*sg - (g_vpost + acc_v)*s
 *   acc_v'  = gpre*beta + acc_w*omega;       acc_w'  = acc_w*beta - gpre*omega
 * States are recomputed per tile from the checkpoints. g_vpost may be NULL; a
 * gradient for W is not taken (the reference ignores it, :1114).
 */
int nsb_plif_rf_bwd(const void* beta, const void* omega, const void* u, const void* v_th,
                    const float* v_ckpt, const float* w_ckpt, const void* g_spike,
                    const void* g_vpost, void* g_beta, void* g_omega, void* g_u, void* g_vth,
                    float* g_vinit, float* g_winit, int64_t T, int64_t cols, int dtype,
                    int ckpt_interval, int surrogate, float alpha, uint32_t* chain_scratch,
                    void* stream);

/*
 * FP16 boundary codec (atomic_ops/fp16_codec.py).
 *
 * nsb_fp16_encode        fp16_encode (:17-46): values [B,S,D] in dtype_in ->
 *                        frames [S*16,B,D] in dtype_out, {0,1}, MSB first.
 * nsb_fp16_decode_fwd    fp16_decode (:49-98): frames -> values [B,S,D], same
 *                        dtype; an all-ones exponent decodes as a normal
 *                        number. With bf16 frames the mantissa sum, 1+m and the
 *                        result are rounded to bf16 as the reference's eager
 *                        arithmetic does.
 * nsb_fp16_decode_bwd    autograd of that formula: g_values [B,S,D] and the
 *                        frames -> g_frames [S*16,B,D].
 * nsb_binary_residual    binary_residual / _binary_residual_fwd (:115-197):
 *                        encode(decode(a)+decode(b)); `rounding` is one of
 *                        NSB_RESIDUAL_* (it matters for bf16 frames only).
 * nsb_encode_ste_bwd     _BinaryEncodeSTE.backward (:220-224): mean over the 16
 *                        frames of each token.
 */
int nsb_fp16_encode(const void* values, void* frames, int64_t B, int64_t S, int64_t D,
                    int dtype_in, int dtype_out, void* stream);
int nsb_fp16_decode_fwd(const void* frames, void* values, int64_t B, int64_t S, int64_t D,
                        int dtype, void* stream);
int nsb_fp16_decode_bwd(const void* frames, const void* g_values, void* g_frames,
                        int64_t B, int64_t S, int64_t D, int dtype, void* stream);
int nsb_binary_residual(const void* frames_a, const void* frames_b, void* frames_out,
                        int64_t B, int64_t S, int64_t D, int dtype, int rounding, void* stream);
int nsb_encode_ste_bwd(const void* g_frames, void* g_values, int64_t B, int64_t S,
                       int64_t D, int dtype, void* stream);

/*
 * Lateral inhibition = divisive normalisation = RMSNorm
 * (atomic_ops/lateral_inhibition.py:50-119, 122-171; atomic_ops/rms_norm.py).
 *   out = x * rsqrt(mean(x^2) + eps) * gain        rows of D, fp32 math
 * Backward: g_x as the reference's kernel; g_gain [D] fp32 is reduced over the
 * rows inside the call (the reference materialises a rows x D tensor and sums
 * it afterwards). `partial` is caller-provided scratch of
 * nsb_li_bwd_scratch_floats(rows, D) floats.
 * gain is [D] in `gain_dtype`; x, out, g_out, g_x in `dtype`.
 */
int nsb_lateral_inhibition_fwd(const void* x, const void* gain, void* out, int64_t rows,
                               int64_t D, float eps, int dtype, int gain_dtype,
                               void* stream);
int64_t nsb_li_bwd_scratch_floats(int64_t rows, int64_t D);
int nsb_lateral_inhibition_bwd(const void* g_out, const void* x, const void* gain,
                               void* g_x, float* g_gain, float* partial, int64_t rows,
                               int64_t D, float eps, int dtype, int gain_dtype,
                               void* stream);

/*
 * nsb_lateral_inhibition_bwd for callers that cannot allocate device memory.
 * (No counterpart in the reference: its backward allocates a rows x D tensor.)
 *
 * Same inputs, outputs and results as nsb_lateral_inhibition_bwd, but without the
 * `partial` argument: the per-CTA partial sums of g_gain are kept in a fixed
 * array inside the library image instead. It is meant for hosts that own all
 * device memory themselves or may not call the CUDA allocator where they run
 * this (a server that pre-reserved the device for its own pool, a plugin that
 * only receives input/output buffers, a loop in which cudaMalloc/cudaFree are
 * ruled out because they synchronise the device). The call itself allocates
 * nothing, neither through CUDA nor through any library.
 *
 * Cost and limits:
 *  - the array is 524 288 floats (2 MiB) of device memory on every GPU that
 *    loads the library, held until the process exits;
 *  - D may not exceed 58 112 (NSB_ERR_TOO_LARGE otherwise): one warp's fp32 row of
 *    partial sums has to fit the 227 KB of shared memory a CTA can have, which is
 *    the bound of nsb_lateral_inhibition_bwd as well; the array itself would hold
 *    rows of up to 524 288. When (CTAs the normal entry point would use) * D
 *    exceeds the array, fewer CTAs are launched, so rows wider than 1 771 floats
 *    run slower than with caller scratch;
 *  - the first call on each device looks up the array's device address
 *    (with that device current). Make that first call outside any stream
 *    capture; later calls do no set-up;
 *  - all calls on a device share the one array. Nothing in it has to be zeroed:
 *    each call writes every element it later reads. But two calls that overlap
 *    on the GPU (different streams, or one stream per thread) race on it and
 *    corrupt each other's g_gain — serialise them.
 */
int nsb_lateral_inhibition_bwd_static(const void* g_out, const void* x, const void* gain,
                                      void* g_x, float* g_gain, int64_t rows, int64_t D,
                                      float eps, int dtype, int gain_dtype, void* stream);

/*
 * Modulation + scan in one pass. Replaces the pair the reference runs between
 * its input projections and W_out in SNNBlock.forward_parallel: the inductor
 * kernel of _fused_modulation_rf (atomic_ops/snn_block.py:52-76, called at
 * :237-241) followed by rf_plif_parallel_forward_recompute (:252-256); with
 * raw_omega == NULL, the first-order pair _fused_modulation + plif_parallel_forward
 * (archive/atomic_ops_v75_pre/snn_block.py:41-47, 186-199).
 *   beta  = sigmoid(raw_beta + b_beta)       alpha = softplus(raw_alpha + b_alpha)
 *   v_th  = v_th_min + |raw_th + b_th|       omega = softplus(raw_omega + b_omega)
 *   r2 = beta^2 + omega^2; if r2 > 0.999^2: (beta, omega) *= 0.999 * rsqrt(r2)
 *   u = alpha * I
 * and then the selective scan (u-form) or the resonate-and-fire scan on those
 * values, which stay in registers: beta, u, v_th, omega are never written to
 * memory (the reference writes and re-reads these four [T, cols] tensors, the
 * largest of a layer, and their gradients).
 * raw_* and cur are [T, cols] in `dtype`; the biases are fp32 [channels] with
 * cols = batch * channels (column c uses bias c % channels); v_init / w_init
 * [cols] fp32. Outputs as nsb_plif_rf_fwd, without v_post / w_out.
 * ckpt_interval is 8 or 32.
 * Numerics: all arithmetic in fp32; sigmoid, softplus and rsqrt use the
 * hardware approximations: beta within 1e-6 relative of correct rounding,
 * alpha and omega within 1e-6 relative or 2.5e-7 absolute, v_th exact;
 * the modulated values are not rounded to `dtype` (the reference rounds them
 * when its parameters are bf16).
 * Adaptive surrogate slope (optional; both pointers or neither): the reference
 * derives it from `u_hidden.std()` (atomic_ops/plif_node.py:93-100), a tensor
 * that no longer exists here. The kernel accumulates the moments of
 * u = alpha*I while it streams and *alpha_out (device) receives
 * clamp(alpha0 * sigma0 / max(std(u), 1e-6), 1, 20), std taken at fp32;
 * u_stats is scratch of nsb_plif_modulated_fwd_stats_doubles(cols) doubles.
 * Give alpha_out to nsb_plif_modulated_bwd as alpha_dev.
 */
int64_t nsb_plif_modulated_fwd_stats_doubles(int64_t cols);
int nsb_plif_modulated_fwd(const void* raw_beta, const void* raw_alpha, const void* raw_th,
                           const void* raw_omega, const void* cur, const float* b_beta,
                           const float* b_alpha, const float* b_th, const float* b_omega,
                           float v_th_min, int64_t channels, const float* v_init,
                           const float* w_init, void* spike_dense, uint32_t* spike_packed,
                           float* v_ckpt, float* w_ckpt, float* v_last, float* w_last,
                           float alpha0, float sigma0, double* u_stats, float* alpha_out, int64_t T,
                           int64_t cols, int dtype, int ckpt_interval, float* split_scratch,
                           void* stream);

/* Floats of scratch nsb_plif_modulated_bwd needs when any bias gradient is asked for. */
int64_t nsb_plif_modulated_bwd_scratch_floats(int64_t cols);

/*
 * Reverse pass of nsb_plif_modulated_fwd for a gradient arriving on the spikes:
 * recomputes modulation and membrane state tile by tile from the checkpoints,
 * runs the scan's adjoint and pushes it through the modulation in registers.
 * Outputs (each optional): gradients of the raw projections and of I
 * ([T, cols], `dtype`), of the biases (fp32 [channels], summed over time and
 * batch in a fixed order; needs `scratch`), of v_init / w_init (fp32 [cols]).
 * Replaces the autograd backward of the two reference functions named above.
 * alpha_dev, when not NULL, is a device float that overrides `alpha`.
 */
int nsb_plif_modulated_bwd(const void* raw_beta, const void* raw_alpha, const void* raw_th,
                           const void* raw_omega, const void* cur, const float* b_beta,
                           const float* b_alpha, const float* b_th, const float* b_omega,
                           float v_th_min, int64_t channels, const float* v_ckpt,
                           const float* w_ckpt, const void* g_spike, void* g_raw_beta,
                           void* g_raw_alpha, void* g_raw_th, void* g_raw_omega, void* g_cur,
                           float* g_b_beta, float* g_b_alpha, float* g_b_th, float* g_b_omega,
                           float* scratch, float* g_vinit, float* g_winit, int64_t T, int64_t cols,
                           int dtype, int ckpt_interval, int surrogate, float alpha,
                           const float* alpha_dev, void* stream);

/*
 * Adaptive surrogate slope without a host round trip. Replaces the
 * `u.std().item()` of PLIFNode.get_surrogate (atomic_ops/plif_node.py:78-101):
 *   *alpha_out = clamp(alpha0 * sigma0 / max(std(u), 1e-6), 1, 20)
 * with std the unbiased standard deviation of the n elements of u, rounded to
 * `dtype` as torch's `u.std()` of such a tensor is. alpha_out is device memory
 * (one float); scratch holds nsb_surrogate_alpha_scratch_doubles() doubles.
 * Deterministic (fixed launch shape and summation order). n < 2 gives 20.
 * The *_dalpha backward entry points below take that device float in place of
 * the `alpha` argument and are otherwise identical to their namesakes.
 */
int64_t nsb_surrogate_alpha_scratch_doubles(void);
int nsb_surrogate_alpha(const void* u, int64_t n, int dtype, float alpha0, float sigma0,
                        double* scratch, float* alpha_out, void* stream);
int nsb_plif_rowparam_bwd_dalpha(const float* beta_row, const void* u, const float* vth_row,
                                 const float* v_ckpt, const void* g_spike, const void* g_vpost,
                                 float* g_beta_row, void* g_u, float* g_vth_row, float* g_vinit,
                                 int64_t T, int64_t cols, int dtype, int ckpt_interval,
                                 int surrogate, const float* alpha_dev,
                                 float* split_scratch, void* stream);
int nsb_plif_rf_bwd_dalpha(const void* beta, const void* omega, const void* u, const void* v_th,
                           const float* v_ckpt, const float* w_ckpt, const void* g_spike,
                           const void* g_vpost, void* g_beta, void* g_omega, void* g_u,
                           void* g_vth, float* g_vinit, float* g_winit, int64_t T, int64_t cols,
                           int dtype, int ckpt_interval, int surrogate, const float* alpha_dev,
                           uint32_t* chain_scratch, void* stream);

/*
 * Spikes packed in time: the 16 frames of one token and column as one uint16, the IEEE half bit
 * pattern they spell (frame 0 = sign = bit 15), in [S, B, D] (S = T/16) - 2 bytes per value
 * where the reference's dense frames (atomic_ops/fp16_codec.py:17-46) take 16 elements. The
 * reference has no packed form: it moves {0,1} frames in the activation dtype between layers
 * (atomic_ops/snn_block.py:281-285, atomic_ops/snn_ffn.py:188-195, model.py:155-157). These
 * entry points keep the reference's arithmetic and change only the storage:
 *
 * nsb_frames_pack / nsb_frames_unpack   dense frames [S*16,B,D] in `dtype` <-> patterns.
 * nsb_fp16_decode_packed_fwd            fp16_decode (:49-98) from patterns: values [B,S,D] in
 *                                       `dtype`, with the roundings that dtype's frames give.
 * nsb_fp16_decode_packed_bwd            its autograd: g_values [B,S,D] -> the 16 frame gradients of
 *                                       every value, dense [S*16,B,D] (what a scan's backward takes
 *                                       as g_spike).
 * nsb_binary_residual_packed            binary_residual (:115-197) on two pattern arrays of n values;
 *                                       `frame_dtype` names the frame dtype whose roundings apply,
 *                                       `rounding` is NSB_RESIDUAL_*.
 * nsb_plif_rowparam_pattern_fwd         the row-parameter scan (plif_rowparam_forward_recompute,
 *                                       atomic_ops/parallel_scan.py:1499-1535) writing its spikes as
 *                                       patterns [T/16, cols]; with patterns_in (may be NULL) the
 *                                       binary residual with that array is applied first, as
 *                                       nsb_plif_rowparam_residual_fwd does on frames. u is [T, cols]
 *                                       in `dtype`, T a multiple of 16, ckpt_interval 16 or 32; the
 *                                       backward is nsb_plif_rowparam_bwd on dense frame gradients.
 */
int nsb_frames_pack(const void* frames, uint16_t* patterns, int64_t B, int64_t S, int64_t D, int dtype,
                    void* stream);
int nsb_frames_unpack(const uint16_t* patterns, void* frames, int64_t B, int64_t S, int64_t D, int dtype,
                      void* stream);
int nsb_fp16_decode_packed_fwd(const uint16_t* patterns, void* values, int64_t B, int64_t S, int64_t D,
                               int dtype, void* stream);
int nsb_fp16_decode_packed_bwd(const uint16_t* patterns, const void* g_values, void* g_frames,
                               int64_t B, int64_t S, int64_t D, int dtype, void* stream);
int nsb_binary_residual_packed(const uint16_t* patterns_a, const uint16_t* patterns_b,
                               uint16_t* patterns_out, int64_t n, int frame_dtype, int rounding,
                               void* stream);
int nsb_plif_rowparam_pattern_fwd(const float* beta_row, const void* u, const float* vth_row,
                                  const float* v_init, const uint16_t* patterns_in,
                                  uint16_t* patterns_out, float* v_ckpt, float* v_last, int64_t T,
                                  int64_t cols, int dtype, int ckpt_interval, int frame_dtype,
                                  int rounding, float* split_scratch, void* stream);

/*
 * Row-parameter scan followed by the binary residual, in one pass. Replaces the
 * pair that ends SNNBlock.forward_parallel and SNNFFN.forward_parallel
 * (atomic_ops/snn_block.py:281-285, atomic_ops/snn_ffn.py:188-195):
 *   spike_out, V_last = plif_rowparam_forward_recompute(beta_row, u, v_th_row, v_init, alpha)
 *   return binary_residual(spike_out, spike_in_seq)          (atomic_ops/fp16_codec.py:115-197)
 * Every 16 steps of a column are one IEEE half bit pattern (frame 0 = sign):
 * frames_out = encode(decode(spikes) + decode(frames_in)), with the reference's
 * roundings for frames stored in `dtype` (`rounding`: NSB_RESIDUAL_*, as for
 * nsb_binary_residual). The spikes themselves are never
 * written. u, frames_in, frames_out are [T, cols] in `dtype`, T a multiple of
 * 16; ckpt_interval is 16 or 32; v_ckpt ([T/ckpt_interval, cols] fp32) is what
 * nsb_plif_rowparam_bwd needs - the residual's backward is the identity on both
 * inputs (straight-through, :171-173), so the gradient arriving for frames_out is
 * at once the gradient of frames_in and the g_spike of that call.
 */
int nsb_plif_rowparam_residual_fwd(const float* beta_row, const void* u, const float* vth_row,
                                   const float* v_init, const void* frames_in, void* frames_out,
                                   float* v_ckpt, float* v_last, int64_t T, int64_t cols, int dtype,
                                   int ckpt_interval, int rounding, float* split_scratch, void* stream);

/*
 * Linear recurrence V[k] = beta[k]*V[k-1] + u[k], V[-1] = v_init. Replaces
 * _fwd_recurrence_kernel / _bwd_recurrence_kernel / _TritonLinearRecurrence and
 * the CUDA branch of linear_recurrence (atomic_ops/parallel_scan.py:65-190,
 * 1282-1302). beta, u, v_out [T, cols] in `dtype` (state in fp32, each step one
 * rounded multiply and one rounded add); v_init, v_last [cols] fp32. The
 * backward recomputes V tile by tile from v_ckpt ([ceil(T/ckpt_interval), cols]
 * fp32, written by the forward when given) instead of reading a saved V:
 *   g += dV[k]; grad_u[k] = g; grad_beta[k] = g * V[k-1]; g *= beta[k]   (:110-141)
 * ckpt_interval is 8 or 32. chain_scratch: see nsb_set_chain_chunks (NULL = one CTA per column
 * block walks all of T).
 */
int nsb_linear_recurrence_fwd(const void* beta, const void* u, const float* v_init, void* v_out,
                              float* v_ckpt, float* v_last, int64_t T, int64_t cols, int dtype,
                              int ckpt_interval, void* stream);
int nsb_linear_recurrence_bwd(const void* beta, const void* u, const float* v_ckpt, const void* g_v,
                              void* g_beta, void* g_u, float* g_vinit, int64_t T, int64_t cols,
                              int dtype, int ckpt_interval, uint32_t* chain_scratch, void* stream);

/*
 * Mixture-of-experts output combine and its backward. Replaces
 * _moe_combine_fwd_kernel, _moe_combine_bwd_expert_kernel,
 * _moe_combine_bwd_weights_kernel and MoECombine (atomic_ops/moe_kernels.py:35-224):
 *   out[n, d] = shared[n, d] + sum_e experts[e, n, d] * weights[n, e]
 *   g_experts[e, n, d] = g_out[n, d] * weights[n, e]
 *   g_weights[n, e]    = sum_d g_out[n, d] * experts[e, n, d]
 * (grad of shared is g_out itself). shared / out / g_out [N, D], experts /
 * g_experts [E, N, D] contiguous in `dtype`; weights / g_weights [N, E] fp32.
 * fp32 accumulation. g_experts or g_weights may be NULL.
 */
int nsb_moe_combine_fwd(const void* shared, const void* experts, const float* weights, void* out,
                        int64_t N, int64_t D, int E, int dtype, void* stream);
int nsb_moe_combine_bwd(const void* g_out, const void* experts, const float* weights,
                        void* g_experts, float* g_weights, int64_t N, int64_t D, int E, int dtype,
                        void* stream);

/*
 * Expert merge of the mixture-of-experts SNN FFN in the frame domain
 * (atomic_ops/moe_snn_ffn.py:377-393, training branch: fp16_decode of the
 * shared output, of every expert's output and of the block input, weighted sum,
 * two additions, binary_encode_ste), as one kernel per direction.
 *   shared, residual, out: frames [S*16, B, D]; experts: [E, S*16, B, D];
 *   weights: [S, B, E] (the reference's full_weights), all in `dtype`; E <= 16.
 *   out = encode(((decode(shared) + sum_e decode(experts[e]) * w[e]) + decode(residual)))
 * with every product, the sum over experts and both additions rounded to
 * `dtype` as the reference's tensor arithmetic rounds them. Experts whose
 * weight for a token is exactly 0 are not read.
 * Backward (straight-through encode, atomic_ops/fp16_codec.py:208-226): g_total
 * = mean over a value's 16 output-frame gradients; g_shared / g_residual =
 * decode'(frames) * g_total; g_experts[e] = decode'(experts[e]) * g_total * w[e];
 * g_weights[s, b, e] = sum_d g_total * decode(experts[e]) (fp32 sum, fixed
 * order). Any of the four outputs may be NULL.
 */
int nsb_frames_combine_fwd(const void* shared, const void* experts, const void* weights,
                           const void* residual, void* out, int64_t B, int64_t S, int64_t D, int E,
                           int dtype, void* stream);
int nsb_frames_combine_bwd(const void* g_out, const void* shared, const void* experts,
                           const void* weights, const void* residual, void* g_shared, void* g_experts,
                           void* g_weights, void* g_residual, int64_t B, int64_t S, int64_t D, int E,
                           int dtype, void* stream);

/*
 * The modulation alone, written out: beta, u, v_th (and omega when raw_omega is
 * given) as [rows, channels] tensors in dtype_out (NSB_F32, or dtype_in). A
 * drop-in for the reference's _fused_modulation(_rf) functions in code that
 * keeps the unfused scan; it evaluates exactly what the fused scan evaluates
 * in registers.
 */
int nsb_modulation_fwd(const void* raw_beta, const void* raw_alpha, const void* raw_th,
                       const void* raw_omega, const void* cur, const float* b_beta,
                       const float* b_alpha, const float* b_th, const float* b_omega,
                       float v_th_min, int64_t rows, int64_t channels, void* beta, void* u,
                       void* v_th, void* omega, int dtype_in, int dtype_out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* NEURONSPARK_B200_H_ */
