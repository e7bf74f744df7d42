"""Modulation of the SNN block and its fusion into the PLIF scans.

NeuronSpark's ``SNNBlock.forward_parallel`` (atomic_ops/snn_block.py:216-256) turns five
raw projections into the scan's inputs with a torch.compile'd elementwise function and
then calls the scan:

    beta, u, v_th, omega = _fused_modulation_rf(raw_beta, b_beta, raw_alpha, b_alpha,
                                                raw_th, b_th, v_th_min, I_all, raw_omega, b_omega)
    s, v_last, w_last = rf_plif_parallel_forward_recompute(beta, omega, u, v_th, v_init, w_init,
                                                           surrogate_function=...)

``modulated_rf_plif_forward`` below computes the same two steps in one kernel: the raw
projections are streamed once, beta / u / v_th / omega live in registers only, and the
backward pushes the scan's adjoint through the modulation in the same pass. The
first-order pair of the v7.5 block (archive/atomic_ops_v75_pre/snn_block.py:41-47,
186-199) is ``modulated_plif_forward``.

``_fused_modulation`` / ``_fused_modulation_rf`` are forward-only drop-ins for the
reference's functions of the same names (they evaluate exactly what the fused scans
evaluate in registers); they refuse inputs that require grad, because this package has
no unfused modulation backward.
"""
from __future__ import annotations

import torch

from . import _lib
from ._lib import NSBError
from . import parallel_scan as ps


def _bias_f32(b: torch.Tensor, channels: int) -> torch.Tensor:
    if b.numel() != channels:
        raise NSBError(f"bias has {b.numel()} elements, expected {channels}")
    return b.detach().reshape(channels).to(torch.float32).contiguous()


def _launch_modulation(raw_beta, b_beta, raw_alpha, b_alpha, raw_th, b_th, v_th_min, I_all,
                       raw_omega=None, b_omega=None, out_dtype=None):
    rf = raw_omega is not None
    streams = [raw_beta, raw_alpha, raw_th, I_all] + ([raw_omega] if rf else [])
    if torch.is_grad_enabled() and any(t.requires_grad for t in streams + [b_beta, b_alpha, b_th]):
        raise NSBError("the stand-alone modulation is forward-only; use modulated_plif_forward / "
                       "modulated_rf_plif_forward for training")
    dt = ps._common_stream_dtype(*streams)
    streams = [ps._as_stream(t, dt) for t in streams]
    dev = _lib.require_cuda(*streams)
    ch = I_all.shape[-1]
    rows = I_all.numel() // ch
    biases = [_bias_f32(b, ch) for b in (b_beta, b_alpha, b_th)] + ([_bias_f32(b_omega, ch)] if rf else [None])
    out_dtype = torch.float32 if out_dtype is None else out_dtype
    if out_dtype not in (torch.float32, dt):
        raise NSBError("out_dtype must be float32 or the inputs' dtype")
    outs = [torch.empty(I_all.shape, dtype=out_dtype, device=dev) for _ in range(4 if rf else 3)]
    rb, ra, rt, ci = streams[:4]
    ro = streams[4] if rf else None
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().nsb_modulation_fwd(
            _lib.ptr(rb), _lib.ptr(ra), _lib.ptr(rt), _lib.ptr(ro), _lib.ptr(ci), _lib.ptr(biases[0]),
            _lib.ptr(biases[1]), _lib.ptr(biases[2]), _lib.ptr(biases[3]), float(v_th_min), rows, ch,
            _lib.ptr(outs[0]), _lib.ptr(outs[1]), _lib.ptr(outs[2]), _lib.ptr(outs[3] if rf else None),
            _lib.dtype_code(dt), _lib.dtype_code(out_dtype), _lib.stream_ptr(dev)), "nsb_modulation_fwd")
    return tuple(outs)


def _fused_modulation(raw_beta, b_beta, raw_alpha, b_alpha, raw_th, b_th, v_th_min, I_all, out_dtype=None):
    """``(beta, u, v_th)``; signature of archive/atomic_ops_v75_pre/snn_block.py:42. fp32 outputs
    unless ``out_dtype`` is the inputs' dtype."""
    return _launch_modulation(raw_beta, b_beta, raw_alpha, b_alpha, raw_th, b_th, v_th_min, I_all,
                              out_dtype=out_dtype)


def _fused_modulation_rf(raw_beta, b_beta, raw_alpha, b_alpha, raw_th, b_th, v_th_min, I_all, raw_omega,
                         b_omega, out_dtype=None):
    """``(beta, u, v_th, omega)``; signature of atomic_ops/snn_block.py:53."""
    return _launch_modulation(raw_beta, b_beta, raw_alpha, b_alpha, raw_th, b_th, v_th_min, I_all,
                              raw_omega, b_omega, out_dtype=out_dtype)


# widest no-grad forward that runs on 8-step tiles so that the library can rotate it among warps
ROTATE_MAX_COLS_RF = 24576
ROTATE_MAX_COLS = 12288


class ModulatedPLIFScan(torch.autograd.Function):
    """Modulation + scan. Inputs: raw_beta, raw_alpha, raw_th, I, raw_omega (or None), b_beta,
    b_alpha, b_th, b_omega (or None), v_init, w_init (or None), v_th_min, alpha, surrogate.
    Returns ``(spike, V_last, W_last)`` (``W_last`` is None for the first-order form).
    Gradients for the five raw tensors, the four biases and the initial states; gradients
    arriving for ``V_last`` / ``W_last`` are ignored, as in the reference's recompute
    Functions (atomic_ops/parallel_scan.py:659, 1204)."""

    @staticmethod
    def forward(ctx, raw_beta, raw_alpha, raw_th, I_all, raw_omega, b_beta, b_alpha, b_th, b_omega,
                v_init, w_init, v_th_min, alpha, surrogate, sigma0=None):
        rf = raw_omega is not None
        streams = [raw_beta, raw_alpha, raw_th, I_all] + ([raw_omega] if rf else [])
        dt = ps._common_stream_dtype(*streams)
        rb, ra, rt, ci = (ps._as_stream(t, dt) for t in streams[:4])
        ro = ps._as_stream(raw_omega, dt) if rf else None
        dev = _lib.require_cuda(rb, ra, rt, ci)
        shape = I_all.shape[1:]
        ch = I_all.shape[-1]
        T, cols = I_all.shape[0], ps._cols(I_all)
        biases = [_bias_f32(b, ch) for b in (b_beta, b_alpha, b_th)] + ([_bias_f32(b_omega, ch)] if rf else [None])
        v0 = ps._row_f32(v_init, shape)
        w0 = ps._row_f32(w_init, shape) if rf else None
        needs_grad = any(ctx.needs_input_grad[:11])
        C = 32 if ps._interval(cols) == 32 else 8
        # Inference over few columns: with 8-step tiles several warps take a column group's tiles in turn
        # (nsb_set_scan_rotation). T=8192, 6144 channels, bf16, forward ms with 32-step tiles -> rotating:
        # resonate-and-fire 0.89 -> 0.50 (one sequence), 0.89 -> 0.57 (two), 1.00 -> 0.88 (four).
        # Wider ones, up to the 49 152 columns of a batch of 8: 32-step tiles (1.22 against 1.46 ms; the 8-step
        # tiles chosen above are for the backward's sake).
        if not needs_grad and ps.CKPT_INTERVAL is None:
            rotating = _lib.scan_rotation_setting() != 1 and cols <= (ROTATE_MAX_COLS_RF if rf else ROTATE_MAX_COLS)
            C = 8 if rotating else (32 if cols <= 49152 else C)
        ctx.interval = C
        spike = torch.empty_like(ci)
        ckv = ckw = None
        if needs_grad:
            ckv = torch.empty((ps._n_tiles(T, C), cols), dtype=torch.float32, device=dev)
            ckw = torch.empty_like(ckv) if rf else None
        v_last = torch.empty(shape, dtype=torch.float32, device=dev)
        w_last = torch.empty_like(v_last) if rf else None
        # adaptive slope: `alpha` is alpha_0; the kernel accumulates the moments of u and the slope
        # lands in a device float that the backward reads (no host round trip)
        stats = alpha_t = None
        if sigma0 is not None and needs_grad:
            stats = torch.empty(int(_lib.lib().nsb_plif_modulated_fwd_stats_doubles(cols)), dtype=torch.float64,
                                device=dev)
            alpha_t = torch.empty((), dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            _lib.check(_lib.lib().nsb_plif_modulated_fwd(
                _lib.ptr(rb), _lib.ptr(ra), _lib.ptr(rt), _lib.ptr(ro), _lib.ptr(ci), _lib.ptr(biases[0]),
                _lib.ptr(biases[1]), _lib.ptr(biases[2]), _lib.ptr(biases[3]), float(v_th_min), ch,
                _lib.ptr(v0), _lib.ptr(w0), _lib.ptr(spike), None, _lib.ptr(ckv), _lib.ptr(ckw),
                _lib.ptr(v_last), _lib.ptr(w_last), float(alpha), float(sigma0 or 0.0), _lib.ptr(stats),
                _lib.ptr(alpha_t), T, cols, _lib.dtype_code(dt), C,
                _lib.ptr(None if stats is not None else ps._split_scratch(T, cols, dev)), _lib.stream_ptr(dev)),
                "nsb_plif_modulated_fwd")
        ctx.alpha_t = alpha_t
        if needs_grad:
            ctx.save_for_backward(rb, ra, rt, ci, ro, *biases[:3], biases[3], ckv, ckw)
        ctx.rf = rf
        ctx.v_th_min = float(v_th_min)
        ctx.alpha = float(alpha)
        ctx.surrogate = ps._surrogate_kind(surrogate)
        ctx.in_dtypes = tuple(None if t is None else t.dtype for t in
                              (raw_beta, raw_alpha, raw_th, I_all, raw_omega, b_beta, b_alpha, b_th, b_omega,
                               v_init, w_init))
        ctx.bias_shapes = tuple(None if b is None else b.shape for b in (b_beta, b_alpha, b_th, b_omega))
        ctx.state_shapes = (v_init.shape, None if w_init is None else w_init.shape)
        spike = ps._cast(spike, I_all.dtype)
        v_last = v_last.to(v_init.dtype)
        if rf:
            w_last = w_last.to(w_init.dtype)
            ctx.mark_non_differentiable(v_last, w_last)
            return spike, v_last, w_last
        ctx.mark_non_differentiable(v_last)
        return spike, v_last, None

    @staticmethod
    def backward(ctx, grad_spike, _gv, _gw):
        rb, ra, rt, ci, ro, bb, ba, bt, bo, ckv, ckw = ctx.saved_tensors
        rf = ctx.rf
        dt, dev = ci.dtype, ci.device
        T, cols = ci.shape[0], ps._cols(ci)
        ch = ci.shape[-1]
        if grad_spike is None:
            grad_spike = torch.zeros_like(ci)
        gs = ps._grad_stream(grad_spike, ci, dt)
        g_rb, g_ra, g_rt, g_ci = (torch.empty_like(ci) for _ in range(4))
        g_ro = torch.empty_like(ci) if rf else None
        g_bias = [torch.empty(ch, dtype=torch.float32, device=dev) for _ in range(4 if rf else 3)]
        scratch = torch.empty(int(_lib.lib().nsb_plif_modulated_bwd_scratch_floats(cols)),
                              dtype=torch.float32, device=dev)
        g_v0 = torch.empty(ci.shape[1:], dtype=torch.float32, device=dev)
        g_w0 = torch.empty_like(g_v0) if rf else None
        with torch.cuda.device(dev):
            _lib.check(_lib.lib().nsb_plif_modulated_bwd(
                _lib.ptr(rb), _lib.ptr(ra), _lib.ptr(rt), _lib.ptr(ro), _lib.ptr(ci), _lib.ptr(bb),
                _lib.ptr(ba), _lib.ptr(bt), _lib.ptr(bo), ctx.v_th_min, ch, _lib.ptr(ckv), _lib.ptr(ckw),
                _lib.ptr(gs), _lib.ptr(g_rb), _lib.ptr(g_ra), _lib.ptr(g_rt), _lib.ptr(g_ro), _lib.ptr(g_ci),
                _lib.ptr(g_bias[0]), _lib.ptr(g_bias[1]), _lib.ptr(g_bias[2]),
                _lib.ptr(g_bias[3] if rf else None), _lib.ptr(scratch), _lib.ptr(g_v0), _lib.ptr(g_w0),
                T, cols, _lib.dtype_code(dt), ctx.interval, ctx.surrogate, ctx.alpha, _lib.ptr(ctx.alpha_t),
                _lib.stream_ptr(dev)), "nsb_plif_modulated_bwd")
        d = ctx.in_dtypes
        sh = ctx.bias_shapes

        def bias_out(i):
            return g_bias[i].to(d[5 + i]).reshape(sh[i])

        return (ps._cast(g_rb, d[0]), ps._cast(g_ra, d[1]), ps._cast(g_rt, d[2]), ps._cast(g_ci, d[3]),
                ps._cast(g_ro, d[4]) if rf else None, bias_out(0), bias_out(1), bias_out(2),
                bias_out(3) if rf else None, g_v0.to(d[9]).reshape(ctx.state_shapes[0]),
                g_w0.to(d[10]).reshape(ctx.state_shapes[1]) if rf else None, None, None, None, None)


def _apply(raw_beta, raw_alpha, raw_th, I_all, raw_omega, b_beta, b_alpha, b_th, b_omega, v_init, w_init,
           v_th_min, surrogate_function, adaptive_sigma0=None):
    if surrogate_function is None:
        with torch.no_grad():
            return ModulatedPLIFScan.apply(raw_beta, raw_alpha, raw_th, I_all, raw_omega, b_beta, b_alpha,
                                           b_th, b_omega, v_init, w_init, v_th_min, 0.0, "sigmoid")
    alpha, kind = ps._alpha_and_kind(surrogate_function)
    return ModulatedPLIFScan.apply(raw_beta, raw_alpha, raw_th, I_all, raw_omega, b_beta, b_alpha, b_th,
                                   b_omega, v_init, w_init, v_th_min, float(alpha), kind, adaptive_sigma0)


def modulated_plif_forward(raw_beta, b_beta, raw_alpha, b_alpha, raw_th, b_th, v_th_min, I_all, v_init,
                           surrogate_function=None, adaptive_sigma0=None):
    """First-order modulation + selective scan: ``_fused_modulation(...)`` followed by
    ``plif_parallel_forward(beta, u, v_th, v_init, surrogate_function=...)``
    (archive/atomic_ops_v75_pre/snn_block.py:186-199). Argument order of the modulation
    function, then the scan's state. Returns ``(spike, V_last)``. ``adaptive_sigma0``: see
    ``modulated_rf_plif_forward``."""
    s, v_last, _ = _apply(raw_beta, raw_alpha, raw_th, I_all, None, b_beta, b_alpha, b_th, None, v_init, None,
                          v_th_min, surrogate_function, adaptive_sigma0)
    return s, v_last


def modulated_rf_plif_forward(raw_beta, b_beta, raw_alpha, b_alpha, raw_th, b_th, v_th_min, I_all, raw_omega,
                              b_omega, v_init, w_init, surrogate_function=None, adaptive_sigma0=None):
    """Second-order modulation + resonate-and-fire scan: ``_fused_modulation_rf(...)`` followed by
    ``rf_plif_parallel_forward_recompute(...)`` (atomic_ops/snn_block.py:237-256). Returns
    ``(spike, V_last, W_last)``.

    ``adaptive_sigma0``: the reference adapts the surrogate slope to ``u_hidden.std()``
    (``hidden_neuron.get_surrogate(u_hidden)``, atomic_ops/plif_node.py:78-101), a tensor the fused
    kernel never writes. Pass the neuron's FIXED surrogate (slope alpha_0) as ``surrogate_function`` and
    its ``sigma_0`` here: the kernel accumulates the moments of u while it streams, and the backward
    uses ``clamp(alpha_0 * sigma_0 / max(std(u), 1e-6), 1, 20)`` read from device memory."""
    return _apply(raw_beta, raw_alpha, raw_th, I_all, raw_omega, b_beta, b_alpha, b_th, b_omega, v_init,
                  w_init, v_th_min, surrogate_function, adaptive_sigma0)
