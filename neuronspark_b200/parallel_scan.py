"""PLIF scan operators with the call signatures of NeuronSpark's
``atomic_ops/parallel_scan.py``, backed by the sm_100a CUDA kernels.

Drop-in surface (same names, argument order, return arity and gradient
semantics as the reference):

    _TritonPLIFForward.apply(beta, u, v_th, v_init, alpha) -> (spike, V_post)
        reference: atomic_ops/parallel_scan.py:690-768
    _TritonPLIFRowParamForward.apply(beta_row, u, v_th_row, v_init, alpha) -> (spike, V_post)
        reference: :415-486
    _TritonPLIFRowParamRecompute.apply(beta_row, u, v_th_row, v_init, alpha) -> (spike, V_last)
        reference: :614-688
    plif_parallel_forward, plif_rowparam_forward, plif_rowparam_forward_alpha,
    plif_rowparam_forward_recompute, plif_fixed_param_forward
        reference: :1309-1412, :1415-1453, :1456-1495, :1499-1535, :1538-1603
    _TritonRFPLIFForward / _TritonRFPLIFRecompute .apply(beta, omega, u, v_th, v_init, w_init, alpha)
    rf_plif_parallel_forward, rf_plif_parallel_forward_recompute
        reference: :1071-1233, :1610-1726 (second-order resonate-and-fire scan)

Differences, all deliberate:
  * CUDA only. A CPU tensor raises; nothing falls back to PyTorch ops.
  * The backward recomputes the membrane trajectory from one fp32 checkpoint
    per time tile instead of reading a stored V_post, so no [T, ...] state
    tensor is kept between forward and backward.
  * The recompute variant returns a freshly allocated grad_u; the reference
    hands back the saved ``u`` buffer overwritten in place (:687-688).
  * Arithmetic is fp32 with separately rounded multiply and add, which is what
    the reference's eager PyTorch time loop computes, so spikes are bit-exact
    against that loop.
Extras that the reference does not have: the alpha*I form with separate
gradients for the write gain and the current (`plif_selective_scan_ai`), an
arctangent surrogate, and the bit-packed inference scans.
"""
from __future__ import annotations

import torch

from . import _lib, fp16_codec
from ._lib import NSBError

#: Steps per time tile = spacing of the fp32 state checkpoints kept for backward
#: (8, 16 or 32). None = chosen per call from the number of columns: problems with few
#: columns are bound by per-tile latency and run faster with long tiles, problems with
#: many columns are bound by HBM bandwidth and want the widest (8-step) kernels.
CKPT_INTERVAL = None


def _interval(cols: int, row_param: bool = False) -> int:
    """Tile length for a problem with ``cols`` columns. Thresholds from forward+backward
    timings on B200 (bf16, T=8192): 32-step tiles win up to ~32 K columns for the selective
    scans and ~64 K for the row-parameter scan (one streamed input), 16-step tiles in a band above
    (the resonate-and-fire scan at 49 152 columns: 2.16 ms forward + backward against 2.51 with
    8-step tiles), 8-step tiles beyond."""
    if CKPT_INTERVAL is not None:
        return int(CKPT_INTERVAL)
    if row_param:
        return 32 if cols <= 65536 else (16 if cols <= 131072 else 8)
    return 32 if cols <= 32768 else (16 if cols < 98304 else 8)  # 98 304 columns: 3.66 ms with 8, 3.77 with 16

_SURROGATES = {"sigmoid": _lib.SURR_SIGMOID, "atan": _lib.SURR_ATAN}


# ----------------------------------------------------------------- helpers


def _cols(t: torch.Tensor) -> int:
    n = 1
    for s in t.shape[1:]:
        n *= s
    return n


def _common_stream_dtype(*tensors: torch.Tensor) -> torch.dtype:
    """The single element type the kernel will stream. Tensors of one low-precision
    type are streamed as they are; mixed inputs are widened to fp32, which is exact
    (the reference widens every load to fp32 individually, :223-225)."""
    dts = {t.dtype for t in tensors if t is not None}
    if len(dts) == 1:
        (dt,) = dts
        if dt in (torch.float32, torch.bfloat16, torch.float16):
            return dt
    return torch.float32


def _as_stream(t, dt):
    """Contiguous tensor of the call's stream dtype; a differing dtype is converted by the library's
    own kernel (``nsb_convert``), not by a framework op."""
    if t is None:
        return None
    if t.dtype != dt:
        return _lib.convert(t, dt)
    return t.contiguous()


def _cast(t, dt):
    """Output or gradient in the dtype the reference would hand back (``empty_like`` of the input)."""
    if t is None or t.dtype == dt:
        return t
    return _lib.convert(t, dt)


def _row_f32(t: torch.Tensor, shape) -> torch.Tensor:
    """Per-column vector as contiguous fp32 of the given trailing shape."""
    if tuple(t.shape) != tuple(shape):
        t = t.expand(shape)
    return t.detach().to(torch.float32).contiguous()


def _surrogate_kind(surrogate) -> int:
    if isinstance(surrogate, int):
        return surrogate
    try:
        return _SURROGATES[surrogate]
    except KeyError:
        raise NSBError(f"unknown surrogate {surrogate!r}; expected 'sigmoid' or 'atan'") from None


def adaptive_alpha(u: torch.Tensor, alpha0: float = 4.0, sigma0: float = 0.4) -> torch.Tensor:
    """Adaptive surrogate slope ``clamp(alpha0 * sigma0 / max(u.std(), 1e-6), 1, 20)`` of
    ``PLIFNode.get_surrogate`` (atomic_ops/plif_node.py:78-101) as a 0-dim float32 CUDA tensor,
    computed without the ``.item()`` the reference pays per scan call. Pass the tensor as
    ``alpha`` to the row-parameter scans, or as the ``.alpha`` of the surrogate object given to
    the resonate-and-fire scans: their backward then reads the slope on the device."""
    dev = _lib.require_cuda(u)
    dt = u.dtype if u.dtype in (torch.float32, torch.bfloat16, torch.float16) else torch.float32
    u_c = _as_stream(u.detach(), dt)
    L = _lib.lib()
    scratch = torch.empty(int(L.nsb_surrogate_alpha_scratch_doubles()), dtype=torch.float64, device=dev)
    out = torch.empty((), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _lib.check(L.nsb_surrogate_alpha(_lib.ptr(u_c), u_c.numel(), _lib.dtype_code(dt), float(alpha0),
                                         float(sigma0), _lib.ptr(scratch), _lib.ptr(out),
                                         _lib.stream_ptr(dev)), "nsb_surrogate_alpha")
    return out


def _split_alpha(alpha):
    """(float, None) for a host number, (0.0, tensor) for a device-resident slope."""
    if isinstance(alpha, torch.Tensor):
        if alpha.numel() != 1:
            raise NSBError("a tensor alpha must have one element")
        if not alpha.is_cuda:
            return float(alpha), None
        return 0.0, alpha.detach().reshape(()).to(torch.float32)
    return float(alpha), None


def _n_tiles(T: int, interval: int) -> int:
    return (T + interval - 1) // interval


def _launch_selective_fwd(beta, drive, gain, v_th, v_init32, *, want_spike, want_packed, want_vpost,
                          want_ckpt):
    """Runs nsb_plif_selective_fwd. Streams must already share dtype and be contiguous."""
    dev = _lib.require_cuda(beta, drive, gain, v_th, v_init32)
    T, cols = drive.shape[0], _cols(drive)
    dt = drive.dtype
    spike = torch.empty_like(drive) if want_spike else None
    packed = (torch.empty((T, (cols + 31) // 32), dtype=torch.int32, device=dev)
              if want_packed else None)
    vpost = torch.empty_like(drive) if want_vpost else None
    C = _interval(cols)
    ckpt = (torch.empty((_n_tiles(T, C), cols), dtype=torch.float32, device=dev) if want_ckpt else None)
    v_last = torch.empty(drive.shape[1:], dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().nsb_plif_selective_fwd(
            _lib.ptr(beta), _lib.ptr(drive), _lib.ptr(gain), _lib.ptr(v_th), _lib.ptr(v_init32),
            _lib.ptr(spike), _lib.ptr(packed), _lib.ptr(vpost), _lib.ptr(ckpt), _lib.ptr(v_last),
            T, cols, _lib.dtype_code(dt), C, _lib.ptr(None if gain is not None else _split_scratch(T, cols, dev)),
            _lib.stream_ptr(dev)), "nsb_plif_selective_fwd")
    return spike, packed, vpost, ckpt, v_last, C


def _launch_rowparam_fwd(beta_row32, u, vth_row32, v_init32, *, want_spike, want_packed, want_vpost,
                         want_ckpt):
    dev = _lib.require_cuda(beta_row32, u, vth_row32, v_init32)
    T, cols = u.shape[0], _cols(u)
    spike = torch.empty_like(u) if want_spike else None
    packed = (torch.empty((T, (cols + 31) // 32), dtype=torch.int32, device=dev)
              if want_packed else None)
    vpost = torch.empty_like(u) if want_vpost else None
    C = _interval(cols, row_param=True)
    ckpt = (torch.empty((_n_tiles(T, C), cols), dtype=torch.float32, device=dev) if want_ckpt else None)
    v_last = torch.empty(u.shape[1:], dtype=torch.float32, device=dev)
    scratch = None if want_vpost else _split_scratch(T, cols, dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().nsb_plif_rowparam_fwd(
            _lib.ptr(beta_row32), _lib.ptr(u), _lib.ptr(vth_row32), _lib.ptr(v_init32),
            _lib.ptr(spike), _lib.ptr(packed), _lib.ptr(vpost), _lib.ptr(ckpt), _lib.ptr(v_last),
            T, cols, _lib.dtype_code(u.dtype), C, _lib.ptr(scratch), _lib.stream_ptr(dev)),
            "nsb_plif_rowparam_fwd")
    return spike, packed, vpost, ckpt, v_last, C


#: Scans over at most this many columns and at least this many steps are given scratch memory,
#: which lets the library cut them along time (see nsb_set_time_split); 592 warp schedulers x 4
#: warps / 2 segments x 32 columns, and a scan several warm-ups long.
TIME_SPLIT_MAX_COLS = 37888
TIME_SPLIT_MIN_STEPS = 4096


def _split_scratch(T: int, cols: int, dev):
    if cols > TIME_SPLIT_MAX_COLS or T < TIME_SPLIT_MIN_STEPS:
        return None
    return torch.empty(int(_lib.lib().nsb_time_split_scratch_floats(cols)), dtype=torch.float32, device=dev)


#: Backward scans over at least this many columns and steps get the few KB of scratch that let the
#: library chain chunks of the time axis (see nsb_set_chain_chunks); narrower or shorter scans gain
#: nothing from it.
CHAIN_MIN_COLS = 49152
CHAIN_MIN_STEPS = 512


def _chain_scratch(T: int, cols: int, dev):
    if cols < CHAIN_MIN_COLS or T < CHAIN_MIN_STEPS:
        return None
    return torch.empty(int(_lib.lib().nsb_chain_scratch_words(cols)), dtype=torch.int32, device=dev)


def _grad_stream(g, like, dt):
    """An incoming gradient as a contiguous stream tensor (None stays None)."""
    return _as_stream(g, dt)


# ------------------------------------------------------- selective scan (u-form)


class PLIFSelectiveScan(torch.autograd.Function):
    """Selective PLIF scan with per-step beta / u / v_th.

    Same contract as the reference's ``_TritonPLIFForward``
    (atomic_ops/parallel_scan.py:690-768): returns ``(spike, V_post)`` in ``u``'s
    dtype; backward returns ``(grad_beta, grad_u, grad_v_th, grad_v_init, None)``
    with the hard spike treated as a constant in the reset path.
    """

    surrogate = _lib.SURR_SIGMOID

    @staticmethod
    def forward(ctx, beta, u, v_th, v_init, alpha):
        out_dtype = u.dtype
        dt = _common_stream_dtype(beta, u, v_th)
        beta_c, u_c, vth_c = (_as_stream(t, dt) for t in (beta, u, v_th))
        v0 = _row_f32(v_init, u.shape[1:])
        needs_grad = any(ctx.needs_input_grad[:4])
        spike, _, vpost, ckpt, _, ctx.interval = _launch_selective_fwd(
            beta_c, u_c, None, vth_c, v0, want_spike=True, want_packed=False, want_vpost=True,
            want_ckpt=needs_grad)
        if needs_grad:
            ctx.save_for_backward(beta_c, u_c, vth_c, ckpt)
        ctx.alpha = float(alpha)
        ctx.in_dtypes = (beta.dtype, u.dtype, v_th.dtype, v_init.dtype)
        ctx.v_init_shape = v_init.shape
        return _cast(spike, out_dtype), _cast(vpost, out_dtype)

    @staticmethod
    def backward(ctx, grad_spike, grad_V_post):
        beta_c, u_c, vth_c, ckpt = ctx.saved_tensors
        dt = u_c.dtype
        dev = u_c.device
        T, cols = u_c.shape[0], _cols(u_c)
        if grad_spike is None:
            grad_spike = torch.zeros_like(u_c)
        gs = _grad_stream(grad_spike, u_c, dt)
        gv = _grad_stream(grad_V_post, u_c, dt)
        g_beta, g_u, g_vth = (torch.empty_like(u_c) for _ in range(3))
        g_v0 = torch.empty(u_c.shape[1:], dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            _lib.check(_lib.lib().nsb_plif_selective_bwd(
                _lib.ptr(beta_c), _lib.ptr(u_c), None, _lib.ptr(vth_c), _lib.ptr(ckpt), _lib.ptr(gs),
                _lib.ptr(gv), _lib.ptr(g_beta), _lib.ptr(g_u), None, _lib.ptr(g_vth), _lib.ptr(g_v0),
                T, cols, _lib.dtype_code(dt), ctx.interval, ctx_surrogate(ctx), ctx.alpha,
                _lib.ptr(_chain_scratch(T, cols, dev)), _lib.stream_ptr(dev)), "nsb_plif_selective_bwd")
        db, du, dth, dv = ctx.in_dtypes
        return (_cast(g_beta, db), _cast(g_u, du), _cast(g_vth, dth),
                g_v0.to(dv).reshape(ctx.v_init_shape), None)


def ctx_surrogate(ctx) -> int:
    return getattr(ctx, "surrogate", _lib.SURR_SIGMOID)


class PLIFSelectiveScanAI(torch.autograd.Function):
    """Selective scan with the write gain and the current as separate inputs:
    ``v_pre = beta*v + gain*cur`` (SelectivePLIFNode.single_step_forward,
    atomic_ops/selective_plif.py:127). Returns ``(spike, V_last)``; gradients for
    beta, cur, gain, v_th and v_init. ``surrogate`` is 'sigmoid' or 'atan'."""

    @staticmethod
    def forward(ctx, beta, cur, gain, v_th, v_init, alpha, surrogate):
        out_dtype = cur.dtype
        dt = _common_stream_dtype(beta, cur, gain, v_th)
        beta_c, cur_c, gain_c, vth_c = (_as_stream(t, dt) for t in (beta, cur, gain, v_th))
        v0 = _row_f32(v_init, cur.shape[1:])
        needs_grad = any(ctx.needs_input_grad[:5])
        spike, _, _, ckpt, v_last, ctx.interval = _launch_selective_fwd(
            beta_c, cur_c, gain_c, vth_c, v0, want_spike=True, want_packed=False, want_vpost=False,
            want_ckpt=needs_grad)
        if needs_grad:
            ctx.save_for_backward(beta_c, cur_c, gain_c, vth_c, ckpt)
        ctx.alpha = float(alpha)
        ctx.surrogate = _surrogate_kind(surrogate)
        ctx.in_dtypes = (beta.dtype, cur.dtype, gain.dtype, v_th.dtype, v_init.dtype)
        ctx.v_init_shape = v_init.shape
        ctx.mark_non_differentiable(v_last)
        return _cast(spike, out_dtype), v_last.to(v_init.dtype)

    @staticmethod
    def backward(ctx, grad_spike, _grad_v_last):
        beta_c, cur_c, gain_c, vth_c, ckpt = ctx.saved_tensors
        dt = cur_c.dtype
        dev = cur_c.device
        T, cols = cur_c.shape[0], _cols(cur_c)
        if grad_spike is None:
            grad_spike = torch.zeros_like(cur_c)
        gs = _grad_stream(grad_spike, cur_c, dt)
        g_beta, g_cur, g_gain, g_vth = (torch.empty_like(cur_c) for _ in range(4))
        g_v0 = torch.empty(cur_c.shape[1:], dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            _lib.check(_lib.lib().nsb_plif_selective_bwd(
                _lib.ptr(beta_c), _lib.ptr(cur_c), _lib.ptr(gain_c), _lib.ptr(vth_c), _lib.ptr(ckpt),
                _lib.ptr(gs), None, _lib.ptr(g_beta), _lib.ptr(g_cur), _lib.ptr(g_gain),
                _lib.ptr(g_vth), _lib.ptr(g_v0), T, cols, _lib.dtype_code(dt), ctx.interval,
                ctx.surrogate, ctx.alpha, _lib.ptr(_chain_scratch(T, cols, dev)), _lib.stream_ptr(dev)),
                "nsb_plif_selective_bwd")
        db, dc, dg, dth, dv = ctx.in_dtypes
        return (_cast(g_beta, db), _cast(g_cur, dc), _cast(g_gain, dg), _cast(g_vth, dth),
                g_v0.to(dv).reshape(ctx.v_init_shape), None, None)


# ------------------------------------------------------------- linear recurrence


class PLIFLinearRecurrence(torch.autograd.Function):
    """``V[k] = beta[k]*V[k-1] + u[k]``; contract of the reference's ``_TritonLinearRecurrence``
    (atomic_ops/parallel_scan.py:143-190): returns V ``[K, ...]`` in ``u``'s dtype, gradients for
    beta, u and v_init. The backward recomputes V from fp32 checkpoints instead of re-reading it."""

    @staticmethod
    def forward(ctx, beta, u, v_init):
        dt = _common_stream_dtype(beta, u)
        beta_c, u_c = _as_stream(beta, dt), _as_stream(u, dt)
        shape = u.shape[1:]
        v0 = _row_f32(v_init, shape)
        dev = _lib.require_cuda(beta_c, u_c, v0)
        T, cols = u_c.shape[0], _cols(u_c)
        needs_grad = any(ctx.needs_input_grad[:3])
        C = ctx.interval = 32 if _interval(cols) == 32 else 8
        V = torch.empty_like(u_c)
        ckpt = torch.empty((_n_tiles(T, C), cols), dtype=torch.float32, device=dev) if needs_grad else None
        v_last = torch.empty(shape, dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            _lib.check(_lib.lib().nsb_linear_recurrence_fwd(
                _lib.ptr(beta_c), _lib.ptr(u_c), _lib.ptr(v0), _lib.ptr(V), _lib.ptr(ckpt), _lib.ptr(v_last),
                T, cols, _lib.dtype_code(dt), C, _lib.stream_ptr(dev)), "nsb_linear_recurrence_fwd")
        if needs_grad:
            ctx.save_for_backward(beta_c, u_c, ckpt)
        ctx.in_dtypes = (beta.dtype, u.dtype, v_init.dtype)
        ctx.v_init_shape = v_init.shape
        return _cast(V, u.dtype)

    @staticmethod
    def backward(ctx, grad_V):
        beta_c, u_c, ckpt = ctx.saved_tensors
        dt, dev = u_c.dtype, u_c.device
        T, cols = u_c.shape[0], _cols(u_c)
        if grad_V is None:
            grad_V = torch.zeros_like(u_c)
        gv = _grad_stream(grad_V, u_c, dt)
        g_beta, g_u = torch.empty_like(u_c), torch.empty_like(u_c)
        g_v0 = torch.empty(u_c.shape[1:], dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            _lib.check(_lib.lib().nsb_linear_recurrence_bwd(
                _lib.ptr(beta_c), _lib.ptr(u_c), _lib.ptr(ckpt), _lib.ptr(gv), _lib.ptr(g_beta), _lib.ptr(g_u),
                _lib.ptr(g_v0), T, cols, _lib.dtype_code(dt), ctx.interval,
                _lib.ptr(_chain_scratch(T, cols, dev)), _lib.stream_ptr(dev)), "nsb_linear_recurrence_bwd")
        db, du, dv = ctx.in_dtypes
        return _cast(g_beta, db), _cast(g_u, du), g_v0.to(dv).reshape(ctx.v_init_shape)


_TritonLinearRecurrence = PLIFLinearRecurrence  # the reference's name for the same contract


def linear_recurrence(beta: torch.Tensor, u: torch.Tensor, v_init: torch.Tensor) -> torch.Tensor:
    """Reference: atomic_ops/parallel_scan.py:1282-1302. Returns V ``(K, *shape)``."""
    return PLIFLinearRecurrence.apply(beta, u, v_init)


# ------------------------------------------------------------- row-param scans


def _rowparam_backward(ctx, grad_spike, grad_V_post):
    beta32, vth32, u_c, ckpt = ctx.saved_tensors
    dt = u_c.dtype
    dev = u_c.device
    T, cols = u_c.shape[0], _cols(u_c)
    if grad_spike is None:
        grad_spike = torch.zeros_like(u_c)
    gs = _grad_stream(grad_spike, u_c, dt)
    gv = _grad_stream(grad_V_post, u_c, dt)
    g_u = torch.empty_like(u_c)
    g_beta, g_vth, g_v0 = (torch.empty(u_c.shape[1:], dtype=torch.float32, device=dev)
                           for _ in range(3))
    alpha_t = getattr(ctx, "alpha_t", None)
    # few columns: the time split (not built for a V_post gradient); many: the chained chunks
    scratch = None
    if cols >= CHAIN_MIN_COLS and T >= CHAIN_MIN_STEPS:
        scratch = torch.empty(int(_lib.lib().nsb_time_split_scratch_floats(cols)), dtype=torch.float32, device=dev)
    elif gv is None:
        scratch = _split_scratch(T, cols, dev)
    with torch.cuda.device(dev):
        if alpha_t is not None:
            _lib.check(_lib.lib().nsb_plif_rowparam_bwd_dalpha(
                _lib.ptr(beta32), _lib.ptr(u_c), _lib.ptr(vth32), _lib.ptr(ckpt), _lib.ptr(gs),
                _lib.ptr(gv), _lib.ptr(g_beta), _lib.ptr(g_u), _lib.ptr(g_vth), _lib.ptr(g_v0), T, cols,
                _lib.dtype_code(dt), ctx.interval, ctx_surrogate(ctx), _lib.ptr(alpha_t), _lib.ptr(scratch),
                _lib.stream_ptr(dev)), "nsb_plif_rowparam_bwd_dalpha")
        else:
            _lib.check(_lib.lib().nsb_plif_rowparam_bwd(
                _lib.ptr(beta32), _lib.ptr(u_c), _lib.ptr(vth32), _lib.ptr(ckpt), _lib.ptr(gs),
                _lib.ptr(gv), _lib.ptr(g_beta), _lib.ptr(g_u), _lib.ptr(g_vth), _lib.ptr(g_v0), T, cols,
                _lib.dtype_code(dt), ctx.interval, ctx_surrogate(ctx), ctx.alpha, _lib.ptr(scratch),
                _lib.stream_ptr(dev)), "nsb_plif_rowparam_bwd")
    db, du, dth, dv = ctx.in_dtypes
    return (g_beta.to(db).reshape(ctx.row_shapes[0]), _cast(g_u, du),
            g_vth.to(dth).reshape(ctx.row_shapes[1]), g_v0.to(dv).reshape(ctx.row_shapes[2]), None)


def _rowparam_forward(ctx, beta_row, u, v_th_row, v_init, alpha, want_vpost):
    shape = u.shape[1:]
    for name, t in (("beta_row", beta_row), ("v_th_row", v_th_row), ("v_init", v_init)):
        if tuple(t.shape) != tuple(shape):
            raise NSBError(f"{name} has shape {tuple(t.shape)}, expected {tuple(shape)}")
    dt = _common_stream_dtype(u)
    u_c = _as_stream(u, dt)
    beta32, vth32, v0 = (_row_f32(t, shape) for t in (beta_row, v_th_row, v_init))
    needs_grad = any(ctx.needs_input_grad[:4])
    spike, _, vpost, ckpt, v_last, ctx.interval = _launch_rowparam_fwd(
        beta32, u_c, vth32, v0, want_spike=True, want_packed=False, want_vpost=want_vpost,
        want_ckpt=needs_grad)
    if needs_grad:
        ctx.save_for_backward(beta32, vth32, u_c, ckpt)
    ctx.alpha, ctx.alpha_t = _split_alpha(alpha)
    ctx.in_dtypes = (beta_row.dtype, u.dtype, v_th_row.dtype, v_init.dtype)
    ctx.row_shapes = (beta_row.shape, v_th_row.shape, v_init.shape)
    return _cast(spike, u.dtype), _cast(vpost, u.dtype), v_last


class PLIFRowParamScan(torch.autograd.Function):
    """Row-parameter PLIF scan returning ``(spike, V_post)``; contract of the
    reference's ``_TritonPLIFRowParamForward`` (atomic_ops/parallel_scan.py:415-486)."""

    @staticmethod
    def forward(ctx, beta_row, u, v_th_row, v_init, alpha):
        spike, vpost, _ = _rowparam_forward(ctx, beta_row, u, v_th_row, v_init, alpha, True)
        return spike, vpost

    @staticmethod
    def backward(ctx, grad_spike, grad_V_post):
        return _rowparam_backward(ctx, grad_spike, grad_V_post)


class PLIFRowParamRecomputeScan(torch.autograd.Function):
    """Row-parameter PLIF scan returning ``(spike, V_last)``; contract of the
    reference's ``_TritonPLIFRowParamRecompute`` (:614-688): the gradient that
    arrives for ``V_last`` is ignored (:659)."""

    @staticmethod
    def forward(ctx, beta_row, u, v_th_row, v_init, alpha):
        spike, _, v_last = _rowparam_forward(ctx, beta_row, u, v_th_row, v_init, alpha, False)
        return spike, v_last.to(v_init.dtype)

    @staticmethod
    def backward(ctx, grad_spike, _grad_V_last_unused):
        return _rowparam_backward(ctx, grad_spike, None)


# ------------------------------------------------- resonate-and-fire (second-order) scan


def _rf_forward(ctx, beta, omega, u, v_th, v_init, w_init, alpha, want_states):
    out_dtype = u.dtype
    dt = _common_stream_dtype(beta, omega, u, v_th)
    beta_c, omega_c, u_c, vth_c = (_as_stream(t, dt) for t in (beta, omega, u, v_th))
    shape = u.shape[1:]
    v0, w0 = _row_f32(v_init, shape), _row_f32(w_init, shape)
    dev = _lib.require_cuda(beta_c, omega_c, u_c, vth_c, v0, w0)
    T, cols = u_c.shape[0], _cols(u_c)
    needs_grad = any(ctx.needs_input_grad[:6])
    spike = torch.empty_like(u_c)
    vpost = torch.empty_like(u_c) if want_states else None
    wout = torch.empty_like(u_c) if want_states else None
    ckv = ckw = None
    C = ctx.interval = _interval(cols)
    if needs_grad:
        ckv = torch.empty((_n_tiles(T, C), cols), dtype=torch.float32, device=dev)
        ckw = torch.empty_like(ckv)
    v_last = torch.empty(shape, dtype=torch.float32, device=dev)
    w_last = torch.empty_like(v_last)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().nsb_plif_rf_fwd(
            _lib.ptr(beta_c), _lib.ptr(omega_c), _lib.ptr(u_c), _lib.ptr(vth_c), _lib.ptr(v0), _lib.ptr(w0),
            _lib.ptr(spike), None, _lib.ptr(vpost), _lib.ptr(wout), _lib.ptr(ckv), _lib.ptr(ckw),
            _lib.ptr(v_last), _lib.ptr(w_last), T, cols, _lib.dtype_code(dt), C,
            _lib.ptr(_split_scratch(T, cols, dev)), _lib.stream_ptr(dev)), "nsb_plif_rf_fwd")
    if needs_grad:
        ctx.save_for_backward(beta_c, omega_c, u_c, vth_c, ckv, ckw)
    ctx.alpha, ctx.alpha_t = _split_alpha(alpha)
    ctx.in_dtypes = tuple(t.dtype for t in (beta, omega, u, v_th, v_init, w_init))
    ctx.state_shapes = (v_init.shape, w_init.shape)
    return _cast(spike, out_dtype), _cast(vpost, out_dtype), _cast(wout, out_dtype), v_last, w_last


def _rf_backward(ctx, grad_spike, grad_V_post):
    beta_c, omega_c, u_c, vth_c, ckv, ckw = ctx.saved_tensors
    dt, dev = u_c.dtype, u_c.device
    T, cols = u_c.shape[0], _cols(u_c)
    if grad_spike is None:
        grad_spike = torch.zeros_like(u_c)
    gs = _grad_stream(grad_spike, u_c, dt)
    gv = _grad_stream(grad_V_post, u_c, dt)
    g_beta, g_omega, g_u, g_vth = (torch.empty_like(u_c) for _ in range(4))
    g_v0 = torch.empty(u_c.shape[1:], dtype=torch.float32, device=dev)
    g_w0 = torch.empty_like(g_v0)
    alpha_t = getattr(ctx, "alpha_t", None)
    with torch.cuda.device(dev):
        fn = _lib.lib().nsb_plif_rf_bwd if alpha_t is None else _lib.lib().nsb_plif_rf_bwd_dalpha
        _lib.check(fn(
            _lib.ptr(beta_c), _lib.ptr(omega_c), _lib.ptr(u_c), _lib.ptr(vth_c), _lib.ptr(ckv),
            _lib.ptr(ckw), _lib.ptr(gs), _lib.ptr(gv), _lib.ptr(g_beta), _lib.ptr(g_omega), _lib.ptr(g_u),
            _lib.ptr(g_vth), _lib.ptr(g_v0), _lib.ptr(g_w0), T, cols, _lib.dtype_code(dt), ctx.interval,
            ctx_surrogate(ctx), ctx.alpha if alpha_t is None else _lib.ptr(alpha_t),
            _lib.ptr(_chain_scratch(T, cols, dev)), _lib.stream_ptr(dev)), "nsb_plif_rf_bwd")
    db, do, du, dth, dv, dw = ctx.in_dtypes
    return (_cast(g_beta, db), _cast(g_omega, do), _cast(g_u, du), _cast(g_vth, dth),
            g_v0.to(dv).reshape(ctx.state_shapes[0]), g_w0.to(dw).reshape(ctx.state_shapes[1]), None)


class PLIFRFScan(torch.autograd.Function):
    """Resonate-and-fire PLIF scan returning ``(spike, V_post, W)``; contract of the
    reference's ``_TritonRFPLIFForward`` (atomic_ops/parallel_scan.py:1071-1148). A
    gradient arriving for ``W`` is ignored, as in the reference (:1114)."""

    @staticmethod
    def forward(ctx, beta, omega, u, v_th, v_init, w_init, alpha):
        spike, vpost, wout, _, _ = _rf_forward(ctx, beta, omega, u, v_th, v_init, w_init, alpha, True)
        return spike, vpost, wout

    @staticmethod
    def backward(ctx, grad_spike, grad_V_post, _grad_W):
        return _rf_backward(ctx, grad_spike, grad_V_post)


class PLIFRFRecomputeScan(torch.autograd.Function):
    """Resonate-and-fire PLIF scan returning ``(spike, V_last, W_last)``; contract of
    the reference's ``_TritonRFPLIFRecompute`` (:1150-1233). Gradients arriving for the
    final states are ignored (:1203); grad_u and grad_v_th are new tensors, not the
    saved inputs overwritten in place (:1232-1233)."""

    @staticmethod
    def forward(ctx, beta, omega, u, v_th, v_init, w_init, alpha):
        spike, _, _, v_last, w_last = _rf_forward(ctx, beta, omega, u, v_th, v_init, w_init, alpha, False)
        return spike, v_last.to(v_init.dtype), w_last.to(w_init.dtype)

    @staticmethod
    def backward(ctx, grad_spike, _gv, _gw):
        return _rf_backward(ctx, grad_spike, None)


# Names the reference's callers import (snn_block.py, snn_ffn.py, test_recompute.py ...).
_TritonRFPLIFForward = PLIFRFScan
_TritonRFPLIFRecompute = PLIFRFRecomputeScan
_TritonPLIFForward = PLIFSelectiveScan
_TritonPLIFRowParamForward = PLIFRowParamScan
_TritonPLIFRowParamRecompute = PLIFRowParamRecomputeScan
_HAS_TRITON = False  # nothing here uses Triton


# ------------------------------------------------------------ public functions


def _alpha_and_kind(surrogate_function):
    """(alpha, kind) of a SpikingJelly-style surrogate object, by class name as
    the reference does (atomic_ops/parallel_scan.py:1347-1349)."""
    name = type(surrogate_function).__name__
    if not hasattr(surrogate_function, "alpha"):
        raise NSBError(f"surrogate {name} has no .alpha")
    a = surrogate_function.alpha
    if not (isinstance(a, torch.Tensor) and a.is_cuda):  # a device-resident slope stays on the device
        a = float(a)
    if name == "Sigmoid":
        return a, _lib.SURR_SIGMOID
    if name == "ATan":
        return a, _lib.SURR_ATAN
    raise NSBError(f"surrogate {name} is not supported (Sigmoid or ATan)")


class _SelectiveScanATan(PLIFSelectiveScan):
    """u-form selective scan with the arctangent surrogate in the backward."""

    @staticmethod
    def forward(ctx, beta, u, v_th, v_init, alpha):
        ctx.surrogate = _lib.SURR_ATAN
        return PLIFSelectiveScan.forward(ctx, beta, u, v_th, v_init, alpha)


def plif_parallel_forward(beta, u, v_th, v_init, max_iter: int = 3, surrogate_function=None):
    """Selective PLIF forward; returns ``(spike, V_post, None)`` like the reference's
    fused path (atomic_ops/parallel_scan.py:1309-1352). ``max_iter`` is accepted
    for signature compatibility and unused: the sequential scan is exact. With
    ``surrogate_function=None`` the outputs carry no gradient."""
    del max_iter
    if surrogate_function is None:
        with torch.no_grad():
            spike, vpost = PLIFSelectiveScan.apply(beta, u, v_th, v_init, 0.0)
        return spike, vpost, None
    alpha, kind = _alpha_and_kind(surrogate_function)
    fn = PLIFSelectiveScan if kind == _lib.SURR_SIGMOID else _SelectiveScanATan
    spike, vpost = fn.apply(beta, u, v_th, v_init, alpha)
    return spike, vpost, None


def _rows(u, *rows):
    """Per-column arguments may be given per channel ([D]) or already expanded to
    ``u.shape[1:]``; broadcasting here keeps their gradients flowing through expand."""
    shape = u.shape[1:]
    return tuple(r if tuple(r.shape) == tuple(shape) else r.expand(shape) for r in rows)


def plif_rowparam_forward(beta_row, u, v_th_row, v_init, surrogate_function=None):
    """Reference: atomic_ops/parallel_scan.py:1415-1453. Returns ``(spike, V_post)``."""
    beta_row, v_th_row, v_init = _rows(u, beta_row, v_th_row, v_init)
    if surrogate_function is None:
        with torch.no_grad():
            return PLIFRowParamScan.apply(beta_row, u, v_th_row, v_init, 0.0)
    alpha, kind = _alpha_and_kind(surrogate_function)
    if kind != _lib.SURR_SIGMOID:
        raise NSBError("row-parameter scans support the Sigmoid surrogate only")
    return PLIFRowParamScan.apply(beta_row, u, v_th_row, v_init, alpha)


def plif_rowparam_forward_alpha(beta_row, u, v_th_row, v_init, alpha: float):
    """Reference: atomic_ops/parallel_scan.py:1456-1495. Returns ``(spike, V_post)``."""
    beta_row, v_th_row, v_init = _rows(u, beta_row, v_th_row, v_init)
    return PLIFRowParamScan.apply(beta_row, u, v_th_row, v_init, alpha)


def plif_rowparam_forward_recompute(beta_row, u, v_th_row, v_init, alpha: float):
    """Reference: atomic_ops/parallel_scan.py:1499-1535. Returns ``(spike, V_last)``."""
    beta_row, v_th_row, v_init = _rows(u, beta_row, v_th_row, v_init)
    return PLIFRowParamRecomputeScan.apply(beta_row, u, v_th_row, v_init, alpha)


class PLIFRowParamResidualScan(torch.autograd.Function):
    """Row-parameter scan + binary residual in one kernel: what the reference computes as
    ``binary_residual(plif_rowparam_forward_recompute(...)[0], spike_in)`` at the end of
    ``SNNBlock.forward_parallel`` and ``SNNFFN.forward_parallel`` (atomic_ops/snn_block.py:281-285,
    atomic_ops/snn_ffn.py:188-195). Returns ``(frames_out, V_last)``. The residual's backward is
    the identity on both of its inputs (atomic_ops/fp16_codec.py:171-173): the gradient arriving
    for ``frames_out`` is returned for ``spike_in`` and drives the scan's backward."""

    @staticmethod
    def forward(ctx, beta_row, u, v_th_row, v_init, spike_in, alpha):
        shape = u.shape[1:]
        if spike_in.shape != u.shape or u.shape[0] % 16:
            raise NSBError("spike_in must have u's shape (T*16, ...)")
        dt = u.dtype if u.dtype in (torch.float32, torch.bfloat16, torch.float16) else torch.float32
        u_c = _as_stream(u, dt)
        fin = _as_stream(spike_in, dt)
        beta32, vth32, v0 = (_row_f32(t, shape) for t in (beta_row, v_th_row, v_init))
        dev = _lib.require_cuda(u_c, fin, beta32, vth32, v0)
        T, cols = u_c.shape[0], _cols(u_c)
        needs_grad = any(ctx.needs_input_grad[:4])
        C = ctx.interval = 32 if _interval(cols, row_param=True) == 32 else 16
        out = torch.empty_like(u_c)
        ckpt = torch.empty((_n_tiles(T, C), cols), dtype=torch.float32, device=dev) if needs_grad else None
        v_last = torch.empty(shape, dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            _lib.check(_lib.lib().nsb_plif_rowparam_residual_fwd(
                _lib.ptr(beta32), _lib.ptr(u_c), _lib.ptr(vth32), _lib.ptr(v0), _lib.ptr(fin), _lib.ptr(out),
                _lib.ptr(ckpt), _lib.ptr(v_last), T, cols, _lib.dtype_code(dt), C,
                fp16_codec.residual_rounding_code(), _lib.ptr(_split_scratch(T, cols, dev)), _lib.stream_ptr(dev)),
                "nsb_plif_rowparam_residual_fwd")
        if needs_grad:
            ctx.save_for_backward(beta32, vth32, u_c, ckpt)
        ctx.alpha, ctx.alpha_t = _split_alpha(alpha)
        ctx.in_dtypes = (beta_row.dtype, u.dtype, v_th_row.dtype, v_init.dtype)
        ctx.row_shapes = (beta_row.shape, v_th_row.shape, v_init.shape)
        ctx.spike_in_dtype = spike_in.dtype
        v_last = v_last.to(v_init.dtype)
        ctx.mark_non_differentiable(v_last)
        return _cast(out, u.dtype), v_last

    @staticmethod
    def backward(ctx, grad_out, _grad_v_last):
        g_spike_in = None
        if ctx.needs_input_grad[4] and grad_out is not None:
            g_spike_in = grad_out.to(ctx.spike_in_dtype)
        if not any(ctx.needs_input_grad[:4]):
            return None, None, None, None, g_spike_in, None
        return _rowparam_backward(ctx, grad_out, None)[:4] + (g_spike_in, None)


def plif_rowparam_residual_forward(beta_row, u, v_th_row, v_init, spike_in, alpha: float):
    """``(binary_residual(spike, spike_in), V_last)`` with ``spike`` the output of the row-parameter
    scan, in one kernel; arguments of ``plif_rowparam_forward_recompute`` plus ``spike_in``."""
    beta_row, v_th_row, v_init = _rows(u, beta_row, v_th_row, v_init)
    return PLIFRowParamResidualScan.apply(beta_row, u, v_th_row, v_init, spike_in, alpha)


@torch.no_grad()
def plif_rowparam_forward_patterns(beta_row, u, v_th_row, v_init, patterns_in=None,
                                   frame_dtype: torch.dtype = None, want_ckpt: bool = False):
    """The row-parameter scan with its spikes packed in time: returns ``(patterns, V_last, ckpt)``
    where ``patterns`` is int16 ``(T/16, ...)`` - per token and column the half bit pattern the 16
    spikes spell (``fp16_codec.pack_frames`` of the dense spikes). With ``patterns_in`` the binary
    residual with that array is applied first (``frame_dtype``: the frame dtype whose roundings
    apply, default ``u``'s). ``ckpt`` (when asked for) and ``(beta_row, u, v_th_row)`` are what
    ``plif_rowparam_patterns_backward`` needs."""
    beta_row, v_th_row, v_init = _rows(u, beta_row, v_th_row, v_init)
    shape = u.shape[1:]
    if u.shape[0] % 16:
        raise NSBError("T must be a multiple of 16")
    dt = u.dtype if u.dtype in (torch.float32, torch.bfloat16, torch.float16) else torch.float32
    u_c = _as_stream(u, dt)
    beta32, vth32, v0 = (_row_f32(t, shape) for t in (beta_row, v_th_row, v_init))
    dev = _lib.require_cuda(u_c, beta32, vth32, v0, patterns_in)
    T, cols = u_c.shape[0], _cols(u_c)
    if patterns_in is not None:
        if patterns_in.dtype != torch.int16 or tuple(patterns_in.shape) != (T // 16, *shape):
            raise NSBError("patterns_in must be int16 of shape (T/16, ...)")
        patterns_in = patterns_in.contiguous()
    C = 32 if _interval(cols, row_param=True) == 32 else 16
    out = torch.empty((T // 16, *shape), dtype=torch.int16, device=dev)
    ckpt = torch.empty((_n_tiles(T, C), cols), dtype=torch.float32, device=dev) if want_ckpt else None
    v_last = torch.empty(shape, dtype=torch.float32, device=dev)
    fdt = frame_dtype if frame_dtype is not None else dt
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().nsb_plif_rowparam_pattern_fwd(
            _lib.ptr(beta32), _lib.ptr(u_c), _lib.ptr(vth32), _lib.ptr(v0), _lib.ptr(patterns_in), _lib.ptr(out),
            _lib.ptr(ckpt), _lib.ptr(v_last), T, cols, _lib.dtype_code(dt), C, _lib.dtype_code(fdt),
            fp16_codec.residual_rounding_code(), _lib.ptr(_split_scratch(T, cols, dev)), _lib.stream_ptr(dev)),
            "nsb_plif_rowparam_pattern_fwd")
    return out, v_last, (ckpt, C)


@torch.no_grad()
def plif_rowparam_patterns_backward(beta_row, u, v_th_row, ckpt, grad_frames, alpha: float):
    """Backward of ``plif_rowparam_forward_patterns``: ``grad_frames`` is the dense ``(T, ...)``
    gradient of the spikes (e.g. from ``fp16_codec.fp16_decode_packed_backward``); ``ckpt`` the third
    value the forward returned. Returns ``(grad_beta_row, grad_u, grad_v_th_row, grad_v_init)``."""
    ck, C = ckpt
    beta_row, v_th_row = _rows(u, beta_row, v_th_row)
    shape = u.shape[1:]
    dt = u.dtype if u.dtype in (torch.float32, torch.bfloat16, torch.float16) else torch.float32
    u_c = _as_stream(u, dt)
    gs = _as_stream(grad_frames, dt)
    beta32, vth32 = _row_f32(beta_row, shape), _row_f32(v_th_row, shape)
    dev = _lib.require_cuda(u_c, gs, beta32, vth32, ck)
    T, cols = u_c.shape[0], _cols(u_c)
    g_u = torch.empty_like(u_c)
    g_beta, g_vth, g_v0 = (torch.empty(shape, dtype=torch.float32, device=dev) for _ in range(3))
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().nsb_plif_rowparam_bwd(
            _lib.ptr(beta32), _lib.ptr(u_c), _lib.ptr(vth32), _lib.ptr(ck), _lib.ptr(gs), None, _lib.ptr(g_beta),
            _lib.ptr(g_u), _lib.ptr(g_vth), _lib.ptr(g_v0), T, cols, _lib.dtype_code(dt), C, _lib.SURR_SIGMOID,
            float(alpha), _lib.ptr(_split_scratch(T, cols, dev)), _lib.stream_ptr(dev)), "nsb_plif_rowparam_bwd")
    return g_beta, g_u, g_vth, g_v0


def _rf_apply(fn, beta, omega, u, v_th, v_init, w_init, surrogate_function):
    if surrogate_function is None:
        with torch.no_grad():
            return fn.apply(beta, omega, u, v_th, v_init, w_init, 0.0)
    alpha, kind = _alpha_and_kind(surrogate_function)
    if kind != _lib.SURR_SIGMOID:
        raise NSBError("the resonate-and-fire scan supports the Sigmoid surrogate only")
    return fn.apply(beta, omega, u, v_th, v_init, w_init, alpha)


def rf_plif_parallel_forward(beta, omega, u, v_th, v_init, w_init, surrogate_function=None):
    """Reference: atomic_ops/parallel_scan.py:1610-1683. Returns ``(spike, V_post, W)``.
    With ``surrogate_function=None`` the outputs carry no gradient."""
    return _rf_apply(PLIFRFScan, beta, omega, u, v_th, v_init, w_init, surrogate_function)


def rf_plif_parallel_forward_recompute(beta, omega, u, v_th, v_init, w_init, surrogate_function=None):
    """Reference: atomic_ops/parallel_scan.py:1690-1726. Returns ``(spike, V_last, W_last)``."""
    return _rf_apply(PLIFRFRecomputeScan, beta, omega, u, v_th, v_init, w_init, surrogate_function)


def plif_fixed_param_forward(beta, u, v_th, v_init, max_iter: int = 3, surrogate_function=None):
    """Reference: atomic_ops/parallel_scan.py:1538-1603. Scalar (float or 0-dim
    tensor) beta and v_th take the row-parameter kernel; anything else is expanded
    to ``u``'s shape and takes the selective kernel. Returns ``(spike, V_post)``."""
    K = u.shape[0]
    shape = u.shape[1:]

    def is_scalar(x):
        return (not isinstance(x, torch.Tensor)) or x.dim() == 0

    if is_scalar(beta) and is_scalar(v_th):
        def row(x):
            if isinstance(x, torch.Tensor):
                return x.expand(*shape)
            return torch.full(shape, float(x), device=u.device, dtype=u.dtype)
        return plif_rowparam_forward(row(beta), u, row(v_th), v_init, surrogate_function)

    def full(x):
        if isinstance(x, torch.Tensor):
            return x.expand(K, *shape) if x.dim() == 0 else x
        return torch.full_like(u, float(x))
    spike, vpost, _ = plif_parallel_forward(full(beta), u, full(v_th), v_init, max_iter,
                                            surrogate_function)
    return spike, vpost


# ---------------------------------------------------------- B200-native extras


def plif_selective_scan_ai(beta, cur, gain, v_th, v_init, alpha: float = 4.0,
                           surrogate: str = "sigmoid"):
    """Selective scan in the alpha*I form with gradients for beta, cur, gain, v_th
    and v_init. Returns ``(spike, V_last)``."""
    return PLIFSelectiveScanAI.apply(beta, cur, gain, v_th, v_init, alpha, surrogate)


@torch.no_grad()
def plif_selective_forward_packed(beta, drive, v_th, v_init, gain=None):
    """Inference scan with bit-packed spikes.

    Returns ``(packed, V_last)``: ``packed`` is int32 ``[T, ceil(cols/32)]`` where
    bit i of word w is column 32*w+i of the flattened trailing dims (tail bits
    zero) and ``V_last`` is fp32 — pass it as ``v_init`` of the next call to carry
    the state across calls (per-token decoding)."""
    dt = _common_stream_dtype(beta, drive, v_th, gain)
    beta_c, drive_c, vth_c, gain_c = (_as_stream(t, dt) for t in (beta, drive, v_th, gain))
    v0 = _row_f32(v_init, drive.shape[1:])
    _, packed, _, _, v_last, _ = _launch_selective_fwd(
        beta_c, drive_c, gain_c, vth_c, v0, want_spike=False, want_packed=True, want_vpost=False,
        want_ckpt=False)
    return packed, v_last


@torch.no_grad()
def plif_rowparam_forward_packed(beta_row, u, v_th_row, v_init):
    """Row-parameter inference scan with bit-packed spikes; see
    :func:`plif_selective_forward_packed` for the layout."""
    shape = u.shape[1:]
    u_c = _as_stream(u, _common_stream_dtype(u))
    beta32, vth32, v0 = (_row_f32(t, shape) for t in (beta_row, v_th_row, v_init))
    _, packed, _, _, v_last, _ = _launch_rowparam_fwd(
        beta32, u_c, vth32, v0, want_spike=False, want_packed=True, want_vpost=False,
        want_ckpt=False)
    return packed, v_last


def unpack_spikes(packed: torch.Tensor, shape, dtype=torch.float32) -> torch.Tensor:
    """Expands bit-packed spikes ``[T, ceil(cols/32)]`` to a dense ``[T, *shape]``
    tensor of {0,1}. A convenience for tests and debugging (plain PyTorch ops)."""
    T = packed.shape[0]
    cols = 1
    for s in shape:
        cols *= s
    bits = torch.arange(32, device=packed.device, dtype=torch.int32)
    dense = ((packed.unsqueeze(-1) >> bits) & 1).reshape(T, -1)[:, :cols]
    return dense.to(dtype).reshape(T, *shape)
