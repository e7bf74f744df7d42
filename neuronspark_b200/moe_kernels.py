"""Mixture-of-experts output combine (mirror of the reference's ``atomic_ops/moe_kernels.py``), and
the same merge done on spike frames (``frames_combine``: what ``MoESNNFFN.forward_parallel`` computes
with fp16_decode, a weighted sum and binary_encode_ste, ``atomic_ops/moe_snn_ffn.py:377-393``).

    out[n, d] = shared[n, d] + sum_e experts[e, n, d] * weights[n, e]

``MoECombine`` keeps the reference's Function contract (:131-207): inputs ``shared (N, D)``,
``experts (E, N, D)``, ``weights (N, E)``; gradients for all three, the one of ``shared`` being the
incoming gradient itself.
"""
from __future__ import annotations

import torch

from . import _lib
from ._lib import NSBError


class MoECombine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, shared, experts, weights):
        if experts.dim() != 3 or shared.dim() != 2 or weights.dim() != 2:
            raise NSBError("moe_combine expects shared (N, D), experts (E, N, D), weights (N, E)")
        E, N, D = experts.shape
        if shared.shape != (N, D) or weights.shape != (N, E):
            raise NSBError("moe_combine: inconsistent shapes")
        dt = shared.dtype if shared.dtype in (torch.float32, torch.bfloat16, torch.float16) else torch.float32
        s_c = shared.to(dt).contiguous()
        e_c = experts.to(dt).contiguous()
        w32 = weights.detach().to(torch.float32).contiguous()
        dev = _lib.require_cuda(s_c, e_c, w32)
        out = torch.empty_like(s_c)
        with torch.cuda.device(dev):
            _lib.check(_lib.lib().nsb_moe_combine_fwd(_lib.ptr(s_c), _lib.ptr(e_c), _lib.ptr(w32), _lib.ptr(out),
                                                      N, D, E, _lib.dtype_code(dt), _lib.stream_ptr(dev)),
                       "nsb_moe_combine_fwd")
        ctx.save_for_backward(e_c, w32)
        ctx.in_dtypes = (shared.dtype, experts.dtype, weights.dtype)
        return out if out.dtype == shared.dtype else out.to(shared.dtype)

    @staticmethod
    def backward(ctx, grad_out):
        e_c, w32 = ctx.saved_tensors
        E, N, D = e_c.shape
        dt, dev = e_c.dtype, e_c.device
        g = grad_out.to(dt).contiguous()
        need_e, need_w = ctx.needs_input_grad[1], ctx.needs_input_grad[2]
        g_e = torch.empty_like(e_c) if need_e else None
        g_w = torch.empty((N, E), dtype=torch.float32, device=dev) if need_w else None
        if need_e or need_w:
            with torch.cuda.device(dev):
                _lib.check(_lib.lib().nsb_moe_combine_bwd(_lib.ptr(g), _lib.ptr(e_c), _lib.ptr(w32), _lib.ptr(g_e),
                                                          _lib.ptr(g_w), N, D, E, _lib.dtype_code(dt),
                                                          _lib.stream_ptr(dev)), "nsb_moe_combine_bwd")
        ds, de, dw = ctx.in_dtypes
        return (grad_out.to(ds) if ctx.needs_input_grad[0] else None,
                g_e.to(de) if need_e else None, g_w.to(dw) if need_w else None)


def moe_combine(shared: torch.Tensor, experts: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
    """Reference: atomic_ops/moe_kernels.py:210-224."""
    return MoECombine.apply(shared, experts, weights)


class FramesCombine(torch.autograd.Function):
    """``binary_encode_ste(decode(shared) + sum_e decode(experts[e]) * w[e] + decode(residual))`` on
    frames, one kernel each way. ``shared`` / ``residual``: (T*16, B, D) frames, ``experts``:
    (E, T*16, B, D), ``weights``: (T, B, E) (the reference's ``full_weights``)."""

    @staticmethod
    def forward(ctx, shared, experts, weights, residual):
        if shared.dim() != 3 or experts.dim() != 4 or weights.dim() != 3 or residual.shape != shared.shape:
            raise NSBError("frames_combine expects shared/residual (T*16, B, D), experts (E, T*16, B, D), "
                           "weights (T, B, E)")
        TK, B, D = shared.shape
        E = experts.shape[0]
        if TK % 16 or experts.shape[1:] != shared.shape or weights.shape != (TK // 16, B, E) or E > 16:
            raise NSBError("frames_combine: inconsistent shapes")
        dt = shared.dtype if shared.dtype in (torch.float32, torch.bfloat16, torch.float16) else torch.float32
        a, x, w, r = (t.to(dt).contiguous() for t in (shared, experts, weights, residual))
        dev = _lib.require_cuda(a, x, w, r)
        out = torch.empty_like(a)
        with torch.cuda.device(dev):
            _lib.check(_lib.lib().nsb_frames_combine_fwd(_lib.ptr(a), _lib.ptr(x), _lib.ptr(w), _lib.ptr(r),
                                                         _lib.ptr(out), B, TK // 16, D, E, _lib.dtype_code(dt),
                                                         _lib.stream_ptr(dev)), "nsb_frames_combine_fwd")
        ctx.save_for_backward(a, x, w, r)
        ctx.in_dtypes = tuple(t.dtype for t in (shared, experts, weights, residual))
        return out if out.dtype == shared.dtype else out.to(shared.dtype)

    @staticmethod
    def backward(ctx, grad_out):
        a, x, w, r = ctx.saved_tensors
        TK, B, D = a.shape
        E, dt, dev = x.shape[0], a.dtype, a.device
        g = grad_out.to(dt).contiguous()
        need = ctx.needs_input_grad
        outs = [torch.empty_like(t) if n else None for t, n in zip((a, x, w, r), need)]
        if any(need):
            with torch.cuda.device(dev):
                _lib.check(_lib.lib().nsb_frames_combine_bwd(
                    _lib.ptr(g), _lib.ptr(a), _lib.ptr(x), _lib.ptr(w), _lib.ptr(r), _lib.ptr(outs[0]),
                    _lib.ptr(outs[1]), _lib.ptr(outs[2]), _lib.ptr(outs[3]), B, TK // 16, D, E,
                    _lib.dtype_code(dt), _lib.stream_ptr(dev)), "nsb_frames_combine_bwd")
        return tuple(o.to(d) if o is not None else None for o, d in zip(outs, ctx.in_dtypes))


def frames_combine(shared: torch.Tensor, experts: torch.Tensor, weights: torch.Tensor,
                   residual: torch.Tensor) -> torch.Tensor:
    """Reference: atomic_ops/moe_snn_ffn.py:377-393 (the training branch's decode / combine / add
    residual / binary_encode_ste sequence)."""
    return FramesCombine.apply(shared, experts, weights, residual)
