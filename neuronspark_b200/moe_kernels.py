"""Mixture-of-experts output combine (mirror of the reference's ``atomic_ops/moe_kernels.py``).

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
