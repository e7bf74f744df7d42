"""Lateral inhibition (divisive normalisation) and RMSNorm with the interfaces
of NeuronSpark's ``atomic_ops/lateral_inhibition.py`` and ``atomic_ops/rms_norm.py``,
backed by the sm_100a CUDA kernels.

    _LateralInhibitionTriton.apply(x, gain, eps)   reference lateral_inhibition.py:122-171
    LateralInhibition(dim, eps)                    reference :178-215
    RMSNorm(dim, eps)                              reference rms_norm.py:20-46

The modules are plain ``torch.nn.Module`` (the reference derives
LateralInhibition from SpikingJelly's stateless MemoryModule; it has no state).
CUDA tensors only.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from . import _lib
from ._lib import NSBError


class LateralInhibitionFunction(torch.autograd.Function):
    """out = x * rsqrt(mean(x^2, -1) + eps) * gain, fp32 math, stored in x's dtype.
    grad_gain is reduced over rows inside the call, deterministically."""

    @staticmethod
    def forward(ctx, x, gain, eps):
        dev = _lib.require_cuda(x, gain)
        if x.dtype not in (torch.float32, torch.bfloat16, torch.float16):
            raise NSBError(f"unsupported dtype {x.dtype}")
        D = x.shape[-1]
        if gain.numel() != D:
            raise NSBError(f"gain has {gain.numel()} elements, expected {D}")
        x2 = x.reshape(-1, D).contiguous()
        g = gain.detach().contiguous()
        if g.dtype not in (torch.float32, torch.bfloat16, torch.float16):
            g = g.float()
        out = torch.empty_like(x2)
        with torch.cuda.device(dev):
            _lib.check(_lib.lib().nsb_lateral_inhibition_fwd(
                _lib.ptr(x2), _lib.ptr(g), _lib.ptr(out), x2.shape[0], D, float(eps),
                _lib.dtype_code(x2.dtype), _lib.dtype_code(g.dtype), _lib.stream_ptr(dev)),
                "nsb_lateral_inhibition_fwd")
        ctx.save_for_backward(x2, g)
        ctx.eps = float(eps)
        ctx.orig_shape = x.shape
        ctx.gain_dtype = gain.dtype
        ctx.gain_shape = gain.shape
        return out.reshape(x.shape)

    @staticmethod
    def backward(ctx, grad_output):
        x2, g = ctx.saved_tensors
        dev = x2.device
        rows, D = x2.shape
        go = grad_output.reshape(rows, D).to(x2.dtype).contiguous()
        dx = torch.empty_like(x2)
        dgain = torch.empty(D, dtype=torch.float32, device=dev)
        n = int(_lib.lib().nsb_li_bwd_scratch_floats(rows, D))
        scratch = torch.empty(max(n, 1), dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            _lib.check(_lib.lib().nsb_lateral_inhibition_bwd(
                _lib.ptr(go), _lib.ptr(x2), _lib.ptr(g), _lib.ptr(dx), _lib.ptr(dgain),
                _lib.ptr(scratch), rows, D, ctx.eps, _lib.dtype_code(x2.dtype),
                _lib.dtype_code(g.dtype), _lib.stream_ptr(dev)), "nsb_lateral_inhibition_bwd")
        return dx.reshape(ctx.orig_shape), dgain.to(ctx.gain_dtype).reshape(ctx.gain_shape), None


# Name used by the reference's modules.
_LateralInhibitionTriton = LateralInhibitionFunction


class LateralInhibition(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.gain = nn.Parameter(torch.ones(dim))
        self.eps = eps
        self.dim = dim

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        return LateralInhibitionFunction.apply(h, self.gain, self.eps)

    def extra_repr(self):
        return f"dim={self.dim}, eps={self.eps}"


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return LateralInhibitionFunction.apply(x, self.weight, self.eps)
