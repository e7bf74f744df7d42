"""FP16 boundary codec with the call signatures of NeuronSpark's
``atomic_ops/fp16_codec.py``, backed by the sm_100a CUDA kernels.

    fp16_encode(emb, K=16)              reference :17-46
    fp16_decode(spikes, seq_len, K=16)  reference :49-98 (differentiable)
    binary_residual(a, b)               reference :115-205 (STE backward)
    binary_encode_ste(x)                reference :208-241

CUDA tensors only; K must be 16 (one frame per bit of an IEEE half).

bf16 frames and the residual: the reference's ``binary_residual`` runs
``torch.compile(_binary_residual_fwd)`` (:168-186), and on a GPU inductor's fused kernel keeps
the decode in fp32 and rounds only the sum to bf16, whereas the same function called eagerly
(or ``_binary_residual_naive``, :103-112) rounds every intermediate to bf16 - the two differ in
about 1 % of the frames of real layer activations. ``binary_residual`` here follows the compiled
behaviour, since that is what the reference's layers get; ``RESIDUAL_ROUNDING = "eager"`` (or
the ``rounding`` argument of ``binary_residual_with``) selects the other. fp32 and fp16 frames
are unaffected: all their intermediates are exact.
"""
from __future__ import annotations

import torch

from . import _lib
from ._lib import NSBError


#: "compiled" (default) or "eager": rounding of the residual on bf16 frames, see the module text.
RESIDUAL_ROUNDING = "compiled"

_ROUNDINGS = {"eager": _lib.RESIDUAL_EAGER, "compiled": _lib.RESIDUAL_COMPILED}


def residual_rounding_code(rounding=None) -> int:
    r = RESIDUAL_ROUNDING if rounding is None else rounding
    try:
        return _ROUNDINGS[r]
    except KeyError:
        raise NSBError(f"unknown residual rounding {r!r}; expected 'compiled' or 'eager'") from None


def _check_k(K: int) -> None:
    if K != 16:
        raise NSBError("the FP16 codec has exactly 16 frames per token (K must be 16)")


def _encode(emb: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    dev = _lib.require_cuda(emb)
    if emb.dim() != 3:
        raise NSBError("fp16_encode expects (batch, seq_len, D)")
    if emb.dtype not in (torch.float32, torch.bfloat16, torch.float16):
        emb = emb.float()
    emb_c = emb.detach().contiguous()
    B, S, D = emb_c.shape
    frames = torch.empty((S * 16, B, D), dtype=out_dtype, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().nsb_fp16_encode(
            _lib.ptr(emb_c), _lib.ptr(frames), B, S, D, _lib.dtype_code(emb_c.dtype),
            _lib.dtype_code(out_dtype), _lib.stream_ptr(dev)), "nsb_fp16_encode")
    return frames


def fp16_encode(emb: torch.Tensor, K: int = 16) -> torch.Tensor:
    """(batch, seq_len, D) values -> (seq_len*16, batch, D) frames in {0,1}, in
    ``emb``'s dtype, detached. Values are clamped to +-65504 and rounded to half
    (nearest even) first; frame t*16+k is bit 15-k (sign, exponent, mantissa)."""
    _check_k(K)
    out_dtype = emb.dtype if emb.dtype in (torch.float32, torch.bfloat16, torch.float16) \
        else torch.float32
    return _encode(emb, out_dtype)


class _FP16Decode(torch.autograd.Function):
    @staticmethod
    def forward(ctx, spikes, seq_len):
        dev = _lib.require_cuda(spikes)
        TK, B, D = spikes.shape
        if TK != seq_len * 16:
            raise NSBError(f"spikes has {TK} frames, expected seq_len*16 = {seq_len * 16}")
        if spikes.dtype not in (torch.float32, torch.bfloat16, torch.float16):
            raise NSBError(f"unsupported dtype {spikes.dtype}")
        sp = spikes.contiguous()
        out = torch.empty((B, seq_len, D), dtype=sp.dtype, device=dev)
        with torch.cuda.device(dev):
            _lib.check(_lib.lib().nsb_fp16_decode_fwd(
                _lib.ptr(sp), _lib.ptr(out), B, seq_len, D, _lib.dtype_code(sp.dtype),
                _lib.stream_ptr(dev)), "nsb_fp16_decode_fwd")
        if ctx.needs_input_grad[0]:
            ctx.save_for_backward(sp)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        (sp,) = ctx.saved_tensors
        dev = sp.device
        TK, B, D = sp.shape
        g = grad_out.to(sp.dtype).contiguous()
        g_frames = torch.empty_like(sp)
        with torch.cuda.device(dev):
            _lib.check(_lib.lib().nsb_fp16_decode_bwd(
                _lib.ptr(sp), _lib.ptr(g), _lib.ptr(g_frames), B, TK // 16, D,
                _lib.dtype_code(sp.dtype), _lib.stream_ptr(dev)), "nsb_fp16_decode_bwd")
        return g_frames, None


def fp16_decode(spikes: torch.Tensor, seq_len: int, K: int = 16) -> torch.Tensor:
    """(seq_len*16, batch, D) frames -> (batch, seq_len, D) values, differentiable
    w.r.t. the frames. An all-ones exponent decodes as an ordinary normal number."""
    _check_k(K)
    return _FP16Decode.apply(spikes, seq_len)


class _BinaryResidual(torch.autograd.Function):
    """encode(decode(a) + decode(b)); backward passes the gradient to both inputs
    unchanged (straight-through), as the reference's class of the same name."""

    @staticmethod
    def forward(ctx, spike_a, spike_b, rounding=None):
        dev = _lib.require_cuda(spike_a, spike_b)
        if spike_a.shape != spike_b.shape or spike_a.dim() != 3 or spike_a.shape[0] % 16:
            raise NSBError("binary_residual expects two (T*16, B, D) tensors of equal shape")
        dt = spike_a.dtype
        if dt not in (torch.float32, torch.bfloat16, torch.float16):
            raise NSBError(f"unsupported dtype {dt}")
        a = spike_a.contiguous()
        b = spike_b.to(dt).contiguous()
        TK, B, D = a.shape
        out = torch.empty_like(a)
        with torch.cuda.device(dev):
            _lib.check(_lib.lib().nsb_binary_residual(
                _lib.ptr(a), _lib.ptr(b), _lib.ptr(out), B, TK // 16, D, _lib.dtype_code(dt),
                residual_rounding_code(rounding), _lib.stream_ptr(dev)), "nsb_binary_residual")
        return out

    @staticmethod
    def backward(ctx, grad_output):
        return grad_output, grad_output, None


def binary_residual(spike_a: torch.Tensor, spike_b: torch.Tensor) -> torch.Tensor:
    """Reference: atomic_ops/fp16_codec.py:189-205."""
    return _BinaryResidual.apply(spike_a, spike_b)


def binary_residual_with(spike_a: torch.Tensor, spike_b: torch.Tensor, rounding: str) -> torch.Tensor:
    """``binary_residual`` with the rounding for bf16 frames given explicitly: "compiled" or "eager"."""
    return _BinaryResidual.apply(spike_a, spike_b, rounding)


class _BinaryEncodeSTE(torch.autograd.Function):
    """Exact encode forward; backward averages the 16 frame gradients of a token."""

    @staticmethod
    def forward(ctx, continuous_btd):
        ctx.in_dtype = continuous_btd.dtype
        return fp16_encode(continuous_btd, 16)

    @staticmethod
    def backward(ctx, grad_output):
        dev = grad_output.device
        g = grad_output.contiguous()
        if g.dtype not in (torch.float32, torch.bfloat16, torch.float16):
            g = g.float()
        TK, B, D = g.shape
        out = torch.empty((B, TK // 16, D), dtype=g.dtype, device=dev)
        with torch.cuda.device(dev):
            _lib.check(_lib.lib().nsb_encode_ste_bwd(
                _lib.ptr(g), _lib.ptr(out), B, TK // 16, D, _lib.dtype_code(g.dtype),
                _lib.stream_ptr(dev)), "nsb_encode_ste_bwd")
        return out.to(ctx.in_dtype)


def binary_encode_ste(continuous_btd: torch.Tensor) -> torch.Tensor:
    return _BinaryEncodeSTE.apply(continuous_btd)
