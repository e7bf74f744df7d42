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


# ------------------------------------------------------------ spikes packed in time
#
# The 16 frames of a token and channel as one int16 (the IEEE half bit pattern they spell,
# frame 0 = sign = bit 15): (S, B, D) patterns for (S*16, B, D) frames, 2 bytes per value instead
# of 16 elements. The reference moves dense frames between layers (atomic_ops/snn_block.py:281-285,
# atomic_ops/snn_ffn.py:188-195, model.py:155-157); these functions keep its arithmetic and change
# only the storage. Patterns are integers, so autograd does not flow through them: the backward
# pieces are plain functions for a caller that wires its own Function.


def _frame_dtype(dt: torch.dtype) -> torch.dtype:
    if dt not in (torch.float32, torch.bfloat16, torch.float16):
        raise NSBError(f"unsupported frame dtype {dt}")
    return dt


@torch.no_grad()
def pack_frames(frames: torch.Tensor) -> torch.Tensor:
    """(S*16, B, D) frames in {0,1} -> (S, B, D) int16 patterns."""
    dev = _lib.require_cuda(frames)
    if frames.dim() != 3 or frames.shape[0] % 16:
        raise NSBError("pack_frames expects (S*16, B, D)")
    f = frames.contiguous()
    _frame_dtype(f.dtype)
    TK, B, D = f.shape
    out = torch.empty((TK // 16, B, D), dtype=torch.int16, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().nsb_frames_pack(_lib.ptr(f), _lib.ptr(out), B, TK // 16, D, _lib.dtype_code(f.dtype),
                                              _lib.stream_ptr(dev)), "nsb_frames_pack")
    return out


def _patterns(p: torch.Tensor):
    dev = _lib.require_cuda(p)
    if p.dtype != torch.int16 or p.dim() != 3:
        raise NSBError("patterns are (S, B, D) int16")
    return dev, p.contiguous()


@torch.no_grad()
def unpack_frames(patterns: torch.Tensor, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """(S, B, D) int16 patterns -> (S*16, B, D) frames in {0,1} of ``dtype``."""
    dev, p = _patterns(patterns)
    S, B, D = p.shape
    out = torch.empty((S * 16, B, D), dtype=_frame_dtype(dtype), device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().nsb_frames_unpack(_lib.ptr(p), _lib.ptr(out), B, S, D, _lib.dtype_code(dtype),
                                                _lib.stream_ptr(dev)), "nsb_frames_unpack")
    return out


@torch.no_grad()
def fp16_decode_packed(patterns: torch.Tensor, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """``fp16_decode(unpack_frames(patterns, dtype), S)`` without the frames: (B, S, D) values."""
    dev, p = _patterns(patterns)
    S, B, D = p.shape
    out = torch.empty((B, S, D), dtype=_frame_dtype(dtype), device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().nsb_fp16_decode_packed_fwd(_lib.ptr(p), _lib.ptr(out), B, S, D, _lib.dtype_code(dtype),
                                                         _lib.stream_ptr(dev)), "nsb_fp16_decode_packed_fwd")
    return out


@torch.no_grad()
def fp16_decode_packed_backward(patterns: torch.Tensor, grad_values: torch.Tensor) -> torch.Tensor:
    """Gradient of the decode with respect to the 16 frames of every value: (B, S, D) value
    gradients -> (S*16, B, D) frame gradients in ``grad_values``' dtype."""
    dev, p = _patterns(patterns)
    S, B, D = p.shape
    g = grad_values.contiguous()
    if tuple(g.shape) != (B, S, D):
        raise NSBError(f"grad_values has shape {tuple(g.shape)}, expected {(B, S, D)}")
    out = torch.empty((S * 16, B, D), dtype=_frame_dtype(g.dtype), device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().nsb_fp16_decode_packed_bwd(_lib.ptr(p), _lib.ptr(g), _lib.ptr(out), B, S, D,
                                                         _lib.dtype_code(g.dtype), _lib.stream_ptr(dev)),
                   "nsb_fp16_decode_packed_bwd")
    return out


@torch.no_grad()
def binary_residual_packed(patterns_a: torch.Tensor, patterns_b: torch.Tensor,
                           frame_dtype: torch.dtype = torch.bfloat16, rounding=None) -> torch.Tensor:
    """``pack_frames(binary_residual(unpack(a), unpack(b)))`` on the patterns themselves; ``frame_dtype``
    names the frame dtype whose roundings apply (they matter for bfloat16 only)."""
    dev, a = _patterns(patterns_a)
    _, b = _patterns(patterns_b)
    if a.shape != b.shape:
        raise NSBError("pattern arrays of different shapes")
    out = torch.empty_like(a)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().nsb_binary_residual_packed(_lib.ptr(a), _lib.ptr(b), _lib.ptr(out), a.numel(),
                                                         _lib.dtype_code(_frame_dtype(frame_dtype)),
                                                         residual_rounding_code(rounding), _lib.stream_ptr(dev)),
                   "nsb_binary_residual_packed")
    return out
