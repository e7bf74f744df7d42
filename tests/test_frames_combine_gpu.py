"""GPU parity of the expert merge in the frame domain (nsb_frames_combine_fwd / _bwd): frames
identical to the golden vectors made with the reference's fp16_decode / binary_encode_ste and to the
CPU oracle (which restates every rounding of the reference's tensor arithmetic); gradients to a
tolerance; agreement with the unfused sequence built from this package's own codec kernels."""
import numpy as np
import pytest
import torch

import neuronspark_b200 as nsb
from neuronspark_b200 import fp16_codec as codec
from neuronspark_b200 import moe_kernels as mk
from oracle import oracle as orc
from util import assert_close, f32

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
STORAGE = {torch.float32: "f32", torch.bfloat16: "bf16", torch.float16: "f16"}


def cuda(a, dtype):
    return torch.as_tensor(np.asarray(a), device=DEV).to(dtype)


def inputs(S, B, D, E, dtype, seed, top_k=2):
    """Frames of random values (spread over the half range, a few subnormal) and routing weights
    with E - top_k exact zeros per token, as scatter_add of top-k softmax weights leaves them."""
    g = torch.Generator(device=DEV).manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g, device=DEV)

    def frames(scale):
        vals = rn(B, S, D) * scale * torch.pow(10.0, torch.randint(-6, 2, (B, S, D), generator=g, device=DEV).float())
        return codec.fp16_encode(vals.to(dtype))

    shared, residual = frames(1.0), frames(2.0)
    experts = torch.stack([frames(0.7) for _ in range(E)]) if E else torch.zeros(0, S * 16, B, D, device=DEV, dtype=dtype)
    w = torch.rand(S, B, E, generator=g, device=DEV)
    if E > top_k:
        drop = torch.rand(S, B, E, generator=g, device=DEV).argsort(-1) >= top_k
        w = w.masked_fill(drop, 0.0)
    return shared, experts, w.to(dtype), residual


@pytest.mark.parametrize("tag,dtype", [("f32", torch.float32), ("bf16", torch.bfloat16)])
def test_golden(golden, tag, dtype):
    g = golden(f"frames_combine_{tag}")
    leaves = [cuda(g[k], dtype).requires_grad_() for k in ("shared", "experts", "weights", "residual")]
    out = mk.frames_combine(*leaves)
    assert out.dtype == dtype and np.array_equal(f32(out), g["out"])
    out.backward(cuda(g["g_out"], dtype))
    tol = 1e-5 if tag == "f32" else 2.0 ** -6  # the reference's bf16 autograd rounds every intermediate
    for t, k in zip(leaves, ("g_shared", "g_experts", "g_weights", "g_residual")):
        assert_close(f32(t.grad), g[k], tol, k)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(1, 1, 1, 1), (3, 2, 40, 4), (5, 3, 33, 2), (2, 2, 768, 8), (4, 1, 130, 0),
                                   (2, 3, 64, 16)])
def test_vs_oracle(dtype, shape):
    S, B, D, E = shape
    shared, experts, w, residual = inputs(S, B, D, E, dtype, 100 + D + E)
    leaves = [t.clone().requires_grad_() for t in (shared, experts, w, residual)]
    out = mk.frames_combine(*leaves)
    want, _ = orc.frames_combine_fwd(f32(shared), f32(experts), f32(w), f32(residual), storage=STORAGE[dtype])
    assert np.array_equal(f32(out), want), "frames must be identical"
    g_out = (torch.randn(S * 16, B, D, device=DEV) * 0.1).to(dtype)
    out.backward(g_out)
    gs, ge, gw, gr = orc.frames_combine_bwd(f32(g_out), f32(shared), f32(experts), f32(w), f32(residual),
                                            storage=STORAGE[dtype])
    tol = 1e-5 if dtype == torch.float32 else 2.0 ** -7
    assert_close(f32(leaves[0].grad), gs, tol, "g_shared")
    assert_close(f32(leaves[3].grad), gr, tol, "g_residual")
    if E:
        assert_close(f32(leaves[1].grad), ge, tol, "g_experts")
        assert_close(f32(leaves[2].grad), gw, tol, "g_weights")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_equals_the_unfused_sequence(dtype):
    """decode every stream, weighted sum, add, add, encode - with this package's codec kernels and
    torch arithmetic on the GPU. torch may associate the sum over experts differently, so a frame
    may differ where that moves a rounding: at most 1 value in 1000."""
    S, B, D, E = 8, 4, 256, 4
    shared, experts, w, residual = inputs(S, B, D, E, dtype, 7)
    out = mk.frames_combine(shared, experts, w, residual)
    vals = torch.stack([codec.fp16_decode(experts[e], S) for e in range(E)])
    total = codec.fp16_decode(shared, S) + (vals * w.permute(2, 1, 0).unsqueeze(-1)).sum(0)
    total = total + codec.fp16_decode(residual, S)
    ref = codec.fp16_encode(total)
    same = (out.view(S, 16, B, D) == ref.view(S, 16, B, D)).all(1)
    assert float(same.float().mean()) > 0.999
    assert_close(f32(codec.fp16_decode(out, S)), f32(codec.fp16_decode(ref, S)), 2.0 ** -7, "decoded")


def test_deterministic_and_partial_grads():
    S, B, D, E = 4, 2, 768, 4
    shared, experts, w, residual = inputs(S, B, D, E, torch.bfloat16, 9)
    g_out = (torch.randn(S * 16, B, D, device=DEV) * 0.1).bfloat16()

    def grads(needs):
        leaves = [t.clone().requires_grad_(n) for t, n in zip((shared, experts, w, residual), needs)]
        mk.frames_combine(*leaves).backward(g_out)
        return [t.grad for t in leaves]

    a, b = grads((True,) * 4), grads((True,) * 4)
    assert all(torch.equal(x, y) for x, y in zip(a, b))
    only_w = grads((False, False, True, False))
    assert only_w[0] is None and only_w[1] is None and torch.equal(only_w[2], a[2])
    only_e = grads((False, True, False, False))
    assert torch.equal(only_e[1], a[1])


def test_unaligned_and_arguments():
    S, B, D, E = 2, 2, 66, 2
    shared, experts, w, residual = inputs(S, B, D, E, torch.bfloat16, 3)
    buf = torch.zeros(shared.numel() + 1, device=DEV, dtype=torch.bfloat16)
    odd = buf[1:].view_as(shared)
    odd.copy_(shared)                                     # 2-byte aligned only
    assert torch.equal(mk.frames_combine(odd, experts, w, residual), mk.frames_combine(shared, experts, w, residual))
    with pytest.raises(nsb.NSBError):
        mk.frames_combine(shared, experts, w[:1], residual)
    with pytest.raises(nsb.NSBError):
        mk.frames_combine(shared[:17], experts[:, :17], w, residual[:17])
    empty = mk.frames_combine(shared[:0], experts[:, :0], w[:0], residual[:0])
    assert empty.shape == (0, B, D)
