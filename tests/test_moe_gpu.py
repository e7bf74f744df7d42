"""GPU parity of the MoE output combine against the golden vectors (reference's `moe_combine` +
autograd) and the CPU oracle."""
import numpy as np
import pytest
import torch

import neuronspark_b200 as nsb
from neuronspark_b200 import moe_kernels as mk
from oracle import oracle as orc
from util import assert_close, assert_close_lowp, f32

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def cuda(a, dtype=torch.float32):
    return torch.as_tensor(np.asarray(a), device=DEV).to(dtype)


def test_golden(golden):
    g = golden("moe_a")
    leaves = [cuda(g[k]).requires_grad_() for k in ("shared", "experts", "weights")]
    out = mk.moe_combine(*leaves)
    assert_close(f32(out), g["out"], 1e-5, "out")
    out.backward(cuda(g["g_out"]))
    for t, k in zip(leaves, ("g_shared", "g_experts", "g_weights")):
        assert_close(f32(t.grad), g[k], 1e-5, k)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(1, 1, 1), (4, 33, 40), (8, 100, 768), (3, 7, 1001), (16, 5, 256)])
def test_vs_oracle(dtype, shape):
    E, N, D = shape
    g = torch.Generator(device=DEV).manual_seed(E * 1000 + N)
    rn = lambda *s: torch.randn(*s, generator=g, device=DEV)
    shared, experts = rn(N, D).to(dtype), rn(E, N, D).to(dtype)
    weights = torch.softmax(rn(N, E), -1)
    leaves = [t.clone().requires_grad_() for t in (shared, experts, weights)]
    out = mk.moe_combine(*leaves)
    want = orc.moe_combine_fwd(f32(shared), f32(experts), f32(weights))
    assert out.dtype == dtype
    assert_close_lowp(f32(out), want, dtype, "out")
    g_out = rn(N, D).to(dtype)
    out.backward(g_out)
    ge, gw = orc.moe_combine_bwd(f32(g_out), f32(experts), f32(weights))
    assert torch.equal(leaves[0].grad, g_out)
    assert_close_lowp(f32(leaves[1].grad), ge, dtype, "g_experts")
    assert_close(f32(leaves[2].grad), gw, 1e-5, "g_weights")


def test_unaligned_and_partial_grads():
    E, N, D = 3, 9, 130
    buf = torch.randn(E * N * D + 1, device=DEV).bfloat16()
    experts = buf[1:].view(E, N, D)                      # 2-byte aligned only
    shared = torch.randn(N, D, device=DEV).bfloat16()
    weights = torch.rand(N, E, device=DEV)
    out = mk.moe_combine(shared, experts, weights)
    assert_close_lowp(f32(out), orc.moe_combine_fwd(f32(shared), f32(experts), f32(weights)), torch.bfloat16, "out")
    w = weights.clone().requires_grad_()                 # only the weights need a gradient
    mk.moe_combine(shared, experts, w).sum().backward()
    _, gw = orc.moe_combine_bwd(np.ones((N, D), np.float32), f32(experts), f32(weights))
    assert_close(f32(w.grad), gw, 1e-5, "g_weights")
    with pytest.raises(nsb.NSBError):
        mk.moe_combine(shared, experts, weights[:, :2])
