"""GPU parity of the linear recurrence V[k] = beta[k]*V[k-1] + u[k] against the golden vectors
(reference's `linear_recurrence` + autograd) and the CPU oracle."""
import numpy as np
import pytest
import torch

import neuronspark_b200 as nsb
from neuronspark_b200 import parallel_scan as ps
from oracle import oracle as orc
from util import assert_close, assert_close_lowp, f32

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(autouse=True)
def _reset():
    nsb.set_tuning()
    ps.CKPT_INTERVAL = None
    yield
    nsb.set_tuning()
    ps.CKPT_INTERVAL = None
    assert nsb.device_error_word() == 0


def cuda(a, dtype=torch.float32):
    return torch.as_tensor(np.asarray(a), device=DEV).to(dtype)


def inputs(T, B, D, dtype, seed):
    g = torch.Generator(device=DEV).manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g, device=DEV)
    return torch.sigmoid(rn(T, B, D) + 1.0).to(dtype), rn(T, B, D).to(dtype), rn(B, D)


def test_golden(golden):
    g = golden("linrec_a")
    leaves = [cuda(g[k]).requires_grad_() for k in ("beta", "u", "v_init")]
    V = ps.linear_recurrence(*leaves)
    assert_close(f32(V), g["V"], 1e-5, "V")
    V.backward(cuda(g["g_V"]))
    for t, k in zip(leaves, ("g_beta", "g_u", "g_vinit")):
        assert_close(f32(t.grad), g[k], 1e-5, k)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(1, 1, 1), (9, 2, 31), (100, 3, 40), (130, 1, 1536), (33, 2, 99)])
def test_vs_oracle(dtype, shape):
    T, B, D = shape
    beta, u, v0 = inputs(T, B, D, dtype, 5)
    leaves = [t.clone().requires_grad_() for t in (beta, u, v0)]
    V = ps.linear_recurrence(*leaves)
    want = orc.linear_recurrence_fwd(f32(beta), f32(u), f32(v0))
    if dtype == torch.float32:
        assert np.array_equal(f32(V), want)   # same rounded multiply, same rounded add
    else:
        assert torch.equal(V, torch.as_tensor(want, device=DEV).to(dtype))  # the fp32 state rounded once
    gV = torch.randn(T, B, D, device=DEV).to(dtype)
    V.backward(gV)
    gb, gu, gv0 = orc.linear_recurrence_bwd(f32(beta), f32(u), f32(v0), f32(gV))
    for t, w, name in zip(leaves, (gb, gu, gv0), ("g_beta", "g_u", "g_vinit")):
        if t.grad.dtype == torch.float32:
            assert_close(f32(t.grad), w, 1e-5, name)
        else:
            assert_close_lowp(f32(t.grad), w, dtype, name)


@pytest.mark.parametrize("tile", [8, 32])
@pytest.mark.parametrize("lanes,direct", [(1, 0), (2, 0), (4, 0), (0, 1)])
def test_every_instantiation(tile, lanes, direct):
    if tile == 32 and lanes > 1:
        pytest.skip("32-step tiles are built for 1 lane per thread")
    T, B, D = 70, 2, 520
    beta, u, v0 = inputs(T, B, D, torch.bfloat16, 7)
    want = torch.as_tensor(orc.linear_recurrence_fwd(f32(beta), f32(u), f32(v0)), device=DEV).bfloat16()
    gV = torch.randn(T, B, D, device=DEV).bfloat16()
    gb, gu, gv0 = orc.linear_recurrence_bwd(f32(beta), f32(u), f32(v0), f32(gV))
    ps.CKPT_INTERVAL = tile
    nsb.set_tuning(lanes_per_thread=lanes, force_direct=direct)
    leaves = [t.clone().requires_grad_() for t in (beta, u, v0)]
    V = ps.linear_recurrence(*leaves)
    info = nsb.last_launch_info()
    assert info["tile_steps"] == tile and info["used_tma"] == (0 if direct else 1)
    assert torch.equal(V, want)
    V.backward(gV)
    assert_close_lowp(f32(leaves[0].grad), gb, torch.bfloat16, "g_beta")
    assert_close_lowp(f32(leaves[1].grad), gu, torch.bfloat16, "g_u")
    assert_close(f32(leaves[2].grad), gv0, 1e-5, "g_vinit")


def test_edges():
    beta, u, v0 = inputs(0, 2, 64, torch.bfloat16, 1)
    assert ps.linear_recurrence(beta, u, v0).shape == (0, 2, 64)
    with torch.no_grad():   # no checkpoints are written when nothing needs a gradient
        beta, u, v0 = inputs(20, 2, 64, torch.float32, 2)
        V = ps.linear_recurrence(beta, u, v0)
        assert np.array_equal(f32(V), orc.linear_recurrence_fwd(f32(beta), f32(u), f32(v0)))
