"""Adaptive surrogate slope computed on the device (nsb_surrogate_alpha) and the backward entry
points that read it from device memory."""
import numpy as np
import pytest
import torch

import neuronspark_b200 as nsb
from neuronspark_b200 import parallel_scan as ps
from oracle import oracle as orc
from util import f32, rowparam_inputs

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {0: torch.float32, 1: torch.bfloat16, 2: torch.float16}
NAME = {torch.float32: "f32", torch.bfloat16: "bf16", torch.float16: "f16"}


class _Sigmoid:
    def __init__(self, alpha):
        self.alpha = alpha


_Sigmoid.__name__ = "Sigmoid"


@pytest.fixture(autouse=True)
def _reset():
    nsb.set_tuning()
    ps.CKPT_INTERVAL = None
    yield
    assert nsb.device_error_word() == 0


def test_golden(golden):
    """Against the numbers the reference's own lines produce (atomic_ops/plif_node.py:93-100)."""
    g = golden("surrogate_alpha")
    for i in range(int(g["n"])):
        dt = DT[int(g[f"dtype{i}"])]
        u = torch.as_tensor(g[f"u{i}"], device=DEV).to(dt)
        a = ps.adaptive_alpha(u, float(g["alpha_0"]), float(g["sigma_0"]))
        assert a.shape == () and a.dtype == torch.float32 and a.is_cuda
        want = float(g[f"alpha{i}"])
        assert abs(float(a) - want) <= 2e-6 * want, (i, float(a), want)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("n,offset", [(1 << 20, 0), (1 << 20, 1), (12345, 3), (7, 0), (1, 0), (0, 0)])
def test_vs_oracle(dtype, n, offset):
    g = torch.Generator(device=DEV).manual_seed(n + offset)
    buf = (torch.randn(n + offset, generator=g, device=DEV) * 0.21 + 0.05).to(dtype)
    u = buf[offset:]   # offset 1 / 3: not 16-byte aligned
    a = float(ps.adaptive_alpha(u, 4.0, 0.4))
    want = orc.surrogate_alpha(f32(u), 4.0, 0.4, NAME[dtype])
    assert abs(a - want) <= 2e-6 * want, (a, want)
    assert float(ps.adaptive_alpha(u, 4.0, 0.4)) == a   # fixed summation order


def test_rowparam_backward_reads_device_alpha():
    T, B, D = 64, 2, 96
    beta_row, u, vth_row, v0 = rowparam_inputs(T, B, D, torch.bfloat16, DEV)
    u = u * 3
    gS = (torch.randn(T, B, D, device=DEV) * 0.1).bfloat16()
    alpha_t = ps.adaptive_alpha(u, 4.0, 0.4)
    alpha_f = float(alpha_t)
    assert 1.0 < alpha_f < 20.0

    def grads(alpha):
        leaves = [t.clone().requires_grad_() for t in (beta_row, u, vth_row, v0)]
        s, _ = ps.plif_rowparam_forward_recompute(*leaves, alpha)
        s.backward(gS)
        return [t.grad for t in leaves]

    for a, b in zip(grads(alpha_t), grads(alpha_f)):
        assert torch.equal(a, b)
    other = grads(alpha_f * 1.5)
    assert not torch.equal(other[1], grads(alpha_f)[1])


def test_rf_backward_reads_device_alpha():
    T, B, D = 48, 2, 64
    g = torch.Generator(device=DEV).manual_seed(3)
    rn = lambda *s: torch.randn(*s, generator=g, device=DEV)
    beta = (0.9 * torch.sigmoid(rn(T, B, D))).bfloat16()
    omega = (0.2 * torch.abs(rn(T, B, D))).bfloat16()
    u, vth = rn(T, B, D).bfloat16(), (torch.abs(rn(T, B, D)) + 0.1).bfloat16()
    v0, w0 = rn(B, D), rn(B, D)
    gS = (rn(T, B, D) * 0.1).bfloat16()
    alpha_t = ps.adaptive_alpha(u, 4.0, 0.4)

    def grads(alpha):
        leaves = [t.clone().requires_grad_() for t in (beta, omega, u, vth, v0, w0)]
        s, _, _ = ps.rf_plif_parallel_forward_recompute(*leaves, surrogate_function=_Sigmoid(alpha))
        s.backward(gS)
        return [t.grad for t in leaves]

    for a, b in zip(grads(alpha_t), grads(float(alpha_t))):
        assert torch.equal(a, b)
