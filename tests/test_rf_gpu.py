"""GPU parity of the resonate-and-fire (second-order) scan against the golden
vectors (reference's CPU loop) and the CPU oracle."""
import numpy as np
import pytest
import torch

import neuronspark_b200 as nsb
from neuronspark_b200 import parallel_scan as ps
from oracle import oracle as orc
from util import assert_close, assert_close_lowp, f32

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


class _Sigmoid:
    def __init__(self, alpha):
        self.alpha = alpha


_Sigmoid.__name__ = "Sigmoid"


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


def rf_inputs(T, B, D, dtype, seed):
    """The distribution of the reference's own check (test_recompute.py:87-101) with its
    stability rescale sqrt(beta^2+omega^2) <= 0.999."""
    g = torch.Generator(device=DEV).manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g, device=DEV)
    beta = torch.sigmoid(rn(T, B, D))
    omega = torch.abs(rn(T, B, D)) * 0.3
    r_sq = beta * beta + omega * omega
    scale = torch.where(r_sq > 0.999 ** 2, 0.999 * torch.rsqrt(r_sq.clamp(min=1e-12)), torch.ones_like(r_sq))
    beta, omega = (beta * scale).to(dtype), (omega * scale).to(dtype)
    u = rn(T, B, D).to(dtype)
    vth = (torch.abs(rn(T, B, D)) + 0.1).to(dtype)
    return beta, omega, u, vth, rn(B, D), rn(B, D)


def test_golden_rf(golden):
    g = golden("rf_a")
    names = ("beta", "omega", "u", "vth", "v_init", "w_init")
    ins = [cuda(g[k]).requires_grad_() for k in names]
    spike, vpost, w = ps.rf_plif_parallel_forward(*ins, _Sigmoid(float(g["alpha"])))
    assert np.array_equal(f32(spike), g["spike"])
    assert np.array_equal(f32(vpost), g["vpost"]) and np.array_equal(f32(w), g["w"])
    ((spike * cuda(g["g_spike"])).sum() + (vpost * cuda(g["g_vpost"])).sum()).backward()
    for t, k in zip(ins, ("g_beta", "g_omega", "g_u", "g_vth", "g_vinit", "g_winit")):
        assert_close(f32(t.grad), g[k], what=k)


def test_rf_recompute_and_materialising_variants_agree_bitwise():
    """test_recompute.py:80-152 of the reference: K=16, batch=2, dim=256, fp32, seed 42;
    torch.equal on spikes / V_last / W_last and zero tolerance on all six gradients."""
    base = rf_inputs(16, 2, 256, torch.float32, 42)
    a = [t.clone().requires_grad_() for t in base]
    b = [t.clone().requires_grad_() for t in base]
    s1, v1, w1 = ps.rf_plif_parallel_forward(*a, _Sigmoid(4.0))
    s1.sum().backward()
    s2, vl, wl = ps.rf_plif_parallel_forward_recompute(*b, _Sigmoid(4.0))
    s2.sum().backward()
    assert torch.equal(s1, s2) and torch.equal(v1[-1], vl) and torch.equal(w1[-1], wl)
    for x, y in zip(a, b):
        assert torch.equal(x.grad, y.grad)


@pytest.mark.parametrize("shape", [(1, 1, 1), (9, 2, 40), (33, 3, 33), (64, 2, 256), (130, 1, 520),
                                   (1024, 2, 768)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rf_vs_oracle(shape, dtype):
    T, B, D = shape
    beta, omega, u, vth, v0, w0 = rf_inputs(T, B, D, dtype, T + D)
    rs, rv, rw, rvl, rwl = orc.plif_rf_fwd(*(f32(t) for t in (beta, omega, u, vth, v0, w0)))
    ins = [t.requires_grad_() for t in (beta, omega, u, vth, v0, w0)]
    spike, vpost, w = ps.rf_plif_parallel_forward(*ins, _Sigmoid(4.0))
    assert np.array_equal(f32(spike), rs), "spikes must be bit-exact"
    if dtype == torch.float32:
        assert np.array_equal(f32(vpost), rv) and np.array_equal(f32(w), rw)
    else:
        assert_close_lowp(f32(vpost), rv, dtype, "V_post")
        assert_close_lowp(f32(w), rw, dtype, "W")
    g = torch.Generator(device=DEV).manual_seed(3)
    gS = torch.randn(T, B, D, generator=g, device=DEV).to(dtype)
    gV = (0.3 * torch.randn(T, B, D, generator=g, device=DEV)).to(dtype)
    ((spike.float() * gS.float()).sum() + (vpost.float() * gV.float()).sum()).backward()
    ref = orc.plif_rf_bwd(*(f32(t) for t in (beta, omega, u, vth, v0, w0)), f32(gS), f32(gV), 4.0)
    for t, e, n in zip(ins, ref, ("g_beta", "g_omega", "g_u", "g_vth", "g_vinit", "g_winit")):
        if n in ("g_vinit", "g_winit"):
            assert_close(f32(t.grad), e, what=n)
        else:
            assert_close_lowp(f32(t.grad), e, dtype, what=n)
    # recompute variant: same spikes, final states exact
    with torch.no_grad():
        s2, vl, wl = ps.rf_plif_parallel_forward_recompute(beta, omega, u, vth, v0, w0)
    assert torch.equal(s2, spike.detach())
    assert np.array_equal(f32(vl), rvl) and np.array_equal(f32(wl), rwl)


@pytest.mark.parametrize("lanes,stages,wpc", [(1, 2, 1), (2, 3, 2), (4, 2, 1)])
def test_rf_paths_agree(lanes, stages, wpc):
    ps.CKPT_INTERVAL = 8
    beta, omega, u, vth, v0, w0 = rf_inputs(70, 2, 384, torch.bfloat16, 9)
    nsb.set_tuning(force_direct=True)
    ref = ps.rf_plif_parallel_forward(beta, omega, u, vth, v0, w0)
    assert nsb.last_launch_info()["used_tma"] == 0
    nsb.set_tuning(warps_per_cta=wpc, stages=stages, lanes_per_thread=lanes)
    got = ps.rf_plif_parallel_forward(beta, omega, u, vth, v0, w0)
    assert nsb.last_launch_info()["used_tma"] == 1
    for a, b in zip(ref, got):
        assert torch.equal(a, b)
    # backward: the TMA path at this lane count against the direct path
    gS = torch.randn(70, 2, 384, device=DEV).bfloat16()
    grads = []
    for direct in (True, False):
        nsb.set_tuning(warps_per_cta=wpc, stages=stages, lanes_per_thread=lanes, force_direct=direct)
        ins = [t.clone().requires_grad_() for t in (beta, omega, u, vth, v0, w0)]
        s_, _, _ = ps.rf_plif_parallel_forward_recompute(*ins, _Sigmoid(4.0))
        s_.backward(gS)
        assert nsb.last_launch_info()["used_tma"] == (0 if direct else 1)
        grads.append([t.grad for t in ins])
    for a, b in zip(*grads):
        assert torch.equal(a, b)


def test_rf_with_zero_omega_is_the_first_order_scan():
    beta, omega, u, vth, v0, w0 = rf_inputs(40, 2, 128, torch.float32, 5)
    z = torch.zeros_like(omega)
    s1, v1, _ = ps.rf_plif_parallel_forward(beta, z, u, vth, v0, torch.zeros_like(w0))
    s2, v2, _ = ps.plif_parallel_forward(beta, u, vth, v0)
    assert torch.equal(s1, s2) and torch.equal(v1, v2)
