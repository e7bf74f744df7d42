"""Backward scans whose time axis is cut into chunks that different CTAs walk, chained through the
per-column outputs (nsb_set_chain_chunks): every gradient equals the unchained launch's bit for bit,
for every scan family that takes the scratch, with ragged T and with more chunks than CTAs can hold."""
import pytest
import torch

import neuronspark_b200 as nsb
from neuronspark_b200 import _lib, parallel_scan as ps, snn_block as sb
from util import selective_inputs

from test_modulated_gpu import _Sigmoid, mod_inputs
from test_rf_gpu import rf_inputs

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)


@pytest.fixture(autouse=True)
def _clean(monkeypatch):
    # the Python layer hands out the scratch only for scans that can exceed the GPU; here every scan gets it
    monkeypatch.setattr(ps, "CHAIN_MIN_COLS", 0)
    monkeypatch.setattr(ps, "CHAIN_MIN_STEPS", 0)
    nsb.set_tuning()
    _lib.set_chain_chunks()
    ps.CKPT_INTERVAL = None
    yield
    nsb.set_tuning()
    _lib.set_chain_chunks()
    ps.CKPT_INTERVAL = None
    assert nsb.device_error_word() == 0


def grads_of(fn, leaves, g_out, chunks):
    _lib.set_chain_chunks(chunks)
    ins = [t.clone().requires_grad_() for t in leaves]
    out = fn(*ins)
    out.backward(g_out)
    torch.cuda.synchronize()
    assert _lib.last_chain_chunks() == chunks, (_lib.last_chain_chunks(), chunks)
    return [t.grad for t in ins]


def check(fn, leaves, g_out, chunk_counts):
    ref = grads_of(fn, leaves, g_out, 1)
    for q in chunk_counts:
        got = grads_of(fn, leaves, g_out, q)
        for i, (a, b) in enumerate(zip(ref, got)):
            assert torch.equal(a, b), (q, i, float((a.float() - b.float()).abs().max()))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("shape", [(256, 2, 512), (203, 3, 200)])
def test_selective_scan_chained_equals_unchained(dtype, shape):
    T, B, D = shape
    beta, cur, gain, vth, v0 = selective_inputs(T, B, D, dtype, DEV, seed=3, zero_init=False)
    gS = (torch.randn(T, B, D, device=DEV) * 0.1).to(dtype)
    ps.CKPT_INTERVAL = 8
    # u-form (three streams) and gain*cur form (four streams)
    check(lambda b, u, th, v: ps.plif_parallel_forward(b, u, th, v, surrogate_function=_Sigmoid(4.0))[0],
          [beta, cur, vth, v0], gS, (2, 3, 7))
    check(lambda b, c, g, th, v: ps.plif_selective_scan_ai(b, c, g, th, v, 2.0, "atan")[0],
          [beta, cur, gain, vth, v0], gS, (2, 5))

    # with a gradient arriving through V_post as well (one more streamed input in the backward)
    def spike_and_vpost(b, u, th, v):
        s, vp, _ = ps.plif_parallel_forward(b, u, th, v, surrogate_function=_Sigmoid(4.0))
        return s + 0.5 * vp

    check(spike_and_vpost, [beta, cur, vth, v0], gS, (3,))


@pytest.mark.parametrize("lanes", [1, 2])
def test_resonate_and_fire_chained_equals_unchained(lanes):
    T, B, D = 180, 2, 384
    beta, omega, u, vth, v0, w0 = rf_inputs(T, B, D, torch.bfloat16, 11)
    gS = (torch.randn(T, B, D, device=DEV) * 0.1).bfloat16()
    ps.CKPT_INTERVAL = 8
    nsb.set_tuning(lanes_per_thread=lanes)
    check(lambda *a: ps.rf_plif_parallel_forward_recompute(*a, _Sigmoid(4.0))[0],
          [beta, omega, u, vth, v0, w0], gS, (2, 4))


@pytest.mark.parametrize("rf", [False, True])
@pytest.mark.parametrize("lanes", [1, 2])
def test_modulated_scans_chained_equal_unchained(rf, lanes):
    T, B, D = 150, 2, 264
    d, b, v0, w0 = mod_inputs(T, B, D, torch.bfloat16, 17, rf)
    gS = (torch.randn(T, B, D, device=DEV) * 0.1).bfloat16()
    names = list(d) + list(b)
    leaves = [d[k] for k in d] + [b[k] for k in b] + [v0] + ([w0] if rf else [])
    ps.CKPT_INTERVAL = 8
    nsb.set_tuning(lanes_per_thread=lanes)

    def fn(*a):
        dd = dict(zip(names, a[:len(names)]))
        rest = a[len(names):]
        args = (dd["raw_beta"], dd["b_beta"], dd["raw_alpha"], dd["b_alpha"], dd["raw_th"], dd["b_th"], 0.1, dd["cur"])
        if rf:
            return sb.modulated_rf_plif_forward(*args, dd["raw_omega"], dd["b_omega"], rest[0], rest[1],
                                                _Sigmoid(4.0))[0]
        return sb.modulated_plif_forward(*args, rest[0], _Sigmoid(4.0))[0]

    check(fn, leaves, gS, (2, 3))


def test_automatic_choice_needs_more_ctas_than_the_gpu_holds():
    """A launch that fits the GPU is not chained (the full-size test covers one that does not fit)."""
    T, B, D = 256, 2, 512
    beta, cur, gain, vth, v0 = selective_inputs(T, B, D, torch.bfloat16, DEV, seed=5)
    ins = [t.clone().requires_grad_() for t in (beta, cur, vth, v0)]
    s, _, _ = ps.plif_parallel_forward(*ins, surrogate_function=_Sigmoid(4.0))
    s.backward(torch.ones_like(s))
    torch.cuda.synchronize()
    assert _lib.last_chain_chunks() == 1


def test_rowparam_and_linear_recurrence_chained_equal_unchained():
    """The row-parameter backward takes the counters from its split scratch, the linear recurrence from
    its own argument; both chained launches equal the unchained ones bit for bit."""
    from util import rowparam_inputs
    T, B, D = 192, 2, 640
    br, u, tr, v0 = rowparam_inputs(T, B, D, torch.bfloat16, DEV, seed=23)
    gS = (torch.randn(T, B, D, device=DEV) * 0.1).bfloat16()
    nsb.set_time_split(1)  # (few columns: without this the scan would be split, not chained)
    try:
        check(lambda *a: ps.plif_rowparam_forward_recompute(*a, 4.0)[0], [br, u, tr, v0], gS, (2, 3))
    finally:
        nsb.set_time_split()
    ps.CKPT_INTERVAL = 8
    beta = torch.sigmoid(torch.randn(T, B, D, device=DEV) + 2).bfloat16()
    check(lambda b, x, v: ps.linear_recurrence(b, x, v), [beta, u, v0], gS, (2, 5))
