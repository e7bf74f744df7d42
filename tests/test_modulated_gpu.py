"""GPU parity of the modulation and of the scans with the modulation fused in.

Three links:
 1. the stand-alone modulation kernel against the CPU oracle (which is pinned to the
    reference's functions by golden vectors): beta within 1e-6 relative, alpha*I and omega within
    1e-6 relative or 3e-7 absolute (hardware exp / log / reciprocal / rsqrt), v_th exact;
 2. the fused scan against [stand-alone modulation (fp32 outputs) -> plain scan on those
    fp32 tensors]: BIT-EXACT, at every size, because both evaluate the same device
    functions and the same scan arithmetic;
 3. the fused scan against the oracle end to end: spikes equal except lanes that come within
    1e-4 * V_th of the threshold (a 1e-6 error on beta moves V by up to beta/(1-beta) times
    that), gradients to 2e-5 of the largest on the lanes whose spikes agree.
"""
import numpy as np
import pytest
import torch

import neuronspark_b200 as nsb
from neuronspark_b200 import parallel_scan as ps
from neuronspark_b200 import snn_block as sb
from oracle import oracle as orc
from util import assert_close, assert_spikes_match, f32

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
V_TH_MIN = 0.1


class _Sigmoid:
    def __init__(self, alpha):
        self.alpha = alpha


_Sigmoid.__name__ = "Sigmoid"


class _ATan:
    def __init__(self, alpha):
        self.alpha = alpha


_ATan.__name__ = "ATan"


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


def mod_inputs(T, B, D, dtype, seed, rf):
    """Raw projections as a trained block produces them (unit-scale activations), biases with
    the reference's initial means (b_beta ~ 2 so that beta ~ 0.88; omega small); every so
    often a large raw_omega so that the stability rescale is active."""
    g = torch.Generator(device=DEV).manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g, device=DEV)
    d = {"raw_beta": rn(T, B, D), "raw_alpha": rn(T, B, D), "raw_th": rn(T, B, D) * 0.5, "cur": rn(T, B, D)}
    if rf:
        ro = rn(T, B, D) - 1.0
        ro = torch.where(torch.rand(T, B, D, generator=g, device=DEV) < 0.05, ro + 3.0, ro)
        d["raw_omega"] = ro
    d = {k: v.to(dtype) for k, v in d.items()}
    b = {"b_beta": 2.0 + 0.5 * rn(D), "b_alpha": 0.3 * rn(D), "b_th": 0.3 * rn(D)}
    if rf:
        b["b_omega"] = -1.0 + 0.5 * rn(D)
    v0 = 0.1 * rn(B, D)
    w0 = 0.1 * rn(B, D) if rf else None
    return d, b, v0, w0


def oracle_mod(d, b, rf):
    extra = dict(raw_omega=f32(d["raw_omega"]), b_omega=f32(b["b_omega"])) if rf else {}
    return orc.modulation_fwd(f32(d["raw_beta"]), f32(d["raw_alpha"]), f32(d["raw_th"]), f32(d["cur"]),
                              f32(b["b_beta"]), f32(b["b_alpha"]), f32(b["b_th"]), V_TH_MIN, **extra)


def run_modulation(d, b, rf, out_dtype=None):
    if rf:
        return sb._fused_modulation_rf(d["raw_beta"], b["b_beta"], d["raw_alpha"], b["b_alpha"], d["raw_th"],
                                       b["b_th"], V_TH_MIN, d["cur"], d["raw_omega"], b["b_omega"],
                                       out_dtype=out_dtype)
    return sb._fused_modulation(d["raw_beta"], b["b_beta"], d["raw_alpha"], b["b_alpha"], d["raw_th"],
                                b["b_th"], V_TH_MIN, d["cur"], out_dtype=out_dtype)


def run_fused(d, b, v0, w0, rf, surrogate=None):
    if rf:
        return sb.modulated_rf_plif_forward(d["raw_beta"], b["b_beta"], d["raw_alpha"], b["b_alpha"],
                                            d["raw_th"], b["b_th"], V_TH_MIN, d["cur"], d["raw_omega"],
                                            b["b_omega"], v0, w0, surrogate)
    s, vl = sb.modulated_plif_forward(d["raw_beta"], b["b_beta"], d["raw_alpha"], b["b_alpha"], d["raw_th"],
                                      b["b_th"], V_TH_MIN, d["cur"], v0, surrogate)
    return s, vl, None


def run_unfused(d, b, v0, w0, rf):
    """Stand-alone modulation (fp32) followed by the plain scan kernels on fp32 streams."""
    mod = run_modulation(d, b, rf)
    if rf:
        beta, u, vth, omega = mod
        s, vl, wl = ps.rf_plif_parallel_forward_recompute(beta, omega, u, vth, v0, w0)
        return s, vl, wl
    beta, u, vth = mod
    s, vpost, _ = ps.plif_parallel_forward(beta, u, vth, v0)
    return s, vpost[-1], None


def rel(a, e):
    a, e = np.asarray(a, np.float64), np.asarray(e, np.float64)
    return np.abs(a - e) / np.maximum(np.abs(e), 1e-30)


# ------------------------------------------------------------ 1. modulation vs oracle


@pytest.mark.parametrize("name", ["modulation_rf", "modulation_first_order"])
def test_modulation_golden(golden, name):
    """On the golden inputs (which include saturated sigmoids, the softplus threshold and both
    sides of the stability rescale) against the reference's own outputs."""
    g = golden(name)
    rf = "raw_omega" in g
    d = {k: cuda(g[k]) for k in ("raw_beta", "raw_alpha", "raw_th", "cur") + (("raw_omega",) if rf else ())}
    b = {k: cuda(g[k]) for k in ("b_beta", "b_alpha", "b_th") + (("b_omega",) if rf else ())}
    out = run_modulation(d, b, rf)
    for mine, ref in zip(out, ("beta", "u", "vth", "omega")):
        mine, want = f32(mine), g[ref]
        if ref == "vth":
            assert np.array_equal(mine, want)
            continue
        # 2e-6 relative; the softplus outputs (alpha inside u, omega) also 3e-7 absolute (times |I| for
        # u); beta 1e-37 absolute where the reference's value is a subnormal / zero
        floor = {"beta": 1e-37, "omega": 3e-7}.get(ref, 3e-7 * np.abs(g["cur"]).astype(np.float64))
        bad = (rel(mine, want) > 2e-6) & (np.abs(mine.astype(np.float64) - want) > floor)
        assert not bad.any(), (ref, rel(mine, want).max())


@pytest.mark.parametrize("rf", [False, True])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_modulation_vs_oracle(rf, dtype):
    d, b, _, _ = mod_inputs(64, 3, 200, dtype, 5, rf)
    out = run_modulation(d, b, rf)
    want = oracle_mod(d, b, rf)
    for i, (mine, ref) in enumerate(zip(out, want)):
        if i == 2:
            assert np.array_equal(f32(mine), ref)
        else:
            floor = 0.0 if i == 0 else (3e-7 * np.abs(f32(d["cur"])) if i == 1 else 3e-7)
            err = np.abs(f32(mine).astype(np.float64) - ref)
            assert (err <= 1e-6 * np.abs(ref) + floor).all(), (i, rel(f32(mine), ref).max())
    if dtype != torch.float32:  # low-precision outputs are the fp32 values rounded once
        low = run_modulation(d, b, rf, out_dtype=dtype)
        for a, c in zip(out, low):
            assert torch.equal(a.to(dtype), c)


def test_modulation_is_forward_only():
    d, b, _, _ = mod_inputs(8, 1, 64, torch.float32, 1, False)
    d["raw_beta"].requires_grad_()
    with pytest.raises(nsb.NSBError):
        run_modulation(d, b, False)


# -------------------------------------- 2. fused scan == modulation kernel + plain scan


SHAPES = [(64, 2, 96), (37, 3, 40), (256, 1, 2048), (16, 4, 776)]


@pytest.mark.parametrize("rf", [False, True])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", SHAPES)
def test_fused_forward_bit_exact(rf, dtype, shape):
    T, B, D = shape
    d, b, v0, w0 = mod_inputs(T, B, D, dtype, 11, rf)
    s, vl, wl = run_fused(d, b, v0, w0, rf)
    s2, vl2, wl2 = run_unfused(d, b, v0, w0, rf)
    assert s.dtype == dtype and torch.equal(s.float(), s2.float())
    assert torch.equal(vl, vl2)
    if rf:
        assert torch.equal(wl, wl2)
    assert 0.01 < float(s.float().mean()) < 0.9


@pytest.mark.parametrize("rf", [False, True])
@pytest.mark.parametrize("tile", [8, 32])
@pytest.mark.parametrize("lanes,direct", [(1, 0), (2, 0), (4, 0), (0, 1)])
def test_fused_forward_variants(rf, tile, lanes, direct):
    """Every kernel instantiation (lanes per thread, tile length, the non-TMA path) gives the
    same bits."""
    if tile == 32 and lanes > 1:
        pytest.skip("32-step tiles are built for 1 lane per thread")
    T, B, D = 100, 2, 520
    d, b, v0, w0 = mod_inputs(T, B, D, torch.bfloat16, 21, rf)
    ref = run_unfused(d, b, v0, w0, rf)
    ps.CKPT_INTERVAL = tile
    nsb.set_tuning(lanes_per_thread=lanes, force_direct=direct)
    s, vl, wl = run_fused(d, b, v0, w0, rf)
    info = nsb.last_launch_info()
    assert info["tile_steps"] == tile and info["used_tma"] == (0 if direct else 1)
    if lanes:
        assert info["lanes_per_thread"] == lanes
    assert torch.equal(s.float(), ref[0].float()) and torch.equal(vl, ref[1])
    if rf:
        assert torch.equal(wl, ref[2])


# ---------------------------------------------------- 3. fused scan vs oracle, end to end


@pytest.mark.parametrize("rf", [False, True])
def test_fused_forward_vs_oracle(rf):
    T, B, D = 128, 2, 256
    d, b, v0, w0 = mod_inputs(T, B, D, torch.float32, 31, rf)
    s, vl, wl = run_fused(d, b, v0, w0, rf)
    mod = oracle_mod(d, b, rf)
    if rf:
        beta, u, vth, omega = mod
        so, vpo, _, vlo, wlo = orc.plif_rf_fwd(beta, omega, u, vth, f32(v0), f32(w0))
    else:
        beta, u, vth = mod
        so, vpo, vlo = orc.plif_selective_fwd(beta, u, vth, f32(v0))
    n_amb = assert_spikes_match(f32(s), so, vpo, vth, "fused spikes", margin=1e-4)
    assert n_amb <= 0.002 * B * D
    same = (f32(s) == so).all(0).reshape(-1)
    assert same.mean() > 0.995
    assert_close(f32(vl).reshape(-1)[same], vlo.reshape(-1)[same], 1e-4, "V_last")
    if rf:
        assert_close(f32(wl).reshape(-1)[same], wlo.reshape(-1)[same], 1e-4, "W_last")


def _oracle_grads(d, b, v0, w0, gS, alpha, kind, rf):
    """Scan adjoint (oracle, double) on the modulated values THE KERNEL computes - so that both
    sides see the same spikes - followed by the oracle's modulation adjoint."""
    mod = run_modulation(d, b, rf)
    raws = {k: f32(v) for k, v in d.items()}
    bias = {k: f32(v) for k, v in b.items()}
    if rf:
        beta, u, vth, omega = (f32(t) for t in mod)
        gb, go, gu, gt, gv, gw = orc.plif_rf_bwd(beta, omega, u, vth, f32(v0), f32(w0), f32(gS), None, alpha, kind)
        out = orc.modulation_bwd(raws["raw_beta"], raws["raw_alpha"], raws["raw_th"], raws["cur"], bias["b_beta"],
                                 bias["b_alpha"], bias["b_th"], gb, gu, gt, raws["raw_omega"], bias["b_omega"], go)
        out["v_init"], out["w_init"] = gv, gw
        return out
    beta, u, vth = (f32(t) for t in mod)
    gb, gu, gt, gv = orc.plif_selective_bwd(beta, u, vth, f32(v0), f32(gS), None, alpha, kind)
    out = orc.modulation_bwd(raws["raw_beta"], raws["raw_alpha"], raws["raw_th"], raws["cur"], bias["b_beta"],
                             bias["b_alpha"], bias["b_th"], gb, gu, gt)
    out["v_init"] = gv
    return out


def _fused_grads(d, b, v0, w0, gS, surrogate, rf):
    leaves = {k: v.clone().requires_grad_() for k, v in {**d, **b}.items()}
    v0l = v0.clone().requires_grad_()
    w0l = w0.clone().requires_grad_() if rf else None
    s, _, _ = run_fused({k: leaves[k] for k in d}, {k: leaves[k] for k in b}, v0l, w0l, rf, surrogate)
    s.backward(gS)
    out = {k: leaves[k].grad for k in leaves}
    out["v_init"] = v0l.grad
    if rf:
        out["w_init"] = w0l.grad
    return out


@pytest.mark.parametrize("rf", [False, True])
@pytest.mark.parametrize("surr", ["sigmoid", "atan"])
@pytest.mark.parametrize("shape", [(64, 2, 96), (100, 3, 264)])
def test_fused_backward_vs_oracle(rf, surr, shape):
    T, B, D = shape
    d, b, v0, w0 = mod_inputs(T, B, D, torch.float32, 41, rf)
    gS = torch.randn(T, B, D, device=DEV) * 0.1
    surrogate = _Sigmoid(4.0) if surr == "sigmoid" else _ATan(2.0)
    kind = orc.SURR_SIGMOID if surr == "sigmoid" else orc.SURR_ATAN
    mine = _fused_grads(d, b, v0, w0, gS, surrogate, rf)
    want = _oracle_grads(d, b, v0, w0, gS, surrogate.alpha, kind, rf)
    names = {"raw_beta": "raw_beta", "raw_alpha": "raw_alpha", "raw_th": "raw_th", "cur": "cur",
             "b_beta": "b_beta", "b_alpha": "b_alpha", "b_th": "b_th", "v_init": "v_init"}
    if rf:
        names.update(raw_omega="raw_omega", b_omega="b_omega", w_init="w_init")
    for k in names:
        tol = 1e-4 if k.startswith("b_") else 2e-5  # bias sums run over T*B terms in fp32
        assert_close(f32(mine[k]).reshape(-1), np.asarray(want[k], np.float64).reshape(-1), tol, k)


@pytest.mark.parametrize("rf", [False, True])
@pytest.mark.parametrize("tile", [8, 32])
@pytest.mark.parametrize("lanes,direct", [(1, 0), (2, 0), (4, 0), (0, 1)])
def test_fused_backward_variants(rf, tile, lanes, direct):
    if tile == 32 and lanes > 1:
        pytest.skip("32-step tiles are built for 1 lane per thread")
    T, B, D = 70, 2, 520
    d, b, v0, w0 = mod_inputs(T, B, D, torch.bfloat16, 51, rf)
    gS = (torch.randn(T, B, D, device=DEV) * 0.1).bfloat16()
    want = _oracle_grads(d, b, v0, w0, gS, 4.0, orc.SURR_SIGMOID, rf)
    ps.CKPT_INTERVAL = tile
    nsb.set_tuning(lanes_per_thread=lanes, force_direct=direct)
    mine = _fused_grads(d, b, v0, w0, gS, _Sigmoid(4.0), rf)
    info = nsb.last_launch_info()
    assert info["tile_steps"] == tile and info["used_tma"] == (0 if direct else 1)
    for k, w in want.items():
        if w is None:
            continue
        w = np.asarray(w, np.float64).reshape(-1)
        a = f32(mine[k]).reshape(-1)
        if mine[k].dtype == torch.bfloat16:
            bound = 2.0 ** -8 * np.abs(w) + 2e-5 * np.abs(w).max()
            assert (np.abs(a - w) <= bound).all(), k
        else:
            assert_close(a, w, 1e-4 if k.startswith("b_") else 2e-5, k)


@pytest.mark.parametrize("rf", [False, True])
def test_fused_backward_launch_shapes(rf):
    """The 2-lane backward kernels run as pairs of warps on one TMA box: any CTA size (odd requests
    are rounded up to whole pairs) and ring depth gives the same bits, also where the last box is
    only partly inside the tensor (1040 = 8 boxes of 128 columns + 16) and the last tile is short."""
    T, B, D = 70, 2, 520
    d, b, v0, w0 = mod_inputs(T, B, D, torch.bfloat16, 61, rf)
    gS = (torch.randn(T, B, D, device=DEV) * 0.1).bfloat16()
    ps.CKPT_INTERVAL = 8
    nsb.set_tuning(lanes_per_thread=2)
    base = _fused_grads(d, b, v0, w0, gS, _Sigmoid(4.0), rf)
    for wpc, stages in [(1, 2), (2, 3), (3, 2), (4, 4), (6, 3), (8, 2)]:
        nsb.set_tuning(warps_per_cta=wpc, stages=stages, lanes_per_thread=2)
        got = _fused_grads(d, b, v0, w0, gS, _Sigmoid(4.0), rf)
        for k, v in base.items():
            if v is not None:
                assert torch.equal(v, got[k]), (wpc, stages, k)


@pytest.mark.parametrize("rf", [False, True])
def test_fused_edge_cases(rf):
    # T = 0: the states pass through, nothing else is touched
    d, b, v0, w0 = mod_inputs(0, 2, 64, torch.bfloat16, 3, rf)
    s, vl, wl = run_fused(d, b, v0, w0, rf)
    assert s.shape == (0, 2, 64) and torch.equal(vl, v0)
    if rf:
        assert torch.equal(wl, w0)
    # a column count that is not a multiple of 32, and one that breaks 16-byte row alignment
    for D in (40, 33):
        d, b, v0, w0 = mod_inputs(20, 3, D, torch.bfloat16, 4, rf)
        ref = run_unfused(d, b, v0, w0, rf)
        s, vl, wl = run_fused(d, b, v0, w0, rf)
        assert torch.equal(s.float(), ref[0].float()) and torch.equal(vl, ref[1])
    # bias of the wrong length
    with pytest.raises(nsb.NSBError):
        bad = dict(b)
        bad["b_beta"] = b["b_beta"][:-1]
        run_fused(d, bad, v0, w0, rf)


@pytest.mark.parametrize("rf", [False, True])
def test_adaptive_slope_from_the_kernel(rf):
    """With adaptive_sigma0 the forward accumulates the moments of u = alpha*I and the backward uses
    clamp(alpha_0*sigma_0/std(u), 1, 20): same gradients as passing that slope by hand."""
    T, B, D = 96, 2, 264
    d, b, v0, w0 = mod_inputs(T, B, D, torch.bfloat16, 61, rf)
    gS = (torch.randn(T, B, D, device=DEV) * 0.1).bfloat16()
    u = run_modulation(d, b, rf)[1]                 # fp32 u as the kernel forms it
    want_alpha = orc.surrogate_alpha(f32(u), 4.0, 0.4, "f32")
    assert 1.0 < want_alpha < 20.0

    def grads(surrogate, sigma0):
        leaves = {k: v.clone().requires_grad_() for k, v in {**d, **b}.items()}
        args = ([leaves[k] for k in ("raw_beta",)] + [leaves["b_beta"], leaves["raw_alpha"], leaves["b_alpha"],
                                                       leaves["raw_th"], leaves["b_th"], V_TH_MIN, leaves["cur"]])
        if rf:
            s, _, _ = sb.modulated_rf_plif_forward(*args, leaves["raw_omega"], leaves["b_omega"], v0, w0,
                                                   surrogate, adaptive_sigma0=sigma0)
        else:
            s, _ = sb.modulated_plif_forward(*args, v0, surrogate, adaptive_sigma0=sigma0)
        s.backward(gS)
        return {k: leaves[k].grad for k in leaves}

    mine = grads(_Sigmoid(4.0), 0.4)
    ref = grads(_Sigmoid(want_alpha), None)
    for k in ref:
        a, w = f32(mine[k]).reshape(-1), f32(ref[k]).astype(np.float64).reshape(-1)
        # both sides are bf16-rounded: they may sit one unit in the last place apart (2^-7 relative)
        bound = (2.0 ** -7 * np.abs(w) if mine[k].dtype == torch.bfloat16 else 0.0) + 1e-5 * np.abs(w).max()
        assert (np.abs(a - w) <= bound).all(), k
    fixed = grads(_Sigmoid(4.0), None)   # and it is not the fixed slope
    assert not torch.equal(fixed["cur"], mine["cur"])
