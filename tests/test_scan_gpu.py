"""GPU parity of the PLIF scan kernels against the CPU oracle and the golden
vectors. Everything here goes through the C ABI (via the ctypes binding)."""
import itertools

import numpy as np
import pytest
import torch

import neuronspark_b200 as nsb
import neuronspark_b200._lib  # noqa: F401  (nsb._lib)
from neuronspark_b200 import parallel_scan as ps
from oracle import oracle as orc
from util import (REL_TOL, assert_close, assert_close_lowp, assert_spikes_match, f32,
                  oracle_selective, rowparam_inputs, selective_inputs)

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(autouse=True)
def _reset_tuning():
    nsb.set_tuning()
    ps.CKPT_INTERVAL = None
    yield
    nsb.set_tuning()
    ps.CKPT_INTERVAL = None
    assert nsb.device_error_word() == 0


def cuda(a, dtype=torch.float32):
    return torch.as_tensor(np.asarray(a), device=DEV).to(dtype)


# ------------------------------------------------------------ golden vectors


@pytest.mark.parametrize("name", ["scan_fwd_a", "scan_fwd_b"])
def test_golden_selective_forward(golden, name):
    g = golden(name)
    spike, vpost, none = ps.plif_parallel_forward(cuda(g["beta"]), cuda(g["u"]), cuda(g["vth"]),
                                                  cuda(g["v_init"]))
    assert none is None
    assert np.array_equal(f32(spike), g["spike"])
    assert np.array_equal(f32(vpost), g["vpost"])


def test_golden_selective_ai_forward(golden):
    g = golden("scan_fwd_c0")
    spike, v_last = ps.plif_selective_scan_ai(cuda(g["beta"]), cuda(g["cur"]), cuda(g["gain"]),
                                              cuda(g["vth"]), cuda(g["v_init"]))
    assert np.array_equal(f32(spike), g["spike"])
    assert np.array_equal(f32(v_last), g["vpost"][-1])


class _Sigmoid:  # stands in for spikingjelly.activation_based.surrogate.Sigmoid
    def __init__(self, alpha):
        self.alpha = alpha


_Sigmoid.__name__ = "Sigmoid"


@pytest.mark.parametrize("name,with_gv", [("scan_bwd_a", True), ("scan_bwd_ones", False)])
def test_golden_selective_backward(golden, name, with_gv):
    g = golden(name)
    beta, u, vth, v0 = (cuda(g[k]).requires_grad_() for k in ("beta", "u", "vth", "v_init"))
    spike, vpost, _ = ps.plif_parallel_forward(beta, u, vth, v0, 3, _Sigmoid(float(g["alpha"])))
    if with_gv:
        loss = (spike * cuda(g["g_spike"])).sum() + (vpost * cuda(g["g_vpost"])).sum()
    else:
        loss = spike.sum() + vpost.sum()  # the loss of exp/verify_fused_plif.py:101
    loss.backward()
    for t, k in ((beta, "g_beta"), (u, "g_u"), (vth, "g_vth"), (v0, "g_vinit")):
        assert_close(f32(t.grad), g[k], what=k)
        # the reference's own acceptance bound (exp/verify_fused_plif.py:137)
        assert np.abs(f32(t.grad) - g[k]).max() < 1e-3


def test_golden_ai_backward(golden):
    g = golden("scan_ai_bwd")
    ins = [cuda(g[k]).requires_grad_() for k in ("beta", "cur", "gain", "vth", "v_init")]
    spike, _ = ps.plif_selective_scan_ai(*ins, alpha=float(g["alpha"]), surrogate="sigmoid")
    assert np.array_equal(f32(spike), g["spike"])
    (spike * cuda(g["g_spike"])).sum().backward()
    for t, k in zip(ins, ("g_beta", "g_cur", "g_gain", "g_vth", "g_vinit")):
        assert_close(f32(t.grad), g[k], what=k)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_golden_ai_backward_atan(golden, dtype):
    """Arctangent surrogate, alpha = 2 (the headline benchmark's): gradients against torch autograd
    through the surrogate's primitive (tests/golden/make_golden.py, fixture scan_ai_bwd_atan)."""
    g = golden("scan_ai_bwd_atan")
    ins = [cuda(g[k]).requires_grad_() for k in ("beta", "cur", "gain", "vth", "v_init")]
    if dtype != torch.float32:
        # bf16 streams: round the inputs, regenerate the expectation from the oracle (itself pinned to
        # the fixture in fp32 by tests/test_oracle_golden.py) on the rounded values
        ins = [t.detach().to(dtype).requires_grad_() for t in ins[:4]] + [ins[4]]
    spike, _ = ps.plif_selective_scan_ai(*ins, alpha=float(g["alpha"]), surrogate="atan")
    gs = cuda(g["g_spike"]).to(dtype)
    (spike.float() * gs.float()).sum().backward()
    if dtype == torch.float32:
        assert np.array_equal(f32(spike), g["spike"])
        for t, k in zip(ins, ("g_beta", "g_cur", "g_gain", "g_vth", "g_vinit")):
            assert_close(f32(t.grad), g[k], what=k)
    else:
        hb, hc, hg, ht, hv = (f32(t) for t in ins)
        s, _, _ = orc.plif_selective_ai_fwd(hb, hc, hg, ht, hv)
        assert np.array_equal(f32(spike), s)
        ref = orc.plif_selective_ai_bwd(hb, hc, hg, ht, hv, f32(gs), None, float(g["alpha"]), orc.SURR_ATAN)
        for t, e, k in zip(ins, ref, ("g_beta", "g_cur", "g_gain", "g_vth", "g_vinit")):
            assert_close_lowp(f32(t.grad), e, t.dtype, what=k)


@pytest.mark.parametrize("name", ["rowparam_a", "rowparam_c1"])
@pytest.mark.parametrize("recompute", [False, True])
def test_golden_rowparam(golden, name, recompute):
    g = golden(name)
    has_gv = "g_vpost" in g
    if recompute and has_gv:
        pytest.skip("the recompute variant ignores the V gradient")
    br, u, tr, v0 = (cuda(g[k]).requires_grad_() for k in ("beta_row", "u", "vth_row", "v_init"))
    alpha = float(g["alpha"])
    if recompute:
        spike, v_last = ps.plif_rowparam_forward_recompute(br, u, tr, v0, alpha)
        assert np.array_equal(f32(v_last), g["vpost"][-1])
        vpost = None
    else:
        spike, vpost = ps.plif_rowparam_forward_alpha(br, u, tr, v0, alpha)
        assert np.array_equal(f32(vpost), g["vpost"])
    assert np.array_equal(f32(spike), g["spike"])
    gS = cuda(g["g_spike"]) if "g_spike" in g else torch.ones_like(spike)
    loss = (spike * gS).sum()
    if has_gv:
        loss = loss + (vpost * cuda(g["g_vpost"])).sum()
    loss.backward()
    for t, k in ((br, "g_beta_row"), (u, "g_u"), (tr, "g_vth_row"), (v0, "g_vinit")):
        assert_close(f32(t.grad), g[k], what=k)


def test_recompute_and_materialising_variants_agree_bitwise():
    """test_recompute.py:20-73 of the reference: torch.equal on spikes and V_last,
    zero tolerance on every gradient (K=16, batch=2, dim=256, fp32, seed 42)."""
    torch.manual_seed(42)
    K, B, D = 16, 2, 256
    base = [torch.sigmoid(torch.randn(B, D)), torch.randn(K, B, D),
            torch.abs(torch.randn(B, D)) + 0.1, torch.randn(B, D)]
    a = [t.to(DEV).requires_grad_() for t in base]
    b = [t.to(DEV).requires_grad_() for t in base]
    s1, v1 = ps.plif_rowparam_forward_alpha(*a, 4.0)
    s1.sum().backward()
    s2, vl = ps.plif_rowparam_forward_recompute(*b, 4.0)
    s2.sum().backward()
    assert torch.equal(s1, s2) and torch.equal(v1[-1], vl)
    for x, y in zip(a, b):
        assert torch.equal(x.grad, y.grad)


# ------------------------------------------------- seeded sweeps vs the oracle

SHAPES = [
    (1, 1, 1), (3, 1, 5), (8, 2, 32), (9, 2, 40), (17, 3, 33), (64, 2, 64),
    (100, 2, 200), (256, 2, 768), (33, 1, 1000), (16, 4, 1536),
]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("form", ["u", "ai"])
def test_selective_forward_vs_oracle(shape, dtype, form):
    T, B, D = shape
    beta, cur, gain, vth, v0 = selective_inputs(T, B, D, dtype, DEV, seed=T * 131 + D, zero_init=False)
    if form == "u":
        u = (gain.float() * cur.float()).to(dtype)
        rs, rv, rl = oracle_selective(beta, u, None, vth, v0)
        spike, vpost, _ = ps.plif_parallel_forward(beta, u, vth, v0)
        assert spike.dtype == dtype and vpost.dtype == dtype
        assert_close_lowp(f32(vpost), rv, dtype, "V_post")
        if dtype == torch.float32:
            assert np.array_equal(f32(vpost), rv)
    else:
        rs, rv, rl = oracle_selective(beta, cur, gain, vth, v0)
        spike, v_last = ps.plif_selective_scan_ai(beta, cur, gain, vth, v0)
        assert np.array_equal(f32(v_last), rl)
    assert np.array_equal(f32(spike), rs), "spikes must be bit-exact"


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rowparam_forward_vs_oracle(shape, dtype):
    T, B, D = shape
    br, u, tr, v0 = rowparam_inputs(T, B, D, dtype, DEV, seed=T + 7 * D)
    rs, rv, rl = orc.plif_rowparam_fwd(f32(br), f32(u), f32(tr), f32(v0))
    spike, vpost = ps.plif_rowparam_forward_alpha(br, u, tr, v0, 4.0)
    assert np.array_equal(f32(spike), rs)
    assert_close_lowp(f32(vpost), rv, dtype, "V_post")
    spike2, v_last = ps.plif_rowparam_forward_recompute(br, u, tr, v0, 4.0)
    assert torch.equal(spike, spike2)
    assert np.array_equal(f32(v_last), rl)
    # per-channel ([D]) parameters broadcast to the same thing
    spike3, _ = ps.plif_rowparam_forward_alpha(br[0], u, tr[0], v0, 4.0)
    assert torch.equal(spike, spike3)


@pytest.mark.parametrize("shape", [(1, 1, 1), (9, 2, 40), (17, 3, 33), (64, 2, 64), (130, 2, 96),
                                   (40, 1, 520)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("form,surrogate", [("u", "sigmoid"), ("ai", "sigmoid"), ("ai", "atan"),
                                            ("u", "atan")])
def test_selective_backward_vs_oracle(shape, dtype, form, surrogate):
    T, B, D = shape
    beta, cur, gain, vth, v0 = selective_inputs(T, B, D, dtype, DEV, seed=T * 17 + D, zero_init=False)
    g = torch.Generator(device=DEV).manual_seed(5)
    gS = (0.1 * torch.randn(T, B, D, generator=g, device=DEV)).to(dtype)
    alpha = 4.0 if surrogate == "sigmoid" else 2.0
    kind = orc.SURR_SIGMOID if surrogate == "sigmoid" else orc.SURR_ATAN
    v0 = v0.requires_grad_()
    if form == "u":
        u = (gain.float() * cur.float()).to(dtype).requires_grad_()
        beta, vth = beta.requires_grad_(), vth.requires_grad_()

        class S:
            pass
        S.__name__ = "Sigmoid" if surrogate == "sigmoid" else "ATan"
        s = S()
        s.alpha = alpha
        gV = (0.05 * torch.randn(T, B, D, generator=g, device=DEV)).to(dtype)
        spike, vpost, _ = ps.plif_parallel_forward(beta, u, vth, v0, 3, s)
        ((spike.float() * gS.float()).sum() + (vpost.float() * gV.float()).sum()).backward()
        ref = orc.plif_selective_bwd(f32(beta), f32(u), f32(vth), f32(v0), f32(gS), f32(gV), alpha, kind)
        got = (beta.grad, u.grad, vth.grad, v0.grad)
        names = ("g_beta", "g_u", "g_vth", "g_vinit")
    else:
        ins = [t.requires_grad_() for t in (beta, cur, gain, vth)]
        spike, _ = ps.plif_selective_scan_ai(*ins, v0, alpha=alpha, surrogate=surrogate)
        (spike.float() * gS.float()).sum().backward()
        ref = orc.plif_selective_ai_bwd(f32(beta), f32(cur), f32(gain), f32(vth), f32(v0), f32(gS),
                                        None, alpha, kind)
        got = tuple(t.grad for t in ins) + (v0.grad,)
        names = ("g_beta", "g_cur", "g_gain", "g_vth", "g_vinit")
    for a, e, n in zip(got, ref, names):
        if n == "g_vinit":
            assert_close(f32(a), e, what=n)
        else:
            assert_close_lowp(f32(a), e, dtype, what=n)


@pytest.mark.parametrize("shape", [(1, 1, 1), (16, 2, 256), (23, 3, 50), (100, 2, 320)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("surrogate", ["sigmoid"])
def test_rowparam_backward_vs_oracle(shape, dtype, surrogate):
    T, B, D = shape
    br, u, tr, v0 = rowparam_inputs(T, B, D, dtype, DEV, seed=T + 3 * D)
    g = torch.Generator(device=DEV).manual_seed(9)
    gS = torch.randn(T, B, D, generator=g, device=DEV).to(dtype)
    gV = (0.1 * torch.randn(T, B, D, generator=g, device=DEV)).to(dtype)
    ins = [t.clone().requires_grad_() for t in (br, u, tr, v0)]
    spike, vpost = ps.plif_rowparam_forward_alpha(*ins, 4.0)
    ((spike.float() * gS.float()).sum() + (vpost.float() * gV.float()).sum()).backward()
    ref = orc.plif_rowparam_bwd(f32(br), f32(u), f32(tr), f32(v0), f32(gS), f32(gV), 4.0)
    for t, e, n in zip(ins, ref, ("g_beta_row", "g_u", "g_vth_row", "g_vinit")):
        if n == "g_u":
            assert_close_lowp(f32(t.grad), e, dtype, what=n)
        else:
            assert_close(f32(t.grad), e, what=n)
    # recompute variant: V gradient ignored
    ins2 = [t.clone().requires_grad_() for t in (br, u, tr, v0)]
    spike2, _ = ps.plif_rowparam_forward_recompute(*ins2, 4.0)
    (spike2.float() * gS.float()).sum().backward()
    ref2 = orc.plif_rowparam_bwd(f32(br), f32(u), f32(tr), f32(v0), f32(gS), None, 4.0)
    for t, e, n in zip(ins2, ref2, ("g_beta_row", "g_u", "g_vth_row", "g_vinit")):
        if n == "g_u":
            assert_close_lowp(f32(t.grad), e, dtype, what=n)
        else:
            assert_close(f32(t.grad), e, what=n)


# ----------------------------------------------------- kernel variants agree


@pytest.mark.parametrize("lanes,stages,wpc", [(1, 2, 1), (2, 3, 3), (4, 2, 2), (2, 4, 8), (1, 6, 4)])
def test_tuning_variants_bitwise_identical(lanes, stages, wpc):
    ps.CKPT_INTERVAL = 8  # the lane count is forced below; 8-step tiles exist for every lane count
    T, B, D = 70, 2, 384
    beta, cur, gain, vth, v0 = selective_inputs(T, B, D, torch.bfloat16, DEV, seed=3)
    nsb.set_tuning(force_direct=True)
    ref_spike, ref_last = ps.plif_selective_scan_ai(beta, cur, gain, vth, v0)
    assert nsb.last_launch_info()["used_tma"] == 0
    nsb.set_tuning(warps_per_cta=wpc, stages=stages, lanes_per_thread=lanes)
    spike, last = ps.plif_selective_scan_ai(beta, cur, gain, vth, v0)
    info = nsb.last_launch_info()
    assert info["used_tma"] == 1 and info["lanes_per_thread"] == lanes and info["stages"] == stages
    assert torch.equal(spike, ref_spike) and torch.equal(last, ref_last)
    packed, last2 = ps.plif_selective_forward_packed(beta, cur, vth, v0, gain=gain)
    assert torch.equal(ps.unpack_spikes(packed, (B, D), torch.bfloat16), ref_spike)
    assert torch.equal(last2, ref_last.float())


@pytest.mark.parametrize("lanes", [1, 2, 4])
@pytest.mark.parametrize("surrogate", ["sigmoid", "atan"])
def test_backward_direct_and_tma_paths_agree(lanes, surrogate):
    ps.CKPT_INTERVAL = 8
    T, B, D = 45, 2, 192
    base = selective_inputs(T, B, D, torch.float32, DEV, seed=11, zero_init=False)
    gS = 0.1 * torch.randn(T, B, D, device=DEV)
    outs = []
    for direct in (True, False):
        nsb.set_tuning(lanes_per_thread=lanes, force_direct=direct)
        ins = [t.clone().requires_grad_() for t in base]
        spike, _ = ps.plif_selective_scan_ai(*ins, alpha=2.0, surrogate=surrogate)
        (spike * gS).sum().backward()
        assert nsb.last_launch_info()["used_tma"] == (0 if direct else 1)
        outs.append([t.grad for t in ins])
    for a, b in zip(*outs):
        assert torch.equal(a, b)


@pytest.mark.parametrize("shape", [(5, 1, 31), (40, 2, 100), (64, 3, 64), (16, 2, 1024)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_packed_spikes_layout(shape, dtype):
    T, B, D = shape
    beta, cur, gain, vth, v0 = selective_inputs(T, B, D, dtype, DEV, seed=21)
    u = (gain.float() * cur.float()).to(dtype)
    rs, _, rl = oracle_selective(beta, u, None, vth, v0)
    packed, v_last = ps.plif_selective_forward_packed(beta, u, vth, v0)
    cols = B * D
    assert packed.shape == (T, (cols + 31) // 32) and packed.dtype == torch.int32
    words = packed.cpu().numpy().view(np.uint32)
    bits = ((words[:, :, None] >> np.arange(32, dtype=np.uint32)) & 1).reshape(T, -1)
    assert np.array_equal(bits[:, :cols], rs.reshape(T, cols).astype(np.uint32))
    assert not bits[:, cols:].any(), "tail bits must be zero"
    assert np.array_equal(f32(v_last), rl)
    br, ur, tr, v0r = rowparam_inputs(T, B, D, dtype, DEV, seed=22)
    rs2, _, _ = orc.plif_rowparam_fwd(f32(br), f32(ur), f32(tr), f32(v0r))
    packed2, _ = ps.plif_rowparam_forward_packed(br, ur, tr, v0r)
    assert np.array_equal(f32(ps.unpack_spikes(packed2, (B, D))), rs2)


def test_state_carry_across_calls_is_exact():
    """Per-token decoding: T=16 calls that carry V equal one long scan."""
    T, B, D = 16 * 6, 4, 256
    beta, cur, gain, vth, v0 = selective_inputs(T, B, D, torch.bfloat16, DEV, seed=5)
    whole, last = ps.plif_selective_forward_packed(beta, cur, vth, v0, gain=gain)
    v = v0
    parts = []
    for i in range(0, T, 16):
        sl = slice(i, i + 16)
        p, v = ps.plif_selective_forward_packed(beta[sl], cur[sl], vth[sl], v, gain=gain[sl])
        parts.append(p)
    assert torch.equal(torch.cat(parts), whole) and torch.equal(v, last)


def test_mixed_dtypes_widen_exactly():
    """fp32 beta/v_th with a bf16 drive (plain autocast) is legal: every input is
    widened to fp32, outputs come back in u's dtype."""
    T, B, D = 24, 2, 64
    beta, cur, gain, vth, v0 = selective_inputs(T, B, D, torch.float32, DEV, seed=8)
    u = (gain * cur).bfloat16()
    rs, rv, _ = oracle_selective(beta, u, None, vth, v0)
    spike, vpost, _ = ps.plif_parallel_forward(beta, u, vth, v0)
    assert spike.dtype == torch.bfloat16
    assert np.array_equal(f32(spike), rs)
    assert_close_lowp(f32(vpost), rv, torch.bfloat16)


def test_expanded_v_init_gradient_flows_through_expand():
    """v_init arrives as an expanded view of a [D] parameter
    (atomic_ops/selective_plif.py:68-70)."""
    T, B, D = 12, 3, 64
    beta, cur, gain, vth, _ = selective_inputs(T, B, D, torch.float32, DEV, seed=4)
    param = (0.1 * torch.randn(D, device=DEV)).requires_grad_()
    v0 = param.unsqueeze(0).expand(B, -1)
    assert not v0.is_contiguous()
    spike, _ = ps.plif_selective_scan_ai(beta, cur, gain, vth, v0)
    spike.sum().backward()
    ref = orc.plif_selective_ai_bwd(f32(beta), f32(cur), f32(gain), f32(vth), f32(v0),
                                    np.ones((T, B, D), np.float32), None, 4.0)
    assert_close(f32(param.grad), ref[4].sum(0), what="grad of the [D] parameter")


def test_fixed_param_dispatch():
    T, B, D = 20, 2, 96
    u = 0.5 * torch.randn(T, B, D, device=DEV)
    v0 = torch.zeros(B, D, device=DEV)
    s1, v1 = ps.plif_fixed_param_forward(0.9, u, 0.3, v0)
    s2, v2 = ps.plif_fixed_param_forward(torch.tensor(0.9, device=DEV), u, torch.tensor(0.3, device=DEV), v0)
    rs, rv, _ = orc.plif_rowparam_fwd(np.full((B, D), 0.9, np.float32), f32(u),
                                      np.full((B, D), 0.3, np.float32), f32(v0))
    assert np.array_equal(f32(s1), rs) and np.array_equal(f32(v1), rv)
    assert torch.equal(s1, s2) and torch.equal(v1, v2)
    full_beta = torch.full_like(u, 0.9)
    s3, v3 = ps.plif_fixed_param_forward(full_beta, u, 0.3, v0)
    assert torch.equal(s1, s3) and torch.equal(v1, v3)


def test_cpu_tensor_is_rejected():
    with pytest.raises(nsb.NSBError):
        ps.plif_parallel_forward(torch.ones(2, 1, 4), torch.ones(2, 1, 4), torch.ones(2, 1, 4),
                                 torch.zeros(1, 4))


def test_empty_time_axis_and_empty_columns():
    """T = 0: nothing to scan, the final state is the initial state and the gradient of the
    initial state is zero; zero columns: a no-op."""
    B, D = 2, 64
    v0 = torch.randn(B, D, device=DEV)
    e = torch.empty(0, B, D, device=DEV)
    packed, v_last = ps.plif_selective_forward_packed(e, e, e, v0)
    assert packed.shape == (0, B * D // 32) and torch.equal(v_last, v0)
    spike, v_l = ps.plif_rowparam_forward_recompute(torch.rand(B, D, device=DEV), e, torch.rand(B, D, device=DEV),
                                                    v0, 4.0)
    assert spike.shape == (0, B, D) and torch.equal(v_l, v0)
    z = torch.empty(4, 0, 8, device=DEV)
    s, v, _ = ps.plif_parallel_forward(z, z, z, torch.empty(0, 8, device=DEV))
    assert s.shape == (4, 0, 8) and v.shape == (4, 0, 8)
    L = nsb._lib.lib()
    g = torch.full((B, D), 7.0, device=DEV)
    dummy = torch.zeros(8, device=DEV)
    st = L.nsb_plif_selective_bwd(nsb._lib.ptr(dummy), nsb._lib.ptr(dummy), None, nsb._lib.ptr(dummy),
                                  nsb._lib.ptr(dummy), nsb._lib.ptr(dummy), None, None, None, None, None,
                                  nsb._lib.ptr(g), 0, B * D, 0, 8, 0, 4.0, None, nsb._lib.stream_ptr(torch.device(DEV)))
    assert st == 0 and float(g.abs().max()) == 0.0


def test_unaligned_views_take_the_direct_path_and_stay_exact():
    """A tensor view that starts 2 bytes into an allocation cannot be a TMA source."""
    T, B, D = 24, 2, 64
    beta, cur, gain, vth, v0 = selective_inputs(T, B, D, torch.bfloat16, DEV, seed=12)
    u = (gain.float() * cur.float()).bfloat16()
    flat = torch.empty(T * B * D + 1, dtype=torch.bfloat16, device=DEV)
    u_off = flat[1:].view(T, B, D)
    u_off.copy_(u)
    assert u_off.data_ptr() % 16 != 0 and u_off.is_contiguous()
    s_ref, v_ref, _ = ps.plif_parallel_forward(beta, u, vth, v0)
    assert nsb.last_launch_info()["used_tma"] == 1
    s, v, _ = ps.plif_parallel_forward(beta, u_off, vth, v0)
    assert nsb.last_launch_info()["used_tma"] == 0
    assert torch.equal(s, s_ref) and torch.equal(v, v_ref)


@pytest.mark.parametrize("interval", [8, 16, 32])
@pytest.mark.parametrize("shape", [(5, 1, 31), (33, 2, 64), (100, 2, 200), (257, 1, 512)])
def test_every_tile_length_vs_oracle(interval, shape):
    """The checkpoint spacing / tile length (8, 16, 32 steps) never changes a result bit."""
    ps.CKPT_INTERVAL = interval
    T, B, D = shape
    beta, cur, gain, vth, v0 = selective_inputs(T, B, D, torch.float32, DEV, seed=T + interval, zero_init=False)
    rs, _, rl = oracle_selective(beta, cur, gain, vth, v0)
    ins = [t.requires_grad_() for t in (beta, cur, gain, vth, v0)]
    spike, v_last = ps.plif_selective_scan_ai(*ins, alpha=4.0, surrogate="sigmoid")
    assert nsb.last_launch_info()["tile_steps"] == interval
    assert np.array_equal(f32(spike), rs) and np.array_equal(f32(v_last), rl)
    gS = torch.randn(T, B, D, device=DEV)
    (spike * gS).sum().backward()
    ref = orc.plif_selective_ai_bwd(*(f32(t) for t in ins), f32(gS), None, 4.0)
    for t, e, n in zip(ins, ref, ("g_beta", "g_cur", "g_gain", "g_vth", "g_vinit")):
        assert_close(f32(t.grad), e, what=n)
    packed, _ = ps.plif_selective_forward_packed(beta.detach(), cur.detach(), vth.detach(), v0.detach(),
                                                 gain=gain.detach())
    assert np.array_equal(f32(ps.unpack_spikes(packed, (B, D))), rs)
    br, u, tr, v0r = rowparam_inputs(T, B, D, torch.bfloat16, DEV, seed=3)
    s2, vl2 = ps.plif_rowparam_forward_recompute(br, u, tr, v0r, 4.0)
    r2 = orc.plif_rowparam_fwd(f32(br), f32(u), f32(tr), f32(v0r), want_vpost=False)
    assert np.array_equal(f32(s2), r2[0]) and np.array_equal(f32(vl2), r2[2])
