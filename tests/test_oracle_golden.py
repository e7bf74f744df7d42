"""The CPU oracle against the golden vectors produced by the reference's code.

This is what pins the oracle: forward scans and the codec must agree bit for
bit, the backward passes and the normaliser to 1e-5 relative (fp32)."""
import numpy as np
import pytest

from oracle import oracle as orc
from conftest import rel_err

TOL = 1e-5  # relative, fp32


@pytest.mark.parametrize("name", ["scan_fwd_a", "scan_fwd_b"])
def test_selective_fwd_bit_exact(golden, name):
    g = golden(name)
    s, v, vl = orc.plif_selective_fwd(g["beta"], g["u"], g["vth"], g["v_init"])
    assert np.array_equal(s, g["spike"])
    assert np.array_equal(v, g["vpost"])
    assert np.array_equal(vl, g["vpost"][-1])


def test_selective_ai_fwd_bit_exact(golden):
    g = golden("scan_fwd_c0")
    s, v, vl = orc.plif_selective_ai_fwd(g["beta"], g["cur"], g["gain"], g["vth"], g["v_init"])
    assert np.array_equal(s, g["spike"])
    assert np.array_equal(v, g["vpost"])
    # u-form on the pre-multiplied drive gives the same thing
    u = (g["gain"] * g["cur"]).astype(np.float32)
    s2, v2, _ = orc.plif_selective_fwd(g["beta"], u, g["vth"], g["v_init"])
    assert np.array_equal(s2, s) and np.array_equal(v2, v)
    assert 0.01 < s.mean() < 0.99


def test_selective_bwd(golden):
    g = golden("scan_bwd_a")
    gb, gu, gt, gv = orc.plif_selective_bwd(g["beta"], g["u"], g["vth"], g["v_init"],
                                            g["g_spike"], g["g_vpost"], float(g["alpha"]))
    for mine, ref in ((gb, "g_beta"), (gu, "g_u"), (gt, "g_vth"), (gv, "g_vinit")):
        assert rel_err(mine, g[ref]) < TOL, ref


def test_selective_bwd_reference_loss(golden):
    """Loss = spike.sum() + V_post.sum(), as in exp/verify_fused_plif.py:101."""
    g = golden("scan_bwd_ones")
    ones = np.ones_like(g["u"])
    gb, gu, gt, gv = orc.plif_selective_bwd(g["beta"], g["u"], g["vth"], g["v_init"],
                                            ones, ones, float(g["alpha"]))
    for mine, ref in ((gb, "g_beta"), (gu, "g_u"), (gt, "g_vth"), (gv, "g_vinit")):
        assert rel_err(mine, g[ref]) < TOL, ref


def test_selective_ai_bwd(golden):
    g = golden("scan_ai_bwd")
    s, v, _ = orc.plif_selective_ai_fwd(g["beta"], g["cur"], g["gain"], g["vth"], g["v_init"])
    assert np.array_equal(s, g["spike"]) and np.array_equal(v, g["vpost"])
    out = orc.plif_selective_ai_bwd(g["beta"], g["cur"], g["gain"], g["vth"], g["v_init"],
                                    g["g_spike"], None, float(g["alpha"]))
    for mine, ref in zip(out, ("g_beta", "g_cur", "g_gain", "g_vth", "g_vinit")):
        assert rel_err(mine, g[ref]) < TOL, ref


def test_selective_ai_backward_atan(golden):
    """The arctangent surrogate (alpha = 2, the headline benchmark's) against torch autograd through
    the surrogate's primitive atan(pi/2*alpha*x)/pi + 1/2: the oracle's hand-written derivative
    (alpha/2)/(1+(pi/2*alpha*x)^2) is what autograd derives."""
    g = golden("scan_ai_bwd_atan")
    s, _, _ = orc.plif_selective_ai_fwd(g["beta"], g["cur"], g["gain"], g["vth"], g["v_init"])
    assert np.array_equal(s, g["spike"])
    out = orc.plif_selective_ai_bwd(g["beta"], g["cur"], g["gain"], g["vth"], g["v_init"],
                                    g["g_spike"], None, float(g["alpha"]), orc.SURR_ATAN)
    for mine, ref in zip(out, ("g_beta", "g_cur", "g_gain", "g_vth", "g_vinit")):
        assert rel_err(mine, g[ref]) < TOL, ref
    # and it is not the sigmoid surrogate that passes
    wrong = orc.plif_selective_ai_bwd(g["beta"], g["cur"], g["gain"], g["vth"], g["v_init"],
                                      g["g_spike"], None, float(g["alpha"]), orc.SURR_SIGMOID)
    assert rel_err(wrong[1], g["g_cur"]) > 1e-2


@pytest.mark.parametrize("name", ["rowparam_a", "rowparam_c1"])
def test_rowparam(golden, name):
    g = golden(name)
    s, v, vl = orc.plif_rowparam_fwd(g["beta_row"], g["u"], g["vth_row"], g["v_init"])
    assert np.array_equal(s, g["spike"])
    assert np.array_equal(v, g["vpost"])
    gS = g.get("g_spike", np.ones_like(g["u"]))
    out = orc.plif_rowparam_bwd(g["beta_row"], g["u"], g["vth_row"], g["v_init"], gS,
                                g.get("g_vpost"), float(g["alpha"]))
    for mine, ref in zip(out, ("g_beta_row", "g_u", "g_vth_row", "g_vinit")):
        assert rel_err(mine, g[ref]) < TOL, ref


def test_codec(golden):
    g = golden("codec_a")
    fa, fb = orc.fp16_encode(g["xa"]), orc.fp16_encode(g["xb"])
    assert np.array_equal(fa, g["frames_a"]) and np.array_equal(fb, g["frames_b"])
    assert np.array_equal(orc.fp16_decode(fa), g["decoded_a"])
    res = orc.binary_residual(fa, fb)
    assert np.array_equal(res, g["residual"])
    assert set(np.unique(res)) <= {0.0, 1.0}
    assert np.array_equal(orc.fp16_decode(res), g["decoded_residual"])
    # the reference's own acceptance checks (test_binary_residual.py:24-31, 90-95)
    half = lambda x: x.astype(np.float16).astype(np.float32)
    assert np.abs(g["decoded_residual"] - half(half(g["xa"]) + half(g["xb"]))).max() < 1e-2
    assert np.abs(g["decoded_a"] - half(g["xa"])).max() < 1e-3
    assert rel_err(orc.fp16_decode_bwd(fa, g["g_out"]), g["g_frames"]) < 1e-6
    assert rel_err(orc.encode_ste_bwd(g["g_frames_in"]), g["g_ste"]) < 1e-6


def test_codec_edges(golden):
    g = golden("codec_edge")
    f = orc.fp16_encode(g["x"])
    assert np.array_equal(f, g["frames"])
    assert np.array_equal(orc.fp16_decode(f), g["decoded"])
    assert np.array_equal(orc.binary_residual(f, g["frames_b"]), g["residual"])
    # exponent pattern 31 decodes as a normal number, no inf/nan
    assert np.array_equal(orc.fp16_decode(g["frames_e31"]), g["decoded_e31"])
    assert np.isfinite(g["decoded_e31"]).all()
    assert np.array_equal(orc.binary_residual(g["frames_e31"], g["frames_b"]), g["residual_e31"])
    # 70000 clamps to 65504
    assert orc.fp16_decode(orc.fp16_encode(np.full((1, 1, 1), 70000.0)))[0, 0, 0] == 65504.0


def test_codec_bf16_frames(golden):
    g = golden("codec_bf16")
    assert np.array_equal(orc.fp16_decode(g["frames_a"], True), g["decoded_a"])
    assert np.array_equal(orc.fp16_decode(g["frames_e"], True), g["decoded_e"])
    assert np.array_equal(orc.binary_residual(g["frames_a"], g["frames_b"], True), g["residual"])
    fb = golden("codec_edge")["frames_b"]
    assert np.array_equal(orc.binary_residual(g["frames_e"], fb, True), g["residual_e"])


def test_lateral_inhibition(golden):
    g = golden("li_a")
    out = orc.li_fwd(g["x"], g["gain"], float(g["eps"]))
    assert rel_err(out, g["out"]) < TOL
    gx, gg = orc.li_bwd(g["g_out"], g["x"], g["gain"], float(g["eps"]))
    assert rel_err(gx, g["g_x"]) < TOL
    assert rel_err(gg, g["g_gain"]) < TOL


def test_rf_scan(golden):
    g = golden("rf_a")
    s, v, w, vl, wl = orc.plif_rf_fwd(g["beta"], g["omega"], g["u"], g["vth"], g["v_init"], g["w_init"])
    assert np.array_equal(s, g["spike"]) and np.array_equal(v, g["vpost"]) and np.array_equal(w, g["w"])
    assert np.array_equal(vl, g["vpost"][-1]) and np.array_equal(wl, g["w"][-1])
    out = orc.plif_rf_bwd(g["beta"], g["omega"], g["u"], g["vth"], g["v_init"], g["w_init"],
                          g["g_spike"], g["g_vpost"], float(g["alpha"]))
    for mine, ref in zip(out, ("g_beta", "g_omega", "g_u", "g_vth", "g_vinit", "g_winit")):
        assert rel_err(mine, g[ref]) < TOL, ref
    # omega = 0, w_init = 0 is the first-order scan
    z = np.zeros_like(g["u"])
    s1, v1, _, _, _ = orc.plif_rf_fwd(g["beta"], z, g["u"], g["vth"], g["v_init"], z[0])
    s2, v2, _ = orc.plif_selective_fwd(g["beta"], g["u"], g["vth"], g["v_init"])
    assert np.array_equal(s1, s2) and np.array_equal(v1, v2)


def _ulp_distance(a, b):
    ai = np.asarray(a, np.float32).view(np.int32).astype(np.int64)
    bi = np.asarray(b, np.float32).view(np.int32).astype(np.int64)
    return np.abs(ai - bi)


@pytest.mark.parametrize("name", ["modulation_rf", "modulation_first_order"])
def test_modulation(golden, name):
    """The reference evaluates sigmoid / softplus / rsqrt with PyTorch's vectorised CPU
    routines (1-2 ulp each); the oracle rounds a double evaluation once. Allowed distance:
    4 ulp on the modulated values, |z| + v_th_min exact; gradients 1e-6 of the largest."""
    g = golden(name)
    rf = "raw_omega" in g
    extra = dict(raw_omega=g["raw_omega"], b_omega=g["b_omega"]) if rf else {}
    out = orc.modulation_fwd(g["raw_beta"], g["raw_alpha"], g["raw_th"], g["cur"], g["b_beta"], g["b_alpha"],
                             g["b_th"], float(g["v_th_min"]), **extra)
    for mine, ref in zip(out, ("beta", "u", "vth", "omega")):
        assert _ulp_distance(mine, g[ref]).max() <= 4, ref
    assert np.array_equal(out[2], g["vth"])
    if rf:
        extra["g_omega"] = g["g_omega"]
        # the stability rescale is exercised on both sides of its threshold
        r2 = g["beta"].astype(np.float64) ** 2 + g["omega"].astype(np.float64) ** 2
        assert (r2 > 0.9979).any() and (r2 < 0.99).any()
    grads = orc.modulation_bwd(g["raw_beta"], g["raw_alpha"], g["raw_th"], g["cur"], g["b_beta"], g["b_alpha"],
                               g["b_th"], g["g_beta"], g["g_u"], g["g_vth"], **extra)
    for k, v in grads.items():
        if v is not None:
            assert rel_err(v, g["grad_" + k]) < 1e-6, k
    # rounding the modulated values to bf16 is the fp32 result rounded once
    import torch
    outb = orc.modulation_fwd(g["raw_beta"], g["raw_alpha"], g["raw_th"], g["cur"], g["b_beta"], g["b_alpha"],
                              g["b_th"], float(g["v_th_min"]), mod_round="bf16",
                              **{k: v for k, v in extra.items() if k != "g_omega"})
    for a, b in zip(out, outb):
        assert np.array_equal(torch.from_numpy(a).bfloat16().float().numpy(), b)
    outh = orc.modulation_fwd(g["raw_beta"], g["raw_alpha"], g["raw_th"], g["cur"], g["b_beta"], g["b_alpha"],
                              g["b_th"], float(g["v_th_min"]), mod_round="f16",
                              **{k: v for k, v in extra.items() if k != "g_omega"})
    for a, b in zip(out, outh):
        assert np.array_equal(torch.from_numpy(a).half().float().numpy(), b)


def test_surrogate_alpha(golden):
    g = golden("surrogate_alpha")
    for i in range(int(g["n"])):
        storage = ("f32", "bf16", "f16")[int(g[f"dtype{i}"])]
        mine = orc.surrogate_alpha(g[f"u{i}"], float(g["alpha_0"]), float(g["sigma_0"]), storage)
        assert abs(mine - float(g[f"alpha{i}"])) <= 2e-6 * float(g[f"alpha{i}"]), (i, mine, float(g[f"alpha{i}"]))


def test_linear_recurrence(golden):
    """The reference's CPU branch is a Hillis-Steele scan (another association of the same
    products), so the comparison is to a tolerance: 1e-5 of the largest value."""
    g = golden("linrec_a")
    V = orc.linear_recurrence_fwd(g["beta"], g["u"], g["v_init"])
    assert rel_err(V, g["V"]) < TOL
    gb, gu, gv0 = orc.linear_recurrence_bwd(g["beta"], g["u"], g["v_init"], g["g_V"])
    assert rel_err(gb, g["g_beta"]) < TOL and rel_err(gu, g["g_u"]) < TOL and rel_err(gv0, g["g_vinit"]) < TOL


def test_moe_combine(golden):
    g = golden("moe_a")
    assert rel_err(orc.moe_combine_fwd(g["shared"], g["experts"], g["weights"]), g["out"]) < TOL
    ge, gw = orc.moe_combine_bwd(g["g_out"], g["experts"], g["weights"])
    assert rel_err(ge, g["g_experts"]) < TOL and rel_err(gw, g["g_weights"]) < TOL
    assert np.array_equal(g["g_shared"], g["g_out"])


@pytest.mark.parametrize("tag", ["f32", "bf16"])
def test_frames_combine(golden, tag):
    """Expert merge in the frame domain against the reference's own decode / weighted sum / add /
    binary_encode_ste sequence: the re-encoded frames and the value they encode must be identical
    (every rounding of the reference's tensor arithmetic is restated); gradients to a tolerance
    (fp32: 1e-5 of the largest; bf16: the reference's autograd rounds every intermediate to bf16,
    so 2^-6 of the largest)."""
    g = golden(f"frames_combine_{tag}")
    out, total = orc.frames_combine_fwd(g["shared"], g["experts"], g["weights"], g["residual"], storage=tag)
    assert np.array_equal(total, g["total"])
    assert np.array_equal(out, g["out"])
    gs, ge, gw, gr = orc.frames_combine_bwd(g["g_out"], g["shared"], g["experts"], g["weights"], g["residual"],
                                            storage=tag)
    tol = TOL if tag == "f32" else 2.0 ** -6
    assert rel_err(gs, g["g_shared"]) < tol and rel_err(gr, g["g_residual"]) < tol
    assert rel_err(ge, g["g_experts"]) < tol and rel_err(gw, g["g_weights"]) < tol
