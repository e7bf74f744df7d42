"""Helpers shared by the GPU parity tests: seeded inputs with the benchmark
configurations' distributions, oracle adapters and the acceptance rules."""
from __future__ import annotations

import numpy as np
import torch

from oracle import oracle as orc

#: fp32 tolerance on membrane state and gradients, relative to the largest
#: magnitude of the reference tensor (the measure the reference's own check
#: uses, exp/verify_fused_plif.py:62-63) and applied element-wise with that scale.
REL_TOL = 1e-5


def f32(t: torch.Tensor) -> np.ndarray:
    return t.detach().float().cpu().numpy()


def selective_inputs(T, B, D, dtype, device, seed=1234, zero_init=True):
    """I ~ N(0,1); beta = sigmoid(N(2,0.5)); gain = softplus(N(0,1));
    v_th = 0.1 + softplus(N(0,1)); all per (t,b,d), rounded to `dtype`."""
    g = torch.Generator(device=device).manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g, device=device, dtype=torch.float32)
    cur = rn(T, B, D)
    beta = torch.sigmoid(2 + 0.5 * rn(T, B, D))
    gain = torch.nn.functional.softplus(rn(T, B, D))
    vth = 0.1 + torch.nn.functional.softplus(rn(T, B, D))
    v0 = torch.zeros(B, D, device=device) if zero_init else 0.1 * rn(B, D)
    return tuple(t.to(dtype) for t in (beta, cur, gain, vth)) + (v0,)


def rowparam_inputs(T, B, D, dtype, device, seed=1234):
    """Per-channel beta = sigmoid(N(2,0.5)), v_th = max(0.05, 0.5+0.1 N(0,1)),
    I ~ N(0,1), u = (1-beta)*I formed by the caller as the reference does
    (atomic_ops/snn_ffn.py:182)."""
    g = torch.Generator(device=device).manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g, device=device, dtype=torch.float32)
    bd = torch.sigmoid(2 + 0.5 * rn(D))
    td = (0.5 + 0.1 * rn(D)).clamp(min=0.05)
    cur = rn(T, B, D).to(dtype)
    u = ((1 - bd) * cur.float()).to(dtype)
    beta_row = bd.expand(B, D).contiguous()
    vth_row = td.expand(B, D).contiguous()
    v0 = torch.zeros(B, D, device=device)
    return beta_row, u, vth_row, v0


def assert_close(actual, expected, tol=REL_TOL, what=""):
    a = np.asarray(actual, np.float64)
    e = np.asarray(expected, np.float64)
    assert a.shape == e.shape, f"{what}: shape {a.shape} vs {e.shape}"
    scale = np.abs(e).max() + 1e-30
    err = np.abs(a - e).max() / scale
    assert err <= tol, f"{what}: relative error {err:.3e} > {tol:.1e}"


def assert_close_lowp(actual, expected, dtype, what="", scale=None):
    """Outputs stored in bf16/fp16: the kernel's fp32 value may round to the
    neighbouring representable number, so allow one unit in the last place
    (2^-8 for bf16, 2^-11 for fp16, relative) on top of REL_TOL."""
    ulp = {torch.bfloat16: 2.0 ** -8, torch.float16: 2.0 ** -11, torch.float32: 0.0}[dtype]
    a = np.asarray(actual, np.float64)
    e = np.asarray(expected, np.float64)
    if scale is None:
        scale = np.abs(e).max() + 1e-30
    if dtype == torch.float16:
        # values at the edge of the half range store as 65504 or inf; compare the rest
        keep = np.abs(e) < 65504.0 * (1 - 2.0 ** -11)
        a, e = a[keep], e[keep]
    # fp16 stores small magnitudes as subnormals with a fixed spacing of 2^-24
    floor = 2.0 ** -24 if dtype == torch.float16 else 0.0
    bound = ulp * np.abs(e) + REL_TOL * scale + floor
    bad = np.abs(a - e) > bound
    assert not bad.any(), (f"{what}: {bad.sum()} of {bad.size} elements off by more than one "
                           f"{dtype} ulp; worst {np.abs(a - e).max():.3e}")


def assert_spikes_match(spike, ref_spike, ref_vpost, vth, what="", margin=1e-5):
    """Spikes must be bit-exact, except that a lane may diverge from the first
    step at which |V_pre - V_th| < margin*|V_th| in the oracle (a legitimately
    ambiguous threshold crossing changes that lane's future)."""
    s = np.asarray(spike, np.float32).reshape(ref_spike.shape[0], -1)
    r = np.asarray(ref_spike, np.float32).reshape(s.shape)
    if np.array_equal(s, r):
        return 0
    vp = np.asarray(ref_vpost, np.float32).reshape(s.shape)
    th = np.broadcast_to(np.asarray(vth, np.float32), ref_spike.shape).reshape(s.shape)
    x = vp - th * (1.0 - r)  # V_pre - V_th
    near = np.abs(x) < margin * np.abs(th)
    ambiguous_from = np.where(near.any(0), near.argmax(0), s.shape[0])
    mism = s != r
    first_bad = np.where(mism.any(0), mism.argmax(0), s.shape[0])
    illegal = first_bad < ambiguous_from
    assert not illegal.any(), (f"{what}: {illegal.sum()} lanes differ from the oracle before any "
                               f"near-threshold step ({mism.sum()} spike mismatches in total)")
    return int(mism.any(0).sum())


def oracle_selective(beta, drive, gain, vth, v0):
    """(spike, V_post, V_last) from the CPU oracle on widened copies of the inputs."""
    if gain is None:
        return orc.plif_selective_fwd(f32(beta), f32(drive), f32(vth), f32(v0))
    return orc.plif_selective_ai_fwd(f32(beta), f32(drive), f32(gain), f32(vth), f32(v0))
