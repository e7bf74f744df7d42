"""Python face of the CPU oracle (``plif_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by the test suite, by the smoke check and by
the benchmark's CPU-baseline leg, never by the shipped package. Parity of the
C restatement against the reference is pinned by the committed golden vectors
(see ``tests/golden/make_golden.py``); the arctangent surrogate, which the reference's fused
kernels lack, is pinned to torch autograd through its published primitive by the same script.

Every function takes and returns ``numpy.float32`` arrays in the reference's
layouts: scans are time-major ``[T, ...]`` with the trailing dims flattened to
columns, codec frames are ``[S*16, B, D]``, codec values are ``[B, S, D]``.
Low-precision inputs must be widened to fp32 by the caller (exact), which is
what the reference's kernels do per load (atomic_ops/parallel_scan.py:223-225).
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_SRC = _HERE / "plif_oracle.c"
_LIB = _HERE / "liborc.so"

SURR_SIGMOID = 0
SURR_ATAN = 1

_lib = None


def build(force: bool = False) -> Path:
    """Compile the C restatement with gcc (no FMA contraction, OpenMP)."""
    if force or not _LIB.exists() or _LIB.stat().st_mtime < _SRC.stat().st_mtime:
        cmd = ["gcc", "-O3", "-mavx2", "-ffp-contract=off", "-fopenmp", "-shared",
               "-fPIC", "-Wall", "-o", str(_LIB), str(_SRC), "-lm"]
        subprocess.run(cmd, check=True)
    return _LIB


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not _LIB.exists():
            build()
        _lib = ctypes.CDLL(str(_LIB))
        _lib.orc_max_threads.restype = ctypes.c_int
    return _lib


def max_threads() -> int:
    return int(lib().orc_max_threads())


def set_threads(n: int) -> None:
    lib().orc_set_threads(ctypes.c_int(int(n)))


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a, dtype=np.float32))


def _p(a):
    if a is None:
        return ctypes.c_void_p(0)
    return a.ctypes.data_as(ctypes.c_void_p)


def _i64(x) -> ctypes.c_int64:
    return ctypes.c_int64(int(x))


def _tc(a: np.ndarray):
    T = a.shape[0]
    cols = int(np.prod(a.shape[1:])) if a.ndim > 1 else 1
    return T, cols


# ---------------------------------------------------------------- scans


def plif_selective_fwd(beta, u, vth, v_init, want_vpost=True):
    """(spike [T,...], V_post [T,...] or None, V_last [...]) — u-form."""
    beta, u, vth, v_init = _f32(beta), _f32(u), _f32(vth), _f32(v_init)
    T, cols = _tc(u)
    spike = np.empty_like(u)
    vpost = np.empty_like(u) if want_vpost else None
    vlast = np.empty_like(v_init)
    lib().orc_plif_selective_fwd(_p(beta), _p(u), _p(vth), _p(v_init), _p(spike),
                                 _p(vpost), _p(vlast), _i64(T), _i64(cols))
    return spike, vpost, vlast


def plif_selective_ai_fwd(beta, cur, gain, vth, v_init, want_vpost=True, out=None):
    """Selective scan with separate write gain and current (alpha*I form).
    ``out`` = (spike, vpost-or-None, vlast) reuses caller buffers (timing loops)."""
    beta, cur, gain, vth, v_init = map(_f32, (beta, cur, gain, vth, v_init))
    T, cols = _tc(cur)
    if out is not None:
        spike, vpost, vlast = out
    else:
        spike = np.empty_like(cur)
        vpost = np.empty_like(cur) if want_vpost else None
        vlast = np.empty_like(v_init)
    lib().orc_plif_selective_ai_fwd(_p(beta), _p(cur), _p(gain), _p(vth), _p(v_init),
                                    _p(spike), _p(vpost), _p(vlast), _i64(T), _i64(cols))
    return spike, vpost, vlast


def plif_rowparam_fwd(beta_row, u, vth_row, v_init, want_vpost=True):
    beta_row, u, vth_row, v_init = map(_f32, (beta_row, u, vth_row, v_init))
    T, cols = _tc(u)
    assert beta_row.size == cols and vth_row.size == cols and v_init.size == cols
    spike = np.empty_like(u)
    vpost = np.empty_like(u) if want_vpost else None
    vlast = np.empty_like(v_init)
    lib().orc_plif_rowparam_fwd(_p(beta_row), _p(u), _p(vth_row), _p(v_init), _p(spike),
                                _p(vpost), _p(vlast), _i64(T), _i64(cols))
    return spike, vpost, vlast


def plif_selective_bwd(beta, u, vth, v_init, g_spike, g_vpost, alpha, kind=SURR_SIGMOID):
    """(g_beta, g_u, g_vth, g_vinit). g_spike / g_vpost may be None."""
    beta, u, vth, v_init = map(_f32, (beta, u, vth, v_init))
    g_spike = None if g_spike is None else _f32(g_spike)
    g_vpost = None if g_vpost is None else _f32(g_vpost)
    T, cols = _tc(u)
    gb, gu, gt = np.empty_like(u), np.empty_like(u), np.empty_like(u)
    gv = np.empty_like(v_init)
    lib().orc_plif_selective_bwd(_p(beta), _p(u), _p(vth), _p(v_init), _p(g_spike),
                                 _p(g_vpost), _p(gb), _p(gu), _p(gt), _p(gv), _i64(T),
                                 _i64(cols), ctypes.c_double(alpha), ctypes.c_int(kind))
    return gb, gu, gt, gv


def plif_selective_ai_bwd(beta, cur, gain, vth, v_init, g_spike, g_vpost, alpha,
                          kind=SURR_SIGMOID, out=None):
    """(g_beta, g_cur, g_gain, g_vth, g_vinit). ``out`` reuses caller buffers."""
    beta, cur, gain, vth, v_init = map(_f32, (beta, cur, gain, vth, v_init))
    g_spike = None if g_spike is None else _f32(g_spike)
    g_vpost = None if g_vpost is None else _f32(g_vpost)
    T, cols = _tc(cur)
    if out is not None:
        gb, gc, gg, gt, gv = out
    else:
        gb, gc, gg, gt = (np.empty_like(cur) for _ in range(4))
        gv = np.empty_like(v_init)
    lib().orc_plif_selective_ai_bwd(_p(beta), _p(cur), _p(gain), _p(vth), _p(v_init),
                                    _p(g_spike), _p(g_vpost), _p(gb), _p(gc), _p(gg),
                                    _p(gt), _p(gv), _i64(T), _i64(cols),
                                    ctypes.c_double(alpha), ctypes.c_int(kind))
    return gb, gc, gg, gt, gv


def plif_rowparam_bwd(beta_row, u, vth_row, v_init, g_spike, g_vpost, alpha,
                      kind=SURR_SIGMOID):
    """(g_beta_row, g_u, g_vth_row, g_vinit)."""
    beta_row, u, vth_row, v_init = map(_f32, (beta_row, u, vth_row, v_init))
    g_spike = None if g_spike is None else _f32(g_spike)
    g_vpost = None if g_vpost is None else _f32(g_vpost)
    T, cols = _tc(u)
    gb, gt, gv = np.empty_like(v_init), np.empty_like(v_init), np.empty_like(v_init)
    gu = np.empty_like(u)
    lib().orc_plif_rowparam_bwd(_p(beta_row), _p(u), _p(vth_row), _p(v_init), _p(g_spike),
                                _p(g_vpost), _p(gb), _p(gu), _p(gt), _p(gv), _i64(T),
                                _i64(cols), ctypes.c_double(alpha), ctypes.c_int(kind))
    return gb, gu, gt, gv


def plif_rf_fwd(beta, omega, u, vth, v_init, w_init, want_states=True):
    """Resonate-and-fire scan: (spike, V_post or None, W or None, V_last, W_last)."""
    beta, omega, u, vth, v_init, w_init = map(_f32, (beta, omega, u, vth, v_init, w_init))
    T, cols = _tc(u)
    spike = np.empty_like(u)
    vpost = np.empty_like(u) if want_states else None
    wout = np.empty_like(u) if want_states else None
    vlast, wlast = np.empty_like(v_init), np.empty_like(w_init)
    lib().orc_plif_rf_fwd(_p(beta), _p(omega), _p(u), _p(vth), _p(v_init), _p(w_init), _p(spike),
                          _p(vpost), _p(wout), _p(vlast), _p(wlast), _i64(T), _i64(cols))
    return spike, vpost, wout, vlast, wlast


def plif_rf_bwd(beta, omega, u, vth, v_init, w_init, g_spike, g_vpost, alpha, kind=SURR_SIGMOID):
    """(g_beta, g_omega, g_u, g_vth, g_vinit, g_winit)."""
    beta, omega, u, vth, v_init, w_init = map(_f32, (beta, omega, u, vth, v_init, w_init))
    g_spike = None if g_spike is None else _f32(g_spike)
    g_vpost = None if g_vpost is None else _f32(g_vpost)
    T, cols = _tc(u)
    gb, go, gu, gt = (np.empty_like(u) for _ in range(4))
    gv, gw = np.empty_like(v_init), np.empty_like(w_init)
    lib().orc_plif_rf_bwd(_p(beta), _p(omega), _p(u), _p(vth), _p(v_init), _p(w_init), _p(g_spike),
                          _p(g_vpost), _p(gb), _p(go), _p(gu), _p(gt), _p(gv), _p(gw), _i64(T),
                          _i64(cols), ctypes.c_double(alpha), ctypes.c_int(kind))
    return gb, go, gu, gt, gv, gw


# ------------------------------------------------------------ linear recurrence


def linear_recurrence_fwd(beta, u, v_init):
    """V [T, ...] of V[k] = beta[k]*V[k-1] + u[k] (atomic_ops/parallel_scan.py:1282-1302)."""
    beta, u, v_init = map(_f32, (beta, u, v_init))
    T, cols = _tc(u)
    out = np.empty_like(u)
    lib().orc_linear_recurrence_fwd(_p(beta), _p(u), _p(v_init), _p(out), _i64(T), _i64(cols))
    return out


def linear_recurrence_bwd(beta, u, v_init, g_v):
    """(g_beta, g_u, g_vinit) for a gradient arriving on V."""
    beta, u, v_init, g_v = map(_f32, (beta, u, v_init, g_v))
    T, cols = _tc(u)
    gb, gu = np.empty_like(u), np.empty_like(u)
    gv0 = np.empty_like(v_init)
    lib().orc_linear_recurrence_bwd(_p(beta), _p(u), _p(v_init), _p(g_v), _p(gb), _p(gu), _p(gv0),
                                    _i64(T), _i64(cols))
    return gb, gu, gv0


# ------------------------------------------------------------------ MoE combine


def moe_combine_fwd(shared, experts, weights):
    """out (N, D) = shared + sum_e experts[e] * weights[:, e] (atomic_ops/moe_kernels.py:210-224)."""
    shared, experts, weights = map(_f32, (shared, experts, weights))
    E, N, D = experts.shape
    out = np.empty_like(shared)
    lib().orc_moe_combine_fwd(_p(shared), _p(experts), _p(weights), _p(out), _i64(N), _i64(D), _i64(E))
    return out


def moe_combine_bwd(g_out, experts, weights):
    """(g_experts (E, N, D), g_weights (N, E)); the gradient of ``shared`` is ``g_out``."""
    g_out, experts, weights = map(_f32, (g_out, experts, weights))
    E, N, D = experts.shape
    ge, gw = np.empty_like(experts), np.empty_like(weights)
    lib().orc_moe_combine_bwd(_p(g_out), _p(experts), _p(weights), _p(ge), _p(gw), _i64(N), _i64(D), _i64(E))
    return ge, gw


# ------------------------------------------------------- adaptive surrogate slope


def surrogate_alpha(u, alpha0, sigma0, storage="f32"):
    """``clamp(alpha0 * sigma0 / max(std(u), 1e-6), 1, 20)`` as PLIFNode.get_surrogate computes it
    (atomic_ops/plif_node.py:93-100): unbiased std; ``u.std()`` of a bf16 / fp16 tensor is itself a
    bf16 / fp16 number, and so is the 1e-6 floor."""
    import torch
    dt = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}[storage]
    x = np.asarray(u, dtype=np.float64).ravel()
    sd = float(np.std(x, ddof=1)) if x.size > 1 else 0.0
    rnd = lambda v: float(torch.tensor(v, dtype=torch.float64).to(torch.float32).to(dt).double())
    sd = max(rnd(sd), rnd(1e-6))
    return float(np.float32(min(max(alpha0 * sigma0 / sd, 1.0), 20.0)))


# ---------------------------------------------------------------- codec


# ----------------------------------------------------------- modulation

MOD_ROUND = {None: 0, "f32": 0, "bf16": 1, "f16": 2}


def modulation_fwd(raw_beta, raw_alpha, raw_th, cur, b_beta, b_alpha, b_th, v_th_min,
                   raw_omega=None, b_omega=None, mod_round=None):
    """(beta, u, v_th[, omega]) from raw projections ``[..., ch]`` and biases ``[ch]``
    (atomic_ops/snn_block.py:52-76; first-order form without ``raw_omega``)."""
    raw_beta, raw_alpha, raw_th, cur = map(_f32, (raw_beta, raw_alpha, raw_th, cur))
    b_beta, b_alpha, b_th = map(_f32, (b_beta, b_alpha, b_th))
    rf = raw_omega is not None
    raw_omega = _f32(raw_omega) if rf else None
    b_omega = _f32(b_omega) if rf else None
    ch = b_beta.size
    rows = cur.size // ch
    beta, u, vth = np.empty_like(cur), np.empty_like(cur), np.empty_like(cur)
    omega = np.empty_like(cur) if rf else None
    lib().orc_modulation_fwd(_p(raw_beta), _p(raw_alpha), _p(raw_th), _p(raw_omega), _p(cur),
                             _p(b_beta), _p(b_alpha), _p(b_th), _p(b_omega),
                             ctypes.c_float(v_th_min), _i64(rows), _i64(ch),
                             ctypes.c_int(MOD_ROUND[mod_round]), _p(beta), _p(u), _p(vth), _p(omega))
    return (beta, u, vth, omega) if rf else (beta, u, vth)


def modulation_bwd(raw_beta, raw_alpha, raw_th, cur, b_beta, b_alpha, b_th, g_beta, g_u, g_vth,
                   raw_omega=None, b_omega=None, g_omega=None):
    """Gradients of the raw projections, of I and of the biases given the gradients of the
    modulated values. Returns a dict (bias gradients as float64 ``[ch]``)."""
    raw_beta, raw_alpha, raw_th, cur = map(_f32, (raw_beta, raw_alpha, raw_th, cur))
    b_beta, b_alpha, b_th = map(_f32, (b_beta, b_alpha, b_th))
    g_beta, g_u, g_vth = map(_f32, (g_beta, g_u, g_vth))
    rf = raw_omega is not None
    raw_omega = _f32(raw_omega) if rf else None
    b_omega = _f32(b_omega) if rf else None
    g_omega = _f32(g_omega) if rf else None
    ch = b_beta.size
    rows = cur.size // ch
    out = {k: np.empty_like(cur) for k in ("raw_beta", "raw_alpha", "raw_th", "cur")}
    out["raw_omega"] = np.empty_like(cur) if rf else None
    for k in ("b_beta", "b_alpha", "b_th"):
        out[k] = np.zeros(ch, dtype=np.float64)
    out["b_omega"] = np.zeros(ch, dtype=np.float64) if rf else None
    lib().orc_modulation_bwd(_p(raw_beta), _p(raw_alpha), _p(raw_th), _p(raw_omega), _p(cur),
                             _p(b_beta), _p(b_alpha), _p(b_th), _p(b_omega), _i64(rows), _i64(ch),
                             _p(g_beta), _p(g_u), _p(g_vth), _p(g_omega), _p(out["raw_beta"]),
                             _p(out["raw_alpha"]), _p(out["raw_th"]), _p(out["raw_omega"]),
                             _p(out["cur"]), _p(out["b_beta"]), _p(out["b_alpha"]), _p(out["b_th"]),
                             _p(out["b_omega"]))
    return out


def modulated_scan_fwd(raw_beta, raw_alpha, raw_th, cur, b_beta, b_alpha, b_th, v_th_min, v_init,
                       raw_omega=None, b_omega=None, w_init=None, mod_round=None):
    """Modulation followed by the selective scan (u-form) or the resonate-and-fire scan:
    what ``SNNBlock.forward_parallel`` computes between its projections and ``W_out``
    (atomic_ops/snn_block.py:237-256). Returns the scan's outputs and the modulated values."""
    mod = modulation_fwd(raw_beta, raw_alpha, raw_th, cur, b_beta, b_alpha, b_th, v_th_min,
                         raw_omega, b_omega, mod_round)
    if raw_omega is None:
        beta, u, vth = mod
        return plif_selective_fwd(beta, u, vth, v_init), mod
    beta, u, vth, omega = mod
    return plif_rf_fwd(beta, omega, u, vth, v_init, w_init), mod


def modulated_scan_bwd(raw_beta, raw_alpha, raw_th, cur, b_beta, b_alpha, b_th, v_th_min, v_init,
                       g_spike, alpha, raw_omega=None, b_omega=None, w_init=None, kind=SURR_SIGMOID,
                       mod_round=None):
    """Adjoint of ``modulated_scan_fwd`` for a gradient arriving on the spikes. Returns the
    dict of ``modulation_bwd`` plus ``v_init`` (and ``w_init``)."""
    mod = modulation_fwd(raw_beta, raw_alpha, raw_th, cur, b_beta, b_alpha, b_th, v_th_min,
                         raw_omega, b_omega, mod_round)
    if raw_omega is None:
        beta, u, vth = mod
        gb, gu, gt, gv = plif_selective_bwd(beta, u, vth, v_init, g_spike, None, alpha, kind)
        out = modulation_bwd(raw_beta, raw_alpha, raw_th, cur, b_beta, b_alpha, b_th, gb, gu, gt)
        out["v_init"] = gv
        return out
    beta, u, vth, omega = mod
    gb, go, gu, gt, gv, gw = plif_rf_bwd(beta, omega, u, vth, v_init, w_init, g_spike, None, alpha, kind)
    out = modulation_bwd(raw_beta, raw_alpha, raw_th, cur, b_beta, b_alpha, b_th, gb, gu, gt,
                         raw_omega, b_omega, go)
    out["v_init"], out["w_init"] = gv, gw
    return out


def fp16_encode(emb):
    """[B,S,D] values -> [S*16,B,D] frames in {0,1}."""
    emb = _f32(emb)
    B, S, D = emb.shape
    frames = np.empty((S * 16, B, D), np.float32)
    lib().orc_fp16_encode(_p(emb), _p(frames), _i64(B), _i64(S), _i64(D))
    return frames


def fp16_decode(frames, bf16_intermediates=False):
    """[S*16,B,D] frames -> [B,S,D] values."""
    frames = _f32(frames)
    TK, B, D = frames.shape
    S = TK // 16
    out = np.empty((B, S, D), np.float32)
    lib().orc_fp16_decode(_p(frames), _p(out), _i64(B), _i64(S), _i64(D),
                          ctypes.c_int(1 if bf16_intermediates else 0))
    return out


def fp16_decode_bwd(frames, g_out):
    frames, g_out = _f32(frames), _f32(g_out)
    TK, B, D = frames.shape
    S = TK // 16
    g = np.empty_like(frames)
    lib().orc_fp16_decode_bwd(_p(frames), _p(g_out), _p(g), _i64(B), _i64(S), _i64(D))
    return g


def binary_residual(fa, fb, bf16_intermediates=False, bf16_compiled=False):
    """encode(decode(fa) + decode(fb)). For bf16 frames the reference has two behaviours:
    ``bf16_intermediates`` = its ops run one by one (every intermediate rounded to bf16),
    ``bf16_compiled`` = its torch.compile'd residual as a GPU evaluates it (decode in fp32, the
    sum rounded to bf16). Neither flag = fp32 / fp16 frames (no intermediate rounds there)."""
    fa, fb = _f32(fa), _f32(fb)
    TK, B, D = fa.shape
    out = np.empty_like(fa)
    mode = 2 if bf16_compiled else (1 if bf16_intermediates else 0)
    lib().orc_binary_residual(_p(fa), _p(fb), _p(out), _i64(B), _i64(TK // 16), _i64(D),
                              ctypes.c_int(mode))
    return out


def encode_ste_bwd(g_frames):
    g_frames = _f32(g_frames)
    TK, B, D = g_frames.shape
    S = TK // 16
    g = np.empty((B, S, D), np.float32)
    lib().orc_encode_ste_bwd(_p(g_frames), _p(g), _i64(B), _i64(S), _i64(D))
    return g


def _round_storage(x, storage):
    """fp32 array rounded through the storage dtype ("f32", "bf16" or "f16"), nearest even."""
    x = np.ascontiguousarray(x, np.float32)
    if storage == "bf16":
        u = x.view(np.uint32).astype(np.uint64)
        u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
        return u.astype(np.uint32).view(np.float32)
    if storage == "f16":
        return x.astype(np.float16).astype(np.float32)
    return x


def frames_combine_fwd(shared, experts, weights, residual, storage="f32"):
    """(out frames (T*16, B, D), total (B, T, D)) of the expert merge in the frame domain
    (atomic_ops/moe_snn_ffn.py:377-393): every product, the sum over the experts (accumulated in
    fp32 in expert order, as a sum over the leading dimension is) and both additions rounded to the
    tensors' dtype. weights is the reference's full_weights, (T, B, E)."""
    rnd = lambda a: _round_storage(a, storage)
    dec = lambda f: rnd(fp16_decode(f, bf16_intermediates=(storage == "bf16")))
    weights = _f32(weights)
    acc = np.zeros_like(dec(shared))
    for e in range(len(experts)):
        w = weights[:, :, e].T[:, :, None]          # (B, T, 1)
        acc = (acc + rnd(dec(experts[e]) * w)).astype(np.float32)
    total = rnd(rnd(dec(shared) + rnd(acc)) + dec(residual))
    return fp16_encode(total), total


def frames_combine_bwd(g_out, shared, experts, weights, residual, storage="f32"):
    """(g_shared, g_experts, g_weights, g_residual): straight-through encode (mean over the 16 frame
    gradients, atomic_ops/fp16_codec.py:222-226), then the decode adjoint of every stream."""
    rnd = lambda a: _round_storage(a, storage)
    weights = _f32(weights)
    g_total = rnd(encode_ste_bwd(g_out))
    g_shared, g_res = fp16_decode_bwd(shared, g_total), fp16_decode_bwd(residual, g_total)
    g_exp, g_w = [], np.zeros_like(weights)
    for e in range(len(experts)):
        w = weights[:, :, e].T[:, :, None]
        g_exp.append(fp16_decode_bwd(experts[e], rnd(g_total * w)))
        val = rnd(fp16_decode(experts[e], bf16_intermediates=(storage == "bf16")))
        g_w[:, :, e] = (g_total.astype(np.float64) * val).sum(-1).T
    g_exp = np.stack(g_exp) if g_exp else np.zeros((0,) + g_shared.shape, np.float32)
    return g_shared, g_exp, rnd(g_w), g_res


# ---------------------------------------------------------------- normaliser


def li_fwd(x, gain, eps=1e-6):
    x, gain = _f32(x), _f32(gain)
    D = x.shape[-1]
    out = np.empty_like(x)
    lib().orc_li_fwd(_p(x), _p(gain), _p(out), _i64(x.size // D), _i64(D),
                     ctypes.c_double(eps))
    return out


def li_bwd(g_out, x, gain, eps=1e-6):
    g_out, x, gain = _f32(g_out), _f32(x), _f32(gain)
    D = x.shape[-1]
    gx = np.empty_like(x)
    gg = np.empty(D, np.float64)
    lib().orc_li_bwd(_p(g_out), _p(x), _p(gain), _p(gx), _p(gg), _i64(x.size // D),
                     _i64(D), ctypes.c_double(eps))
    return gx, gg


if __name__ == "__main__":
    print(build(force=True))
