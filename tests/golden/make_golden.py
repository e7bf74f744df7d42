"""Generate the golden vectors under tests/golden/ from the reference's own code.

Run once, where the reference checkout and PyTorch (CPU) are available; the
checkout's path comes from the first argument or from NEURONSPARK_REF:

    python tests/golden/make_golden.py <path to the NeuronSpark checkout>

The reference's ``atomic_ops`` package cannot be imported as a package here
(it depends on SpikingJelly, which is not installed), so the two files that
matter are loaded by path: ``parallel_scan.py`` and ``fp16_codec.py`` import
only torch at module level.

What each fixture is produced by:
  scan_fwd_*      rf_plif_parallel_forward(..., omega=0, w_init=0,
                  surrogate_function=None): the reference's executable CPU time
                  loop (atomic_ops/parallel_scan.py:1655-1683), which with
                  omega = 0 is the first-order selective scan.
  scan_bwd_*      torch autograd through the loop the reference's own test
                  uses as ground truth (exp/verify_fused_plif.py:111-124: hard
                  spike detached in the reset, surrogate spike as output), with
                  a local sigmoid surrogate that restates SpikingJelly's
                  (heaviside forward, alpha*sig*(1-sig) backward).
  scan_ai_*       the same loop with v_pre = beta*v + alpha*x
                  (atomic_ops/selective_plif.py:127).
  scan_ai_bwd_atan the same loop with the arctangent surrogate (BASELINE config 2: atan,
                  alpha = 2; the reference's fused kernels have sigmoid only). The surrogate is
                  given by its PRIMITIVE, g(x) = atan(pi/2 * alpha * x) / pi + 1/2 (the published
                  form of SpikingJelly's ATan), and torch autograd derives g' from it: no
                  hand-written derivative enters the fixture. Inputs with config 2's distributions.
  rowparam_*      the same loops with per-column beta / v_th.
  codec_*         fp16_encode, fp16_decode (+ autograd), _binary_residual_fwd,
                  _binary_residual_naive, _BinaryEncodeSTE from
                  atomic_ops/fp16_codec.py, in fp32 and bf16.
  modulation_*    _fused_modulation_rf (atomic_ops/snn_block.py:52-76) and
                  _fused_modulation (archive/atomic_ops_v75_pre/snn_block.py:41-47),
                  taken out of their files by name with ``ast`` (the modules need
                  SpikingJelly to import) and run eagerly, without their
                  torch.compile decorator, + autograd.
  moe_a           moe_combine (atomic_ops/moe_kernels.py:210-224; its CPU branch) + autograd.
  frames_combine_* the training branch of MoESNNFFN.forward_parallel that merges the experts
                  (atomic_ops/moe_snn_ffn.py:377-393: fp16_decode of every stream, weighted
                  sum, + shared, + residual, binary_encode_ste), restated with the
                  reference's own fp16_decode / binary_encode_ste, in fp32 and bf16, + autograd.
  linrec_a        linear_recurrence (atomic_ops/parallel_scan.py:1282-1302; on CPU the
                  Hillis-Steele scan, :1238-1275) + autograd.
  surrogate_alpha the four lines of PLIFNode.get_surrogate that derive the slope from
                  u.std() (atomic_ops/plif_node.py:93-100; the method itself needs
                  SpikingJelly), on fp32, bf16 and fp16 tensors.
  li_*            the PyTorch fallback of LateralInhibition.forward
                  (atomic_ops/lateral_inhibition.py:208-212) + autograd.
"""
import importlib.util
import os
import sys
from pathlib import Path

import numpy as np
import torch

if len(sys.argv) < 2 and "NEURONSPARK_REF" not in os.environ:
    raise SystemExit("usage: make_golden.py <path to the NeuronSpark checkout>  (or set NEURONSPARK_REF)")
REF = Path(sys.argv[1] if len(sys.argv) > 1 else os.environ["NEURONSPARK_REF"])
OUT = Path(__file__).resolve().parent
# optional: `--only PREFIX` rewrites just the fixtures whose name starts with PREFIX
ONLY = sys.argv[sys.argv.index("--only") + 1] if "--only" in sys.argv else ""


def load(name, rel):
    spec = importlib.util.spec_from_file_location(name, REF / rel)
    m = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(m)
    return m


class SigmoidSurrogate(torch.autograd.Function):
    """heaviside(x) forward, alpha*sigmoid(alpha x)(1-sigmoid(alpha x)) backward."""

    @staticmethod
    def forward(ctx, x, alpha):
        ctx.save_for_backward(x)
        ctx.alpha = alpha
        return (x >= 0).to(x.dtype)

    @staticmethod
    def backward(ctx, g):
        (x,) = ctx.saved_tensors
        s = torch.sigmoid(ctx.alpha * x)
        return g * ctx.alpha * s * (1 - s), None


class PrimitiveSurrogate(torch.autograd.Function):
    """heaviside(x) forward; backward multiplies by the derivative of ``primitive`` at x, which
    torch autograd computes from the primitive itself."""

    @staticmethod
    def forward(ctx, x, primitive):
        ctx.save_for_backward(x)
        ctx.primitive = primitive
        return (x >= 0).to(x.dtype)

    @staticmethod
    def backward(ctx, g):
        (x,) = ctx.saved_tensors
        with torch.enable_grad():
            xx = x.detach().requires_grad_()
            (d,) = torch.autograd.grad(ctx.primitive(xx).sum(), xx)
        return g * d, None


def atan_primitive(alpha):
    import math
    return lambda x: torch.atan(math.pi / 2 * alpha * x) / math.pi + 0.5


def seq_loop(beta, u, vth, v_init, alpha, rowparam=False, gain=None, cur=None, primitive=None):
    """The reference test's ground-truth loop (exp/verify_fused_plif.py:111-124)."""
    v = v_init
    T = (u if u is not None else cur).shape[0]
    S, V = [], []
    for k in range(T):
        b = beta if rowparam else beta[k]
        th = vth if rowparam else vth[k]
        drive = u[k] if u is not None else gain[k] * cur[k]
        v_pre = b * v + drive
        sp = (v_pre.detach() >= th.detach()).to(v_pre.dtype)
        v = v_pre - th * sp
        S.append(SigmoidSurrogate.apply(v_pre - th, alpha) if primitive is None
                 else PrimitiveSurrogate.apply(v_pre - th, primitive))
        V.append(v)
    return torch.stack(S), torch.stack(V)


def function_from_source(rel, name):
    """Compiles one top-level function of a reference file, without its decorators, in a
    namespace that has only torch and torch.nn.functional."""
    import ast
    tree = ast.parse((REF / rel).read_text())
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name == name:
            node.decorator_list = []
            mod = ast.Module(body=[node], type_ignores=[])
            ns = {"torch": torch, "F": torch.nn.functional}
            exec(compile(ast.fix_missing_locations(mod), str(REF / rel), "exec"), ns)
            return ns[name]
    raise KeyError(f"{name} not found in {rel}")


def npz(name, **arrs):
    if not name.startswith(ONLY):
        return
    out = {}
    for k, v in arrs.items():
        if isinstance(v, torch.Tensor):
            v = v.detach().float().numpy()
        out[k] = np.asarray(v)
    np.savez_compressed(OUT / f"{name}.npz", **out)
    print(f"wrote {name}.npz", {k: v.shape for k, v in out.items()})


def main():
    torch.set_num_threads(1)
    ps = load("ref_parallel_scan", "atomic_ops/parallel_scan.py")
    codec = load("ref_fp16_codec", "atomic_ops/fp16_codec.py")

    # ---- forward, the distribution of exp/verify_fused_plif.py:41-46 (seed 42)
    for tag, (T, B, D) in {"a": (64, 2, 32), "b": (200, 3, 20)}.items():
        torch.manual_seed(42)
        beta = torch.sigmoid(torch.randn(T, B, D))
        u = torch.randn(T, B, D) * 0.1
        vth = 0.1 + torch.abs(torch.randn(T, B, D)) * 0.5
        v0 = torch.randn(B, D) * 0.1
        z = torch.zeros(B, D)
        s, V, _ = ps.rf_plif_parallel_forward(beta, torch.zeros_like(beta), u, vth, v0, z, None)
        npz(f"scan_fwd_{tag}", beta=beta, u=u, vth=vth, v_init=v0, spike=s, vpost=V)

    # ---- forward, BASELINE config-0 distribution at reduced size
    g = torch.Generator().manual_seed(1234)
    T, B, D = 256, 2, 40
    cur = torch.randn(T, B, D, generator=g)
    beta = torch.sigmoid(2 + 0.5 * torch.randn(T, B, D, generator=g))
    gain = torch.nn.functional.softplus(torch.randn(T, B, D, generator=g))
    vth = 0.1 + torch.nn.functional.softplus(torch.randn(T, B, D, generator=g))
    z = torch.zeros(B, D)
    u = gain * cur
    s, V, _ = ps.rf_plif_parallel_forward(beta, torch.zeros_like(beta), u, vth, z, z, None)
    with torch.no_grad():
        s_ai, V_ai = seq_loop(beta, None, vth, z, 4.0, gain=gain, cur=cur)
    assert torch.equal(s, s_ai) and torch.equal(V, V_ai)
    npz("scan_fwd_c0", beta=beta, cur=cur, gain=gain, vth=vth, v_init=z, spike=s, vpost=V)

    # ---- backward (sigmoid alpha=4), loss = sum(spike*gS) + sum(V*gV)
    torch.manual_seed(42)
    T, B, D = 64, 2, 32
    beta = torch.sigmoid(torch.randn(T, B, D)).requires_grad_()
    u = (torch.randn(T, B, D) * 0.3).requires_grad_()
    vth = (0.1 + torch.abs(torch.randn(T, B, D)) * 0.5).requires_grad_()
    v0 = (torch.randn(B, D) * 0.1).requires_grad_()
    gS = torch.randn(T, B, D)
    gV = torch.randn(T, B, D)
    S, V = seq_loop(beta, u, vth, v0, 4.0)
    ((S * gS).sum() + (V * gV).sum()).backward()
    npz("scan_bwd_a", beta=beta, u=u, vth=vth, v_init=v0, g_spike=gS, g_vpost=gV,
        alpha=np.float64(4.0), g_beta=beta.grad, g_u=u.grad, g_vth=vth.grad, g_vinit=v0.grad)
    # the reference test's own loss: spike.sum() + V_post.sum()
    for t in (beta, u, vth, v0):
        t.grad = None
    S, V = seq_loop(beta, u, vth, v0, 4.0)
    (S.sum() + V.sum()).backward()
    npz("scan_bwd_ones", beta=beta, u=u, vth=vth, v_init=v0, alpha=np.float64(4.0),
        g_beta=beta.grad, g_u=u.grad, g_vth=vth.grad, g_vinit=v0.grad)

    # ---- alpha*I form backward
    torch.manual_seed(7)
    T, B, D = 48, 2, 24
    cur = torch.randn(T, B, D).requires_grad_()
    beta = torch.sigmoid(2 + 0.5 * torch.randn(T, B, D)).requires_grad_()
    gain = torch.nn.functional.softplus(torch.randn(T, B, D)).requires_grad_()
    vth = (0.1 + torch.nn.functional.softplus(torch.randn(T, B, D))).requires_grad_()
    v0 = (torch.randn(B, D) * 0.1).requires_grad_()
    gS = torch.randn(T, B, D) * 0.1
    S, V = seq_loop(beta, None, vth, v0, 4.0, gain=gain, cur=cur)
    (S * gS).sum().backward()
    npz("scan_ai_bwd", beta=beta, cur=cur, gain=gain, vth=vth, v_init=v0, g_spike=gS,
        alpha=np.float64(4.0), spike=S, vpost=V, g_beta=beta.grad, g_cur=cur.grad,
        g_gain=gain.grad, g_vth=vth.grad, g_vinit=v0.grad)

    # ---- alpha*I form backward, arctangent surrogate (alpha = 2) through its primitive, config-2 inputs
    g = torch.Generator().manual_seed(2024)
    T, B, D = 96, 2, 48
    rn = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
    cur = rn(T, B, D).requires_grad_()
    beta = torch.sigmoid(2 + 0.5 * rn(T, B, D)).requires_grad_()
    gain = torch.nn.functional.softplus(rn(T, B, D)).requires_grad_()
    vth = (0.1 + torch.nn.functional.softplus(rn(T, B, D))).requires_grad_()
    v0 = (rn(B, D) * 0.1).requires_grad_()
    gS = rn(T, B, D) * 0.1
    # fp32-representable inputs, adjoint in double: the spikes are those of the fp32 recurrence
    # (asserted), the gradients carry no fp32 accumulation error of the generator's own
    with torch.no_grad():
        for t in (cur, beta, gain, vth, v0, gS):
            t.copy_(t.float().double())
        s32, V32 = seq_loop(beta.float(), None, vth.float(), v0.float(), 2.0, gain=gain.float(), cur=cur.float())
    S, V = seq_loop(beta, None, vth, v0, 2.0, gain=gain, cur=cur, primitive=atan_primitive(2.0))
    assert torch.equal(S.detach().float(), s32), "double and fp32 recurrences spike differently on this seed"
    (S * gS).sum().backward()
    npz("scan_ai_bwd_atan", beta=beta, cur=cur, gain=gain, vth=vth, v_init=v0, g_spike=gS,
        alpha=np.float64(2.0), spike=S, g_beta=beta.grad, g_cur=cur.grad, g_gain=gain.grad,
        g_vth=vth.grad, g_vinit=v0.grad)

    # ---- row-param, the inputs of test_recompute.py:27-31 (K=16,B=2,dim=256, seed 42)
    torch.manual_seed(42)
    K, B, D = 16, 2, 256
    beta_row = torch.sigmoid(torch.randn(B, D)).requires_grad_()
    u = torch.randn(K, B, D).requires_grad_()
    vth_row = (torch.abs(torch.randn(B, D)) + 0.1).requires_grad_()
    v0 = torch.randn(B, D).requires_grad_()
    S, V = seq_loop(beta_row, u, vth_row, v0, 4.0, rowparam=True)
    S.sum().backward()
    npz("rowparam_a", beta_row=beta_row, u=u, vth_row=vth_row, v_init=v0, alpha=np.float64(4.0),
        spike=S, vpost=V, g_beta_row=beta_row.grad, g_u=u.grad, g_vth_row=vth_row.grad,
        g_vinit=v0.grad)

    # ---- row-param, BASELINE config-1 distribution at reduced size, with gV
    g = torch.Generator().manual_seed(1234)
    T, B, D = 160, 3, 24
    bd = torch.sigmoid(2 + 0.5 * torch.randn(D, generator=g))
    td = (0.5 + 0.1 * torch.randn(D, generator=g)).clamp(min=0.05)
    beta_row = bd.expand(B, D).contiguous().requires_grad_()
    vth_row = td.expand(B, D).contiguous().requires_grad_()
    cur = torch.randn(T, B, D, generator=g)
    u = ((1 - bd) * cur).requires_grad_()
    v0 = torch.zeros(B, D).requires_grad_()
    gS = torch.randn(T, B, D, generator=g)
    gV = torch.randn(T, B, D, generator=g) * 0.1
    S, V = seq_loop(beta_row, u, vth_row, v0, 4.0, rowparam=True)
    ((S * gS).sum() + (V * gV).sum()).backward()
    npz("rowparam_c1", beta_row=beta_row, u=u, vth_row=vth_row, v_init=v0, g_spike=gS, g_vpost=gV,
        alpha=np.float64(4.0), spike=S, vpost=V, g_beta_row=beta_row.grad, g_u=u.grad,
        g_vth_row=vth_row.grad, g_vinit=v0.grad)

    # ---- resonate-and-fire scan: forward from the reference's CPU loop
    # (rf_plif_parallel_forward, surrogate None); backward from autograd through the
    # same recurrence with the hard spike detached in the reset, which is what the
    # reference's fused kernel computes (atomic_ops/parallel_scan.py:835-848).
    # Inputs as test_recompute.py:87-94 draws them, smaller (seed 42).
    torch.manual_seed(42)
    T, B, D = 48, 2, 40
    beta = torch.sigmoid(torch.randn(T, B, D))
    omega = torch.abs(torch.randn(T, B, D)) * 0.3
    u = torch.randn(T, B, D)
    vth = torch.abs(torch.randn(T, B, D)) + 0.1
    v0, w0 = torch.randn(B, D), torch.randn(B, D) * 0.1
    s, V, W = ps.rf_plif_parallel_forward(beta, omega, u, vth, v0, w0, None)
    leaves = [t.clone().requires_grad_() for t in (beta, omega, u, vth, v0, w0)]
    b_, o_, u_, t_, v, w = leaves
    S_l, V_l = [], []
    for k in range(T):
        v_pre = b_[k] * v - o_[k] * w + u_[k]
        w_new = o_[k] * v + b_[k] * w
        sp = (v_pre.detach() >= t_[k].detach()).to(v_pre.dtype)
        S_l.append(SigmoidSurrogate.apply(v_pre - t_[k], 4.0))
        v = v_pre - t_[k] * sp
        w = w_new
        V_l.append(v)
    S2, V2 = torch.stack(S_l), torch.stack(V_l)
    assert torch.equal(S2.detach(), s) and torch.equal(V2.detach(), V)
    gS = torch.randn(T, B, D)
    gV = torch.randn(T, B, D) * 0.3
    ((S2 * gS).sum() + (V2 * gV).sum()).backward()
    npz("rf_a", beta=beta, omega=omega, u=u, vth=vth, v_init=v0, w_init=w0, spike=s, vpost=V, w=W,
        g_spike=gS, g_vpost=gV, alpha=np.float64(4.0),
        **{f"g_{n}": t.grad for n, t in zip(("beta", "omega", "u", "vth", "vinit", "winit"), leaves)})

    # ---- codec: the inputs of test_binary_residual.py (seed 42) + edge values
    torch.manual_seed(42)
    B, S_, D = 2, 4, 8
    xa = torch.randn(B, S_, D).clamp(-100, 100)
    xb = torch.randn(B, S_, D).clamp(-100, 100)
    fa, fb = codec.fp16_encode(xa, 16), codec.fp16_encode(xb, 16)
    res = codec._binary_residual_fwd(fa, fb)
    assert torch.equal(res, codec._binary_residual_naive(fa, fb))
    dec = codec.fp16_decode(res, S_, 16)
    fr = fa.clone().requires_grad_()
    gout = torch.randn(B, S_, D)
    (codec.fp16_decode(fr, S_, 16) * gout).sum().backward()
    gfr = torch.randn(S_ * 16, B, D)
    xe = xa.clone().requires_grad_()
    (codec.binary_encode_ste(xe) * gfr).sum().backward()
    npz("codec_a", xa=xa, xb=xb, frames_a=fa, frames_b=fb, residual=res, decoded_residual=dec,
        decoded_a=codec.fp16_decode(fa, S_, 16), g_out=gout, g_frames=fr.grad,
        g_frames_in=gfr, g_ste=xe.grad)

    edge = torch.tensor([0.0, -0.0, 1.0, -1.0, 65504.0, -65504.0, 70000.0, -1e9, 6.1035e-05,
                         6.0e-05, 5.9605e-08, 2.9e-08, 3.0e-08, 1e-10, 0.33333334, 2049.0,
                         2051.0, 1.00048828125, 1.0009765625, 65519.9, 100.06, -3.1415927,
                         1e-5, 33000.0], dtype=torch.float32)
    edge = torch.cat([edge, torch.randn(40) * torch.logspace(-8, 4, 40)]).reshape(1, 4, 16)
    fe = codec.fp16_encode(edge, 16)
    fe2 = codec.fp16_encode(edge.flip(2) * 0.75, 16)
    # frames with an all-ones exponent (never produced by encode, legal to decode)
    f31 = fe.clone()
    f31[1:6] = 1.0
    npz("codec_edge", x=edge, frames=fe, decoded=codec.fp16_decode(fe, 4, 16),
        frames_b=fe2, residual=codec._binary_residual_fwd(fe, fe2),
        frames_e31=f31, decoded_e31=codec.fp16_decode(f31, 4, 16),
        residual_e31=codec._binary_residual_fwd(f31, fe2))

    # bf16 frames: the reference computes the decode formula in bf16
    fab, fbb = fa.bfloat16(), fb.bfloat16()
    npz("codec_bf16", frames_a=fab, frames_b=fbb, decoded_a=codec.fp16_decode(fab, S_, 16),
        residual=codec._binary_residual_fwd(fab, fbb),
        frames_e=fe.bfloat16(), decoded_e=codec.fp16_decode(fe.bfloat16(), 4, 16),
        residual_e=codec._binary_residual_fwd(fe.bfloat16(), fe2.bfloat16()))

    # ---- modulation: raw projections + biases -> beta, u, v_th (, omega)
    mod_rf = function_from_source("atomic_ops/snn_block.py", "_fused_modulation_rf")
    mod_1 = function_from_source("archive/atomic_ops_v75_pre/snn_block.py", "_fused_modulation")
    torch.manual_seed(77)
    rows, ch = 96, 40
    names = ("raw_beta", "raw_alpha", "raw_th", "raw_omega", "cur")
    raw = {n: torch.randn(rows, ch) * 1.5 for n in names}
    # softplus threshold (z > 20), saturated sigmoid, |z| at exactly 0, stability rescale on and off
    raw["raw_alpha"][0, :8] = torch.tensor([19.9, 20.0, 20.1, 25.0, -25.0, -90.0, 0.0, 60.0])
    raw["raw_beta"][1, :8] = torch.tensor([30.0, -30.0, 88.0, -88.0, -104.0, 0.0, 5.0, 9.0])
    raw["raw_omega"][2, :8] = torch.tensor([-30.0, 21.0, 0.0, -5.0, 3.0, -2.0, 0.5, -0.5])
    raw["raw_th"][3, :4] = torch.tensor([0.0, -0.0, 1e-8, -1e-8])
    bias = {"b_beta": 2.0 + 0.5 * torch.randn(ch), "b_alpha": 0.3 * torch.randn(ch),
            "b_th": 0.3 * torch.randn(ch), "b_omega": -1.0 + 0.5 * torch.randn(ch)}
    bias["b_alpha"][:8] = 0.0
    bias["b_beta"][:8] = 0.0
    bias["b_omega"][:8] = 0.0
    bias["b_th"][:4] = 0.0
    v_th_min = 0.1
    leaves = {k: v.clone().requires_grad_() for k, v in {**raw, **bias}.items()}
    beta, u, vth, omega = mod_rf(leaves["raw_beta"], leaves["b_beta"], leaves["raw_alpha"], leaves["b_alpha"],
                                 leaves["raw_th"], leaves["b_th"], v_th_min, leaves["cur"],
                                 leaves["raw_omega"], leaves["b_omega"])
    ups = {n: torch.randn(rows, ch) for n in ("g_beta", "g_u", "g_vth", "g_omega")}
    ((beta * ups["g_beta"]).sum() + (u * ups["g_u"]).sum() + (vth * ups["g_vth"]).sum()
     + (omega * ups["g_omega"]).sum()).backward()
    npz("modulation_rf", **raw, **bias, v_th_min=np.float64(v_th_min), beta=beta, u=u, vth=vth, omega=omega,
        **ups, **{f"grad_{k}": v.grad for k, v in leaves.items()})
    leaves = {k: v.clone().requires_grad_() for k, v in {**raw, **bias}.items() if "omega" not in k}
    beta, u, vth = mod_1(leaves["raw_beta"], leaves["b_beta"], leaves["raw_alpha"], leaves["b_alpha"],
                         leaves["raw_th"], leaves["b_th"], v_th_min, leaves["cur"])
    ((beta * ups["g_beta"]).sum() + (u * ups["g_u"]).sum() + (vth * ups["g_vth"]).sum()).backward()
    npz("modulation_first_order", **{k: v for k, v in raw.items() if "omega" not in k},
        **{k: v for k, v in bias.items() if "omega" not in k}, v_th_min=np.float64(v_th_min),
        beta=beta, u=u, vth=vth, **{k: v for k, v in ups.items() if "omega" not in k},
        **{f"grad_{k}": v.grad for k, v in leaves.items()})

    # ---- MoE combine
    moe = load("ref_moe_kernels", "atomic_ops/moe_kernels.py")
    torch.manual_seed(33)
    E_, N_, D_ = 4, 10, 24
    msh = torch.randn(N_, D_).requires_grad_()
    mex = torch.randn(E_, N_, D_).requires_grad_()
    mw = torch.softmax(torch.randn(N_, E_), -1).requires_grad_()
    mout = moe.moe_combine(msh, mex, mw)
    mg = torch.randn(N_, D_)
    (mout * mg).sum().backward()
    npz("moe_a", shared=msh, experts=mex, weights=mw, out=mout, g_out=mg, g_shared=msh.grad, g_experts=mex.grad,
        g_weights=mw.grad)

    # ---- expert merge in the frame domain (atomic_ops/moe_snn_ffn.py:377-393)
    for tag, dt in (("f32", torch.float32), ("bf16", torch.bfloat16)):
        torch.manual_seed(33)
        T_, K_, B_, D_, E_ = 6, 16, 2, 24, 4
        mk = lambda scale: codec.fp16_encode((torch.randn(B_, T_, D_) * scale).to(dt), K_).requires_grad_()
        f_shared, f_res = mk(1.0), mk(2.0)
        f_exp = [mk(0.7) for _ in range(E_)]
        fw = torch.rand(T_, B_, E_) * (torch.rand(T_, B_, E_) < 0.5)      # sparse routing weights
        fw = fw.to(dt).requires_grad_()
        shared_val = codec.fp16_decode(f_shared, T_, K_)
        expert_vals = torch.stack([codec.fp16_decode(f_exp[e], T_, K_) for e in range(E_)], dim=0)
        w = fw.permute(2, 1, 0).unsqueeze(-1)
        combined = shared_val + (expert_vals * w).sum(dim=0)
        total = combined + codec.fp16_decode(f_res, T_, K_)
        out = codec.binary_encode_ste(total)
        g_out = (torch.randn(T_ * K_, B_, D_) * 0.1).to(dt)
        (out.float() * g_out.float()).sum().backward()
        npz(f"frames_combine_{tag}", shared=f_shared, residual=f_res, experts=torch.stack(f_exp), weights=fw,
            total=total, out=out, g_out=g_out, g_shared=f_shared.grad, g_residual=f_res.grad,
            g_experts=torch.stack([f.grad for f in f_exp]), g_weights=fw.grad)

    # ---- linear recurrence (the reference's CPU branch is a Hillis-Steele scan: same numbers up to
    # the association of the products, not bit-comparable with a sequential loop)
    torch.manual_seed(21)
    T, B, D = 37, 2, 24
    lb = torch.sigmoid(torch.randn(T, B, D) + 1.0).requires_grad_()
    lu = torch.randn(T, B, D).requires_grad_()
    lv0 = torch.randn(B, D).requires_grad_()
    Vl = ps.linear_recurrence(lb, lu, lv0)
    gVl = torch.randn(T, B, D)
    (Vl * gVl).sum().backward()
    npz("linrec_a", beta=lb, u=lu, v_init=lv0, V=Vl, g_V=gVl, g_beta=lb.grad, g_u=lu.grad, g_vinit=lv0.grad)

    # ---- adaptive surrogate slope (atomic_ops/plif_node.py:93-100)
    torch.manual_seed(5)
    cases = {}
    for i, (scale, dt) in enumerate([(0.05, torch.float32), (0.4, torch.float32), (3.0, torch.float32),
                                     (0.13, torch.bfloat16), (0.77, torch.bfloat16), (1e-9, torch.bfloat16),
                                     (0.31, torch.float16)]):
        u = (torch.randn(40, 3, 50) * scale + 0.01).to(dt)
        alpha_0, sigma_0 = 4.0, 0.4
        sigma_V = u.std().clamp(min=1e-6)
        alpha_adaptive = alpha_0 * sigma_0 / sigma_V.item()
        alpha_adaptive = max(1.0, min(alpha_adaptive, 20.0))
        cases[f"u{i}"] = u
        cases[f"alpha{i}"] = np.float64(alpha_adaptive)
        cases[f"dtype{i}"] = np.array({torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}[dt])
    npz("surrogate_alpha", n=np.array(7), alpha_0=np.float64(4.0), sigma_0=np.float64(0.4), **cases)

    # ---- lateral inhibition fallback (atomic_ops/lateral_inhibition.py:208-212)
    torch.manual_seed(42)
    x = (torch.randn(6, 5, 48) * 2).requires_grad_()
    gain = (1 + 0.1 * torch.randn(48)).requires_grad_()
    eps = 1e-6
    variance = x.pow(2).mean(-1, keepdim=True)
    out = gain * (x * torch.rsqrt(variance + eps))
    go = torch.randn_like(out)
    (out * go).sum().backward()
    npz("li_a", x=x, gain=gain, eps=np.float64(eps), out=out, g_out=go, g_x=x.grad,
        g_gain=gain.grad)


if __name__ == "__main__":
    sys.exit(main())
