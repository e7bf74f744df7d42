#!/usr/bin/env python
"""Timing of the boundary kernels (FP16 codec, lateral inhibition, adaptive surrogate slope) on one GPU.

    python microbench.py [--dtype bf16|f32] [--iters N] [--only SUBSTRING]
    python microbench.py --triton-reference       the reference's own Triton scans beside this library's

Prints one JSON line per kernel and shape: microseconds per call (CUDA events,
best of N, 256 MB written between calls so that nothing is served from L2),
algorithmic bytes and the bandwidth they imply. Shapes are those of the
reference's 768-wide model: token blocks of (batch 8 or 32, 512 tokens, D 768)
for the codec, (rows, 768) for the normaliser, plus a wide case."""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from neuronspark_b200 import fp16_codec as codec  # noqa: E402
from neuronspark_b200 import lateral_inhibition as li  # noqa: E402
from neuronspark_b200 import parallel_scan as ps  # noqa: E402


def _time(fn, iters, flush):
    fn()
    torch.cuda.synchronize()
    best = float("inf")
    for _ in range(iters):
        flush.fill_(1)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        best = min(best, a.elapsed_time(b))
    return best * 1e3  # us


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "f32"])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--only", default="", help="substring filter on the kernel name")
    ap.add_argument("--triton-reference", action="store_true",
                    help="time the reference's Triton scan kernels (staged under oracle/_ref) and this "
                         "library's on the same inputs; nothing else")
    args = ap.parse_args()
    if args.triton_reference:
        triton_reference(args.iters)
        return
    dt = torch.bfloat16 if args.dtype == "bf16" else torch.float32
    es = 2 if dt == torch.bfloat16 else 4
    dev = torch.device("cuda", 0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def report(name, shape, us, nbytes):
        print(json.dumps({"kernel": name, "shape": list(shape), "dtype": args.dtype, "us": round(us, 2),
                          "algorithmic_bytes": int(nbytes), "GB_per_s": round(nbytes / us / 1e3, 1)}),
              flush=True)

    for shape in [(8, 512, 768), (32, 512, 768), (8, 512, 6144)]:
        B, S, D = shape
        n = B * S * D
        x = torch.randn(B, S, D, device=dev).to(dt)
        fa, fb = codec.fp16_encode(x), codec.fp16_encode(-0.5 * x)
        gv = torch.randn(B, S, D, device=dev).to(dt)
        gf = torch.randn(S * 16, B, D, device=dev).to(dt)
        cases = {
            "fp16_encode": (lambda: codec.fp16_encode(x), n * 17 * es),
            "fp16_decode_fwd": (lambda: codec.fp16_decode(fa, S), n * 17 * es),
            "binary_residual": (lambda: codec.binary_residual(fa, fb), n * 48 * es),
            "fp16_decode_bwd": (lambda: codec._FP16Decode.backward(_Ctx((fa,)), gv), n * 33 * es),
            "encode_ste_bwd": (lambda: codec._BinaryEncodeSTE.backward(_Ctx((), dt), gf), n * 17 * es),
        }
        for name, (fn, nbytes) in cases.items():
            if args.only in name:
                report(name, shape, _time(fn, args.iters, flush), nbytes)

    # spikes packed in time (one int16 pattern per token and channel) beside the dense kernels above
    if args.only in "packed":
        for shape in [(8, 512, 768), (32, 512, 768)]:
            B, S, D = shape
            n = B * S * D
            x = torch.randn(B, S, D, device=dev).to(dt)
            pa = codec.pack_frames(codec.fp16_encode(x))
            pb = codec.pack_frames(codec.fp16_encode(-0.5 * x))
            gv = torch.randn(B, S, D, device=dev).to(dt)
            cases = {
                "packed: fp16_decode_packed": (lambda: codec.fp16_decode_packed(pa, dt), n * (2 + es)),
                "packed: fp16_decode_packed_backward": (lambda: codec.fp16_decode_packed_backward(pa, gv), n * (2 + 17 * es)),
                "packed: binary_residual_packed": (lambda: codec.binary_residual_packed(pa, pb, dt), n * 6),
                "packed: unpack_frames": (lambda: codec.unpack_frames(pa, dt), n * (2 + 16 * es)),
                "packed: pack_frames": (lambda fr=codec.unpack_frames(pa, dt): codec.pack_frames(fr), n * (2 + 16 * es)),
            }
            for name, (fn, nbytes) in cases.items():
                report(name, shape, _time(fn, args.iters, flush), nbytes)
            # the output neuron of a block: scan + residual, dense frames against packed patterns
            T = S * 16
            g = torch.Generator(device=dev).manual_seed(3)
            bd = torch.sigmoid(2 + 0.5 * torch.randn(D, generator=g, device=dev)).expand(B, D).contiguous()
            td = torch.full((B, D), 0.4, device=dev)
            u = (0.5 * torch.randn(T, B, D, generator=g, device=dev)).to(dt)
            v0 = torch.zeros(B, D, device=dev)
            fin = codec.unpack_frames(pb.reshape(S, B, D) if pb.shape == (S, B, D) else pb, dt)
            with torch.no_grad():
                report("packed: row-param scan + residual, dense frames in/out", (T, B, D),
                       _time(lambda: ps.plif_rowparam_residual_forward(bd, u, td, v0, fin, 4.0), args.iters, flush),
                       T * B * D * 3 * es)
                report("packed: row-param scan + residual, patterns in/out", (T, B, D),
                       _time(lambda: ps.plif_rowparam_forward_patterns(bd, u, td, v0, patterns_in=pb), args.iters, flush),
                       T * B * D * es + 2 * n * 2)

    for rows, D in [(4096, 768), (65536, 768), (8192, 6144)]:
        x = torch.randn(rows, D, device=dev).to(dt)
        gain = 1 + 0.1 * torch.randn(D, device=dev)
        go = torch.randn(rows, D, device=dev).to(dt)
        fn = li.LateralInhibitionFunction
        if args.only in "lateral_inhibition_fwd":
            report("lateral_inhibition_fwd", (rows, D),
                   _time(lambda: fn.apply(x, gain, 1e-6), args.iters, flush), rows * D * 2 * es)
        if args.only in "lateral_inhibition_bwd":
            ctx = _Ctx((x, gain))
            ctx.eps, ctx.orig_shape, ctx.gain_dtype, ctx.gain_shape = 1e-6, x.shape, gain.dtype, gain.shape
            report("lateral_inhibition_bwd", (rows, D),
                   _time(lambda: fn.backward(ctx, go), args.iters, flush), rows * D * 4 * es)

    # linear recurrence, forward and forward+backward (2 streams in, 1 out; backward 3 in, 2 out)
    from neuronspark_b200 import moe_kernels as mk
    if args.only in "linear_recurrence":
        T, B, D = 8192, 32, 6144
        beta = torch.rand(T, B, D, device=dev).to(dt)
        u = torch.empty(T, B, D, dtype=dt, device=dev).normal_()
        v0 = torch.zeros(B, D, device=dev)
        with torch.no_grad():
            report("linear_recurrence_fwd", (T, B, D), _time(lambda: ps.linear_recurrence(beta, u, v0), args.iters, flush),
                   T * B * D * 3 * es)
        bl, ul = beta.requires_grad_(), u.requires_grad_()
        gV = torch.empty(T, B, D, dtype=dt, device=dev).normal_()

        def fb():
            ps.linear_recurrence(bl, ul, v0).backward(gV)
            bl.grad = ul.grad = None
        report("linear_recurrence_fwd_bwd", (T, B, D), _time(fb, args.iters, flush), T * B * D * 8 * es)
        del beta, u, gV, bl, ul
    if args.only in "moe_combine":
        for E, N, D in [(4, 65536, 768), (8, 32768, 768)]:
            sh = torch.empty(N, D, dtype=dt, device=dev).normal_()
            ex = torch.empty(E, N, D, dtype=dt, device=dev).normal_()
            w = torch.softmax(torch.randn(N, E, device=dev), -1)
            with torch.no_grad():
                report("moe_combine_fwd", (E, N, D), _time(lambda: mk.moe_combine(sh, ex, w), args.iters, flush),
                       (E + 2) * N * D * es)
            exl, wl = ex.requires_grad_(), w.requires_grad_()
            go = torch.empty(N, D, dtype=dt, device=dev).normal_()
            out = mk.moe_combine(sh, exl, wl)

            def bw():
                out.backward(go, retain_graph=True)
                exl.grad = wl.grad = None
            report("moe_combine_bwd", (E, N, D), _time(bw, args.iters, flush), (2 * E + 1) * N * D * es)
            del sh, ex, w, exl, wl, go, out

    if args.only in "frames_combine":
        for E, top_k, B, S, D in [(4, 2, 8, 512, 768), (8, 2, 8, 512, 768)]:
            mkf = lambda: codec.fp16_encode(torch.empty(B, S, D, dtype=dt, device=dev).normal_())
            sh, rs = mkf(), mkf()
            ex = torch.stack([mkf() for _ in range(E)])
            w = torch.rand(S, B, E, device=dev)
            w = w.masked_fill(torch.rand(S, B, E, device=dev).argsort(-1) >= top_k, 0.0).to(dt)
            fb = B * S * D * 16 * es                      # bytes of one frame tensor
            with torch.no_grad():
                report("frames_combine_fwd", (E, top_k, B, S, D),
                       _time(lambda: mk.frames_combine(sh, ex, w, rs), args.iters, flush), (top_k + 3) * fb)

                def unfused():
                    vals = torch.stack([codec.fp16_decode(ex[e], S) for e in range(E)])
                    tot = codec.fp16_decode(sh, S) + (vals * w.permute(2, 1, 0).unsqueeze(-1)).sum(0)
                    return codec.fp16_encode(tot + codec.fp16_decode(rs, S))
                report("frames_combine_fwd_unfused (codec kernels + torch ops)", (E, top_k, B, S, D),
                       _time(unfused, args.iters, flush), (E + 3) * fb)
            leaves = [t.requires_grad_() for t in (sh, ex, w, rs)]
            go = torch.empty_like(sh).normal_()
            out = mk.frames_combine(*leaves)

            def bw():
                out.backward(go, retain_graph=True)
                for t in leaves:
                    t.grad = None
            report("frames_combine_bwd", (E, top_k, B, S, D), _time(bw, args.iters, flush), (2 * E + 5) * fb)
            del sh, rs, ex, w, leaves, go, out

    # adaptive surrogate slope: one read of u (the reference pays the same pass plus a host sync)
    for shape in [(8192, 8, 768), (8192, 32, 6144)]:
        if args.only in "surrogate_alpha":
            u = torch.empty(shape, dtype=dt, device=dev).normal_()
            report("surrogate_alpha", shape, _time(lambda: ps.adaptive_alpha(u, 4.0, 0.4), args.iters, flush),
                   u.numel() * es)
            del u


def triton_reference(iters):
    """The kernels to beat: ``_TritonPLIFForward`` and ``_TritonPLIFRowParamRecompute`` of the
    reference (atomic_ops/parallel_scan.py:690-768, 614-688), forward + backward, at the shapes of
    the reference's own bench (exp/bench_fused_plif.py:156-158: T=8192, batch 2, D*N = 6144 and
    D = 768, bf16) and at the headline shape (batch 32), next to this library's Functions of the
    same names on the same tensors. One JSON line per (implementation, kernel, shape); where the
    reference cannot run (no staged copy, Triton cannot compile) the line says why."""
    import importlib.util
    ref_file = ROOT / "oracle" / "_ref" / "atomic_ops" / "parallel_scan.py"
    dev = torch.device("cuda", 0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    ref = None
    why = None
    if not ref_file.exists():
        why = "oracle/_ref is empty (python oracle/make_ref.py <NeuronSpark checkout>)"
    else:
        try:
            spec = importlib.util.spec_from_file_location("ref_parallel_scan", ref_file)
            ref = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(ref)
            if not getattr(ref, "_HAS_TRITON", False):
                ref, why = None, "the reference found no Triton"
        except Exception as e:  # noqa: BLE001
            ref, why = None, f"{type(e).__name__}: {e}"

    def inputs(T, B, D, seed):
        g = torch.Generator(device=dev).manual_seed(seed)

        def rn():
            out = torch.empty((T, B, D), dtype=torch.bfloat16, device=dev)
            for t0 in range(0, T, 512):
                out[t0:t0 + 512] = torch.randn(out[t0:t0 + 512].shape, generator=g, device=dev)
            return out
        beta = rn().float().mul_(0.5).add_(2).sigmoid_().bfloat16()
        u = rn()
        vth = torch.nn.functional.softplus(rn().float()).add_(0.1).bfloat16()
        gs = rn().mul_(0.1)
        return beta, u, vth, gs

    def fwd_bwd(fn, tensors, gs, n_out_grads):
        leaves = [t.detach().clone().requires_grad_() for t in tensors]  # the reference overwrites u in place

        def run():
            out = fn(*leaves)
            out[0].backward(gs)
            for t in leaves:
                t.grad = None
        return run

    for T, B, D in [(8192, 2, 6144), (8192, 2, 768), (8192, 32, 6144)]:
        beta, u, vth, gs = inputs(T, B, D, 1234)
        v0 = torch.zeros(B, D, dtype=torch.bfloat16, device=dev)
        beta_row, vth_row = beta[0].contiguous(), vth[0].contiguous()
        ns = T * B * D
        cases = [
            # u-form selective scan: fwd 3 in + spike + V_post out; bwd 3 in + V_post, spike, gS in + 3 out
            ("selective fwd+bwd (_TritonPLIFForward)", "_TritonPLIFForward", (beta, u, vth, v0), None),
            ("row-param recompute fwd+bwd (_TritonPLIFRowParamRecompute)", "_TritonPLIFRowParamRecompute",
             (beta_row, u, vth_row, v0), None),
        ]
        for label, cls, tensors, _ in cases:
            for impl, mod in (("reference-triton", ref), ("neuronspark_b200", ps)):
                line = {"impl": impl, "kernel": label, "shape": [T, B, D], "dtype": "bf16"}
                if mod is None:
                    line["unavailable"] = why
                    print(json.dumps(line), flush=True)
                    continue
                try:
                    f = getattr(mod, cls)
                    run = fwd_bwd(lambda *a, f=f: f.apply(*a, 4.0), tensors, gs, 0)
                    us = _time(run, iters, flush)
                    line.update({"us": round(us, 1), "G_neuron_steps_per_s": round(ns / us / 1e3, 2)})
                except Exception as e:  # noqa: BLE001
                    line["unavailable"] = f"{type(e).__name__}: {str(e)[:300]}"
                    if impl == "reference-triton":
                        ref, why = None, line["unavailable"]
                print(json.dumps(line), flush=True)
        del beta, u, vth, gs


class _Ctx:
    """Just enough of an autograd context to call a Function's backward directly."""

    def __init__(self, saved, in_dtype=None):
        self.saved_tensors = saved
        self.in_dtype = in_dtype
        self.needs_input_grad = (True,)


if __name__ == "__main__":
    main()
