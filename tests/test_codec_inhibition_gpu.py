"""GPU parity of the FP16 codec and the lateral-inhibition kernels against the
golden vectors (produced by the reference's code) and the CPU oracle."""
import numpy as np
import pytest
import torch

import neuronspark_b200 as nsb
from neuronspark_b200 import fp16_codec as codec
from neuronspark_b200 import lateral_inhibition as li
from oracle import oracle as orc
from util import REL_TOL, assert_close, assert_close_lowp, f32

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def cuda(a, dtype=torch.float32):
    return torch.as_tensor(np.asarray(a), device=DEV).to(dtype)


def test_golden_codec(golden):
    g = golden("codec_a")
    fa, fb = codec.fp16_encode(cuda(g["xa"])), codec.fp16_encode(cuda(g["xb"]))
    assert np.array_equal(f32(fa), g["frames_a"]) and np.array_equal(f32(fb), g["frames_b"])
    assert not fa.requires_grad
    assert np.array_equal(f32(codec.fp16_decode(fa, 4)), g["decoded_a"])
    res = codec.binary_residual(fa, fb)
    assert np.array_equal(f32(res), g["residual"])
    assert set(np.unique(f32(res))) <= {0.0, 1.0}          # test_binary_residual.py:36-52
    dec = f32(codec.fp16_decode(res, 4))
    assert np.array_equal(dec, g["decoded_residual"])
    half = lambda x: x.astype(np.float16).astype(np.float32)
    assert np.abs(dec - half(half(g["xa"]) + half(g["xb"]))).max() < 1e-2   # :24-31
    # decode backward
    fr = cuda(g["frames_a"]).requires_grad_()
    (codec.fp16_decode(fr, 4) * cuda(g["g_out"])).sum().backward()
    assert_close(f32(fr.grad), g["g_frames"], 1e-6, "decode grad")
    # STE: identity to both inputs (test_binary_residual.py:55-75)
    a, b = fa.clone().requires_grad_(), fb.clone().requires_grad_()
    codec.binary_residual(a, b).sum().backward()
    assert torch.equal(a.grad, torch.ones_like(a)) and torch.equal(b.grad, torch.ones_like(b))
    # encode STE: forward = encode, backward = mean over the 16 frames (:78-115)
    x = cuda(g["xa"]).requires_grad_()
    sp = codec.binary_encode_ste(x)
    assert np.array_equal(f32(sp), g["frames_a"])
    assert np.abs(f32(codec.fp16_decode(sp, 4)) - half(g["xa"])).max() < 1e-3
    (sp * cuda(g["g_frames_in"])).sum().backward()
    assert x.grad.shape == x.shape
    assert_close(f32(x.grad), g["g_ste"], 1e-6, "encode STE grad")


def test_golden_codec_edges(golden):
    g = golden("codec_edge")
    f = codec.fp16_encode(cuda(g["x"]))
    assert np.array_equal(f32(f), g["frames"])
    assert np.array_equal(f32(codec.fp16_decode(f, 4)), g["decoded"])
    assert np.array_equal(f32(codec.binary_residual(f, cuda(g["frames_b"]))), g["residual"])
    e31 = cuda(g["frames_e31"])
    assert np.array_equal(f32(codec.fp16_decode(e31, 4)), g["decoded_e31"])
    assert np.array_equal(f32(codec.binary_residual(e31, cuda(g["frames_b"]))), g["residual_e31"])
    big = torch.full((1, 1, 1), 70000.0, device=DEV)
    assert codec.fp16_decode(codec.fp16_encode(big), 1).item() == 65504.0


def test_golden_codec_bf16_frames(golden):
    g = golden("codec_bf16")
    e = golden("codec_edge")
    fa, fb = cuda(g["frames_a"], torch.bfloat16), cuda(g["frames_b"], torch.bfloat16)
    assert np.array_equal(f32(codec.fp16_decode(fa, 4)), g["decoded_a"])
    # the golden residuals come from the reference's function run op by op on CPU: "eager" rounding
    assert np.array_equal(f32(codec.binary_residual_with(fa, fb, "eager")), g["residual"])
    fe = cuda(g["frames_e"], torch.bfloat16)
    assert np.array_equal(f32(codec.fp16_decode(fe, 4)), g["decoded_e"])
    assert np.array_equal(f32(codec.binary_residual_with(fe, cuda(e["frames_b"], torch.bfloat16), "eager")),
                          g["residual_e"])


@pytest.mark.parametrize("shape", [(1, 1, 1), (2, 3, 7), (3, 5, 64), (2, 16, 768), (1, 2, 1001)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_codec_vs_oracle(shape, dtype):
    B, S, D = shape
    g = torch.Generator(device=DEV).manual_seed(B * 100 + D)
    scale = torch.logspace(-6, 4, D, device=DEV)
    x = (torch.randn(B, S, D, generator=g, device=DEV) * scale).to(dtype)
    y = (torch.randn(B, S, D, generator=g, device=DEV) * scale.flip(0)).to(dtype)
    fx, fy = codec.fp16_encode(x), codec.fp16_encode(y)
    assert fx.dtype == dtype and fx.shape == (S * 16, B, D)
    ox, oy = orc.fp16_encode(f32(x)), orc.fp16_encode(f32(y))
    assert np.array_equal(f32(fx), ox) and np.array_equal(f32(fy), oy)
    emu = dtype == torch.bfloat16
    dec = codec.fp16_decode(fx, S)
    want = orc.fp16_decode(ox, emu)
    if dtype == torch.float16:
        want = want.astype(np.float16).astype(np.float32)
    assert np.array_equal(f32(dec), want)
    assert np.array_equal(f32(codec.binary_residual_with(fx, fy, "eager")), orc.binary_residual(ox, oy, emu))
    assert np.array_equal(f32(codec.binary_residual(fx, fy)), orc.binary_residual(ox, oy, bf16_compiled=emu))
    # round trip: decode(encode(x)) is x rounded to half (fp32 frames: exactly)
    if dtype == torch.float32:
        assert np.array_equal(f32(dec), f32(x).clip(-65504, 65504).astype(np.float16).astype(np.float32))
    # gradients
    gout = torch.randn(B, S, D, generator=g, device=DEV).to(dtype)
    fr = fx.clone().requires_grad_()
    (codec.fp16_decode(fr, S).float() * gout.float()).sum().backward()
    assert_close_lowp(f32(fr.grad), orc.fp16_decode_bwd(ox, f32(gout)), dtype, "decode grad")
    gfr = torch.randn(S * 16, B, D, generator=g, device=DEV).to(dtype)
    xe = x.clone().requires_grad_()
    (codec.binary_encode_ste(xe).float() * gfr.float()).sum().backward()
    assert_close_lowp(f32(xe.grad), orc.encode_ste_bwd(f32(gfr)), dtype, "STE grad")


def test_golden_lateral_inhibition(golden):
    g = golden("li_a")
    x, gain = cuda(g["x"]).requires_grad_(), cuda(g["gain"]).requires_grad_()
    out = li._LateralInhibitionTriton.apply(x, gain, float(g["eps"]))
    assert_close(f32(out), g["out"], what="out")
    (out * cuda(g["g_out"])).sum().backward()
    assert_close(f32(x.grad), g["g_x"], what="g_x")
    assert_close(f32(gain.grad), g["g_gain"], what="g_gain")


@pytest.mark.parametrize("rows,D", [(1, 1), (3, 7), (17, 768), (4096, 768), (64, 6144), (5, 1001),
                                    (300, 48), (700, 6144), (9, 16384), (33, 4104), (2, 2056)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_lateral_inhibition_vs_oracle(rows, D, dtype):
    g = torch.Generator(device=DEV).manual_seed(rows + D)
    x = (2 * torch.randn(rows, D, generator=g, device=DEV)).to(dtype).requires_grad_()
    mod = li.LateralInhibition(D).to(DEV)
    with torch.no_grad():
        mod.gain.copy_(1 + 0.1 * torch.randn(D, generator=g, device=DEV))
    go = torch.randn(rows, D, generator=g, device=DEV).to(dtype)
    out = mod(x)
    assert out.dtype == dtype
    want = orc.li_fwd(f32(x), f32(mod.gain))
    assert_close_lowp(f32(out), want, dtype, "out")
    (out.float() * go.float()).sum().backward()
    gx, gg = orc.li_bwd(f32(go), f32(x), f32(mod.gain))
    # g_x is a difference of two terms of size |g_out*gain|*rrms that cancel almost
    # completely for tiny D; the tolerance is relative to that size.
    rrms = 1.0 / np.sqrt((f32(x) ** 2).mean(-1) + 1e-6)
    term = np.abs(f32(go) * f32(mod.gain)).max() * rrms.max()
    assert_close_lowp(f32(x.grad), gx, dtype, "g_x", scale=max(term, np.abs(gx).max()))
    assert_close(f32(mod.gain.grad), gg, 2e-5 if dtype == torch.float32 else 1e-4, "g_gain")
    # deterministic: a second backward gives the same bits
    x2 = x.detach().clone().requires_grad_()
    mod.gain.grad = None
    (mod(x2).float() * go.float()).sum().backward()
    assert torch.equal(x2.grad, x.grad)
    # RMSNorm is the same kernel
    rn = li.RMSNorm(D).to(DEV)
    with torch.no_grad():
        rn.weight.copy_(mod.gain)
    assert torch.equal(rn(x.detach()), out.detach())
