"""Spikes packed in time (16 frames of a token and channel = one int16 half bit pattern): every
packed kernel against the dense kernel it stands for (bit for bit) and against the CPU oracle of
the reference's codec and scan."""
import numpy as np
import pytest
import torch

import neuronspark_b200 as nsb
from neuronspark_b200 import fp16_codec as codec
from neuronspark_b200 import parallel_scan as ps
from oracle import oracle as orc
from util import assert_close, assert_close_lowp, f32, rowparam_inputs

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)
DTYPES = [torch.float32, torch.bfloat16, torch.float16]


@pytest.fixture(autouse=True)
def _clean():
    nsb.set_tuning()
    ps.CKPT_INTERVAL = None
    yield
    nsb.set_tuning()
    ps.CKPT_INTERVAL = None
    assert nsb.device_error_word() == 0


def random_patterns(S, B, D, seed):
    """Every kind of half pattern: normals, subnormals, zeros of both signs, an all-ones exponent."""
    g = torch.Generator(device=DEV).manual_seed(seed)
    p = torch.randint(-32768, 32768, (S, B, D), generator=g, device=DEV, dtype=torch.int32)
    p.view(-1)[:8] = torch.tensor([0, -32768, 0x7C00, 0x7FFF, 0x0001, 0x03FF, 0x0400, -1], device=DEV)[: p.numel()][:8]
    return p.to(torch.int16)


def frames_of(p, dtype):
    bits = torch.arange(15, -1, -1, device=p.device, dtype=torch.int32)
    S, B, D = p.shape
    f = ((p.to(torch.int32).unsqueeze(1) >> bits.view(1, 16, 1, 1)) & 1).reshape(S * 16, B, D)
    return f.to(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(1, 1, 1), (3, 2, 7), (5, 3, 64), (16, 8, 768), (2, 1, 1001)])
def test_pack_unpack_decode(dtype, shape):
    S, B, D = shape
    p = random_patterns(S, B, D, S * 131 + D)
    frames = frames_of(p, dtype)
    assert torch.equal(codec.unpack_frames(p, dtype), frames)
    assert torch.equal(codec.pack_frames(frames), p)
    dense = codec.fp16_decode(frames, S)
    packed = codec.fp16_decode_packed(p, dtype)
    assert packed.dtype == dtype and torch.equal(packed.view(torch.int16 if dtype != torch.float32 else torch.int32),
                                                 dense.view(torch.int16 if dtype != torch.float32 else torch.int32))
    want = orc.fp16_decode(f32(frames), dtype == torch.bfloat16)
    if dtype == torch.float16:
        with np.errstate(over="ignore"):
            want = want.astype(np.float16).astype(np.float32)
    assert np.array_equal(f32(packed), want)


@pytest.mark.parametrize("dtype", DTYPES)
def test_decode_backward(dtype):
    S, B, D = 6, 3, 200
    p = random_patterns(S, B, D, 17)
    frames = frames_of(p, dtype).requires_grad_()
    g = (torch.randn(B, S, D, device=DEV) * 0.1).to(dtype)
    codec.fp16_decode(frames, S).backward(g)
    got = codec.fp16_decode_packed_backward(p, g)
    assert got.shape == (S * 16, B, D) and got.dtype == dtype
    assert torch.equal(got.float().nan_to_num(), frames.grad.float().nan_to_num())
    if dtype == torch.float32:
        small = (p.to(torch.int32) & 0x7C00) < 0x7000  # keeps the oracle comparison away from 1e4-sized values
        want = orc.fp16_decode_bwd(f32(frames), f32(g))
        mask = small.unsqueeze(1).expand(S, 16, B, D).reshape(S * 16, B, D).cpu().numpy()
        assert_close(f32(got)[mask], want[mask], what="frame gradients")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rounding", ["compiled", "eager"])
def test_residual_packed(dtype, rounding):
    S, B, D = 9, 2, 333
    pa, pb = random_patterns(S, B, D, 5), random_patterns(S, B, D, 6)
    fa, fb = frames_of(pa, dtype), frames_of(pb, dtype)
    dense = codec.binary_residual_with(fa, fb, rounding)
    got = codec.binary_residual_packed(pa, pb, dtype, rounding)
    assert got.dtype == torch.int16 and torch.equal(got, codec.pack_frames(dense))
    emu = dtype == torch.bfloat16
    want = orc.binary_residual(f32(fa), f32(fb), bf16_intermediates=emu and rounding == "eager",
                               bf16_compiled=emu and rounding == "compiled")
    if dtype != torch.float16:  # (half frames add in half precision; covered by the dense kernel's own test)
        assert np.array_equal(f32(codec.unpack_frames(got, torch.float32)), want)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(1, 2, 64), (3, 2, 96), (10, 3, 40), (4, 1, 2048), (2, 5, 33)])
def test_pattern_scan_equals_dense_scan_and_oracle(dtype, shape):
    S, B, D = shape
    T = S * 16
    beta_row, u, vth_row, v0 = rowparam_inputs(T, B, D, dtype, DEV, seed=7)
    u = u * 3.0
    spikes, v_last = ps.plif_rowparam_forward_recompute(beta_row, u, vth_row, v0, 4.0)
    pats, v_last_p, _ = ps.plif_rowparam_forward_patterns(beta_row, u, vth_row, v0)
    assert pats.shape == (S, B, D) and pats.dtype == torch.int16
    assert torch.equal(pats, codec.pack_frames(spikes)) and torch.equal(v_last_p, v_last.float())
    so, _, vlo = orc.plif_rowparam_fwd(f32(beta_row), f32(u), f32(vth_row), f32(v0), want_vpost=False)
    assert np.array_equal(f32(codec.unpack_frames(pats, torch.float32)), so) and np.array_equal(f32(v_last_p), vlo)
    assert 0.05 < so.mean() < 0.9
    # with the residual: the incoming stream packed as well
    pin = random_patterns(S, B, D, 23)
    fin = frames_of(pin, dtype)
    dense_out, _ = ps.plif_rowparam_residual_forward(beta_row, u, vth_row, v0, fin, 4.0)
    pats_res, v_last_r, _ = ps.plif_rowparam_forward_patterns(beta_row, u, vth_row, v0, patterns_in=pin)
    assert torch.equal(pats_res, codec.pack_frames(dense_out)) and torch.equal(v_last_r, v_last.float())
    if dtype != torch.float16:
        want = orc.binary_residual(so, f32(fin), bf16_compiled=dtype == torch.bfloat16)
        assert np.array_equal(f32(codec.unpack_frames(pats_res, torch.float32)), want)


@pytest.mark.parametrize("tile", [16, 32])
@pytest.mark.parametrize("lanes,direct", [(1, 0), (2, 0), (4, 0), (0, 1)])
def test_every_instantiation(tile, lanes, direct):
    if tile == 32 and lanes > 1:
        pytest.skip("32-step tiles are built for 1 lane per thread")
    S, B, D = 7, 2, 520
    beta_row, u, vth_row, v0 = rowparam_inputs(S * 16, B, D, torch.bfloat16, DEV, seed=9)
    u = u * 3.0
    pin = random_patterns(S, B, D, 29)
    ref, ref_v, _ = ps.plif_rowparam_forward_patterns(beta_row, u, vth_row, v0, patterns_in=pin)
    ps.CKPT_INTERVAL = tile
    nsb.set_tuning(lanes_per_thread=lanes, force_direct=direct)
    out, v_last, _ = ps.plif_rowparam_forward_patterns(beta_row, u, vth_row, v0, patterns_in=pin)
    info = nsb.last_launch_info()
    assert info["tile_steps"] == tile and info["used_tma"] == (0 if direct else 1)
    if lanes:
        assert info["lanes_per_thread"] == lanes
    assert torch.equal(out, ref) and torch.equal(v_last, ref_v)


def test_pattern_scan_backward_equals_dense():
    S, B, D = 6, 2, 264
    T = S * 16
    beta_row, u, vth_row, v0 = rowparam_inputs(T, B, D, torch.bfloat16, DEV, seed=11)
    u = u * 3.0
    g_values = (torch.randn(B, S, D, device=DEV) * 0.1).bfloat16()
    # dense route: scan -> frames -> fp16_decode -> loss
    leaves = [t.clone().requires_grad_() for t in (beta_row, u, vth_row, v0)]
    spikes, _ = ps.plif_rowparam_forward_recompute(*leaves, 4.0)
    codec.fp16_decode(spikes, S).backward(g_values)
    # packed route: the same quantities never materialising the frames forward
    pats, _, ckpt = ps.plif_rowparam_forward_patterns(beta_row, u, vth_row, v0, want_ckpt=True)
    g_frames = codec.fp16_decode_packed_backward(pats, g_values)
    grads = ps.plif_rowparam_patterns_backward(beta_row, u, vth_row, ckpt, g_frames, 4.0)
    for got, leaf, name in zip(grads, leaves, ("beta_row", "u", "v_th_row", "v_init")):
        assert torch.equal(got.to(leaf.grad.dtype), leaf.grad), name


def test_argument_checks():
    beta_row, u, vth_row, v0 = rowparam_inputs(32, 2, 64, torch.bfloat16, DEV, seed=3)
    with pytest.raises(nsb.NSBError):
        ps.plif_rowparam_forward_patterns(beta_row, u[:20], vth_row, v0)
    with pytest.raises(nsb.NSBError):
        ps.plif_rowparam_forward_patterns(beta_row, u, vth_row, v0, patterns_in=torch.zeros(1, 2, 64, dtype=torch.int16,
                                                                                          device=DEV))
    with pytest.raises(nsb.NSBError):
        codec.fp16_decode_packed(torch.zeros(2, 2, 4, dtype=torch.int32, device=DEV))
