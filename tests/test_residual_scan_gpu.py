"""GPU parity of the row-parameter scan with the binary residual fused in
(nsb_plif_rowparam_residual_fwd): bit-exact against the CPU oracle's scan followed by the oracle's
binary residual (both pinned to the reference by golden vectors), and against this package's two
separate kernels; gradients identical to the unfused pair's."""
import numpy as np
import pytest
import torch

import neuronspark_b200 as nsb
from neuronspark_b200 import fp16_codec as codec
from neuronspark_b200 import parallel_scan as ps
from oracle import oracle as orc
from util import f32, rowparam_inputs

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(autouse=True)
def _reset():
    nsb.set_tuning()
    ps.CKPT_INTERVAL = None
    yield
    nsb.set_tuning()
    ps.CKPT_INTERVAL = None
    assert nsb.device_error_word() == 0


def inputs(S, B, D, dtype, seed):
    """Scan inputs as in the reference's row-parameter use, plus the frames of a random residual
    stream (values spread over the half range, some subnormal, some that overflow when added)."""
    T = S * 16
    beta_row, u, vth_row, v0 = rowparam_inputs(T, B, D, dtype, DEV, seed=seed)
    g = torch.Generator(device=DEV).manual_seed(seed + 1)
    vals = torch.randn(B, S, D, generator=g, device=DEV) * torch.pow(
        10.0, torch.randint(-7, 5, (B, S, D), generator=g, device=DEV).float())
    frames_in = codec.fp16_encode(vals.to(dtype))
    return beta_row, u * 3.0, vth_row, v0, frames_in   # a livelier drive: ~30 % spikes


def unfused(beta_row, u, vth_row, v0, frames_in, alpha=4.0):
    s, v_last = ps.plif_rowparam_forward_recompute(beta_row, u, vth_row, v0, alpha)
    return codec.binary_residual(s, frames_in), v_last, s


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(1, 2, 64), (3, 2, 96), (10, 3, 40), (4, 1, 2048), (2, 5, 33)])
def test_fused_equals_oracle_and_unfused(dtype, shape):
    S, B, D = shape
    beta_row, u, vth_row, v0, fin = inputs(S, B, D, dtype, 7)
    out, v_last = ps.plif_rowparam_residual_forward(beta_row, u, vth_row, v0, fin, 4.0)
    ref_out, ref_v, spikes = unfused(beta_row, u, vth_row, v0, fin)
    assert out.dtype == dtype and torch.equal(out, ref_out) and torch.equal(v_last, ref_v)
    assert 0.05 < float(spikes.float().mean()) < 0.9
    so, _, vlo = orc.plif_rowparam_fwd(f32(beta_row), f32(u), f32(vth_row), f32(v0), want_vpost=False)
    want = orc.binary_residual(so, f32(fin), bf16_compiled=(dtype == torch.bfloat16))
    if dtype == torch.float16:  # the reference adds the two decoded values in half precision
        want = f32(codec.binary_residual(torch.as_tensor(so, device=DEV).half(), fin))
    assert np.array_equal(f32(out), want)
    assert np.array_equal(f32(v_last), vlo)


def test_eager_rounding_of_bf16_frames(monkeypatch):
    """The other rounding of the residual on bf16 frames (every intermediate rounded to bf16, as the
    reference's ops give when run one by one) is selectable and differs from the default."""
    beta_row, u, vth_row, v0, fin = inputs(6, 2, 520, torch.bfloat16, 13)
    fin = (torch.rand_like(fin.float()) < 0.5).to(torch.bfloat16)  # full 10-bit mantissas, as layers produce
    default, _ = ps.plif_rowparam_residual_forward(beta_row, u, vth_row, v0, fin, 4.0)
    monkeypatch.setattr(codec, "RESIDUAL_ROUNDING", "eager")
    out, _ = ps.plif_rowparam_residual_forward(beta_row, u, vth_row, v0, fin, 4.0)
    so, _, _ = orc.plif_rowparam_fwd(f32(beta_row), f32(u), f32(vth_row), f32(v0), want_vpost=False)
    assert np.array_equal(f32(out), orc.binary_residual(so, f32(fin), bf16_intermediates=True))
    assert np.array_equal(f32(default), orc.binary_residual(so, f32(fin), bf16_compiled=True))
    assert not torch.equal(out, default)


@pytest.mark.parametrize("tile", [16, 32])
@pytest.mark.parametrize("lanes,direct", [(1, 0), (2, 0), (4, 0), (0, 1)])
def test_every_instantiation(tile, lanes, direct):
    if tile == 32 and lanes > 1:
        pytest.skip("32-step tiles are built for 1 lane per thread")
    S, B, D = 7, 2, 520
    beta_row, u, vth_row, v0, fin = inputs(S, B, D, torch.bfloat16, 9)
    ref_out, ref_v, _ = unfused(beta_row, u, vth_row, v0, fin)
    ps.CKPT_INTERVAL = tile
    nsb.set_tuning(lanes_per_thread=lanes, force_direct=direct)
    out, v_last = ps.plif_rowparam_residual_forward(beta_row, u, vth_row, v0, fin, 4.0)
    info = nsb.last_launch_info()
    assert info["tile_steps"] == tile and info["used_tma"] == (0 if direct else 1)
    if lanes:
        assert info["lanes_per_thread"] == lanes
    assert torch.equal(out, ref_out) and torch.equal(v_last, ref_v)


@pytest.mark.parametrize("tile", [16, 32])
def test_gradients_equal_unfused(tile):
    S, B, D = 6, 2, 264
    beta_row, u, vth_row, v0, fin = inputs(S, B, D, torch.bfloat16, 11)
    ps.CKPT_INTERVAL = tile
    g_out = (torch.randn(S * 16, B, D, device=DEV) * 0.1).bfloat16()

    def grads(fused):
        leaves = [t.clone().requires_grad_() for t in (beta_row, u, vth_row, v0, fin)]
        if fused:
            out, _ = ps.plif_rowparam_residual_forward(*leaves, 4.0)
        else:
            s, _ = ps.plif_rowparam_forward_recompute(*leaves[:4], 4.0)
            out = codec.binary_residual(s, leaves[4])
        out.backward(g_out)
        return [t.grad for t in leaves]

    a, b = grads(True), grads(False)
    for x, y in zip(a, b):
        assert torch.equal(x, y)
    assert torch.equal(a[4], g_out)


def test_argument_checks():
    beta_row, u, vth_row, v0, fin = inputs(2, 2, 64, torch.bfloat16, 3)
    with pytest.raises(nsb.NSBError):  # T not a multiple of 16
        ps.plif_rowparam_residual_forward(beta_row, u[:20], vth_row, v0, fin[:20], 4.0)
    with pytest.raises(nsb.NSBError):  # shapes differ
        ps.plif_rowparam_residual_forward(beta_row, u, vth_row, v0, fin[:16], 4.0)
    out, v_last = ps.plif_rowparam_residual_forward(beta_row, u[:0], vth_row, v0, fin[:0], 4.0)
    assert out.shape[0] == 0 and torch.equal(v_last, v0)
