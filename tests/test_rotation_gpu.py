"""Forward scans with the modulation fused in, over few columns, with the tiles of a column group taken in
turn by several warps (nsb_set_scan_rotation): a warp evaluates its tile's modulation, waits for the state
its predecessor left, runs the tile's steps and hands the state on. Per column the arithmetic and its order
are those of the one-warp scan, so spikes, final states and - through the checkpoints the backward starts
from - every gradient equal the unrotated launch's bit for bit."""
import pytest
import torch

import neuronspark_b200 as nsb
from neuronspark_b200 import parallel_scan as ps, snn_block as sb
from test_modulated_gpu import _Sigmoid, _fused_grads, mod_inputs

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)


@pytest.fixture(autouse=True)
def _clean():
    nsb.set_tuning()
    nsb.set_scan_rotation()
    ps.CKPT_INTERVAL = 8  # the rotating kernels are built for 8-step tiles
    yield
    nsb.set_tuning()
    nsb.set_scan_rotation()
    ps.CKPT_INTERVAL = None
    assert nsb.device_error_word() == 0


def _run(rf, T, B, D, seed, rotation, grads):
    d, b, v0, w0 = mod_inputs(T, B, D, torch.bfloat16, seed, rf)
    nsb.set_tuning(lanes_per_thread=1)  # (the planner may give a thread several columns; rotation is for one)
    nsb.set_scan_rotation(rotation)
    if grads:
        g = torch.Generator(device=DEV).manual_seed(seed + 1)
        gs = (torch.randn((T, B, D), generator=g, device=DEV) * 0.1).to(torch.bfloat16)
        out = _fused_grads(d, b, v0, w0, gs, _Sigmoid(4.0), rf)
        return nsb.last_scan_rotation(), [out[k] for k in sorted(out)]
    args = (d["raw_beta"], b["b_beta"], d["raw_alpha"], b["b_alpha"], d["raw_th"], b["b_th"], 0.1, d["cur"])
    with torch.no_grad():
        out = (sb.modulated_rf_plif_forward(*args, d["raw_omega"], b["b_omega"], v0, w0) if rf
               else sb.modulated_plif_forward(*args, v0))
    return nsb.last_scan_rotation(), [o.clone() for o in out]


@pytest.mark.parametrize("rf", [False, True])
@pytest.mark.parametrize("shape,rotation,expect", [
    ((1032 + 5, 2, 768), 2, 2),   # ragged T
    ((1032 + 5, 2, 768), 3, 3),
    ((1024, 1, 200), 4, 4),       # ragged columns: 6 full warps and one with 8 columns
    ((2048, 8, 768), 0, 4),       # automatic: 192 column warps for 592 schedulers
    ((40, 2, 96), 4, 1),          # 5 tiles: too short to share
    ((8, 1, 64), 2, 1),
])
def test_rotated_forward_equals_the_one_warp_scan(rf, shape, rotation, expect):
    T, B, D = shape
    used, got = _run(rf, T, B, D, seed=11, rotation=rotation, grads=False)
    assert used == expect
    ref_used, ref = _run(rf, T, B, D, seed=11, rotation=1, grads=False)
    assert ref_used == 1
    for a, e in zip(got, ref):
        assert torch.equal(a, e)


@pytest.mark.parametrize("rf", [False, True])
@pytest.mark.parametrize("rotation", [2, 4])
def test_gradients_from_a_rotated_forward_are_the_same_bits(rf, rotation):
    """The backward recomputes from the forward's checkpoints: equal gradients mean equal checkpoints."""
    used, got = _run(rf, 1024 + 16, 2, 384, seed=5, rotation=rotation, grads=True)
    assert used == rotation
    _, ref = _run(rf, 1024 + 16, 2, 384, seed=5, rotation=1, grads=True)
    assert len(got) == len(ref) >= 6
    for a, e in zip(got, ref):
        assert torch.equal(a, e)


@pytest.mark.parametrize("rf", [False, True])
@pytest.mark.parametrize("rotation", [1, 0, 3])
def test_bit_packed_spikes_of_a_rotated_forward(rf, rotation):
    """The same call through the C ABI with bit-packed spikes out (32 columns per word, ballots kept per
    tile): the words spell the dense spikes of the unrotated launch."""
    from neuronspark_b200 import _lib
    T, B, D = 1024 + 8, 2, 768
    cols = B * D
    d, b, v0, w0 = mod_inputs(T, B, D, torch.bfloat16, 9, rf)
    L, p = _lib.lib(), _lib.ptr
    bias = [b["b_beta"].float().contiguous(), b["b_alpha"].float().contiguous(), b["b_th"].float().contiguous(),
            (b["b_omega"].float().contiguous() if rf else None)]
    v0f = v0.float().contiguous()
    w0f = w0.float().contiguous() if rf else None
    v_last = torch.empty_like(v0f)
    w_last = torch.empty_like(v0f) if rf else None

    def call(dense, packed):
        _lib.check(L.nsb_plif_modulated_fwd(
            p(d["raw_beta"]), p(d["raw_alpha"]), p(d["raw_th"]), p(d["raw_omega"]) if rf else None, p(d["cur"]),
            p(bias[0]), p(bias[1]), p(bias[2]), p(bias[3]) if rf else None, 0.1, D, p(v0f), p(w0f) if rf else None,
            p(dense), p(packed), None, None, p(v_last), p(w_last) if rf else None, 4.0, 0.0, None, None, T, cols,
            _lib.BF16, 8, None, _lib.stream_ptr(DEV)), "nsb_plif_modulated_fwd")
        torch.cuda.synchronize()

    nsb.set_scan_rotation(1)
    dense = torch.empty((T, B, D), dtype=torch.bfloat16, device=DEV)
    call(dense, None)
    want_v = v_last.clone()
    nsb.set_scan_rotation(rotation)
    packed = torch.zeros((T, (cols + 31) // 32), dtype=torch.int32, device=DEV)
    call(None, packed)
    assert nsb.last_scan_rotation() == (1 if rotation == 1 else (4 if rotation == 0 else 3))
    assert torch.equal(ps.unpack_spikes(packed, (B, D)), dense.float())
    assert torch.equal(v_last, want_v)
