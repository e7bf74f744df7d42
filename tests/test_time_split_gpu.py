"""Row-parameter forward scans over few columns, cut along time into segments that run side by side
(nsb_set_time_split): results equal the unsplit scan's bit for bit - with the default warm-up, where
no segment needs a second pass, and with a warm-up far too short, where the checking launch finds
the segments whose assumed starting state was wrong and rescans them."""
import numpy as np
import pytest
import torch

import neuronspark_b200 as nsb
from neuronspark_b200 import _lib, fp16_codec as codec, parallel_scan as ps
from oracle import oracle as orc
from util import assert_close, f32, rowparam_inputs

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)


@pytest.fixture(autouse=True)
def _clean():
    nsb.set_tuning()
    nsb.set_time_split()
    ps.CKPT_INTERVAL = None
    yield
    nsb.set_tuning()
    nsb.set_time_split()
    ps.CKPT_INTERVAL = None
    assert nsb.device_error_word() == 0


def unsplit(fn):
    nsb.set_time_split(1)
    try:
        out = fn()
        assert nsb.last_time_split()["segments"] == 1
        return out
    finally:
        nsb.set_time_split()


def test_config1_is_split_and_exact():
    """B=8, T=8192, D=768 (6144 columns = 192 warps for 592 schedulers): three segments, no rescans,
    every packed word and final state equal to the unsplit scan and to the oracle."""
    br, u, tr, v0 = rowparam_inputs(8192, 8, 768, torch.bfloat16, DEV, seed=1234)
    packed, v_last = ps.plif_rowparam_forward_packed(br, u, tr, v0)
    ts = nsb.last_time_split()
    assert ts["segments"] >= 2 and nsb.last_launch_info()["launches"] == 2, ts
    ref_packed, ref_v = unsplit(lambda: ps.plif_rowparam_forward_packed(br, u, tr, v0))
    assert torch.equal(packed, ref_packed) and torch.equal(v_last, ref_v)
    rs, _, rl = orc.plif_rowparam_fwd(f32(br), f32(u), f32(tr), f32(v0), want_vpost=False)
    assert np.array_equal(f32(ps.unpack_spikes(packed, (8, 768))), rs) and np.array_equal(f32(v_last), rl)


def raw_packed_scan(br, u, tr, v0, tile=32):
    """nsb_plif_rowparam_fwd through the C ABI with the test's own scratch, so that the rescan
    counter can be read back."""
    T, cols = u.shape[0], u.shape[1] * u.shape[2]
    L = _lib.lib()
    scratch = torch.zeros(int(L.nsb_time_split_scratch_floats(cols)), dtype=torch.float32, device=DEV)
    packed = torch.empty((T, (cols + 31) // 32), dtype=torch.int32, device=DEV)
    v_last = torch.empty(u.shape[1:], dtype=torch.float32, device=DEV)
    p = _lib.ptr
    _lib.check(L.nsb_plif_rowparam_fwd(p(br), p(u), p(tr), p(v0), None, p(packed), None, None, p(v_last), T, cols,
                                       _lib.dtype_code(u.dtype), tile, p(scratch), _lib.stream_ptr(DEV)), "fwd")
    torch.cuda.synchronize()
    ts = nsb.last_time_split()
    rescans = int(scratch[2 * ts["segments"] * cols:].view(torch.int32)[0]) if ts["segments"] > 1 else 0
    return packed, v_last, ts, rescans


@pytest.mark.parametrize("segments", [2, 3, 5, 16])
def test_too_short_a_warm_up_is_caught_and_repaired(segments):
    br, u, tr, v0 = rowparam_inputs(4096, 2, 200, torch.bfloat16, DEV, seed=segments)
    ref_packed, ref_v, ts0, _ = unsplit(lambda: raw_packed_scan(br, u, tr, v0))
    nsb.set_time_split(segments, 32)  # one tile of warm-up: most lanes have not merged by then
    packed, v_last, ts, rescans = raw_packed_scan(br, u, tr, v0)
    assert ts["segments"] == segments and ts["warm_tiles"] == 1
    assert rescans > 0, "a 32-step warm-up cannot have brought every lane to the exact state"
    assert torch.equal(packed, ref_packed) and torch.equal(v_last, ref_v)
    nsb.set_time_split(segments, 2048 if segments <= 2 else 4096 // segments // 32 * 32)
    packed, v_last, ts, rescans = raw_packed_scan(br, u, tr, v0)
    assert torch.equal(packed, ref_packed) and torch.equal(v_last, ref_v)


@pytest.mark.parametrize("shape", [(4096, 2, 96), (4100, 3, 333), (5000, 1, 1001), (4128, 9, 1024)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("warm", [0, 64])
def test_training_forward_and_gradients_equal_unsplit(shape, dtype, warm):
    T, B, D = shape
    br, u, tr, v0 = rowparam_inputs(T, B, D, dtype, DEV, seed=T + D)
    v0 = 0.1 * torch.randn(B, D, device=DEV)
    g = (torch.randn(T, B, D, device=DEV) * 0.1).to(dtype)

    def run():
        leaves = [t.clone().requires_grad_() for t in (br, u, tr, v0)]
        spike, v_last = ps.plif_rowparam_forward_recompute(*leaves, 4.0)
        spike.backward(g)
        return [spike.detach(), v_last.detach()] + [t.grad for t in leaves]

    ref = unsplit(run)
    nsb.set_time_split(0 if warm == 0 else 4, warm)
    out = run()
    if warm:
        assert nsb.last_launch_info()["launches"] in (1, 2)
    for a, b, name in zip(out, ref, ("spike", "v_last", "g_beta", "g_u", "g_vth", "g_v0")):
        if name in ("g_beta", "g_vth"):
            # sums over time, added up segment by segment in the split backward: the same terms in
            # another association, equal to fp32 rounding
            assert_close(f32(a), f32(b), tol=1e-5, what=name)
        else:
            assert torch.equal(a, b), name
    so, _, vl = orc.plif_rowparam_fwd(f32(br), f32(u), f32(tr), f32(v0), want_vpost=False)
    assert np.array_equal(f32(out[0]), so) and np.array_equal(f32(out[1]), vl)


@pytest.mark.parametrize("warm", [0, 32])
def test_residual_and_pattern_scans_equal_unsplit(warm):
    S, B, D = 256, 4, 768
    br, u, tr, v0 = rowparam_inputs(S * 16, B, D, torch.bfloat16, DEV, seed=21)
    u = u * 3.0
    fin = (torch.rand(S * 16, B, D, device=DEV) < 0.4).to(torch.bfloat16)
    pin = codec.pack_frames(fin)
    ref_res = unsplit(lambda: ps.plif_rowparam_residual_forward(br, u, tr, v0, fin, 4.0))
    ref_pat = unsplit(lambda: ps.plif_rowparam_forward_patterns(br, u, tr, v0, patterns_in=pin))
    nsb.set_time_split(0 if warm == 0 else 6, warm)
    res = ps.plif_rowparam_residual_forward(br, u, tr, v0, fin, 4.0)
    assert nsb.last_time_split()["segments"] >= 2
    pat = ps.plif_rowparam_forward_patterns(br, u, tr, v0, patterns_in=pin)
    assert nsb.last_time_split()["segments"] >= 2
    assert torch.equal(res[0], ref_res[0]) and torch.equal(res[1], ref_res[1])
    assert torch.equal(pat[0], ref_pat[0]) and torch.equal(pat[1], ref_pat[1])
    assert torch.equal(pat[0], codec.pack_frames(res[0]))


def raw_backward(br, u, tr, ckpt, gs, tile, scratch):
    T, cols = u.shape[0], u.shape[1] * u.shape[2]
    L, p = _lib.lib(), _lib.ptr
    g_u = torch.empty_like(u)
    g_b, g_t, g_v = (torch.empty(u.shape[1:], dtype=torch.float32, device=DEV) for _ in range(3))
    _lib.check(L.nsb_plif_rowparam_bwd(p(br), p(u), p(tr), p(ckpt), p(gs), None, p(g_b), p(g_u), p(g_t), p(g_v), T, cols,
                                       _lib.dtype_code(u.dtype), tile, _lib.SURR_SIGMOID, 4.0, p(scratch),
                                       _lib.stream_ptr(DEV)), "bwd")
    torch.cuda.synchronize()
    return g_u, g_v, g_b, g_t


@pytest.mark.parametrize("segments,warm", [(3, 0), (2, 32), (5, 32), (16, 32)])
def test_backward_split_exact_adjoint_and_repaired_speculation(segments, warm):
    """The backward through the C ABI with the test's own scratch: grad_u and grad_v_init equal the serial
    launch's bit for bit, the row sums to rounding; with a one-tile warm-up the checking launch must have
    rescanned segments (counter > 0) and the results are the same."""
    T, B, D, tile = 4096, 2, 200, 32
    br, u, tr, v0 = rowparam_inputs(T, B, D, torch.bfloat16, DEV, seed=40 + segments)
    u = u * 3.0
    cols = B * D
    L, p = _lib.lib(), _lib.ptr
    ckpt = torch.empty((T // tile, cols), dtype=torch.float32, device=DEV)
    spike, v_last = torch.empty_like(u), torch.empty_like(v0)
    nsb.set_time_split(1)
    _lib.check(L.nsb_plif_rowparam_fwd(p(br), p(u), p(tr), p(v0), p(spike), None, None, p(ckpt), p(v_last), T, cols,
                                       _lib.dtype_code(u.dtype), tile, None, _lib.stream_ptr(DEV)), "fwd")
    gs = (torch.randn(T, B, D, device=DEV) * 0.1).bfloat16()
    ref = raw_backward(br, u, tr, ckpt, gs, tile, None)
    assert nsb.last_time_split()["segments"] == 1
    nsb.set_time_split(segments, warm)
    scratch = torch.zeros(int(L.nsb_time_split_scratch_floats(cols)), dtype=torch.float32, device=DEV)
    out = raw_backward(br, u, tr, ckpt, gs, tile, scratch)
    ts = nsb.last_time_split()
    assert ts["segments"] == (segments if warm else 3), ts
    rescans = int(scratch[4 * ts["segments"] * cols:].view(torch.int32)[0])
    assert (rescans > 0) == (warm == 32), rescans
    assert torch.equal(out[0], ref[0]) and torch.equal(out[1], ref[1])
    assert_close(f32(out[2]), f32(ref[2]), tol=1e-5, what="grad beta_row")
    assert_close(f32(out[3]), f32(ref[3]), tol=1e-5, what="grad v_th_row")
    # and against the oracle
    want = orc.plif_rowparam_bwd(f32(br), f32(u), f32(tr), f32(v0), f32(gs), None, 4.0)
    assert_close(f32(out[2]), want[0], what="grad beta_row vs oracle")
    assert_close(f32(out[1]), want[3], what="grad v_init vs oracle")


def test_large_problems_are_left_alone():
    br, u, tr, v0 = rowparam_inputs(4096, 64, 768, torch.bfloat16, DEV, seed=2)  # 49 152 columns
    ps.plif_rowparam_forward_packed(br, u, tr, v0)
    assert nsb.last_time_split()["segments"] == 1 and nsb.last_launch_info()["launches"] == 1


def test_several_warps_per_scheduler():
    """12 288 columns are 384 column warps for 592 schedulers: the split still pays with several warps on
    a scheduler, and stays exact."""
    br, u, tr, v0 = rowparam_inputs(8192, 16, 768, torch.bfloat16, DEV, seed=7)
    packed, v_last = ps.plif_rowparam_forward_packed(br, u, tr, v0)
    assert nsb.last_time_split()["segments"] >= 2 and nsb.last_launch_info()["launches"] == 2
    ref_packed, ref_v = unsplit(lambda: ps.plif_rowparam_forward_packed(br, u, tr, v0))
    assert torch.equal(packed, ref_packed) and torch.equal(v_last, ref_v)


# ---- the scans of the hidden neurons (per-step parameters; forward only)


def _hidden_forward(kind, T, B, D, seed, want_grad=False):
    """(callable returning the scan's outputs as a tuple of tensors) for one of the hidden-neuron scans."""
    from neuronspark_b200 import snn_block as sb
    from test_modulated_gpu import mod_inputs
    from test_rf_gpu import rf_inputs
    from util import selective_inputs
    if kind == "u":
        beta, cur, _, vth, v0 = selective_inputs(T, B, D, torch.bfloat16, DEV, seed=seed, zero_init=False)
        return lambda: ps.plif_selective_forward_packed(beta, cur, vth, v0)
    if kind == "rf":
        beta, omega, u, vth, v0, w0 = rf_inputs(T, B, D, torch.bfloat16, seed)
        return lambda: ps.rf_plif_parallel_forward_recompute(beta, omega, u, vth, v0, w0)
    rf = kind == "rfmod"
    d, b, v0, w0 = mod_inputs(T, B, D, torch.bfloat16, seed, rf)
    args = (d["raw_beta"], b["b_beta"], d["raw_alpha"], b["b_alpha"], d["raw_th"], b["b_th"], 0.1, d["cur"])
    if rf:
        return lambda: sb.modulated_rf_plif_forward(*args, d["raw_omega"], b["b_omega"], v0, w0)
    return lambda: sb.modulated_plif_forward(*args, v0)


@pytest.mark.parametrize("kind", ["u", "rf", "mod", "rfmod"])
@pytest.mark.parametrize("segments,warm", [(0, 0), (4, 0), (7, 64), (3, 32)])
def test_hidden_neuron_scans_split_equal_unsplit(kind, segments, warm):
    """A single sequence of the 768-wide model is 6 144 columns of hidden neurons: on request the
    selective, resonate-and-fire and modulated forward scans are cut along time as the row-parameter
    ones are, with both states (V, W) compared at every boundary; short warm-ups force rescans."""
    T, B, D = 4096 + 40, 2, 768 if kind != "u" else 1024
    run = _hidden_forward(kind, T, B, D, seed=31)
    if kind in ("mod", "rfmod"):
        ps.CKPT_INTERVAL = 32  # (a no-grad modulated forward over few columns takes 8-step tiles by default, which rotate among warps instead)
    nsb.set_time_split(segments, warm)
    with torch.no_grad():
        got = run()
    ts = nsb.last_time_split()
    if segments == 0:  # these neurons' memory may outlast any warm-up: split only on request
        assert ts["segments"] == 1 and nsb.last_launch_info()["launches"] == 1, ts
    else:
        assert ts["segments"] >= 2 and nsb.last_launch_info()["launches"] == 2, ts
    with torch.no_grad():
        ref = unsplit(run)
    for a, b in zip(got, ref):
        if a is not None:
            assert torch.equal(a, b)


def test_a_neuron_that_forgets_slowly_is_left_unsplit_after_one_try():
    """beta = 0.9995 keeps a difference alive for 30 000 steps: every segment of the first split launch
    is rescanned; the launch reports that to the host, and the next calls for the same neuron scan
    unsplit - while a neuron with a short memory, same shape, keeps its split. Results are exact
    throughout."""
    T, B, D = 8192, 8, 768
    br, u, tr, v0 = rowparam_inputs(T, B, D, torch.bfloat16, DEV, seed=77)
    slow = torch.full_like(br, 0.9995)
    u_small = (u.float() * 0.02).to(u.dtype)  # so that the slow neuron spikes now and then, not every step
    ref = unsplit(lambda: ps.plif_rowparam_forward_packed(slow, u_small, tr, v0))
    nsb.set_time_split()  # forget earlier launches
    first = ps.plif_rowparam_forward_packed(slow, u_small, tr, v0)
    assert nsb.last_time_split()["segments"] >= 2
    torch.cuda.synchronize()  # the counters have reached the host
    for _ in range(3):
        again = ps.plif_rowparam_forward_packed(slow, u_small, tr, v0)
        assert nsb.last_time_split()["segments"] == 1
        assert torch.equal(again[0], ref[0]) and torch.equal(again[1], ref[1])
    assert torch.equal(first[0], ref[0]) and torch.equal(first[1], ref[1])
    for _ in range(3):  # another neuron of the same shape is judged by its own launches
        ps.plif_rowparam_forward_packed(br, u, tr, v0)
        assert nsb.last_time_split()["segments"] >= 2
        torch.cuda.synchronize()
