"""Parity at the benchmark configurations' full sizes.

Where the CPU oracle finishes in seconds (configs 0 and 1) the whole output is
compared. At the headline size (config 2: 1.6 G neuron-steps) the oracle runs on
a strided sample of columns that reaches every warp of the forward launch and
every CTA of the backward launch, and the rest is covered by
size-independent properties: gradients are linear in the upstream gradient,
packed and dense spikes agree, and a scan cut in two with the state carried
equals the uncut scan."""
import numpy as np
import pytest
import torch

import bench
import neuronspark_b200 as nsb
from neuronspark_b200 import parallel_scan as ps
from oracle import oracle as orc
from util import assert_close, assert_close_lowp, f32, rowparam_inputs, selective_inputs

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)


@pytest.fixture(autouse=True)
def _clean():
    nsb.set_tuning()
    yield
    torch.cuda.empty_cache()
    assert nsb.device_error_word() == 0


def test_config0_full():
    """B=2, T=1024, D=768, fp32, V0=0: dense spikes and final V, whole output."""
    beta, cur, gain, vth, v0 = selective_inputs(1024, 2, 768, torch.float32, DEV, seed=1234)
    rs, _, rl = orc.plif_selective_ai_fwd(f32(beta), f32(cur), f32(gain), f32(vth), f32(v0))
    spike, v_last = ps.plif_selective_scan_ai(beta, cur, gain, vth, v0)
    assert np.array_equal(f32(spike), rs) and np.array_equal(f32(v_last), rl)
    assert 0.05 < rs.mean() < 0.5


def test_config1_full():
    """B=8, T=8192, D=768, bf16 drive, per-channel parameters, packed spikes, whole output."""
    br, u, tr, v0 = rowparam_inputs(8192, 8, 768, torch.bfloat16, DEV, seed=1234)
    rs, _, rl = orc.plif_rowparam_fwd(f32(br), f32(u), f32(tr), f32(v0), want_vpost=False)
    packed, v_last = ps.plif_rowparam_forward_packed(br, u, tr, v0)
    assert packed.shape == (8192, 8 * 768 // 32)
    assert np.array_equal(f32(ps.unpack_spikes(packed, (8, 768))), rs)
    assert np.array_equal(f32(v_last), rl)


def test_config2_full_size_properties():
    B, T, D = bench.WORKLOADS["c2"]
    inp = bench.make_inputs(B, T, D, DEV, 1234)
    names = ("beta", "cur", "gain", "vth")
    leaves = [inp[k].requires_grad_() for k in names] + [inp["v0"].requires_grad_()]
    spike, v_last = ps.plif_selective_scan_ai(*leaves, alpha=2.0, surrogate="atan")
    nsb_launch = {"fwd": nsb.last_launch_info()}
    spike.backward(inp["g_spike"], retain_graph=True)
    torch.cuda.synchronize()
    # the backward launch has more CTAs than the GPU holds: its time axis is cut into chained chunks
    assert nsb._lib.last_chain_chunks() > 1
    g1 = [t.grad for t in leaves]
    for t in leaves:
        t.grad = None

    # (0) the same backward as one CTA per column block over all of T: every gradient bit-identical
    nsb._lib.set_chain_chunks(1)
    try:
        spike.backward(inp["g_spike"], retain_graph=True)
        torch.cuda.synchronize()
        assert nsb._lib.last_chain_chunks() == 1
    finally:
        nsb._lib.set_chain_chunks()
    for a, t, n in zip(g1, leaves, names + ("v0",)):
        assert torch.equal(a, t.grad), f"chained and unchained backward differ in grad {n}"
        t.grad = None

    # (1) the oracle on columns cut out of the full problem: the two edge blocks, and one column out
    # of every 128 across the whole width - every warp of the forward launch and of the backward
    # launch (32 lanes x 4 columns each) has a column in the sample, and the offset
    # inside the 128 rotates so that all lanes and all four vector positions are hit - over all
    # 8192 steps, forward and the five gradients
    cols = B * D
    # (a warp owns 32 x lanes-per-thread <= 128 consecutive columns in both launches; the backward runs
    # on autograd's thread, so its launch record is not this thread's: ask the planner instead)
    assert 32 * nsb_launch["fwd"]["lanes_per_thread"] <= 128
    assert 32 * nsb._lib.scan_plan(True, 5, 2, T, cols)["lanes_per_thread"] <= 128
    w = np.arange(cols // 128)
    strided = torch.from_numpy(128 * w + (37 * w) % 128).to(DEV)
    assert len(strided) >= 1536 and len(set(((37 * w) % 128).tolist())) == 128
    edges = torch.cat([torch.arange(0, 96), torch.arange(cols - 96, cols)]).to(DEV)
    flat = lambda t: t.detach().reshape(T, cols)
    for idx in (edges, strided):
        pick = lambda t: f32(flat(t).index_select(1, idx))
        ins = [pick(inp[k]) for k in names]
        v0b = f32(inp["v0"].detach().reshape(cols)[idx])
        rs, _, rl = orc.plif_selective_ai_fwd(*ins, v0b, want_vpost=False)
        assert np.array_equal(pick(spike), rs), "spikes must be bit-exact"
        assert np.array_equal(f32(v_last.detach().reshape(cols)[idx]), rl)
        ref = orc.plif_selective_ai_bwd(*ins, v0b, pick(inp["g_spike"]), None, 2.0, orc.SURR_ATAN)
        for g, e, n in zip(g1[:4], ref[:4], names):
            assert_close_lowp(pick(g), e, torch.bfloat16, f"grad {n}")
        assert_close(f32(g1[4].reshape(cols)[idx]), ref[4], what="grad v_init")

    # (2) gradients are linear in the upstream gradient; doubling is exact in binary floating point
    spike2, _ = ps.plif_selective_scan_ai(*leaves, alpha=2.0, surrogate="atan")
    spike2.backward(inp["g_spike"] * 2)
    assert torch.equal(spike2, spike)
    for a, b in zip(g1, [t.grad for t in leaves]):
        assert torch.equal(a * 2, b)
    del spike2
    for t in leaves:
        t.grad = None
        t.requires_grad_(False)

    # (3) packed spikes equal the dense ones, bit for bit, over the whole tensor
    packed, v_last_p = ps.plif_selective_forward_packed(inp["beta"], inp["cur"], inp["vth"], inp["v0"],
                                                        gain=inp["gain"])
    assert torch.equal(v_last_p, v_last.float())
    step = 1024
    for t0 in range(0, T, step):
        dense = ps.unpack_spikes(packed[t0:t0 + step], (B, D), torch.bfloat16)
        assert torch.equal(dense, spike[t0:t0 + step])

    # (4) cutting the scan in two and carrying V gives the same spikes and the same final state
    h = T // 2 + 8
    p1, v_mid = ps.plif_selective_forward_packed(inp["beta"][:h], inp["cur"][:h], inp["vth"][:h],
                                                 inp["v0"], gain=inp["gain"][:h])
    p2, v_end = ps.plif_selective_forward_packed(inp["beta"][h:], inp["cur"][h:], inp["vth"][h:], v_mid,
                                                 gain=inp["gain"][h:])
    assert torch.equal(torch.cat([p1, p2]), packed) and torch.equal(v_end, v_last_p)


def test_decode_variant_carries_state():
    """Per-token decoding (config 4's variant): 16-step calls at B=1024, D=6144 with V carried
    between calls equal one 64-step scan; a column block is also checked against the oracle."""
    B, T, D = 1024, 64, 6144
    inp = bench.make_inputs(B, T, D, DEV, 77)
    whole, v_end = ps.plif_selective_forward_packed(inp["beta"], inp["cur"], inp["vth"], inp["v0"],
                                                    gain=inp["gain"])
    v = inp["v0"]
    parts = []
    for t0 in range(0, T, 16):
        sl = slice(t0, t0 + 16)
        p, v = ps.plif_selective_forward_packed(inp["beta"][sl], inp["cur"][sl], inp["vth"][sl], v,
                                                gain=inp["gain"][sl])
        parts.append(p)
    assert torch.equal(torch.cat(parts), whole) and torch.equal(v, v_end)
    cols = B * D
    sl = slice(cols - 4096, cols)
    ins = [f32(inp[k].reshape(T, cols)[:, sl]) for k in ("beta", "cur", "gain", "vth")]
    rs, _, rl = orc.plif_selective_ai_fwd(*ins, np.zeros(4096, np.float32), want_vpost=False)
    dense = ps.unpack_spikes(whole, (B, D)).reshape(T, cols)[:, sl]
    assert np.array_equal(f32(dense), rs) and np.array_equal(f32(v_end.reshape(cols)[sl]), rl)


def test_more_than_2_31_elements():
    """Tensors of more than 2^31 elements (B=44, T=8192, D=6144: 2.21 G per stream): element offsets
    no longer fit 32 bits. The last column block - whose offsets are the largest - is checked
    against the oracle, forward and backward, and the kernel that addresses global memory itself
    (no tensor maps) must give the same bits as the tiled one over the whole output."""
    B, T, D = 44, 8192, 6144
    cols = B * D
    assert T * cols > 2 ** 31
    inp = bench.make_inputs(B, T, D, DEV, 4321)
    names = ("beta", "cur", "gain", "vth")
    leaves = [inp[k].requires_grad_() for k in names] + [inp["v0"].requires_grad_()]
    spike, v_last = ps.plif_selective_scan_ai(*leaves, alpha=2.0, surrogate="atan")
    assert nsb.last_launch_info()["used_tma"] == 1
    spike.backward(inp["g_spike"])
    flat = lambda t: t.detach().reshape(T, cols)
    sl = slice(cols - 64, cols)
    ins = [f32(flat(inp[k])[:, sl]) for k in names]
    v0b = f32(inp["v0"].detach().reshape(cols)[sl])
    rs, _, rl = orc.plif_selective_ai_fwd(*ins, v0b, want_vpost=False)
    assert np.array_equal(f32(flat(spike)[:, sl]), rs)
    assert np.array_equal(f32(v_last.detach().reshape(cols)[sl]), rl)
    ref = orc.plif_selective_ai_bwd(*ins, v0b, f32(flat(inp["g_spike"])[:, sl]), None, 2.0, orc.SURR_ATAN)
    for t, e, n in zip(leaves[:4], ref[:4], names):
        assert_close_lowp(f32(flat(t.grad)[:, sl]), e, torch.bfloat16, f"grad {n}")
    assert_close(f32(leaves[4].grad.reshape(cols)[sl]), ref[4], what="grad v_init")
    g_tma = [t.grad for t in leaves]
    for t in leaves:
        t.grad = None

    nsb.set_tuning(force_direct=1)
    spike_d, v_last_d = ps.plif_selective_scan_ai(*leaves, alpha=2.0, surrogate="atan")
    assert nsb.last_launch_info()["used_tma"] == 0
    assert torch.equal(spike_d, spike) and torch.equal(v_last_d, v_last)
    spike_d.backward(inp["g_spike"])
    for a, t in zip(g_tma, leaves):
        assert torch.equal(a, t.grad)


def test_codec_more_than_2_31_frames():
    """fp16_encode of 140 M values writes 2.24 G frames; decoding them returns every value rounded
    to half, and the binary residual with an all-zero second stream is the identity."""
    from neuronspark_b200 import fp16_codec as codec
    Bv, S, Dv = 38, 600, 6144
    assert Bv * S * Dv * 16 > 2 ** 31
    g = torch.Generator(device=DEV).manual_seed(5)
    x = (torch.randn(Bv, S, Dv, generator=g, device=DEV) * 3.0).bfloat16()
    x[x.abs() < 1e-3] = 1.0  # keeps every value a normal half that bf16 holds exactly, and no -0
    frames = codec.fp16_encode(x)
    assert frames.shape == (S * 16, Bv, Dv) and frames.dtype == torch.bfloat16
    back = codec.fp16_decode(frames, S)
    assert torch.equal(back, x.half().to(torch.bfloat16))
    # the last value's 16 frames, by hand
    bits = int(x[-1, -1, -1].half().view(torch.int16)) & 0xFFFF
    assert [int(v) for v in frames[-16:, -1, -1].float()] == [(bits >> (15 - k)) & 1 for k in range(16)]
    zeros = torch.zeros_like(frames)
    assert torch.equal(codec.binary_residual(frames, zeros), frames)
