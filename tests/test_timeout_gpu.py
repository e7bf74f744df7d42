"""The device-side timeout path, exercised without a fault: a wait with a short limit that
nothing will ever satisfy runs out, the kernel returns by itself, the host learns of it through
the sticky status of the next scan call, and the library keeps working afterwards."""
import numpy as np
import pytest
import torch

import neuronspark_b200 as nsb
from neuronspark_b200 import NSBError, _lib, parallel_scan as ps
from oracle import oracle as orc
from util import f32, rowparam_inputs

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)


def test_wait_runs_out_is_reported_and_the_library_recovers():
    br, u, tr, v0 = rowparam_inputs(64, 2, 96, torch.bfloat16, DEV, seed=5)
    ps.plif_rowparam_forward_packed(br, u, tr, v0)  # the error word exists from the first scan on
    torch.cuda.synchronize()
    assert nsb.device_error_word() == 0
    nsb.set_wait_limit_ns(1_000_000)  # 1 ms
    try:
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        _lib.check(_lib.lib().nsb_selftest_wait_timeout(_lib.stream_ptr(DEV)), "nsb_selftest_wait_timeout")
        t1.record()
        torch.cuda.synchronize()  # returns: the waiting warp gave up on its own
        assert 0.5 <= t0.elapsed_time(t1) < 200.0  # it did wait, and for about the limit, not for 2 s
        # sticky status: the next scan call refuses to launch and says why
        with pytest.raises(NSBError, match="bounded device-side wait"):
            ps.plif_rowparam_forward_packed(br, u, tr, v0)
        word = nsb.device_error_word()
        assert word & 0x80000000, hex(word)  # the wait for a tile that never arrives
        assert word & 0x40000000, hex(word)  # the wait for a chunk that never finishes (chained backward)
        assert nsb.device_error_word() == 0  # reading cleared it
    finally:
        nsb.set_wait_limit_ns(0)
    # the context is intact and the next real scan is bit-exact
    packed, v_last = ps.plif_rowparam_forward_packed(br, u, tr, v0)
    rs, _, rl = orc.plif_rowparam_fwd(f32(br), f32(u), f32(tr), f32(v0), want_vpost=False)
    assert np.array_equal(f32(ps.unpack_spikes(packed, (2, 96))), rs) and np.array_equal(f32(v_last), rl)
    assert nsb.device_error_word() == 0


def test_tuning_without_a_launch_shape_is_unsupported_not_invalid():
    """lanes_per_thread = 4 with 32-step tiles has no kernel: status 2 (unsupported), and the
    message does not blame the caller's pointers."""
    br, u, tr, v0 = rowparam_inputs(64, 2, 128, torch.bfloat16, DEV, seed=6)
    nsb.set_tuning(lanes_per_thread=4)
    try:
        ps.CKPT_INTERVAL = 32
        with pytest.raises(NSBError, match="unsupported"):
            ps.plif_rowparam_forward_packed(br, u, tr, v0)
    finally:
        ps.CKPT_INTERVAL = None
        nsb.set_tuning()
