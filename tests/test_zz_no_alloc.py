"""The allocation-free backward of the lateral inhibition.

``nsb_lateral_inhibition_bwd_static`` exists for callers that may not allocate
device memory where they run the backward (a process that gave the whole GPU to
its own pool, a plugin that is only handed buffers, a loop where the CUDA
allocator's implicit synchronisation is unacceptable): it keeps its partial
sums in a fixed 2 MiB array inside the library instead of taking scratch from
the caller. This test calls it straight through the C ABI, twice in a row on
different data (the array is shared between calls and keeps old contents), and
compares with the ordinary entry point, which gets its scratch from the caller.

The file is named so that pytest collects it last: a run that stops at the
first failure has then already run every other test.
"""
import ctypes

import numpy as np
import pytest
import torch

from neuronspark_b200 import _lib
from oracle import oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _run_both(rows, D, dtype, seed, gain_dtype=torch.float32, side_stream=False, keep_inputs=None):
    L = _lib.lib()
    g = torch.Generator(device=DEV).manual_seed(seed)
    x = (2 * torch.randn(rows, D, generator=g, device=DEV)).to(dtype)
    go = torch.randn(rows, D, generator=g, device=DEV).to(dtype)
    gain = (1 + 0.1 * torch.randn(D, generator=g, device=DEV)).to(gain_dtype)
    if keep_inputs is not None:
        keep_inputs.update(x=x, go=go, gain=gain)
    torch.cuda.synchronize()
    s = torch.cuda.Stream(device=DEV) if side_stream else torch.cuda.current_stream(torch.device(DEV))
    stream = ctypes.c_void_p(s.cuda_stream)
    code = _lib.dtype_code(dtype)
    gcode = _lib.dtype_code(gain_dtype)

    gx_ref = torch.empty_like(x)
    gg_ref = torch.empty(D, dtype=torch.float32, device=DEV)
    scratch = torch.empty(int(L.nsb_li_bwd_scratch_floats(rows, D)), dtype=torch.float32, device=DEV)
    _lib.check(L.nsb_lateral_inhibition_bwd(_lib.ptr(go), _lib.ptr(x), _lib.ptr(gain), _lib.ptr(gx_ref),
                                            _lib.ptr(gg_ref), _lib.ptr(scratch), rows, D, 1e-6, code,
                                            gcode, stream), "nsb_lateral_inhibition_bwd")
    s.synchronize()

    gx = torch.full_like(x, float("nan"))
    gg = torch.full((D,), float("nan"), dtype=torch.float32, device=DEV)
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    free_before = torch.cuda.mem_get_info()[0]  # the driver's count: a cudaMalloc inside the library would show here
    _lib.check(L.nsb_lateral_inhibition_bwd_static(_lib.ptr(go), _lib.ptr(x), _lib.ptr(gain), _lib.ptr(gx),
                                                   _lib.ptr(gg), rows, D, 1e-6, code, gcode, stream),
               "nsb_lateral_inhibition_bwd_static")
    s.synchronize()
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before
    if _run_both.warm:  # (the very first call looks up the array's address; nothing is allocated then either,
        assert torch.cuda.mem_get_info()[0] >= free_before  # but the context may still be growing its own pools)
    _run_both.warm = True
    return gx_ref, gg_ref, gx, gg


_run_both.warm = False


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_static_scratch_backward_matches_twice_in_a_row(dtype):
    # 1e-5 relative on grad_gain, the tolerance of the normaliser tests; grad_x does not depend on
    # the scratch and must be identical.
    for call, (rows, D, seed) in enumerate([(4096, 768, 1), (777, 1000, 2), (4096, 768, 3)]):
        gx_ref, gg_ref, gx, gg = _run_both(rows, D, dtype, seed)
        assert torch.equal(gx, gx_ref), f"call {call}: grad_x differs"
        a, e = gg.cpu().double().numpy(), gg_ref.cpu().double().numpy()
        assert np.isfinite(a).all()
        assert np.abs(a - e).max() <= 1e-5 * np.abs(e).max(), f"call {call}: grad_gain differs"


def test_static_scratch_other_types_streams_and_the_oracle():
    """Half activations, a bf16 gain, a side stream, a row count that fills the array to the last float
    (256 CTAs x 2048 floats = 524 288), and one direct comparison with the CPU oracle."""
    for rows, D, dtype, gdt, side in [(1500, 768, torch.float16, torch.float32, False),
                                      (1500, 768, torch.bfloat16, torch.bfloat16, True),
                                      (4096, 2048, torch.float32, torch.float32, True)]:
        keep = {}
        gx_ref, gg_ref, gx, gg = _run_both(rows, D, dtype, 11, gain_dtype=gdt, side_stream=side, keep_inputs=keep)
        assert torch.equal(gx, gx_ref)
        e = gg_ref.cpu().double().numpy()
        assert np.abs(gg.cpu().double().numpy() - e).max() <= 1e-5 * np.abs(e).max()
        if dtype == torch.float32:
            f = lambda t: t.float().cpu().numpy()
            want_gx, want_gg = orc.li_bwd(f(keep["go"]), f(keep["x"]), f(keep["gain"]))
            assert np.abs(f(gx) - want_gx).max() <= 1e-5 * np.abs(want_gx).max()
            assert np.abs(f(gg) - want_gg).max() <= 1e-5 * np.abs(want_gg).max()


def test_both_entry_points_share_the_row_width_limit():
    """One warp's fp32 row of partial sums must fit a CTA's 227 KB of shared memory: D <= 58 112, for the
    caller-scratch entry point and the static one alike (status 5 = too large, nothing launched)."""
    L = _lib.lib()
    rows, D = 4, 58113
    x = torch.zeros(rows, D, device=DEV)
    gain = torch.ones(D, device=DEV)
    gx, gg = torch.empty_like(x), torch.empty(D, device=DEV)
    scratch = torch.empty(4 * D, device=DEV)
    st = _lib.stream_ptr(torch.device(DEV))
    p = _lib.ptr
    assert L.nsb_lateral_inhibition_bwd(p(x), p(x), p(gain), p(gx), p(gg), p(scratch), rows, D, 1e-6, 0, 0, st) == 5
    assert L.nsb_lateral_inhibition_bwd_static(p(x), p(x), p(gain), p(gx), p(gg), rows, D, 1e-6, 0, 0, st) == 5
    D = 57344
    x = torch.randn(rows, D, device=DEV)
    gain, gx, gg = torch.ones(D, device=DEV), torch.empty(rows, D, device=DEV), torch.empty(D, device=DEV)
    assert L.nsb_lateral_inhibition_bwd_static(p(x), p(x), p(gain), p(gx), p(gg), rows, D, 1e-6, 0, 0, st) == 0
    torch.cuda.synchronize()
    assert torch.isfinite(gg).all()


def test_static_scratch_uses_fewer_ctas_for_wide_rows_and_rejects_too_wide():
    # 296 CTAs x 6144 floats would not fit 524 288 floats: the call shrinks its grid instead
    gx_ref, gg_ref, gx, gg = _run_both(2000, 6144, torch.bfloat16, 5)
    assert torch.equal(gx, gx_ref)
    e = gg_ref.cpu().double().numpy()
    assert np.abs(gg.cpu().double().numpy() - e).max() <= 1e-5 * np.abs(e).max()
    z = ctypes.c_void_p(0)
    L = _lib.lib()
    assert L.nsb_lateral_inhibition_bwd_static(z, z, z, z, z, 4, (1 << 19) + 1, 1e-6, 0, 0, z) == 5
