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

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _run_both(rows, D, dtype, seed):
    L = _lib.lib()
    g = torch.Generator(device=DEV).manual_seed(seed)
    x = (2 * torch.randn(rows, D, generator=g, device=DEV)).to(dtype)
    go = torch.randn(rows, D, generator=g, device=DEV).to(dtype)
    gain = 1 + 0.1 * torch.randn(D, generator=g, device=DEV)
    stream = _lib.stream_ptr(torch.device(DEV))
    code = _lib.dtype_code(dtype)

    gx_ref = torch.empty_like(x)
    gg_ref = torch.empty(D, dtype=torch.float32, device=DEV)
    scratch = torch.empty(int(L.nsb_li_bwd_scratch_floats(rows, D)), dtype=torch.float32, device=DEV)
    _lib.check(L.nsb_lateral_inhibition_bwd(_lib.ptr(go), _lib.ptr(x), _lib.ptr(gain), _lib.ptr(gx_ref),
                                            _lib.ptr(gg_ref), _lib.ptr(scratch), rows, D, 1e-6, code,
                                            _lib.F32, stream), "nsb_lateral_inhibition_bwd")

    gx = torch.full_like(x, float("nan"))
    gg = torch.full((D,), float("nan"), dtype=torch.float32, device=DEV)
    before = torch.cuda.memory_allocated()
    _lib.check(L.nsb_lateral_inhibition_bwd_static(_lib.ptr(go), _lib.ptr(x), _lib.ptr(gain), _lib.ptr(gx),
                                                   _lib.ptr(gg), rows, D, 1e-6, code, _lib.F32, stream),
               "nsb_lateral_inhibition_bwd_static")
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before
    return gx_ref, gg_ref, gx, gg


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


def test_static_scratch_uses_fewer_ctas_for_wide_rows_and_rejects_too_wide():
    # 296 CTAs x 6144 floats would not fit 524 288 floats: the call shrinks its grid instead
    gx_ref, gg_ref, gx, gg = _run_both(2000, 6144, torch.bfloat16, 5)
    assert torch.equal(gx, gx_ref)
    e = gg_ref.cpu().double().numpy()
    assert np.abs(gg.cpu().double().numpy() - e).max() <= 1e-5 * np.abs(e).max()
    z = ctypes.c_void_p(0)
    L = _lib.lib()
    assert L.nsb_lateral_inhibition_bwd_static(z, z, z, z, z, 4, (1 << 19) + 1, 1e-6, 0, 0, z) == 5
