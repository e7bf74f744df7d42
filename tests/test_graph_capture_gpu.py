"""The library's launches inside a CUDA graph.

Two entry points launch a pair of kernels of which the second is a dependent launch (its CTAs take their
places while the first kernel still runs and wait for it on the device): the lateral-inhibition backward
with the reduction of its partial rows, and a time-split scan with its checking launch. Captured into a
graph and replayed on fresh inputs, both give the results of the eager calls, bit for bit.
"""
import ctypes

import pytest
import torch

import neuronspark_b200 as nsb
from neuronspark_b200 import _lib, parallel_scan as ps
from util import rowparam_inputs

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)


@pytest.fixture(autouse=True)
def _clean():
    nsb.set_tuning()
    nsb.set_time_split()
    yield
    nsb.set_time_split()
    assert nsb.device_error_word() == 0


def _captured(fn):
    """fn() captured on a side stream (after one eager call, so that nothing is allocated or looked up for
    the first time inside the capture); returns the graph and what fn returned during the capture."""
    fn()
    torch.cuda.synchronize()
    side = torch.cuda.Stream(device=DEV)
    side.wait_stream(torch.cuda.current_stream(DEV))
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        out = fn()
    return graph, out


@pytest.mark.parametrize("rows,D", [(4096, 768), (512, 6144)])
def test_lateral_inhibition_backward_replays(rows, D):
    L = _lib.lib()
    g = torch.Generator(device=DEV).manual_seed(5)
    x = torch.empty(rows, D, device=DEV, dtype=torch.bfloat16)
    go = torch.empty_like(x)
    gain = (1 + 0.1 * torch.randn(D, generator=g, device=DEV))
    gx = torch.empty_like(x)
    gg = torch.empty(D, dtype=torch.float32, device=DEV)
    scratch = torch.empty(int(L.nsb_li_bwd_scratch_floats(rows, D)), dtype=torch.float32, device=DEV)
    code = _lib.dtype_code(torch.bfloat16)

    def call():
        stream = ctypes.c_void_p(torch.cuda.current_stream(DEV).cuda_stream)
        _lib.check(L.nsb_lateral_inhibition_bwd(_lib.ptr(go), _lib.ptr(x), _lib.ptr(gain), _lib.ptr(gx), _lib.ptr(gg),
                                                _lib.ptr(scratch), rows, D, 1e-6, code, _lib.dtype_code(torch.float32),
                                                stream), "nsb_lateral_inhibition_bwd")

    def fill(seed):
        gen = torch.Generator(device=DEV).manual_seed(seed)
        x.copy_((2 * torch.randn(rows, D, generator=gen, device=DEV)).to(torch.bfloat16))
        go.copy_(torch.randn(rows, D, generator=gen, device=DEV).to(torch.bfloat16))

    fill(1)
    graph, _ = _captured(call)
    for seed in (2, 3):
        fill(seed)
        call()
        torch.cuda.synchronize()
        want_gx, want_gg = gx.clone(), gg.clone()
        gx.fill_(float("nan"))
        gg.fill_(float("nan"))
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(gx, want_gx) and torch.equal(gg, want_gg)


def test_time_split_scan_replays():
    """B=8, T=8192, D=768 is cut along time (two launches); the captured pair replays to the eager result."""
    br, u, tr, v0 = rowparam_inputs(8192, 8, 768, torch.bfloat16, DEV, seed=21)
    graph, (packed, v_last) = _captured(lambda: ps.plif_rowparam_forward_packed(br, u, tr, v0))
    assert nsb.last_time_split()["segments"] >= 2
    for seed in (22, 23):
        _, u2, _, _ = rowparam_inputs(8192, 8, 768, torch.bfloat16, DEV, seed=seed)
        u.copy_(u2)
        want_packed, want_v = ps.plif_rowparam_forward_packed(br, u, tr, v0)
        torch.cuda.synchronize()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(packed, want_packed) and torch.equal(v_last, want_v)
