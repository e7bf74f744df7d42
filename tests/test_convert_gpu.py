"""nsb_convert: every pairing of fp32 / bf16 / fp16, bit-identical to torch's own conversion (exact
widening, round-to-nearest-even narrowing), on ragged lengths and unaligned starts; and the scan
mirrors use it for inputs whose dtypes differ (no framework op on [T, ...] tensors)."""
import pytest
import torch

from neuronspark_b200 import _lib, parallel_scan as ps

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)
DTYPES = [torch.float32, torch.bfloat16, torch.float16]


@pytest.mark.parametrize("src", DTYPES)
@pytest.mark.parametrize("dst", DTYPES)
@pytest.mark.parametrize("n,offset", [(1, 0), (7, 1), (4096, 0), (100003, 3)])
def test_convert_matches_torch(src, dst, n, offset):
    g = torch.Generator(device=DEV).manual_seed(n)
    base = (torch.randn(n + offset, generator=g, device=DEV) * torch.logspace(-8, 5, n + offset, device=DEV)).to(src)
    base[:: 97] = 0.0
    x = base[offset:]
    got = _lib.convert(x, dst)
    want = x.to(dst)
    assert got.dtype == dst and got.is_contiguous()
    view = torch.int32 if dst == torch.float32 else torch.int16
    assert torch.equal(got.view(view), want.view(view))


def test_mixed_input_dtypes_go_through_the_library(monkeypatch):
    calls = []
    real = _lib.convert
    monkeypatch.setattr(_lib, "convert", lambda t, dt: (calls.append((t.dtype, dt)), real(t, dt))[1])
    T, B, D = 64, 2, 96
    g = torch.Generator(device=DEV).manual_seed(1)
    beta = torch.sigmoid(2 + 0.5 * torch.randn(T, B, D, generator=g, device=DEV))            # fp32
    u = torch.randn(T, B, D, generator=g, device=DEV).bfloat16().requires_grad_()             # bf16
    vth = (0.1 + torch.rand(T, B, D, generator=g, device=DEV)).half()                         # fp16
    v0 = torch.zeros(B, D, device=DEV)
    spike, vpost = ps._TritonPLIFForward.apply(beta, u, vth, v0, 4.0)
    assert spike.dtype == torch.bfloat16  # follows u, as empty_like(u) does in the reference
    spike.float().sum().backward()
    assert u.grad.dtype == torch.bfloat16
    assert (torch.bfloat16, torch.float32) in calls and (torch.float16, torch.float32) in calls
    assert (torch.float32, torch.bfloat16) in calls  # outputs and grad_u converted back by the same kernel
    ref_s, ref_v = ps._TritonPLIFForward.apply(beta, u.detach().float(), vth.float(), v0, 4.0)
    assert torch.equal(spike.float(), ref_s) and torch.equal(vpost.float(), ref_v.bfloat16().float())
