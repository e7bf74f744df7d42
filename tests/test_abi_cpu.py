"""CPU-side checks of the C-ABI library and of the host logic: the shared
object loads, exports every symbol the header declares, and the Python mirror
refuses to run without a CUDA device (no fallback)."""
import ctypes
import re
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def built_lib():
    from neuronspark_b200 import build
    return build.build()


def declared_symbols():
    text = (ROOT / "include" / "neuronspark_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(nsb_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(built_lib):
    handle = ctypes.CDLL(str(built_lib))
    names = declared_symbols()
    assert len(names) >= 18
    for n in names:
        assert hasattr(handle, n), f"{n} is declared in the header but not exported"


def test_binding_covers_the_header(built_lib):
    from neuronspark_b200 import _lib
    assert sorted(_lib.EXPORTED_SYMBOLS) == declared_symbols()
    L = _lib.lib()
    assert L.nsb_version() >= 100
    assert L.nsb_status_string(0) == b"ok"
    for code in range(1, 6):
        assert L.nsb_status_string(code) not in (b"ok", b"unknown status")
    assert L.nsb_status_string(99) == b"unknown status"


def test_argument_validation_needs_no_gpu(built_lib):
    """Bad sizes / enums are rejected before anything touches CUDA."""
    from neuronspark_b200 import _lib
    L = _lib.lib()
    z = ctypes.c_void_p(0)
    assert L.nsb_plif_selective_fwd(z, z, z, z, z, z, z, z, z, z, -1, 8, 0, 8, z, z) == 1
    assert L.nsb_plif_selective_fwd(z, z, z, z, z, z, z, z, z, z, 8, 8, 7, 8, z, z) == 1   # dtype
    assert L.nsb_plif_selective_fwd(z, z, z, z, z, z, z, z, z, z, 8, 8, 0, 5, z, z) == 1   # interval
    assert L.nsb_plif_selective_fwd(z, z, z, z, z, z, z, z, z, z, 8, 8, 0, 8, z, z) == 1   # nulls
    assert L.nsb_plif_selective_fwd(z, z, z, z, z, z, z, z, z, z, 8, 0, 0, 8, z, z) == 0   # empty
    assert L.nsb_plif_selective_bwd(z, z, z, z, z, z, z, z, z, z, z, z, 8, 8, 0, 8, 9, 1.0, z, z) == 1
    assert L.nsb_plif_rowparam_fwd(z, z, z, z, z, z, z, z, z, 4, 4, 0, 8, z, z) == 1
    assert L.nsb_fp16_encode(z, z, 1, 1, 0, 0, 0, z) == 0
    assert L.nsb_fp16_encode(z, z, 1, 1, 4, 0, 0, z) == 1
    assert L.nsb_set_tuning(64, 0, 0, 0) == 1 and L.nsb_set_tuning(0, 0, 3, 0) == 1
    assert L.nsb_set_tuning(0, 0, 0, 0) == 0
    assert L.nsb_set_scan_rotation(5) == 1 and L.nsb_set_scan_rotation(-1) == 1
    assert L.nsb_set_scan_rotation(3) == 0 and L.nsb_set_scan_rotation(0) == 0
    assert 1 <= L.nsb_last_scan_rotation() <= 4  # (1 while this thread has launched no forward scan)
    assert L.nsb_set_chain_chunks(1025) == 1 and L.nsb_set_chain_chunks(0) == 0


def test_no_cpu_fallback(built_lib):
    import neuronspark_b200 as nsb
    from neuronspark_b200 import fp16_codec, lateral_inhibition, parallel_scan
    with pytest.raises(nsb.NSBError):
        parallel_scan.plif_rowparam_forward_alpha(torch.ones(2, 4), torch.ones(3, 2, 4),
                                                  torch.ones(2, 4), torch.zeros(2, 4), 4.0)
    with pytest.raises(nsb.NSBError):
        fp16_codec.fp16_encode(torch.ones(1, 2, 4))
    with pytest.raises(nsb.NSBError):
        lateral_inhibition.LateralInhibition(4)(torch.ones(2, 4))


def test_stream_dtype_rule():
    from neuronspark_b200.parallel_scan import _common_stream_dtype
    b, h, f = (torch.empty(1, dtype=d) for d in (torch.bfloat16, torch.float16, torch.float32))
    assert _common_stream_dtype(b, b, b) == torch.bfloat16
    assert _common_stream_dtype(h, h) == torch.float16
    assert _common_stream_dtype(b, f, b) == torch.float32
    assert _common_stream_dtype(b, h) == torch.float32
    assert _common_stream_dtype(torch.empty(1, dtype=torch.float64)) == torch.float32
    assert _common_stream_dtype(b, None, b) == torch.bfloat16


def test_launch_planner(built_lib):
    """The planner is pure host arithmetic over a B200 description."""
    from neuronspark_b200 import _lib
    _lib.set_tuning()
    # headline shape: 196 608 columns, bf16, gain*cur form
    fwd = _lib.scan_plan(False, 4, 2, 8192, 32 * 6144)
    bwd = _lib.scan_plan(True, 5, 2, 8192, 32 * 6144)
    for p in (fwd, bwd):
        assert p["lanes_per_thread"] in (1, 2, 4) and 2 <= p["stages"] <= 6
        assert p["grid"] * p["warps_per_cta"] * 32 * p["lanes_per_thread"] >= 32 * 6144
        assert p["smem_bytes"] <= 227 * 1024
    # wide TMA tiles (>= 2 KB per stream) are what reaches HBM bandwidth on this shape
    assert fwd["lanes_per_thread"] * 8 * 32 * 2 >= 2048
    # the override is honoured
    _lib.set_tuning(warps_per_cta=3, stages=2, lanes_per_thread=2)
    p = _lib.scan_plan(True, 5, 2, 8192, 32 * 6144)
    assert (p["lanes_per_thread"], p["warps_per_cta"], p["stages"]) == (2, 3, 2)
    _lib.set_tuning()
    # a single tile never asks for a deep ring; tiny problems still get a plan
    assert _lib.scan_plan(False, 1, 4, 5, 7)["grid"] == 1


def test_time_axis_planning(built_lib):
    """The division of the time axis - segments of the row-parameter time split, chained chunks of a
    backward launch - is host arithmetic; the measured cases it was fitted to, without a GPU."""
    from neuronspark_b200 import _lib
    split = lambda bwd, cols, T=8192: _lib.time_plan(bwd, T, cols, tile=32)["segments"]
    # forward / backward segments at T = 8192 (one lane per thread, 32-step tiles, warm-up 1024 steps)
    assert (split(False, 6144), split(True, 6144)) == (8, 6)      # config 1: 192 column warps for 592 schedulers
    assert (split(False, 1536), split(True, 1536)) == (8, 8)
    assert (split(False, 12288), split(True, 12288)) == (6, 3)
    assert (split(False, 24576), split(True, 24576)) == (3, 2)
    assert (split(False, 36864), split(True, 36864)) == (2, 1)
    assert (split(False, 49152), split(True, 49152)) == (1, 1)    # too wide: left alone
    assert split(False, 6144, T=1024) == 1                         # too short for a warm-up of 1024 steps
    p = _lib.time_plan(False, 8192, 6144, tile=32)
    assert p["seg_tiles"] * p["segments"] >= 256 > p["seg_tiles"] * (p["segments"] - 1) and p["warm_tiles"] == 32
    # chained chunks of the backward: 128-step chunks from 98 304 columns on, 512-step chunks from 49 152
    chain = lambda cols, **k: _lib.time_plan(True, 8192, cols, tile=8, **k)["chain_chunks"]
    assert chain(196608, lanes=4, warps_per_cta=2) == 64
    assert chain(98304, lanes=2, warps_per_cta=2) == 64
    assert chain(49152, lanes=2) == 16
    assert chain(24576) == 1
    assert _lib.time_plan(False, 8192, 196608, tile=8, lanes=4, warps_per_cta=4)["chain_chunks"] == 1  # forward: never
    # modulation fused in: only where the launch has more CTAs than the GPU holds (768 for 444)
    assert chain(196608, lanes=2, warps_per_cta=4, modulated=True) == 8
    assert chain(98304, lanes=2, warps_per_cta=4, modulated=True) == 1
    # the hidden neurons' scans (per-step parameters; a memory that may outlast any warm-up) are cut along
    # time only on request
    L = _lib.lib()
    hidden = lambda: _lib.time_plan(False, 8192, 6144, tile=32, modulated=True)["segments"]
    assert hidden() == 1
    try:
        assert L.nsb_set_time_split(4, 0) == 0
        assert 2 <= hidden() <= 4 and 2 <= split(False, 6144) <= 4  # at most that many
        assert L.nsb_set_time_split(1, 0) == 0
        assert hidden() == 1 and split(False, 6144) == 1
        assert L.nsb_set_time_split(17, 0) == 1 and L.nsb_set_time_split(2, -1) == 1  # invalid arguments
    finally:
        assert L.nsb_set_time_split(0, 0) == 0
    # rotation of a modulated forward among the warps of a CTA: about five warps per scheduler, at most four
    # per column group, none beyond 1.5 column warps per scheduler, every warp of a group with a few tiles
    rot = lambda cols, T=8192: L.nsb_scan_rotation_query(T, cols, 8)
    assert [rot(c) for c in (6144, 12288, 24576, 28416, 28448, 49152)] == [4, 4, 4, 3, 1, 1]
    assert rot(6144, T=64) == 2 and rot(6144, T=24) == 1 and rot(0) == 0
    try:
        assert L.nsb_set_scan_rotation(1) == 0 and rot(6144) == 1
        assert L.nsb_set_scan_rotation(3) == 0 and rot(49152) == 3  # (as asked, whether or not it pays)
    finally:
        assert L.nsb_set_scan_rotation(0) == 0
