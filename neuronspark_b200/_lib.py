"""ctypes binding of ``libneuronspark_b200.so`` (the C ABI in
``include/neuronspark_b200.h``).

There is no CPU or PyTorch fallback: if the shared library is missing, or a
tensor is not on a CUDA device, the call raises.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_int32, c_int64, c_uint32, c_void_p
from pathlib import Path

import torch

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "libneuronspark_b200.so"

NSB_OK = 0
F32, BF16, F16 = 0, 1, 2
SURR_SIGMOID, SURR_ATAN = 0, 1
RESIDUAL_EAGER, RESIDUAL_COMPILED = 0, 1

_DTYPES = {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16}

_lib = None

_SIGNATURES = {
    "nsb_version": (c_int, []),
    "nsb_status_string": (ctypes.c_char_p, [c_int]),
    "nsb_last_cuda_error": (ctypes.c_char_p, []),
    "nsb_device_error_word": (c_int, [ctypes.POINTER(c_uint32)]),
    "nsb_set_wait_limit_ns": (c_int, [ctypes.c_uint64]),
    "nsb_selftest_wait_timeout": (c_int, [c_void_p]),
    "nsb_set_tuning": (c_int, [c_int, c_int, c_int, c_int]),
    "nsb_last_launch_info": (c_int, [ctypes.POINTER(c_int32)]),
    "nsb_scan_plan_query": (c_int, [c_int, c_int, c_int, c_int64, c_int64, c_int,
                                    ctypes.POINTER(c_int32)]),
    "nsb_time_plan_query": (c_int, [c_int, c_int, c_int64, c_int64, c_int, c_int, c_int, ctypes.POINTER(c_int32)]),
    "nsb_plif_selective_fwd": (c_int, [c_void_p] * 10 + [c_int64, c_int64, c_int, c_int, c_void_p, c_void_p]),
    "nsb_plif_selective_bwd": (c_int, [c_void_p] * 12 + [c_int64, c_int64, c_int, c_int, c_int,
                                                          c_float, c_void_p, c_void_p]),
    "nsb_chain_scratch_words": (c_int64, [c_int64]),
    "nsb_set_chain_chunks": (c_int, [c_int]),
    "nsb_last_chain_chunks": (c_int, []),
    "nsb_set_scan_rotation": (c_int, [c_int]),
    "nsb_last_scan_rotation": (c_int, []),
    "nsb_scan_rotation_query": (c_int, [c_int64, c_int64, c_int]),
    "nsb_plif_rowparam_fwd": (c_int, [c_void_p] * 9 + [c_int64, c_int64, c_int, c_int, c_void_p, c_void_p]),
    "nsb_convert": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p]),
    "nsb_set_time_split": (c_int, [c_int, c_int]),
    "nsb_time_split_scratch_floats": (c_int64, [c_int64]),
    "nsb_last_time_split": (c_int, [ctypes.POINTER(c_int32)]),
    "nsb_plif_rowparam_bwd": (c_int, [c_void_p] * 10 + [c_int64, c_int64, c_int, c_int, c_int,
                                                         c_float, c_void_p, c_void_p]),
    "nsb_plif_rf_fwd": (c_int, [c_void_p] * 14 + [c_int64, c_int64, c_int, c_int, c_void_p, c_void_p]),
    "nsb_plif_rf_bwd": (c_int, [c_void_p] * 14 + [c_int64, c_int64, c_int, c_int, c_int, c_float,
                                                   c_void_p, c_void_p]),
    "nsb_plif_modulated_fwd_stats_doubles": (c_int64, [c_int64]),
    "nsb_plif_modulated_fwd": (c_int, [c_void_p] * 9 + [c_float, c_int64] + [c_void_p] * 8 +
                               [c_float, c_float, c_void_p, c_void_p, c_int64, c_int64, c_int, c_int, c_void_p, c_void_p]),
    "nsb_plif_modulated_bwd_scratch_floats": (c_int64, [c_int64]),
    "nsb_plif_modulated_bwd": (c_int, [c_void_p] * 9 + [c_float, c_int64] + [c_void_p] * 15 +
                               [c_int64, c_int64, c_int, c_int, c_int, c_float, c_void_p, c_void_p]),
    "nsb_surrogate_alpha_scratch_doubles": (c_int64, []),
    "nsb_surrogate_alpha": (c_int, [c_void_p, c_int64, c_int, c_float, c_float, c_void_p, c_void_p, c_void_p]),
    "nsb_plif_rowparam_bwd_dalpha": (c_int, [c_void_p] * 10 + [c_int64, c_int64, c_int, c_int, c_int,
                                                                c_void_p, c_void_p, c_void_p]),
    "nsb_plif_rf_bwd_dalpha": (c_int, [c_void_p] * 14 + [c_int64, c_int64, c_int, c_int, c_int, c_void_p,
                                                          c_void_p, c_void_p]),
    "nsb_plif_rowparam_residual_fwd": (c_int, [c_void_p] * 8 + [c_int64, c_int64, c_int, c_int, c_int, c_void_p,
                                                                c_void_p]),
    "nsb_frames_pack": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_void_p]),
    "nsb_frames_unpack": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_void_p]),
    "nsb_fp16_decode_packed_fwd": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_void_p]),
    "nsb_fp16_decode_packed_bwd": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int,
                                           c_void_p]),
    "nsb_binary_residual_packed": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p]),
    "nsb_plif_rowparam_pattern_fwd": (c_int, [c_void_p] * 8 + [c_int64, c_int64, c_int, c_int, c_int, c_int,
                                                               c_void_p, c_void_p]),
    "nsb_linear_recurrence_fwd": (c_int, [c_void_p] * 6 + [c_int64, c_int64, c_int, c_int, c_void_p]),
    "nsb_linear_recurrence_bwd": (c_int, [c_void_p] * 7 + [c_int64, c_int64, c_int, c_int, c_void_p, c_void_p]),
    "nsb_moe_combine_fwd": (c_int, [c_void_p] * 4 + [c_int64, c_int64, c_int, c_int, c_void_p]),
    "nsb_moe_combine_bwd": (c_int, [c_void_p] * 5 + [c_int64, c_int64, c_int, c_int, c_void_p]),
    "nsb_frames_combine_fwd": (c_int, [c_void_p] * 5 + [c_int64] * 3 + [c_int, c_int, c_void_p]),
    "nsb_frames_combine_bwd": (c_int, [c_void_p] * 9 + [c_int64] * 3 + [c_int, c_int, c_void_p]),
    "nsb_modulation_fwd": (c_int, [c_void_p] * 9 + [c_float, c_int64, c_int64] + [c_void_p] * 4 +
                           [c_int, c_int, c_void_p]),
    "nsb_fp16_encode": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_int, c_void_p]),
    "nsb_fp16_decode_fwd": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_void_p]),
    "nsb_fp16_decode_bwd": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int,
                                    c_void_p]),
    "nsb_binary_residual": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_int,
                                    c_void_p]),
    "nsb_encode_ste_bwd": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_void_p]),
    "nsb_lateral_inhibition_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_float,
                                           c_int, c_int, c_void_p]),
    "nsb_li_bwd_scratch_floats": (c_int64, [c_int64, c_int64]),
    "nsb_lateral_inhibition_bwd": (c_int, [c_void_p] * 6 + [c_int64, c_int64, c_float, c_int, c_int,
                                                            c_void_p]),
    "nsb_lateral_inhibition_bwd_static": (c_int, [c_void_p] * 5 + [c_int64, c_int64, c_float, c_int,
                                                                   c_int, c_void_p]),
}

EXPORTED_SYMBOLS = tuple(_SIGNATURES)


class NSBError(RuntimeError):
    """A C-ABI call returned a non-zero status."""


def lib() -> ctypes.CDLL:
    """Loads the shared library (once). Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise NSBError(
                f"{LIB_PATH} is missing: build it with `python -m neuronspark_b200.build` "
                "(there is no CPU or PyTorch fallback)")
        handle = ctypes.CDLL(str(LIB_PATH))
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(status: int, what: str) -> None:
    if status != NSB_OK:
        L = lib()
        msg = L.nsb_status_string(status).decode()
        if status == 3:
            msg += " — " + L.nsb_last_cuda_error().decode()
        if status == 4:
            msg += (" — an earlier kernel of this process gave up on a bounded wait; its outputs are "
                    "invalid. device_error_word() reads and clears the record")
        raise NSBError(f"{what}: {msg} (status {status})")


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DTYPES[dt]
    except KeyError:
        raise NSBError(f"unsupported dtype {dt}; expected float32, bfloat16 or float16") from None


def ptr(t) -> c_void_p:
    """Device pointer of a tensor (None -> NULL)."""
    if t is None:
        return c_void_p(0)
    return c_void_p(t.data_ptr())


def stream_ptr(device) -> c_void_p:
    return c_void_p(torch.cuda.current_stream(device).cuda_stream)


def require_cuda(*tensors) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise NSBError("neuronspark_b200 runs on CUDA tensors only (no CPU fallback)")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise NSBError(f"tensors on different devices: {dev} and {t.device}")
    if dev is None:
        raise NSBError("no tensor arguments")
    return dev


def set_tuning(warps_per_cta: int = 0, stages: int = 0, lanes_per_thread: int = 0,
               force_direct: int = 0) -> None:
    """Overrides the scan launch heuristics (0 = automatic). Process-global.

    ``force_direct``: 1 (or True) = no TMA; 2 / 3 = TMA with the ring refilled one
    tile late always / never."""
    check(lib().nsb_set_tuning(warps_per_cta, stages, lanes_per_thread, int(force_direct)),
          "nsb_set_tuning")


def last_launch_info() -> dict:
    out = (c_int32 * 8)()
    check(lib().nsb_last_launch_info(out), "nsb_last_launch_info")
    keys = ("used_tma", "warps_per_cta", "stages", "lanes_per_thread", "grid", "smem_bytes",
            "tile_steps", "launches")
    return dict(zip(keys, out))


def scan_plan(backward: bool, nstreams: int, elem_size: int, T: int, cols: int, tile: int = 8) -> dict:
    """Launch plan the scan kernels would choose on a B200 (host arithmetic only)."""
    out = (c_int32 * 5)()
    check(lib().nsb_scan_plan_query(int(backward), nstreams, elem_size, T, cols, tile, out),
          "nsb_scan_plan_query")
    return dict(zip(("lanes_per_thread", "warps_per_cta", "stages", "grid", "smem_bytes"), out))


def time_plan(backward: bool, T: int, cols: int, tile: int = 32, lanes: int = 1, warps_per_cta: int = 1,
              modulated: bool = False) -> dict:
    """How the library would divide the time axis of such a scan on a B200 (host arithmetic only): the time
    split of a row-parameter scan and the chained chunks of a backward launch."""
    out = (c_int32 * 4)()
    check(lib().nsb_time_plan_query(int(backward), int(modulated), T, cols, tile, lanes, warps_per_cta, out),
          "nsb_time_plan_query")
    return dict(zip(("segments", "seg_tiles", "warm_tiles", "chain_chunks"), out))


def convert(t: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """``t`` as a contiguous tensor of ``dtype`` (fp32 / bf16 / fp16), converted by the library's own
    kernel: no framework elementwise op on the path. Detached; a tensor that already has the type is
    returned as it is (made contiguous)."""
    t = t.detach()
    if t.dtype == dtype:
        return t.contiguous()
    if t.dtype not in _DTYPES or not t.is_cuda:
        return t.to(dtype).contiguous()  # integer / double / CPU inputs: not a stream the kernels take anyway
    src = t.contiguous()
    out = torch.empty(src.shape, dtype=dtype, device=src.device)
    with torch.cuda.device(src.device):
        check(lib().nsb_convert(ptr(src), ptr(out), src.numel(), dtype_code(src.dtype), dtype_code(dtype),
                                stream_ptr(src.device)), "nsb_convert")
    return out


def set_time_split(max_segments: int = 0, warm_steps: int = 0) -> None:
    """Time split of the row-parameter forward scans over few columns: ``max_segments`` 0 = automatic,
    1 = off, 2..16 = at most that many; ``warm_steps`` 0 = default (1024). Process-global."""
    check(lib().nsb_set_time_split(int(max_segments), int(warm_steps)), "nsb_set_time_split")


def last_time_split() -> dict:
    out = (c_int32 * 3)()
    check(lib().nsb_last_time_split(out), "nsb_last_time_split")
    return dict(zip(("segments", "seg_tiles", "warm_tiles"), out))


def set_chain_chunks(chunks: int = 0) -> None:
    """Chained chunks of backward scans over more columns than the GPU holds at once: 0 = automatic,
    1 = never, n = n chunks. Process-global."""
    check(lib().nsb_set_chain_chunks(int(chunks)), "nsb_set_chain_chunks")


def last_chain_chunks() -> int:
    return int(lib().nsb_last_chain_chunks())


_scan_rotation = 0


def set_scan_rotation(warps: int = 0) -> None:
    """Warps that take the tiles of a column group in turn in a modulated forward scan over few columns:
    0 = automatic, 1 = never, 2..4. Process-global."""
    global _scan_rotation
    check(lib().nsb_set_scan_rotation(int(warps)), "nsb_set_scan_rotation")
    _scan_rotation = int(warps)


def scan_rotation_setting() -> int:
    """What was last set through set_scan_rotation (the Python layer picks its tile length by it)."""
    return _scan_rotation


def last_scan_rotation() -> int:
    return int(lib().nsb_last_scan_rotation())


def set_wait_limit_ns(ns: int = 0) -> None:
    """Limit of the kernels' bounded waits in nanoseconds (0 = the default, 2 s). Process-global."""
    check(lib().nsb_set_wait_limit_ns(int(ns)), "nsb_set_wait_limit_ns")


def device_error_word() -> int:
    w = c_uint32(0)
    check(lib().nsb_device_error_word(ctypes.byref(w)), "nsb_device_error_word")
    return int(w.value)
