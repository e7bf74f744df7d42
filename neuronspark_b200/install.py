"""Rebinds NeuronSpark's own modules to the B200 implementations.

The reference's layers import the scan functions by name at import time
(``from .parallel_scan import plif_rowparam_forward_recompute`` in
``atomic_ops/snn_block.py`` and ``atomic_ops/snn_ffn.py``; ``from
atomic_ops.fp16_codec import fp16_encode, fp16_decode`` in ``model.py``), so
replacing the attributes of ``atomic_ops.parallel_scan`` alone is not enough:
every already-imported module that holds one of those names has to be patched
too. ``install()`` does both and returns what it changed; ``uninstall()`` puts
the originals back.

    import atomic_ops, model            # the reference, unmodified
    import neuronspark_b200.install as nsb_install
    nsb_install.install()               # snn_block / snn_ffn / model now call the CUDA kernels

Functions of the reference that this package does not replace (e.g.
``hillis_steele_scan``) are left untouched.
"""
from __future__ import annotations

import sys
from types import ModuleType

from . import fp16_codec, lateral_inhibition, moe_kernels, parallel_scan

#: reference module (by its name inside the ``atomic_ops`` package) -> replacement names
REPLACEMENTS = {
    "parallel_scan": (parallel_scan, (
        "_TritonPLIFForward", "_TritonPLIFRowParamForward", "_TritonPLIFRowParamRecompute",
        "plif_parallel_forward", "plif_rowparam_forward", "plif_rowparam_forward_alpha",
        "plif_rowparam_forward_recompute", "plif_fixed_param_forward",
        "_TritonRFPLIFForward", "_TritonRFPLIFRecompute", "rf_plif_parallel_forward",
        "rf_plif_parallel_forward_recompute", "_TritonLinearRecurrence", "linear_recurrence")),
    "fp16_codec": (fp16_codec, (
        "fp16_encode", "fp16_decode", "binary_residual", "binary_encode_ste", "_BinaryResidual",
        "_BinaryEncodeSTE")),
    "lateral_inhibition": (lateral_inhibition, ("_LateralInhibitionTriton",)),
    "moe_kernels": (moe_kernels, ("MoECombine", "moe_combine")),
}

#: modules of the reference whose ``forward`` takes its kernel branch only when its module-level
#: ``_HAS_TRITON`` is true (atomic_ops/lateral_inhibition.py:206, atomic_ops/rms_norm.py:40). Without
#: Triton the reference does not even define ``_LateralInhibitionTriton`` (:122, under ``if
#: _HAS_TRITON``), so both names are set there regardless of what the import found.
_GATED = {"lateral_inhibition": ("_LateralInhibitionTriton",), "rms_norm": ("_LateralInhibitionTriton",)}

_ABSENT = object()
_undo: list[tuple[ModuleType, str, object]] = []


def _reference_modules(package: str) -> dict[str, ModuleType]:
    found = {}
    for short in REPLACEMENTS:
        m = sys.modules.get(f"{package}.{short}")
        if m is not None:
            found[short] = m
    return found


def install(package: str = "atomic_ops", extra_modules=(), fused_layers: bool = False) -> list[str]:
    """Patches the imported reference modules; returns ``module.name`` strings changed.

    ``package`` is the import name of the reference's operator package.
    ``extra_modules`` are further already-imported modules to scan for
    by-name imports (``model`` is scanned automatically when present).
    ``fused_layers``: also replace ``SNNBlock.forward_parallel`` and ``SNNFFN.forward_parallel`` by
    the bodies of ``neuronspark_b200.layers``, which call the fused kernels (modulation inside the
    resonate-and-fire scan, output scan + residual in one kernel, surrogate slope kept on the
    device). Off by default: it changes the layers' call sequence, not just the kernels under it."""
    refs = _reference_modules(package)
    if not refs:
        raise RuntimeError(f"no module of the reference package {package!r} has been imported")
    originals: dict[int, tuple[str, object]] = {}
    changed: list[str] = []
    for short, ref_mod in refs.items():
        ours, names = REPLACEMENTS[short]
        for name in names:
            if hasattr(ref_mod, name):
                old = getattr(ref_mod, name)
                originals[id(old)] = (name, getattr(ours, name))
                _undo.append((ref_mod, name, old))
                setattr(ref_mod, name, getattr(ours, name))
                changed.append(f"{ref_mod.__name__}.{name}")
    for short, names in _GATED.items():
        mod = sys.modules.get(f"{package}.{short}")
        if mod is None:
            continue
        for name, new in [("_HAS_TRITON", True)] + [(n, getattr(lateral_inhibition, n)) for n in names]:
            old = getattr(mod, name, _ABSENT)
            if old is not new:
                _undo.append((mod, name, old))
                setattr(mod, name, new)
                if name != "_HAS_TRITON" or old is not True:
                    changed.append(f"{mod.__name__}.{name}")
    # modules that did `from .parallel_scan import name` hold their own reference
    scan = [m for n, m in list(sys.modules.items())
            if m is not None and (n == package or n.startswith(package + ".") or n == "model")]
    scan += list(extra_modules)
    for mod in scan:
        if mod in refs.values():
            continue
        for attr, val in list(vars(mod).items()):
            hit = originals.get(id(val))
            if hit is not None and hit[0] == attr:
                _undo.append((mod, attr, val))
                setattr(mod, attr, hit[1])
                changed.append(f"{mod.__name__}.{attr}")
    if fused_layers:
        from . import layers
        for short, cls_name, body in (("snn_block", "SNNBlock", layers.snn_block_forward_parallel),
                                      ("snn_ffn", "SNNFFN", layers.snn_ffn_forward_parallel)):
            mod = sys.modules.get(f"{package}.{short}")
            cls = getattr(mod, cls_name, None) if mod is not None else None
            if cls is not None:
                _undo.append((cls, "forward_parallel", cls.__dict__["forward_parallel"]))
                cls.forward_parallel = body
                changed.append(f"{mod.__name__}.{cls_name}.forward_parallel")
    return changed


def uninstall() -> int:
    """Restores everything ``install()`` changed; returns the number of names restored."""
    n = 0
    while _undo:
        mod, name, old = _undo.pop()
        if old is _ABSENT:
            delattr(mod, name)
        else:
            setattr(mod, name, old)
        n += 1
    return n
