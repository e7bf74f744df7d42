"""Stage the reference's own Python files beside the oracle, untouched, for tests and benches.

    python oracle/make_ref.py <path to the NeuronSpark checkout>     (or NEURONSPARK_REF=<path>)

Test infrastructure, like everything under ``oracle/``: nothing in the
``neuronspark_b200`` package imports from here.

NeuronSpark is pure Python (PyTorch + Triton): there is nothing to compile. What
this recipe does is copy the files that make up the layers around the scan
(``atomic_ops/*.py`` and ``model.py``) byte for byte into ``oracle/_ref/``, which
is ignored by git — the reference's sources never enter this repository's
history — and write ``oracle/_ref/MANIFEST.json`` with a sha256 per file. The
copy exists so that

  * the harness in ``tests/ref_harness.py`` can build the reference's real
    ``SNNBlock`` / ``SNNFFN`` / ``SNNDecoderLayer`` / ``SNNLanguageModel`` and let
    them call this library through ``neuronspark_b200.install``;
  * a bench can time the reference's own Triton kernels on the same GPU;
  * the reference's own test scripts for this path (``test_recompute.py``,
    ``test_binary_residual.py``, ``exp/verify_fused_plif.py``, ``exp/verify_triton_scan.py``) can be run as they are
    against this library;

on machines where the checkout itself is not mounted. Nothing is patched: the
harness supplies a stand-in for the one third-party package the reference
needs and this environment lacks (SpikingJelly) through ``sys.modules``.
"""
from __future__ import annotations

import hashlib
import json
import os
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
DEST = HERE / "_ref"

#: files of the checkout that the harness imports, relative to its root, and the reference's own
#: test scripts for this path (run, unchanged, on this library by tests/test_reference_own_tests_gpu.py)
WANTED = ("model.py", "atomic_ops/*.py", "test_recompute.py", "test_binary_residual.py",
          "exp/verify_fused_plif.py", "exp/verify_triton_scan.py")


def stage(checkout: Path, dest: Path = DEST) -> dict:
    checkout = Path(checkout)
    if not (checkout / "atomic_ops" / "parallel_scan.py").exists():
        raise SystemExit(f"{checkout} does not look like a NeuronSpark checkout")
    if dest.exists():
        shutil.rmtree(dest)
    manifest = {}
    for pattern in WANTED:
        for src in sorted(checkout.glob(pattern)):
            rel = src.relative_to(checkout)
            out = dest / rel
            out.parent.mkdir(parents=True, exist_ok=True)
            data = src.read_bytes()
            out.write_bytes(data)
            manifest[str(rel)] = hashlib.sha256(data).hexdigest()
    (dest / "MANIFEST.json").write_text(json.dumps(manifest, indent=1, sort_keys=True) + "\n")
    return manifest


def available(dest: Path = DEST) -> bool:
    return (dest / "MANIFEST.json").exists() and (dest / "atomic_ops" / "parallel_scan.py").exists()


if __name__ == "__main__":
    if len(sys.argv) < 2 and "NEURONSPARK_REF" not in os.environ:
        raise SystemExit(__doc__)
    m = stage(Path(sys.argv[1] if len(sys.argv) > 1 else os.environ["NEURONSPARK_REF"]))
    print(f"staged {len(m)} files under {DEST}")
