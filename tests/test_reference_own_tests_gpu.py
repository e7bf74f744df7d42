"""The reference's own test scripts for this path, run as they are on this library.

``oracle/make_ref.py`` stages NeuronSpark's ``test_recompute.py`` (recompute and materialising scans
equal to the bit, forward and backward, row-parameter and resonate-and-fire), ``test_binary_residual.py``
(codec round trips, straight-through gradients) and ``exp/verify_fused_plif.py`` (the fused scan against
a sequential PyTorch loop, its gradients against autograd through that loop, the real training shapes)
and ``exp/verify_triton_scan.py`` (the linear recurrence against the Hillis-Steele scan) beside the reference's modules. Here the modules are imported, ``install()`` rebinds their kernels to
this library, and each script is executed as ``__main__``. The scripts' own assertions and verdict lines
are the acceptance. The only lines not executed are two machine-specific ones at the top of
``verify_fused_plif.py`` (a ptxas path and a home directory of the authors' machine)."""
import contextlib
import io
import sys

import pytest
import torch

import neuronspark_b200 as nsb
from neuronspark_b200 import install as inst, parallel_scan as ps
from oracle import ref_harness as rh

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not rh.available(), reason="the reference's files are not staged (oracle/make_ref.py)")]


@pytest.fixture()
def reference_on_this_library():
    rh.unload_reference()
    atomic_ops, _ = rh.load_reference()
    inst.install()
    try:
        yield atomic_ops
    finally:
        inst.uninstall()
        rh.unload_reference()
        assert nsb.device_error_word() == 0


def run_script(name: str, default_device=None) -> str:
    path = rh.REF_DIR / name
    if not path.exists():
        pytest.skip(f"{name} is not staged: re-run oracle/make_ref.py")
    lines = path.read_text().splitlines(keepends=True)
    kept = ["\n" if ("TRITON_PTXAS_PATH" in l or "/home/dgxspark" in l) else l for l in lines]
    out = io.StringIO()
    place = torch.device(default_device) if default_device else contextlib.nullcontext()
    with contextlib.redirect_stdout(out), place:
        exec(compile("".join(kept), str(path), "exec"), {"__name__": "__main__", "__file__": str(path)})
    torch.cuda.synchronize()
    return out.getvalue()


def test_recompute_script(reference_on_this_library):
    scan = sys.modules["atomic_ops.parallel_scan"]
    assert scan.plif_rowparam_forward_recompute is ps.plif_rowparam_forward_recompute
    assert scan.rf_plif_parallel_forward_recompute is ps.rf_plif_parallel_forward_recompute
    text = run_script("test_recompute.py")
    assert "[PASS] PLIF rowparam recompute: 0-bit exact match (forward + backward)" in text, text
    assert "[PASS] RF PLIF recompute: 0-bit exact match (forward + backward)" in text, text
    assert "All tests passed!" in text, text


def test_binary_residual_script(reference_on_this_library):
    codec = sys.modules["atomic_ops.fp16_codec"]
    from neuronspark_b200 import fp16_codec as mine
    assert codec.binary_residual is mine.binary_residual and codec.fp16_decode is mine.fp16_decode
    # the script names no device (the reference's codec is eager PyTorch and runs where its tensors are):
    # here its tensors are created on the GPU, where this library runs
    text = run_script("test_binary_residual.py", default_device="cuda")
    assert "===== ALL TESTS PASSED =====" in text, text


def test_verify_fused_plif_script(reference_on_this_library):
    scan = sys.modules["atomic_ops.parallel_scan"]
    assert scan.plif_parallel_forward is ps.plif_parallel_forward
    text = run_script("exp/verify_fused_plif.py")
    assert "ALL TESTS PASSED" in text and "FAIL" not in text.replace("SOME TESTS FAILED", ""), text


def test_verify_triton_scan_script(reference_on_this_library):
    """The linear recurrence against the reference's Hillis-Steele scan (forward in fp32 and bf16, gradients),
    its no-grad path, and the PLIF forwards built on it, at the real training shapes."""
    scan = sys.modules["atomic_ops.parallel_scan"]
    assert scan.linear_recurrence is ps.linear_recurrence
    text = run_script("exp/verify_triton_scan.py")
    assert "ALL TESTS PASSED" in text and "FAIL" not in text.replace("SOME TESTS FAILED", ""), text
