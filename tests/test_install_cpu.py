"""install()/uninstall() rebind the reference's modules, including names that
callers imported with ``from .parallel_scan import ...`` (CPU test on a
stand-in package with the reference's module layout)."""
import sys
import types

import pytest


@pytest.fixture
def fake_reference():
    pkg = types.ModuleType("fake_atomic_ops")
    pkg.__path__ = []
    ps = types.ModuleType("fake_atomic_ops.parallel_scan")
    for n in ("plif_parallel_forward", "plif_rowparam_forward_recompute", "plif_fixed_param_forward",
              "linear_recurrence", "hillis_steele_scan"):
        setattr(ps, n, (lambda name: (lambda *a, **k: name))(n))
    ps._TritonPLIFForward = type("_TritonPLIFForward", (), {})
    codec = types.ModuleType("fake_atomic_ops.fp16_codec")
    codec.fp16_encode = lambda *a: "ref-encode"
    codec.binary_residual = lambda *a: "ref-residual"
    ffn = types.ModuleType("fake_atomic_ops.snn_ffn")  # from .parallel_scan import ...
    ffn.plif_rowparam_forward_recompute = ps.plif_rowparam_forward_recompute
    ffn.binary_residual = codec.binary_residual
    ffn.unrelated = 7
    mods = {m.__name__: m for m in (pkg, ps, codec, ffn)}
    sys.modules.update(mods)
    yield ps, codec, ffn
    for n in mods:
        sys.modules.pop(n, None)


def test_install_patches_definitions_and_by_name_imports(fake_reference):
    from neuronspark_b200 import fp16_codec, install as inst, parallel_scan
    ps, codec, ffn = fake_reference
    rf = ps.hillis_steele_scan
    changed = inst.install("fake_atomic_ops")
    assert ps.plif_rowparam_forward_recompute is parallel_scan.plif_rowparam_forward_recompute
    assert ps._TritonPLIFForward is parallel_scan._TritonPLIFForward
    assert codec.fp16_encode is fp16_codec.fp16_encode
    # the layer module's own binding follows
    assert ffn.plif_rowparam_forward_recompute is parallel_scan.plif_rowparam_forward_recompute
    assert ffn.binary_residual is fp16_codec.binary_residual
    assert "fake_atomic_ops.snn_ffn.binary_residual" in changed
    # the linear recurrence is rebound too; what this package has no kernel for stays the reference's
    assert ps.linear_recurrence is parallel_scan.linear_recurrence
    assert ps.hillis_steele_scan is rf and ffn.unrelated == 7
    assert inst.uninstall() == len(changed)
    assert ps.plif_rowparam_forward_recompute() == "plif_rowparam_forward_recompute"
    assert ffn.binary_residual() == "ref-residual"


def test_install_requires_the_reference():
    from neuronspark_b200 import install as inst
    with pytest.raises(RuntimeError):
        inst.install("package_that_is_not_imported")
