"""The reference's own modules (staged by ``oracle/make_ref.py``) import through the
SpikingJelly stand-in, run on CPU through their own fallbacks, and are rebound by
``install()`` — the real ``atomic_ops`` / ``model`` modules, not look-alikes."""
import pytest
import torch

from oracle import ref_harness as rh

pytestmark = pytest.mark.skipif(
    not rh.available(), reason="oracle/_ref is empty: python oracle/make_ref.py <NeuronSpark checkout>")


@pytest.fixture
def reference():
    ao, model = rh.load_reference(eager_elementwise=True)
    yield ao, model
    from neuronspark_b200 import install as inst
    inst.uninstall()


def tiny_model(model):
    """The model of the reference's exp/test_e2e.py:16-18 (vocab 256, D 64, N 4, 2 layers, D_ff 128)
    with K = 16: HEAD's fp16_encode has 16 frames per token built in (atomic_ops/fp16_codec.py:39-40),
    so that script's K = 4 no longer runs against its own checkout."""
    torch.manual_seed(0)
    return model.SNNLanguageModel(vocab_size=256, D=64, N=4, K=16, num_layers=2, D_ff=128)


def test_memory_module_semantics():
    rh.install_spikingjelly_shim()
    from spikingjelly.activation_based import base, functional, neuron, surrogate

    class Node(neuron.BaseNode):
        def single_step_forward(self, x):
            self.v_float_to_tensor(x)
            self.v = self.v + x
            return self.surrogate_function(self.v - self.v_threshold)

    n = Node(v_threshold=1.0, v_reset=None, surrogate_function=surrogate.Sigmoid(alpha=4.0))
    assert n.v == 0.0 and "v" not in dict(n.named_parameters()) and "v" not in dict(n.named_buffers())
    x = torch.full((2, 3), 0.6, requires_grad=True)
    assert n(x).sum() == 0 and isinstance(n.v, torch.Tensor)
    s = n(x)
    assert s.sum() == 6
    s.sum().backward()
    sg = 4.0 * torch.sigmoid(torch.tensor(0.8)) * (1 - torch.sigmoid(torch.tensor(0.8)))
    assert torch.allclose(x.grad, 2 * sg.expand(2, 3), atol=1e-6)  # v = x + x at the second step
    holder = torch.nn.Sequential(n)
    functional.reset_net(holder)
    assert n.v == 0.0
    assert isinstance(n, base.MemoryModule)


def test_reference_model_runs_on_cpu_with_the_shim(reference):
    _, model = reference
    m = tiny_model(model)
    x = torch.randint(0, 256, (2, 8))
    y = torch.randint(1, 256, (2, 8))
    loss = m(x, y).last_loss.mean()
    assert torch.isfinite(loss)
    loss.backward()
    missing = [n for n, p in m.named_parameters() if p.grad is None or not p.grad.abs().sum() > 0]
    assert not missing, missing  # the acceptance of exp/test_e2e.py:33-41


def test_install_rebinds_the_real_reference(reference):
    ao, model = reference
    from neuronspark_b200 import fp16_codec, install as inst, lateral_inhibition, moe_kernels, parallel_scan
    ref_recompute = ao.snn_block.plif_rowparam_forward_recompute
    changed = inst.install()
    # definitions ...
    assert ao.parallel_scan._TritonRFPLIFRecompute is parallel_scan._TritonRFPLIFRecompute
    assert ao.parallel_scan.linear_recurrence is parallel_scan.linear_recurrence
    assert ao.moe_kernels.moe_combine is moe_kernels.moe_combine
    assert ao.lateral_inhibition._LateralInhibitionTriton is lateral_inhibition._LateralInhibitionTriton
    # ... and every by-name import the layers made (snn_block.py:35-36, snn_ffn.py:29-30,
    # moe_snn_ffn.py:28-29, model.py:24, rms_norm.py:17, atomic_ops/__init__.py:9-10)
    assert ao.snn_block.rf_plif_parallel_forward_recompute is parallel_scan.rf_plif_parallel_forward_recompute
    assert ao.snn_block.plif_rowparam_forward_recompute is parallel_scan.plif_rowparam_forward_recompute
    assert ao.snn_block.binary_residual is fp16_codec.binary_residual
    assert ao.snn_ffn.plif_rowparam_forward_recompute is parallel_scan.plif_rowparam_forward_recompute
    assert ao.snn_ffn.binary_residual is fp16_codec.binary_residual
    assert ao.moe_snn_ffn.binary_encode_ste is fp16_codec.binary_encode_ste
    assert model.fp16_encode is fp16_codec.fp16_encode and model.fp16_decode is fp16_codec.fp16_decode
    assert ao.rms_norm._LateralInhibitionTriton is lateral_inhibition._LateralInhibitionTriton
    assert ao.plif_rowparam_forward_recompute is parallel_scan.plif_rowparam_forward_recompute
    # what this package has no replacement for stays the reference's
    assert ao.parallel_scan.hillis_steele_scan.__module__ == "atomic_ops.parallel_scan"
    assert inst.uninstall() == len(changed)
    assert ao.snn_block.plif_rowparam_forward_recompute is ref_recompute
    assert model.fp16_encode.__module__ == "atomic_ops.fp16_codec"


def test_fused_layers_are_patched_and_restored(reference):
    ao, _ = reference
    from neuronspark_b200 import install as inst, layers
    block_fwd, ffn_fwd = ao.snn_block.SNNBlock.forward_parallel, ao.snn_ffn.SNNFFN.forward_parallel
    changed = inst.install(fused_layers=True)
    assert ao.snn_block.SNNBlock.forward_parallel is layers.snn_block_forward_parallel
    assert ao.snn_ffn.SNNFFN.forward_parallel is layers.snn_ffn_forward_parallel
    assert inst.uninstall() == len(changed)
    assert ao.snn_block.SNNBlock.forward_parallel is block_fwd and ao.snn_ffn.SNNFFN.forward_parallel is ffn_fwd


def test_library_refuses_cpu_tensors_when_installed(reference):
    """No silent fallback: the reference's model on CPU tensors, once rebound, raises."""
    _, model = reference
    from neuronspark_b200 import NSBError, install as inst
    m = tiny_model(model)
    inst.install()
    with pytest.raises(NSBError):
        m(torch.randint(0, 256, (1, 2)))
