"""Loads the reference's own layers (staged by ``oracle/make_ref.py``) so that tests and
benches can run them, unmodified, on top of this library.

Test infrastructure: used by ``tests/`` and by ``bench.py``'s layer/model workloads; the
``neuronspark_b200`` package never imports it.

The reference's modules derive from SpikingJelly 0.0.0.0.14 (``requirements.txt:4``), which
is not installed here and not vendored by the reference. Only a sliver of its API is
touched by the files on this path:

  ``base.MemoryModule``      ``register_memory(name, value)`` / ``reset()``
                             (atomic_ops/plif_node.py:76, selective_plif.py:66,
                             snn_block.py:79, snn_ffn.py:33, snn_decoder_layer.py:20)
  ``neuron.BaseNode``        constructor fields, the ``v`` memory, ``v_float_to_tensor``,
                             single-step dispatch (atomic_ops/selective_plif.py:28-58, 118)
  ``layer.Linear``           ``nn.Linear`` carrying a ``step_mode`` (atomic_ops/snn_block.py:104-114)
  ``surrogate.Sigmoid``      heaviside forward, ``alpha*s*(1-s)`` backward, ``.alpha``
                             (atomic_ops/plif_node.py:45, 102; parallel_scan.py:1347-1349
                             dispatches on the class NAME ``Sigmoid``)
  ``functional.reset_net``   calls ``reset()`` on every sub-module that has one (model.py:32)

``install_spikingjelly_shim()`` registers a behavioural stand-in for exactly that under the
package's import names. It is a restatement written from the call sites above, not the
pinned package; a real SpikingJelly, when importable, is used instead.
"""
from __future__ import annotations

import copy
import importlib
import math
import sys
import types
from pathlib import Path

import torch
import torch.nn as nn

REF_DIR = Path(__file__).resolve().parent / "_ref"


# ------------------------------------------------------------------ SpikingJelly stand-in


class MemoryModule(nn.Module):
    """Module with named state ("memories") that ``reset()`` puts back to its registered value."""

    def __init__(self):
        super().__init__()
        self._memories_rv = {}

    def register_memory(self, name: str, value):
        self._memories_rv[name] = value
        object.__setattr__(self, name, copy.deepcopy(value))

    def reset(self):
        for name, value in self._memories_rv.items():
            object.__setattr__(self, name, copy.deepcopy(value))

    def __setattr__(self, name, value):
        rv = self.__dict__.get("_memories_rv")
        if rv is not None and name in rv:
            object.__setattr__(self, name, value)  # state, never a parameter/buffer/sub-module
        else:
            super().__setattr__(name, value)


class _SigmoidSurrogateFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, alpha):
        if x.requires_grad:
            ctx.save_for_backward(x)
            ctx.alpha = alpha
        return (x >= 0).to(x)

    @staticmethod
    def backward(ctx, g):
        (x,) = ctx.saved_tensors
        s = torch.sigmoid(ctx.alpha * x)
        return g * ctx.alpha * s * (1.0 - s), None


class Sigmoid(nn.Module):
    """Heaviside step whose gradient is that of ``sigmoid(alpha*x)``."""

    def __init__(self, alpha: float = 4.0, spiking: bool = True):
        super().__init__()
        self.alpha = alpha
        self.spiking = spiking

    def forward(self, x):
        if self.spiking:
            return _SigmoidSurrogateFn.apply(x, self.alpha)
        return torch.sigmoid(self.alpha * x)

    def extra_repr(self):
        return f"alpha={self.alpha}, spiking={self.spiking}"


class _ATanSurrogateFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, alpha):
        if x.requires_grad:
            ctx.save_for_backward(x)
            ctx.alpha = alpha
        return (x >= 0).to(x)

    @staticmethod
    def backward(ctx, g):
        (x,) = ctx.saved_tensors
        return g * (ctx.alpha / 2) / (1 + (math.pi / 2 * ctx.alpha * x) ** 2), None


class ATan(nn.Module):
    """Heaviside step whose gradient is that of ``atan(pi/2*alpha*x)/pi + 1/2``. The reference never
    names it; BASELINE's headline configuration does, and the reference's CPU scan accepts any
    surrogate callable (atomic_ops/parallel_scan.py:1667-1677)."""

    def __init__(self, alpha: float = 2.0, spiking: bool = True):
        super().__init__()
        self.alpha = alpha
        self.spiking = spiking

    def forward(self, x):
        return _ATanSurrogateFn.apply(x, self.alpha)


class BaseNode(MemoryModule):
    def __init__(self, v_threshold: float = 1.0, v_reset=0.0, surrogate_function=None,
                 detach_reset: bool = False, step_mode: str = "s", backend: str = "torch",
                 store_v_seq: bool = False):
        super().__init__()
        self.register_memory("v", 0.0 if v_reset is None else v_reset)
        self.v_threshold = v_threshold
        self.v_reset = v_reset
        self.detach_reset = detach_reset
        self.surrogate_function = surrogate_function if surrogate_function is not None else Sigmoid()
        self.step_mode = step_mode
        self.backend = backend
        self.store_v_seq = store_v_seq

    def v_float_to_tensor(self, x: torch.Tensor):
        if isinstance(self.v, float):
            self.v = torch.full_like(x.data, self.v)

    def forward(self, *args, **kwargs):
        if self.step_mode != "s":
            raise NotImplementedError("the stand-in implements single-step mode only")
        return self.single_step_forward(*args, **kwargs)


class Linear(nn.Linear):
    def __init__(self, in_features, out_features, bias=True, step_mode="s"):
        super().__init__(in_features, out_features, bias=bias)
        self.step_mode = step_mode


def reset_net(net: nn.Module):
    for m in net.modules():
        if hasattr(m, "reset"):
            m.reset()


def install_spikingjelly_shim(force: bool = False) -> bool:
    """Registers the stand-in as ``spikingjelly.activation_based``. Returns True if the stand-in
    is what ``import spikingjelly`` now gives, False if the real package was found and kept."""
    if not force:
        try:
            importlib.import_module("spikingjelly.activation_based")
            return getattr(sys.modules["spikingjelly"], "__nsb_shim__", False)
        except ImportError:
            pass
    top = types.ModuleType("spikingjelly")
    top.__nsb_shim__ = True
    top.__path__ = []
    ab = types.ModuleType("spikingjelly.activation_based")
    ab.__path__ = []
    subs = {}
    for name, members in (("base", {"MemoryModule": MemoryModule}),
                          ("neuron", {"BaseNode": BaseNode}),
                          ("layer", {"Linear": Linear}),
                          ("surrogate", {"Sigmoid": Sigmoid, "ATan": ATan}),
                          ("functional", {"reset_net": reset_net})):
        m = types.ModuleType(f"spikingjelly.activation_based.{name}")
        for k, v in members.items():
            setattr(m, k, v)
        setattr(ab, name, m)
        subs[m.__name__] = m
    top.activation_based = ab
    sys.modules.update({"spikingjelly": top, "spikingjelly.activation_based": ab, **subs})
    return True


# ------------------------------------------------------------------------ the reference


def available() -> bool:
    return (REF_DIR / "atomic_ops" / "parallel_scan.py").exists() and (REF_DIR / "model.py").exists()


def load_reference(eager_elementwise: bool = False):
    """Imports the staged reference: returns ``(atomic_ops, model)`` modules.

    ``eager_elementwise``: the reference decorates a few elementwise helpers with
    ``torch.compile`` (atomic_ops/snn_block.py:40, 52; fp16_codec.py:168). Where the inductor
    toolchain cannot run, ``True`` makes those decorators no-ops for the duration of the import,
    so the helpers run as the eager PyTorch they are written in. The files themselves are not
    touched either way."""
    if not available():
        raise RuntimeError(f"{REF_DIR} is empty: run `python oracle/make_ref.py <NeuronSpark checkout>`")
    install_spikingjelly_shim()
    if "atomic_ops" in sys.modules and "model" in sys.modules:
        return sys.modules["atomic_ops"], sys.modules["model"]
    if str(REF_DIR) not in sys.path:
        sys.path.insert(0, str(REF_DIR))
    real_compile = torch.compile
    if eager_elementwise:
        def passthrough(fn=None, **_kw):
            return fn if fn is not None else (lambda f: f)
        torch.compile = passthrough
    try:
        atomic_ops = importlib.import_module("atomic_ops")
        model = importlib.import_module("model")
    finally:
        torch.compile = real_compile
    return atomic_ops, model


def unload_reference():
    for name in [n for n in sys.modules if n == "model" or n == "atomic_ops" or n.startswith("atomic_ops.")]:
        del sys.modules[name]
