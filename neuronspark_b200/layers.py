"""Fused forwards for NeuronSpark's ``SNNBlock`` and ``SNNFFN`` (opt-in; ``install(fused_layers=True)``).

``install()`` alone swaps kernels under the reference's layers and leaves their call sequence as
it is. Three fusions need that sequence to change, because they remove a tensor the layer
materialises between two calls:

  * ``SNNBlock.forward_parallel`` (atomic_ops/snn_block.py:203-285) turns five raw projections into
    beta / u / v_th / omega with an elementwise kernel (:237-241) and then scans them (:252-256).
    ``modulated_rf_plif_forward`` streams the raw projections once and never writes the four
    modulated tensors - the largest of the layer (and, in training, never their gradients).
  * Both layers end with the output neuron's scan followed by ``binary_residual`` (snn_block.py:281-285,
    snn_ffn.py:188-195). ``plif_rowparam_residual_forward`` does both in one kernel; the neuron's
    spikes are never written.
  * Before every scan the layers take ``float(neuron.get_surrogate(u).alpha)`` (snn_block.py:252-256,
    278-279; snn_ffn.py:161, 186), i.e. ``u.std().item()``: the host waits for the GPU once per scan.
    ``adaptive_alpha`` leaves the slope in device memory, where the backward reads it.

The functions below are drop-in bodies for the two ``forward_parallel`` methods: they read the
module's own parameters, buffers and helpers (the projections stay the reference's ``F.linear``
calls on its own weights, the gate / skip arithmetic stays its own ``_fused_gate_skip_scale``) and
update the neurons' carried state exactly as the reference does. Differences in results, all from
the first fusion: the modulated values are not rounded to the activation dtype between modulation
and scan, and their transcendental functions are the hardware approximations (1e-6 relative),
so a hidden spike can differ where a membrane potential comes within ~1e-6 of its threshold.
"""
from __future__ import annotations

import sys

import torch
import torch.nn.functional as F

from . import parallel_scan as ps
from . import snn_block as sb


def _state(neuron, name, init_name, batch, like):
    """A neuron's carried state, or its learnable initial state expanded to the batch when the
    state is still the float that ``reset_net`` leaves (atomic_ops/plif_node.py:103-115,
    selective_plif.py:68-74)."""
    v = getattr(neuron, name)
    if isinstance(v, float):
        expand = getattr(neuron, f"expand_{init_name}")
        v = expand(batch, like.device, like.dtype)
    return v


def _slope(neuron, u):
    """The surrogate slope the reference would pass (atomic_ops/plif_node.py:78-101), kept on the
    device when it is the adaptive one."""
    alpha0 = float(neuron.surrogate_function.alpha)
    if not getattr(neuron, "adaptive_surrogate", True) or not torch.is_grad_enabled():
        return alpha0  # (without autograd the slope is never used)
    return ps.adaptive_alpha(u, alpha0, float(getattr(neuron, "sigma_0", 1.0)))


def snn_block_forward_parallel(self, spike_in_seq: torch.Tensor) -> torch.Tensor:
    """Body for ``SNNBlock.forward_parallel`` (atomic_ops/snn_block.py:203-285)."""
    TK, batch, D = spike_in_seq.shape
    DN = self.D * self.N
    flat = spike_in_seq.reshape(TK * batch, D)
    x = flat.detach()  # the processing path takes no gradient to its input (:218-223)
    proj = lambda lin, width: F.linear(x, lin.weight).reshape(TK, batch, width)
    I_all, raw_beta, raw_alpha = proj(self.W_in, DN), proj(self.W_beta_x, DN), proj(self.W_alpha_x, DN)
    raw_th, raw_omega = proj(self.W_th_x, DN), proj(self.W_omega_x, DN)
    gate_all = torch.sigmoid(proj(self.W_gate, D))
    I_skip_all = proj(self.W_skip, D)

    hidden = self.hidden_neuron
    v_init = _state(hidden, "v", "v_init", batch, flat)
    w_init = _state(hidden, "w", "w_init", batch, flat)
    s_hidden, v_last, w_last = sb.modulated_rf_plif_forward(
        raw_beta, self.b_beta, raw_alpha, self.b_alpha, raw_th, self.b_th, self.v_th_min, I_all, raw_omega,
        self.b_omega, v_init, w_init, surrogate_function=hidden.surrogate_function,
        adaptive_sigma0=1.0 if torch.is_grad_enabled() else None)  # SelectivePLIFNode: sigma_0 = 1 (:80-85)
    hidden.v, hidden.w = v_last.detach(), w_last.detach()

    out_n = self.output_neuron
    I_out_all = F.linear(s_hidden.reshape(TK * batch, DN), self.W_out.weight).reshape(TK, batch, D)
    beta_out = out_n.beta
    gate_skip_scale = sys.modules[type(self).__module__]._fused_gate_skip_scale  # the layer's own helper (:40-46)
    u_output = gate_skip_scale(I_out_all, gate_all, I_skip_all, 1.0 - beta_out)
    v_init_out = _state(out_n, "v", "v_init", batch, flat)
    out, v_last_out = ps.plif_rowparam_residual_forward(
        beta_out.unsqueeze(0).expand(batch, D), u_output, out_n.v_th.unsqueeze(0).expand(batch, D), v_init_out,
        spike_in_seq, _slope(out_n, u_output))
    out_n.v = v_last_out.detach()
    return out


def snn_ffn_forward_parallel(self, spike_in_seq: torch.Tensor) -> torch.Tensor:
    """Body for ``SNNFFN.forward_parallel`` (atomic_ops/snn_ffn.py:108-195)."""
    TK, batch, D = spike_in_seq.shape
    D_ff = self.D_ff
    flat = spike_in_seq.reshape(TK * batch, D)
    x = flat.detach()
    I_gate = F.linear(x, self.gate_proj.weight).reshape(TK, batch, D_ff)
    I_up = F.linear(x, self.up_proj.weight).reshape(TK, batch, D_ff)
    I_skip = F.linear(x, self.skip_proj.weight).reshape(TK, batch, D)

    gate_n, up_n, out_n = self.gate_neuron, self.up_neuron, self.output_neuron
    beta_gu = torch.cat([gate_n.beta, up_n.beta])
    u_merged = torch.cat([I_gate, I_up], dim=-1) * (1.0 - beta_gu)
    vth_gu = torch.cat([gate_n.v_th, up_n.v_th])
    v_init_gu = torch.cat([_state(gate_n, "v", "v_init", batch, flat), _state(up_n, "v", "v_init", batch, flat)], dim=-1)
    spike_gu, v_last_gu = ps.plif_rowparam_forward_recompute(
        beta_gu.unsqueeze(0).expand(batch, 2 * D_ff), u_merged, vth_gu.unsqueeze(0).expand(batch, 2 * D_ff),
        v_init_gu, _slope(gate_n, u_merged))
    gate_n.v, up_n.v = v_last_gu[:, :D_ff].detach(), v_last_gu[:, D_ff:].detach()

    gated = spike_gu[:, :, :D_ff] * spike_gu[:, :, D_ff:]  # coincidence gate (:176)
    I_out = F.linear(gated.reshape(TK * batch, D_ff), self.down_proj.weight).reshape(TK, batch, D) + I_skip
    beta_out = out_n.beta
    u_out = (1.0 - beta_out) * I_out
    rows = lambda t: t.unsqueeze(0).expand(batch, D)
    v_init_out = _state(out_n, "v", "v_init", batch, flat)
    if self.add_residual:
        out, v_last_out = ps.plif_rowparam_residual_forward(rows(beta_out), u_out, rows(out_n.v_th), v_init_out,
                                                            spike_in_seq, _slope(out_n, u_out))
    else:  # the shared expert of the MoE layer: its caller adds the residual (:193-195)
        out, v_last_out = ps.plif_rowparam_forward_recompute(rows(beta_out), u_out, rows(out_n.v_th), v_init_out,
                                                             _slope(out_n, u_out))
    out_n.v = v_last_out.detach()
    return out
