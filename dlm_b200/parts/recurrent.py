"""Mixers that carry a state of fixed size per request instead of keys and values."""
from __future__ import annotations

import math

import torch

from ..registry import register_part
from .base import Mixer, ParamSpec, RequestState, Runtime, StepContext


class Mamba2Mixer(Mixer):
    """State-space mixer with a scalar decay per head.  ``inner = heads * vdim``; ``W_in h`` is laid out
    ``[z: inner | x: inner | B: groups * state | C: groups * state | dt: heads]``.  x, B and C together pass a
    causal convolution per channel (``conv_taps`` taps with bias, the last tap meets the current token) and silu.
    Per head n (group ``n // (heads / groups)``), with ``dt = softplus(dt + dt_bias)`` (no clamp)::

        S_t = exp(-exp(A_log_n) dt) S_(t-1) + dt B_t x_t^T          (S: state x vdim, 32-bit, zero at the start)
        y_t = S_t^T C_t + D_n x_t

    then ``y * silu(z)``, an RMS norm over ``norm_groups`` equal parts of the channels (the gate comes before the
    norm), times ``norm``, then ``W_o``.  A request's state: S of every head and the convolution's last
    ``conv_taps - 1`` inputs.  Everything between the two projections is 32-bit."""

    def __init__(self, hidden_size: int, heads: int, vdim: int, state: int, groups: int, conv_taps: int,
                 norm_groups: int, eps: float):
        self.hidden, self.H, self.P, self.N, self.G = int(hidden_size), int(heads), int(vdim), int(state), int(groups)
        self.taps, self.ng, self.eps = int(conv_taps), int(norm_groups), float(eps)
        self.inner = self.H * self.P
        self.C = self.inner + 2 * self.G * self.N          # channels that pass the convolution
        if self.H % self.G:
            raise ValueError("heads must be a multiple of groups")
        if self.inner % self.ng:
            raise ValueError("heads * vdim must be a multiple of norm_groups")
        if self.taps < 1:
            raise ValueError("the convolution has at least one tap")
        self.w_in = self.w_o = self.conv_w = self.conv_b = self.dt_bias = self.A_log = self.D = self.norm_w = None

    def param_specs(self):
        return [ParamSpec("in", (2 * self.inner + 2 * self.G * self.N + self.H, self.hidden)),
                ParamSpec("conv", (self.C, self.taps)), ParamSpec("conv.b", (self.C,), init="bias"),
                ParamSpec("dt_bias", (self.H,), init="bias"), ParamSpec("A_log", (self.H,), init="bias"),
                ParamSpec("D", (self.H,), init="norm"), ParamSpec("norm", (self.inner,), init="norm"),
                ParamSpec("o", (self.hidden, self.inner))]

    def load(self, tensors, rt: Runtime):
        self.w_in, self.w_o = rt.matrix(tensors["in"]), rt.matrix(tensors["o"])
        self.conv_w, self.conv_b = rt.vector(tensors["conv"]), rt.vector(tensors["conv.b"])
        self.dt_bias, self.A_log, self.D = (rt.vector(tensors[n]) for n in ("dt_bias", "A_log", "D"))
        self.norm_w = rt.vector(tensors["norm"])

    def state_need(self):
        need = {"ssm": RequestState((self.H, self.N, self.P))}
        if self.taps > 1:
            need["conv"] = RequestState((self.taps - 1, self.C))
        return need

    def forward(self, h, resid, ctx: StepContext, call: int):
        rt, ops, b = ctx.rt, ctx.rt.ops, ctx.batch
        proj = ops.linear(h, self.w_in, None, torch.float32)
        z = proj[:, :self.inner]
        dt = proj[:, self.inner + self.C:]
        conv_state = ctx.state(call, "conv") if self.taps > 1 else torch.empty((0, 0, self.C), device=h.device)
        xbc = ops.causal_conv(proj[:, self.inner:self.inner + self.C], self.conv_w, self.conv_b, conv_state, b,
                              False, True, torch.float32)
        y = ops.ssm_scan(xbc, dt, self.dt_bias, self.A_log, self.D, ctx.state(call, "ssm"), b, self.H, self.P, self.N,
                         self.G)
        g = ops.gated_rmsnorm(y, z, self.norm_w, self.ng, self.eps, "silu_before", rt.dtype)
        ops.linear_add(g, self.w_o, resid)


class GeneralDeltaMixer(Mixer):
    """Delta-rule recurrence with a decay and a removal rate per head and key channel.  ``r, k, v = W h`` (heads x
    dim each); decay ``w = exp(-decay_coef * sigmoid(W_w2 tanh(W_w1 h) + w0))``; removal rate
    ``a = sigmoid(W_a h + a.b)``; unit key ``u = k / sqrt(sum k^2 + unit_eps)`` per head::

        S_t = diag(w) S_(t-1) - (a * u)(u^T S_(t-1)) + k v^T       (S: dim x dim, 32-bit, zero at the start)
        o_t = S_t^T r

    Each head's o is divided by its root mean square, the heads side by side are multiplied by ``norm`` and by
    ``sigmoid(W_g h)``, then ``W_o``.  The width of the decay's bottleneck is whatever ``w1`` has."""

    def __init__(self, hidden_size: int, heads: int, dim: int, eps: float, decay_coef: float = math.exp(-0.5),
                 unit_eps: float = 1e-6, decay_rank: int = 16):
        self.hidden, self.H, self.d, self.eps = int(hidden_size), int(heads), int(dim), float(eps)
        self.decay_coef, self.unit_eps, self.decay_rank = float(decay_coef), float(unit_eps), int(decay_rank)
        self.HD = self.H * self.d
        self.w_in = self.w2 = self.w0 = self.a_b = self.norm_w = self.w_o = None

    def param_specs(self):
        HD, hid = self.HD, self.hidden
        # -1: the size is the checkpoint's (random weights take `arg`)
        return [ParamSpec("r", (HD, hid)), ParamSpec("k", (HD, hid)), ParamSpec("v", (HD, hid)),
                ParamSpec("a", (HD, hid)), ParamSpec("a.b", (HD,), init="bias"), ParamSpec("g", (HD, hid)),
                ParamSpec("w1", (-1, hid), arg=self.decay_rank), ParamSpec("w2", (HD, -1), arg=self.decay_rank),
                ParamSpec("w0", (HD,), init="bias"), ParamSpec("norm", (HD,), init="norm"), ParamSpec("o", (hid, HD))]

    def load(self, tensors, rt: Runtime):
        if tensors["w1"].shape[0] != tensors["w2"].shape[1]:
            raise ValueError("w1 and w2 disagree about the width of the decay's bottleneck")
        self.w_in = torch.cat([rt.matrix(tensors[n]) for n in ("r", "k", "v", "a", "g", "w1")], dim=0).contiguous()
        self.w2, self.w_o = rt.matrix(tensors["w2"]), rt.matrix(tensors["o"])
        self.w0, self.a_b, self.norm_w = rt.vector(tensors["w0"]), rt.vector(tensors["a.b"]), rt.vector(tensors["norm"])

    def state_need(self):
        return {"delta": RequestState((self.H, self.d, self.d))}

    def forward(self, h, resid, ctx: StepContext, call: int):
        rt, ops, b = ctx.rt, ctx.rt.ops, ctx.batch
        HD = self.HD
        proj = ops.linear(h, self.w_in, None, torch.float32)        # [r | k | v | a | g | w1 h]
        bottleneck = ops.activation(proj[:, 5 * HD:], "tanh", rt.dtype)
        lw = ops.linear(bottleneck, self.w2, self.w0, torch.float32)
        o = ops.delta_scan(proj, (0, HD, 2 * HD, 3 * HD), lw, self.a_b, ctx.state(call, "delta"), b, self.H, self.d,
                           self.unit_eps, self.decay_coef)
        g = ops.gated_rmsnorm(o, proj[:, 4 * HD:5 * HD], self.norm_w, self.H, self.eps, "sigmoid_after", rt.dtype)
        ops.linear_add(g, self.w_o, resid)


register_part("mixer", "mamba2", Mamba2Mixer)
register_part("mixer", "general_delta", GeneralDeltaMixer)
