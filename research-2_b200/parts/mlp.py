"""Dense feed-forwards, added to the residual stream: act(h @ w_in + b_in) @ w_out + b_out
(reference: kelpie-models/kelpie_models/models/torch/gpt2.py:94-96), and the gated form with clamped
projections."""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import Runtime, register_feed_forward
from .util import matrix, vector


@register_feed_forward("mlp")
class DenseMLP:
    """params: activation ("gelu_new" | "gelu"). weights: w_in [D, F], b_in, w_out [F, D], b_out,
    both matrices stored [in, out]; the inner width F is the weights' own."""

    def __init__(self, params: dict, weights: dict, rt: Runtime):
        self.activation = params["activation"]
        if self.activation not in ops.ACTIVATIONS or self.activation in (None, "none"):
            raise ValueError(f"mlp: unknown activation {self.activation!r}")
        self.w_in = matrix(weights["w_in"], rt)
        self.b_in = vector(weights["b_in"], rt)
        self.w_out = matrix(weights["w_out"], rt)
        self.b_out = vector(weights["b_out"], rt)
        if self.w_in.shape[1] != self.w_out.shape[0] or self.w_in.shape[0] != self.w_out.shape[1]:
            raise ValueError(f"mlp: w_in {tuple(self.w_in.shape)} and w_out {tuple(self.w_out.shape)} do not fit")

    takes_lazy_norm = True  # the input goes straight into ops.linear

    def matrices(self):
        """The weight matrices in the order in which forward() uses them."""
        return [self.w_in, self.w_out]

    def resident_mlp(self) -> dict:
        return {"w_fc": self.w_in, "b_fc": self.b_in, "w_pr": self.w_out, "b_pr": self.b_out, "act": self.activation,
                "width": self.w_in.shape[0], "inner": self.w_in.shape[1]}

    def forward(self, h, residual, ctx):
        return ops.mlp(h, self.w_in, self.b_in, self.activation, self.w_out, self.b_out, residual=residual)


@register_feed_forward("gated_clamped")
class GatedClampedMLP:
    """W_down y with y = g * sigmoid(alpha * g) * (u + up_offset), g = min(W_gate h, limit) and
    u = clamp(W_up h, -limit, limit). params: limit, alpha, up_offset. weights: w_gate [F, D], w_up [F, D],
    w_down [D, F], all stored [out, in], no biases. The two input projections run as one product over the
    stacked matrix [2 F, D]."""

    def __init__(self, params: dict, weights: dict, rt: Runtime):
        self.limit, self.alpha, self.up_offset = float(params["limit"]), float(params["alpha"]), float(params["up_offset"])
        gate, up, down = weights["w_gate"], weights["w_up"], weights["w_down"]
        if gate.shape != up.shape or down.shape != (gate.shape[1], gate.shape[0]):
            raise ValueError(f"gated feed-forward: w_gate {tuple(gate.shape)}, w_up {tuple(up.shape)} and w_down {tuple(down.shape)} do not fit")
        self.inner = gate.shape[0]
        self.w_gate_up = matrix(torch.cat([gate, up], dim=0), rt)
        self.w_down = matrix(down, rt)

    def matrices(self):
        return [self.w_gate_up, self.w_down]

    def input_matrix(self):
        """The stacked projections of the input, [gate; up] x D stored [out, in] (see `forward_projected`)."""
        return self.w_gate_up

    def forward(self, h, residual, ctx):
        return self.forward_projected(ops.linear(h, self.w_gate_up, None, w_is_nk=True), residual, ctx)

    def forward_projected(self, gate_up, residual, ctx):
        """`gate_up` [T, 2 F]: the input's gate and up projections."""
        y = ops.gated_act(gate_up, self.limit, self.alpha, self.up_offset)
        return ops.linear(y, self.w_down, None, w_is_nk=True, residual=residual)
