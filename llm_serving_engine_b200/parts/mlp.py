"""Dense gated feed-forward (SiLU-gated in the reference, ``src/llmserve/model.py:180-188``)."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.tensor_spec import TensorSpec
from .base import FeedForward, register_feed_forward
from .linear import linear_partials, linear_sums


_DEFAULT_NAMES = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight"}


@register_feed_forward("swiglu")
class SwiGLU(FeedForward):
    """params: ``intermediate_size``; ``activation`` ("silu", the default, "gelu_tanh", "relu", or "clamped_swish":
    g = min(gate, limit), u = clamp(up, -limit, limit), act = g sigmoid(1.702 g) (u + 1), with ``limit`` a parameter);
    ``float32_output`` (the down product leaves float32 sums whatever the compute dtype: for layers that add this
    output to another branch's before the residual takes it); ``tensor_names``
    (the names of the gate, up and down matrices after the part's prefix; default the Qwen2 names).
    y = down(act(gate(x)) * up(x)), no biases; gate and up are stacked into one matrix when the part is
    built (gate rows, then up rows), and the activation kernel adds up the partial sums of their product
    on the way."""

    graph_safe = True

    def __init__(self, params, weights, ctx) -> None:
        super().__init__(params, weights, ctx)
        self.inter = int(params["intermediate_size"])
        self.activation = params.get("activation", "silu")
        if self.activation not in ops.GATE_ACTIVATIONS:
            raise ops.KernelError(f"feed-forward: activation {self.activation!r} is not one of {sorted(ops.GATE_ACTIVATIONS)}")
        self.limit = float(params.get("limit", 0.0))
        if self.activation == "clamped_swish" and not self.limit > 0:
            raise ops.KernelError("feed-forward: clamped_swish needs a positive limit")
        self.float32_output = bool(params.get("float32_output", False))
        names = {**_DEFAULT_NAMES, **params.get("tensor_names", {})}
        self.gate_up_weight = torch.cat([weights[names["gate"]], weights[names["up"]]], dim=0).contiguous()
        self.down_weight = weights[names["down"]].contiguous()

    @classmethod
    def expected_tensors(cls, params, hidden_size):
        inter = int(params["intermediate_size"])
        names = {**_DEFAULT_NAMES, **params.get("tensor_names", {})}
        return {
            names["gate"]: TensorSpec((inter, hidden_size)),
            names["up"]: TensorSpec((inter, hidden_size)),
            names["down"]: TensorSpec((hidden_size, inter)),
        }

    def forward(self, x):
        gate_up = linear_partials(x, self.gate_up_weight)
        act = torch.empty((x.shape[0], self.inter), dtype=x.dtype, device=x.device)
        ops.silu_mul(gate_up, act, self.activation, self.limit)
        return linear_sums(act, self.down_weight) if self.float32_output else linear_partials(act, self.down_weight)


register_feed_forward("gated_mlp", SwiGLU)   # the same part under the name that does not say which activation
