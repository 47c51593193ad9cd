"""Mixture-of-experts feed-forward: a softmax router over experts and identity experts, clamped gated experts, and a
gated shared expert."""
from __future__ import annotations

import os

import torch

from ..kernels import ops
from ..weights.tensor_spec import TensorSpec
from .base import FeedForward, register_feed_forward
from .linear import linear, linear_partials, SKINNY_MAX_ROWS

# Rows of a step from which the rows are grouped by expert (bfloat16).  Below it every expert's product is taken for
# every row: with few rows the experts' weights are what the step waits for, and nearly all of them are read either way.
GROUPED_FROM_ROWS = int(os.environ.get("LSE_MOE_GROUPED_FROM", "128"))

_DEFAULT_NAMES = {"router": "router", "router_bias": "router.b", "correction": "correction", "expert": "e{index}.",
                  "shared": "shared.", "gate": "gate", "up": "up", "down": "down", "shared_gate": "sg"}


@register_feed_forward("clamped_moe")
class ClampedMoE(FeedForward):
    """params: ``experts``, ``identity`` (the router's last ``identity`` outputs stand for experts whose output is the
    input itself), ``top``, ``ff`` and ``limit`` of an expert, ``correction`` (a learned vector added to the scores for
    the choice only; default true), ``shared`` ({"ff", "limit"} or None: an expert that every token uses, times
    sigmoid(w_sg . x)), ``router_bias`` (the router's logits have a bias vector; default false), ``weights``
    ("softmax_all", the default below, or "softmax_chosen": the ``top`` largest logits are chosen and the weights are
    the softmax over the chosen logits only), ``activation`` ("clamped_swish", the default below, or "silu":
    y = W_down (silu(W_gate x) * (W_up x)), nothing clamped, ``limit`` not read; or "squared_relu": experts without a
    gate matrix, y = W_down relu(W_up x)^2), ``scores`` ("softmax", the default, or "sigmoid": scores are sigmoids of the
    logits, the chosen experts' scores are divided by their sum and multiplied by ``router_scale``, and with ``groups``
    {"count", "keep"} the choice is confined to the ``keep`` best of ``count`` equal groups of neighbouring experts, a
    group's score being the sum of its two largest corrected scores), ``tensor_names``.

    Expert: g = min(W_gate x, limit), u = clamp(W_up x, -limit, limit), y = W_down (g sigmoid(1.702 g) (u + 1)).
    Router: s = softmax(W_router x) over all outputs, in float32; the ``top`` outputs with the largest s + correction
    are chosen; the weights are their s, not renormalised.

    The experts' matrices are held once, stacked: [gate; up] expert by expert and then of the shared expert as one
    matrix, and the down matrices side by side as another.  Two ways through them, chosen by the number of rows and the
    precision only (neither depends on the routing, so a step can be replayed from a CUDA graph):

    * few rows (decoding) and float32: all experts side by side as two products; the activation kernel multiplies each
      expert's columns by the token's weight for it (zero where it was not chosen), so that the second product is the
      weighted sum over the experts.  With a handful of tokens nearly every expert's weights are read anyway.
    * many bfloat16 rows: every (token, chosen expert) pair gets a row in a buffer grouped by expert (two small
      kernels), the library's grouped product runs over views of the same stacked matrices, and a kernel adds each
      token's rows times their weights in float32, with the identity experts' share, onto the shared expert's output."""

    graph_safe = True

    def __init__(self, params, weights, ctx) -> None:
        super().__init__(params, weights, ctx)
        p = params
        self.experts, self.identity, self.top = int(p["experts"]), int(p.get("identity", 0)), int(p["top"])
        self.activation = p.get("activation", "clamped_swish")
        if self.activation not in ops.MOE_ACTIVATIONS:
            raise ops.KernelError(f"mixture of experts: activation {self.activation!r} is not one of {sorted(ops.MOE_ACTIVATIONS)}")
        if p.get("weights", "softmax_all") not in ("softmax_all", "softmax_chosen"):
            raise ops.KernelError(f"mixture of experts: weights {p.get('weights')!r} must be softmax_all or softmax_chosen")
        self.over_chosen = p.get("weights", "softmax_all") == "softmax_chosen"
        if p.get("scores", "softmax") not in ("softmax", "sigmoid"):
            raise ops.KernelError(f"mixture of experts: scores {p.get('scores')!r} must be softmax or sigmoid")
        self.sigmoid_scores = p.get("scores", "softmax") == "sigmoid"
        groups = p.get("groups") or {}
        self.group_count, self.group_keep = int(groups.get("count", 1)), int(groups.get("keep", 1))
        self.router_scale = float(p.get("router_scale", 1.0))
        if self.sigmoid_scores and (self.identity or self.over_chosen or p.get("router_bias", False)):
            raise ops.KernelError("mixture of experts: sigmoid scores come without identity experts, a router bias or softmax_chosen")
        self.columns = 1 if self.activation in ops.MOE_UNGATED else 2    # input columns per column of an expert
        self.ff, self.limit = int(p["ff"]), float(p.get("limit", 0.0))
        shared = p.get("shared")
        self.shared_ff = int(shared["ff"]) if shared else 0
        self.shared_limit = float(shared.get("limit", 0.0)) if shared else 0.0
        names = {**_DEFAULT_NAMES, **p.get("tensor_names", {})}
        prefixes = [names["expert"].format(index=index) for index in range(self.experts)]
        if shared:
            prefixes.append(names["shared"])
        roles = ("up",) if self.columns == 1 else ("gate", "up")
        pairs = [weights[prefix + names[which]] for prefix in prefixes for which in roles]
        self.inter = self.experts * self.ff + self.shared_ff
        self.gate_up_weight = torch.cat(pairs, dim=0).contiguous() if prefixes else None
        self.down_weight = torch.cat([weights[prefix + names["down"]] for prefix in prefixes], dim=1).contiguous() if prefixes else None
        # the router's rows, then the shared expert's gate row, padded with zero rows to a multiple of 16: one product
        # gives every logit that the routing kernel reads
        rows = [weights[names["router"]]] + ([weights[names["shared"] + names["shared_gate"]].reshape(1, -1)] if shared else [])
        self.outputs = self.experts + self.identity
        pad = -(self.outputs + len(rows) - 1) % 16
        if pad:
            rows.append(torch.zeros((pad, rows[0].shape[1]), dtype=rows[0].dtype, device=rows[0].device))
        self.router = torch.cat(rows, dim=0).contiguous()
        self.correction = weights[names["correction"]].float().contiguous() if p.get("correction", True) else None
        self.router_bias = weights[names["router_bias"]].float().contiguous() if p.get("router_bias", False) else None
        self.row_scale = None    # after forward: float32 [T] c_t, when c_t x_t is still to be added to the output
        # views of the stacked matrices for the grouped product: [experts, width, 2 ff] and [experts, ff, width]
        self._grouped_gate_up = self._grouped_down = None
        width = self.router.shape[1]
        if (self.experts and self.gate_up_weight.dtype == torch.bfloat16 and width % 8 == 0 and self.ff % 8 == 0
                and self.inter % 8 == 0 and hasattr(torch, "_grouped_mm")):
            routed = self.experts * self.ff
            self._grouped_gate_up = (self.gate_up_weight[:self.columns * routed]
                                     .view(self.experts, self.columns * self.ff, width).transpose(1, 2))
            self._grouped_down = self.down_weight.as_strided((self.experts, self.ff, width), (self.ff, 1, self.inter))

    @classmethod
    def expected_tensors(cls, params, hidden_size):
        p = params
        experts, identity, ff = int(p["experts"]), int(p.get("identity", 0)), int(p["ff"])
        names = {**_DEFAULT_NAMES, **p.get("tensor_names", {})}
        out = {names["router"]: TensorSpec((experts + identity, hidden_size))}
        if p.get("correction", True):
            out[names["correction"]] = TensorSpec((experts + identity,), "bias")
        if p.get("router_bias", False):
            out[names["router_bias"]] = TensorSpec((experts + identity,), "bias")
        sized = [(names["expert"].format(index=index), ff) for index in range(experts)]
        if p.get("shared"):
            sized.append((names["shared"], int(p["shared"]["ff"])))
            out[names["shared"] + names["shared_gate"]] = TensorSpec((1, hidden_size))
        gated = p.get("activation", "clamped_swish") not in ops.MOE_UNGATED
        for prefix, width in sized:
            if gated:
                out[prefix + names["gate"]] = TensorSpec((width, hidden_size))
            out[prefix + names["up"]] = TensorSpec((width, hidden_size))
            out[prefix + names["down"]] = TensorSpec((hidden_size, width))
        return out

    def _grouped(self, x):
        """Rows grouped by expert (see the class)."""
        tokens, width = x.shape
        chosen = torch.empty((tokens, self.top), dtype=torch.int32, device=x.device)
        expert_weights, identity_weight, shared_gate = self._route(x, chosen)
        y = None
        if self.shared_ff:   # the shared expert: two plain products, its gate folded into the activation
            routed = self.experts * self.ff
            gate_up = linear(x, self.gate_up_weight[self.columns * routed:])
            act = torch.empty((tokens, self.shared_ff), dtype=x.dtype, device=x.device)
            ops.moe_gated_act(gate_up, None, shared_gate, act, 0, 8, self.shared_ff, self.limit, self.shared_limit,
                              activation=self.activation)
            y = linear(act, self.down_weight[:, routed:], out_dtype=torch.float32)
        row_of, offsets = ops.moe_group_rows(chosen, self.experts)
        rows = tokens * self.top
        grouped = torch.empty((rows, width), dtype=x.dtype, device=x.device)
        ops.moe_gather_rows(x, row_of, grouped)
        gate_up = torch._grouped_mm(grouped, self._grouped_gate_up, offs=offsets)     # rows beyond the last range stay as they are
        act = torch.empty((rows, self.ff), dtype=x.dtype, device=x.device)
        ops.moe_gated_act(gate_up, None, None, act, 1, self.ff, 0, self.limit, 0.0, valid_rows=offsets[-1:],
                          activation=self.activation)
        down = torch._grouped_mm(act, self._grouped_down, offs=offsets)
        out = y if y is not None else torch.empty((tokens, width), dtype=torch.float32, device=x.device)
        return ops.moe_combine(down, row_of, chosen, expert_weights, identity_weight if self.identity else None, x, out,
                               accumulate=y is not None)

    def _route(self, x, chosen=None):
        """The router's logits as a product with float32 sums (partial sums for few rows), then the routing kernel."""
        if x.dtype != torch.bfloat16:
            logits = linear_partials(x, self.router)
        elif x.shape[0] <= SKINNY_MAX_ROWS and ops.gemm_bf16_skinny_ok(x, self.router):
            logits = ops.gemm_bf16_skinny(x, self.router)     # float32 partial sums, added up by the routing kernel
        else:
            logits = linear(x, self.router, out_dtype=torch.float32)
        if self.sigmoid_scores:
            return ops.moe_route_sigmoid(logits, self.correction, self.experts, self.top, self.group_count,
                                         self.group_keep, self.router_scale, shared_gate=self.shared_ff > 0, chosen=chosen)
        return ops.moe_route(logits, self.correction, self.outputs, self.identity, self.top,
                             shared_gate=self.shared_ff > 0, chosen=chosen, logit_bias=self.router_bias,
                             over_chosen=self.over_chosen)

    def forward(self, x):
        tokens = x.shape[0]
        self.row_scale = None
        if self._grouped_gate_up is not None and x.dtype == torch.bfloat16 and tokens >= GROUPED_FROM_ROWS:
            return self._grouped(x)
        expert_weights, identity_weight, shared_gate = self._route(x)
        if self.inter:
            gate_up = linear_partials(x, self.gate_up_weight)
            act = torch.empty((tokens, self.inter), dtype=x.dtype, device=x.device)
            ops.moe_gated_act(gate_up, expert_weights, shared_gate, act, self.experts, self.ff, self.shared_ff,
                              self.limit, self.shared_limit, activation=self.activation)
            if x.dtype == torch.bfloat16 and tokens > SKINNY_MAX_ROWS:
                y = linear(act, self.down_weight, out_dtype=torch.float32)
            else:
                y = linear_partials(act, self.down_weight)
        else:
            y = torch.zeros((tokens, x.shape[1]), dtype=torch.float32, device=x.device)
        if self.identity:
            self.row_scale = identity_weight     # the identity experts' share w_t x_t: the norm that adds the output adds it
        return y


register_feed_forward("routed_experts", ClampedMoE)   # the same part under a name that does not say which activation
