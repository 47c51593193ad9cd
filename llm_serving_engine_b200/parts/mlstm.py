"""A matrix memory with exponential gates and a float32 state per request (the mLSTM of the xLSTM family)."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.tensor_spec import TensorSpec
from .base import Mixer, RequestState, register_mixer
from .linear import linear_sums, linear_partials, SKINNY_MAX_ROWS

_DEFAULT_NAMES = {"q": "q", "k": "k", "v": "v", "gate": "g", "out": "o", "norm": "norm", "input_gate": "i",
                  "forget_gate": "f", "bias_suffix": ".b"}


@register_mixer("mlstm")
class MatrixMemory(Mixer):
    """params: ``heads``, ``dim`` (of a head's queries and keys), ``vdim`` (of its values), ``gate_cap`` (the gates'
    pre-activations pass cap tanh(z / cap)), ``eps`` (of the per-head output norm), ``tensor_names``.

    Per head, token by token, with i_t = cap tanh((w_i x + b_i) / cap), f_t = logsigmoid(cap tanh((w_f x + b_f) / cap)),
    q = W_q x / sqrt(dim), k = W_k x, v = W_v x and a running maximum m (zero for a new request):
        m_t = max(f_t + m_(t-1), i_t)
        S_t = exp(f_t + m_(t-1) - m_t) S_(t-1) + exp(i_t - m_t) k_t v_t^T        n_t the same with k_t alone
        o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)
    Each head's o is divided by its root mean square; the concatenated heads are multiplied by a weight and by
    sigmoid(W_g x) and projected by W_o.  Kept per request, in float32: S with n as one more column
    ([heads, dim, vdim + 1]) and m ([heads]).

    One stacked product gives [q | k | v | gate | i | f] with float32 results (the gates and whatever enters the
    recurrence are float32 from there on); a small kernel walks the gates and leaves three numbers per token and head;
    the scan is the gated form of the linear-attention scan (chunks side by side for many rows); a last kernel divides,
    norms and gates."""

    graph_safe = True

    def __init__(self, params, weights, ctx) -> None:
        super().__init__(params, weights, ctx)
        self.heads, self.dim, self.vdim = int(params["heads"]), int(params["dim"]), int(params["vdim"])
        self.eps, self.cap = float(params["eps"]), float(params["gate_cap"])
        names = {**_DEFAULT_NAMES, **params.get("tensor_names", {})}
        roles = ("q", "k", "v", "gate", "input_gate", "forget_gate")
        self.in_weight = torch.cat([weights[names[role]] for role in roles], dim=0).contiguous()
        pad = -self.in_weight.shape[0] % 16       # whole tiles of the few-rows product
        if pad:
            self.in_weight = torch.cat([self.in_weight, self.in_weight.new_zeros((pad, self.in_weight.shape[1]))]).contiguous()
        self.out_weight = weights[names["out"]].contiguous()
        self.norm_weight = weights[names["norm"]].to(torch.float32).contiguous()
        self.i_bias = weights[names["input_gate"] + names["bias_suffix"]].to(torch.float32).contiguous()
        self.f_bias = weights[names["forget_gate"] + names["bias_suffix"]].to(torch.float32).contiguous()
        qk, value = self.heads * self.dim, self.heads * self.vdim
        self.q_off, self.k_off, self.v_off, self.g_off = 0, qk, 2 * qk, 2 * qk + value
        self.i_off = 2 * qk + 2 * value
        self.f_off = self.i_off + self.heads

    @classmethod
    def expected_tensors(cls, params, hidden_size):
        heads, dim, vdim = int(params["heads"]), int(params["dim"]), int(params["vdim"])
        names = {**_DEFAULT_NAMES, **params.get("tensor_names", {})}
        suffix = names["bias_suffix"]
        return {
            names["q"]: TensorSpec((heads * dim, hidden_size)),
            names["k"]: TensorSpec((heads * dim, hidden_size)),
            names["v"]: TensorSpec((heads * vdim, hidden_size)),
            names["gate"]: TensorSpec((heads * vdim, hidden_size)),
            names["out"]: TensorSpec((hidden_size, heads * vdim)),
            names["norm"]: TensorSpec((heads * vdim,), "norm"),
            names["input_gate"]: TensorSpec((heads, hidden_size)),
            names["input_gate"] + suffix: TensorSpec((heads,), "bias"),
            names["forget_gate"]: TensorSpec((heads, hidden_size)),
            names["forget_gate"] + suffix: TensorSpec((heads,), "bias"),
        }

    @classmethod
    def cache_requirement(cls, params, hidden_size):
        heads, dim, vdim = int(params["heads"]), int(params["dim"]), int(params["vdim"])
        return (RequestState((heads, dim, vdim + 1), "float32"), RequestState((heads,), "float32"))

    def forward(self, x, step, cache):
        tokens = x.shape[0]
        memory, maximum = cache.parts[0].state, cache.parts[1].state
        proj = input_projection(x, self.in_weight)
        keep, take, floor = ops.mlstm_gates(proj, self.i_off, self.f_off, self.i_bias, self.f_bias, self.cap, maximum,
                                            step.segment_start, step.segment_state_slot, self.heads)
        read = torch.empty((tokens, self.heads * (self.vdim + 1)), dtype=torch.float32, device=x.device)
        ops.gated_linear_attention_scan(proj, self.q_off, self.k_off, self.v_off, keep, take, self.dim ** -0.5, memory,
                                        step.segment_start, step.segment_state_slot, read, self.heads, self.dim, self.vdim)
        gated = torch.empty((tokens, self.heads * self.vdim), dtype=x.dtype, device=x.device)
        ops.mlstm_readout(read, floor, proj, self.g_off, self.norm_weight, self.eps, gated, self.heads, self.vdim,
                          step.segment_of_token)
        return linear_partials(gated, self.out_weight)


def input_projection(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """x W^T with float32 results whatever the compute dtype (``parts.linear.linear_sums``)."""
    return linear_sums(x, weight)
