"""Linear attention with a decay per head and a float32 state per request."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.tensor_spec import TensorSpec
from .base import Mixer, RequestState, register_mixer
from .linear import linear_partials, linear_sums

_DEFAULT_NAMES = {"q": "q", "k": "k", "v": "v", "gate": "g", "out": "o", "norm": "norm"}


@register_mixer("decayed_linear_attention")
class DecayedLinearAttention(Mixer):
    """params: ``heads``, ``dim`` (of a head's queries and keys), ``vdim`` (of its values), ``decay`` (one number per
    head), ``eps`` (of the output norm), ``activation`` ("silu", the default, or "none") on q, k and v,
    ``tensor_names`` (names of the q, k, v, gate and output matrices and of the norm weight after the part's prefix).

    Per head, token by token:  S_t = decay_h S_(t-1) + k_t v_t^T,  o_t = S_t^T q_t  with q, k, v = act(W x).
    The concatenated heads are RMS-normed with a plain weight, multiplied by sigmoid(W_g x) and projected by W_o.
    S is [dim, vdim] per head, float32, zero for a new request, kept in the request's state slot between steps;
    no other scale is applied.  The four input projections are one stacked product."""

    graph_safe = True

    def __init__(self, params, weights, ctx) -> None:
        super().__init__(params, weights, ctx)
        self.heads, self.dim, self.vdim = int(params["heads"]), int(params["dim"]), int(params["vdim"])
        self.eps = float(params["eps"])
        self.activation = params.get("activation", "silu")
        decay = [float(value) for value in params["decay"]]
        if len(decay) != self.heads:
            raise ops.KernelError(f"linear attention: {len(decay)} decays for {self.heads} heads")
        self.decay = torch.tensor(decay, dtype=torch.float64).to(torch.float32).to(ctx.device)
        names = {**_DEFAULT_NAMES, **params.get("tensor_names", {})}
        self.in_weight = torch.cat([weights[names[role]] for role in ("q", "k", "v", "gate")], dim=0).contiguous()
        self.out_weight = weights[names["out"]].contiguous()
        self.norm_weight = weights[names["norm"]].to(torch.float32).contiguous()
        qk, value = self.heads * self.dim, self.heads * self.vdim
        self.offsets = (0, qk, 2 * qk, 2 * qk + value)   # columns of q, k, v and the gate in the stacked product

    @classmethod
    def expected_tensors(cls, params, hidden_size):
        heads, dim, vdim = int(params["heads"]), int(params["dim"]), int(params["vdim"])
        names = {**_DEFAULT_NAMES, **params.get("tensor_names", {})}
        return {
            names["q"]: TensorSpec((heads * dim, hidden_size)),
            names["k"]: TensorSpec((heads * dim, hidden_size)),
            names["v"]: TensorSpec((heads * vdim, hidden_size)),
            names["gate"]: TensorSpec((heads * vdim, hidden_size)),
            names["out"]: TensorSpec((hidden_size, heads * vdim)),
            names["norm"]: TensorSpec((heads * vdim,), "norm"),
        }

    @classmethod
    def cache_requirement(cls, params, hidden_size):
        return RequestState((int(params["heads"]), int(params["dim"]), int(params["vdim"])), "float32")

    def forward(self, x, step, cache):
        tokens = x.shape[0]
        proj = linear_partials(x, self.in_weight)
        q_off, k_off, v_off, g_off = self.offsets
        attended = torch.empty((tokens, self.heads * self.vdim), dtype=torch.float32, device=x.device)
        ops.linear_attention_scan(proj, q_off, k_off, v_off, self.decay, cache.state, step.segment_start,
                                  step.segment_state_slot, attended, self.heads, self.dim, self.vdim, self.activation)
        gated = torch.empty((tokens, self.heads * self.vdim), dtype=x.dtype, device=x.device)
        ops.gated_rmsnorm(attended, proj, g_off, self.norm_weight, self.eps, gated, step.segment_of_token)
        return linear_partials(gated, self.out_weight)


_CHANNEL_DECAY_NAMES = {"q": "q", "k": "k", "v": "v", "gate": "g", "out": "o", "norm": "norm", "decay_down": "a1",
                        "decay_up": "a2", "decay_bias": "a2.b"}


@register_mixer("channel_decay_linear_attention")
class ChannelDecayLinearAttention(Mixer):
    """params: ``heads``, ``dim`` (of a head's queries and keys), ``vdim`` (of its values), ``tau``, ``rank`` (of the
    decay's low-rank map), ``eps`` (of the output norm), ``tensor_names``.

    Gated linear attention: a matrix memory per head whose rows decay by a learned factor per key channel and token,
        keep_t = sigmoid(W_a2 (W_a1 x_t) + b)^(1 / tau)       (heads x dim numbers a token)
        S_t = diag(keep_t) S_(t-1) + k_t v_t^T,   o_t = S_t^T (q_t / sqrt(dim)),
    with q, k, v = W x as they are.  Each head's o is RMS-normed over ``vdim`` with one weight vector for all heads; the
    concatenated heads are multiplied by silu(W_g x) and projected by W_o.  S is [dim, vdim] per head, float32, zero for
    a new request, kept in the request's state slot between steps.  The five input projections are one stacked
    product with float32 results; the decay's second product and everything behind it (logarithm of the sigmoid, the
    power, the scan) are float32."""

    graph_safe = True

    def __init__(self, params, weights, ctx) -> None:
        super().__init__(params, weights, ctx)
        self.heads, self.dim, self.vdim = int(params["heads"]), int(params["dim"]), int(params["vdim"])
        self.tau, self.eps, self.rank = float(params["tau"]), float(params["eps"]), int(params["rank"])
        names = {**_CHANNEL_DECAY_NAMES, **params.get("tensor_names", {})}
        stacked = [weights[names[role]] for role in ("q", "k", "v", "gate", "decay_down")]
        pad = -sum(w.shape[0] for w in stacked) % 16     # whole tiles of the few-rows product
        if pad:
            stacked.append(stacked[0].new_zeros((pad, stacked[0].shape[1])))
        self.in_weight = torch.cat(stacked, dim=0).contiguous()
        up = weights[names["decay_up"]]
        pad = -up.shape[1] % 16
        self.rank_padded = up.shape[1] + pad       # the second product's inner size, in whole tiles too
        self.decay_up = (torch.cat([up, up.new_zeros((up.shape[0], pad))], dim=1) if pad else up).contiguous()
        self.decay_bias = weights[names["decay_bias"]].to(torch.float32).contiguous()
        self.out_weight = weights[names["out"]].contiguous()
        self.norm_weight = weights[names["norm"]].to(torch.float32).contiguous()
        qk, value = self.heads * self.dim, self.heads * self.vdim
        self.offsets = (0, qk, 2 * qk, 2 * qk + value, 2 * qk + 2 * value)   # q, k, v, gate, the decay's low-rank input

    @classmethod
    def expected_tensors(cls, params, hidden_size):
        heads, dim, vdim, rank = int(params["heads"]), int(params["dim"]), int(params["vdim"]), int(params["rank"])
        names = {**_CHANNEL_DECAY_NAMES, **params.get("tensor_names", {})}
        return {
            names["q"]: TensorSpec((heads * dim, hidden_size)),
            names["k"]: TensorSpec((heads * dim, hidden_size)),
            names["v"]: TensorSpec((heads * vdim, hidden_size)),
            names["gate"]: TensorSpec((heads * vdim, hidden_size)),
            names["out"]: TensorSpec((hidden_size, heads * vdim)),
            names["norm"]: TensorSpec((vdim,), "norm"),
            names["decay_down"]: TensorSpec((rank, hidden_size)),
            names["decay_up"]: TensorSpec((heads * dim, rank)),
            names["decay_bias"]: TensorSpec((heads * dim,), "bias"),
        }

    @classmethod
    def cache_requirement(cls, params, hidden_size):
        return RequestState((int(params["heads"]), int(params["dim"]), int(params["vdim"])), "float32")

    def forward(self, x, step, cache):
        tokens = x.shape[0]
        proj = linear_sums(x, self.in_weight)
        q_off, k_off, v_off, g_off, a_off = self.offsets
        low = proj[..., a_off:a_off + self.rank]
        if low.dim() == 3:
            low = low.sum(0)
        padded = torch.zeros((tokens, self.rank_padded), dtype=x.dtype, device=x.device) if self.rank_padded != self.rank else None
        if padded is not None:
            padded[:, :self.rank] = low
            low = padded
        else:
            low = low.to(x.dtype).contiguous()
        keep = ops.sigmoid_power(linear_sums(low, self.decay_up), 0, self.heads * self.dim, self.decay_bias, self.tau)
        attended = torch.empty((tokens, self.heads * self.vdim), dtype=torch.float32, device=x.device)
        ops.channel_decay_scan(proj, q_off, k_off, v_off, keep, self.dim ** -0.5, cache.state, step.segment_start,
                               step.segment_state_slot, attended, self.heads, self.dim, self.vdim)
        gated = torch.empty((tokens, self.heads * self.vdim), dtype=x.dtype, device=x.device)
        ops.gated_group_rmsnorm(attended, proj, g_off, self.norm_weight, self.eps, gated, self.heads, gate_first=False,
                                gate_activation="silu", segment_of_token=step.segment_of_token)
        return linear_sums(gated, self.out_weight)
