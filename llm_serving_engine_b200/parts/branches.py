"""Mixers that can run side by side on one input: a grouped-query attention behind short convolutions, a selective
state-space scan, and the mixer that sums several such branches with a weight each."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.tensor_spec import TensorSpec
from .base import MIXERS, Mixer, PagedKV, RequestState, cache_for, cache_needs, register_mixer
from .latent_attention import rotary_frequencies
from .linear import linear_partials, linear_sums
from .mlstm import input_projection
from .normed_attention import prompt_shape_for_tcgen05


class BranchMixer(Mixer):
    """A mixer of the form  y = W_out inner(W_in x):  its input product and its output product can be shared with other
    mixers that read the same x (their input matrices stacked into one product, their output matrices side by side,
    so that the sum of the branches is one product too).  A subclass sets ``in_weight`` [n_in, H] and ``out_weight``
    [H, n_mid] and implements ``inner(proj, offset, step, cache, out, scale)``: its columns of the stacked
    projection start at ``offset``; it writes ``scale`` times its activations into ``out`` [T, n_mid], which may be
    a column range of a wider tensor."""

    in_weight: torch.Tensor
    out_weight: torch.Tensor

    def inner(self, proj, offset: int, step, cache, out: torch.Tensor, scale: float) -> None:
        raise NotImplementedError

    def forward(self, x, step, cache):
        proj = input_projection(x, self.in_weight)
        mid = torch.empty((x.shape[0], self.out_weight.shape[1]), dtype=x.dtype, device=x.device)
        self.inner(proj, 0, step, cache, mid, 1.0)
        return linear_partials(mid, self.out_weight)


_ATTENTION_NAMES = {"q": "q", "k": "k", "v": "v", "gate": "g", "out": "o", "q_norm": "q.norm", "k_norm": "k.norm",
                    "conv_suffix": ".conv"}


@register_mixer("conv_rotary_attention")
class ConvRotaryAttention(BranchMixer):
    """params: ``heads``, ``kv_heads`` (query head h uses key/value head h // (heads / kv_heads)), ``dim`` (of a head's
    query and key), ``vdim`` (of its value), ``conv`` (taps of the short causal convolution that q, k and v each
    pass, per channel, straight after their projection; 0 or absent: none, and no such tensors), ``eps`` (of the norms), ``rot`` ({base, dims,
    scaling}: the first ``dims`` values of every head are rotated, value i paired with i + dims / 2; see
    ``rotary_frequencies`` for ``scaling``), ``scale`` (on the scores), ``gate`` (head h's output times
    sigmoid(w_g,h x)), ``tensor_names``.

    After the convolutions q and k are RMS-normed over their whole width (all heads at once, weights of that width),
    then rotated; the softmax is the ordinary causal one.  Kept per request: pages of keys and values, and the last
    ``conv - 1`` projected rows [q | k | v] (float32), so that a step may start anywhere.

    One kernel does convolution, norms, rotation, the page write and the gates' sigmoid; the attention itself is the
    engine's paged attention for keys and values of any sizes (tensor cores for bfloat16 shapes that it takes; long
    prompt portions with heads of 64 or 128 on the tcgen05 kernel)."""

    graph_safe = True

    def __init__(self, params, weights, ctx) -> None:
        super().__init__(params, weights, ctx)
        p = params
        self.n_q, self.n_kv = int(p["heads"]), int(p["kv_heads"])
        self.dk, self.dv, self.taps = int(p["dim"]), int(p["vdim"]), max(int(p.get("conv", 0)), 1)
        self.scale, self.eps = float(p["scale"]), float(p["eps"])
        if self.n_q % self.n_kv:
            raise ops.KernelError(f"attention: {self.n_q} query heads do not divide into {self.n_kv} groups")
        rot = p.get("rot") or {"dims": 0, "base": 1.0}
        if int(rot["dims"]) % 2 or int(rot["dims"]) > self.dk:
            raise ops.KernelError(f"attention: {rot['dims']} rotated values of {self.dk}")
        freq, self.rot_factor = rotary_frequencies(rot) if int(rot["dims"]) else (torch.zeros(0, dtype=torch.float64), 1.0)
        self.freq = freq.to(torch.float64).contiguous().to(ctx.device)
        names = {**_ATTENTION_NAMES, **p.get("tensor_names", {})}
        stacked = [weights[names[role]] for role in ("q", "k", "v")]
        self.channels = sum(w.shape[0] for w in stacked)
        self.has_gate = bool(p.get("gate", False))
        if self.has_gate:
            stacked.append(weights[names["gate"]])
        self.in_weight = torch.cat(stacked, dim=0).contiguous()
        if int(p.get("conv", 0)) >= 1:
            self.conv_weight = torch.cat([weights[names[role] + names["conv_suffix"]].to(torch.float32)
                                          for role in ("q", "k", "v")], dim=0).contiguous()
        else:
            self.conv_weight = torch.ones((self.channels, 1), dtype=torch.float32, device=ctx.device)
        self.q_norm = weights[names["q_norm"]].to(torch.float32).contiguous()
        self.k_norm = weights[names["k_norm"]].to(torch.float32).contiguous()
        self.out_weight = weights[names["out"]].contiguous()

    @classmethod
    def expected_tensors(cls, params, hidden_size):
        p = params
        n_q, n_kv, dk, dv, taps = int(p["heads"]), int(p["kv_heads"]), int(p["dim"]), int(p["vdim"]), int(p.get("conv", 0))
        names = {**_ATTENTION_NAMES, **p.get("tensor_names", {})}
        out = {names["q"]: TensorSpec((n_q * dk, hidden_size)), names["k"]: TensorSpec((n_kv * dk, hidden_size)),
               names["v"]: TensorSpec((n_kv * dv, hidden_size)), names["out"]: TensorSpec((hidden_size, n_q * dv)),
               names["q_norm"]: TensorSpec((n_q * dk,), "norm"), names["k_norm"]: TensorSpec((n_kv * dk,), "norm")}
        if taps >= 1:
            for role in ("q", "k", "v"):
                out[names[role] + names["conv_suffix"]] = TensorSpec((out[names[role]].shape[0], taps), "filter")
        if p.get("gate", False):
            out[names["gate"]] = TensorSpec((n_q, hidden_size))
        return out

    @classmethod
    def cache_requirement(cls, params, hidden_size):
        n_q, n_kv, dk, dv = int(params["heads"]), int(params["kv_heads"]), int(params["dim"]), int(params["vdim"])
        taps = int(params.get("conv", 0))
        pages = PagedKV(n_kv, dk, 0, 0 if dv == dk else dv)
        return (pages, RequestState((max(taps - 1, 0), (n_q + n_kv) * dk + n_kv * dv), "float32"))

    def _on_tcgen05(self, segment_counts, page_size=None) -> bool:
        if not prompt_shape_for_tcgen05(self.ctx.dtype, self.dk, self.dv, segment_counts):
            return False
        return page_size is None or ops.attention_tc_supported(self.dk, self.n_q, self.n_kv, page_size, self.ctx.dtype)

    def launch_signature(self, segment_counts):
        return ("tcgen05",) if self._on_tcgen05(segment_counts) else ()

    def inner(self, proj, offset, step, cache, out, scale):
        pages, window = cache.parts[0], cache.parts[1].state
        tokens = out.shape[0]
        q = torch.empty((tokens, self.n_q, self.dk), dtype=out.dtype, device=out.device)
        gate = torch.empty((tokens, self.n_q), dtype=torch.float32, device=out.device) if self.has_gate else None
        ops.conv_qk_norm_rope(proj, offset, offset + self.channels, self.conv_weight, window, self.q_norm, self.k_norm,
                              self.eps, self.freq, self.rot_factor, step, pages.slot_mapping, q, pages.keys, pages.values,
                              gate, self.n_q, self.n_kv, self.dk, self.dv)
        if self.taps > 1:
            ops.short_conv_state(proj, offset, self.channels, self.taps, window, step)
        attended = torch.empty((tokens, self.n_q, self.dv), dtype=out.dtype, device=out.device)
        if (not step.decode_only and step.segments
                and self._on_tcgen05([segment.count for segment in step.segments], pages.keys.shape[2])):
            ops.attention_scored_tc(q, pages.keys, pages.values, attended, pages.block_tables, step.segment_start,
                                    step.segment_first_position, self.scale)
        else:
            ops.attention_scored(q, pages.keys, pages.values, attended, pages.block_tables, step.segment_of_token,
                                 step.positions, self.scale, segment_start=step.segment_start,
                                 segment_first_position=step.segment_first_position)
        ops.head_gate_scale(attended, gate, out, scale, step.segment_of_token)


_SSM_NAMES = {"in": "in", "conv": "conv", "conv_bias": "conv.b", "x": "x", "dt": "dt", "dt_bias": "dt.b",
              "a_log": "A_log", "skip": "D", "out": "o"}


@register_mixer("selective_state_space")
class SelectiveStateSpace(BranchMixer):
    """params: ``inner`` (channels), ``state`` (states per channel), ``dt_rank``, ``conv`` (taps), ``tensor_names``.

    W_in x = [u | z]; u passes a short causal convolution per channel (with bias) and SiLU; W_x u = [low (dt_rank) |
    B (state) | C (state)]; dt = softplus(W_dt low + b_dt) per channel; A = -exp(A_log);
        S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c u_c B_n;      y_c = sum_n S[c, n] C_n + D_c u_c;
    the output is W_out (y * silu(z)).  Kept per request, in float32: S [inner, state] and the last ``conv - 1`` rows
    of u before the convolution.  Step sizes, decays, B, C and the state are float32."""

    graph_safe = True

    def __init__(self, params, weights, ctx) -> None:
        super().__init__(params, weights, ctx)
        p = params
        self.channels, self.states, self.rank, self.taps = int(p["inner"]), int(p["state"]), int(p["dt_rank"]), int(p["conv"])
        names = {**_SSM_NAMES, **p.get("tensor_names", {})}
        self.in_weight = weights[names["in"]].contiguous()
        self.conv_weight = weights[names["conv"]].to(torch.float32).contiguous()
        self.conv_bias = weights[names["conv_bias"]].to(torch.float32).contiguous()
        low = weights[names["x"]]
        pad = -low.shape[0] % 16       # whole tiles of the few-rows product
        self.low_weight = (torch.cat([low, low.new_zeros((pad, low.shape[1]))]) if pad else low).contiguous()
        self.dt_weight_t = weights[names["dt"]].to(torch.float32).t().contiguous()      # [rank, channels]
        self.dt_bias = weights[names["dt_bias"]].to(torch.float32).contiguous()
        self.a_log = weights[names["a_log"]].to(torch.float32).contiguous()
        self.skip = weights[names["skip"]].to(torch.float32).contiguous()
        self.out_weight = weights[names["out"]].contiguous()

    @classmethod
    def expected_tensors(cls, params, hidden_size):
        p = params
        inner, states, rank, taps = int(p["inner"]), int(p["state"]), int(p["dt_rank"]), int(p["conv"])
        names = {**_SSM_NAMES, **p.get("tensor_names", {})}
        return {names["in"]: TensorSpec((2 * inner, hidden_size)), names["conv"]: TensorSpec((inner, taps), "filter"),
                names["conv_bias"]: TensorSpec((inner,), "bias"), names["x"]: TensorSpec((rank + 2 * states, inner)),
                names["dt"]: TensorSpec((inner, rank)), names["dt_bias"]: TensorSpec((inner,), "bias"),
                names["a_log"]: TensorSpec((inner, states), "positive"), names["skip"]: TensorSpec((inner,), "norm"),
                names["out"]: TensorSpec((hidden_size, inner))}

    @classmethod
    def cache_requirement(cls, params, hidden_size):
        inner, states, taps = int(params["inner"]), int(params["state"]), int(params["conv"])
        return (RequestState((inner, states), "float32"), RequestState((max(taps - 1, 0), inner), "float32"))

    def inner(self, proj, offset, step, cache, out, scale):
        state, window = cache.parts[0].state, cache.parts[1].state
        tokens = out.shape[0]
        u = torch.empty((tokens, self.channels), dtype=out.dtype, device=out.device)
        ops.short_conv_act(proj, offset, self.conv_weight, self.conv_bias, window, step, u, "silu")
        if self.taps > 1:
            ops.short_conv_state(proj, offset, self.channels, self.taps, window, step)
        low = input_projection(u, self.low_weight)
        dt = ops.ssm_step_sizes(low, self.dt_weight_t, self.dt_bias)
        ops.selective_scan(u, dt, proj, offset + self.channels, low, self.rank, self.rank + self.states, self.a_log,
                           self.skip, state, step, out, scale)


_HEAD_NORM_NAMES = {"q": "q", "k": "k", "v": "v", "out": "o", "q_norm": "q.norm", "k_norm": "k.norm",
                    "bias_suffix": ".b", "head_bias": "pb"}


@register_mixer("head_norm_rotary_attention")
class HeadNormRotaryAttention(BranchMixer):
    """params: ``heads``, ``kv_heads`` (query head h uses key/value head h // (heads / kv_heads)), ``dim`` (of a head's
    query and key), ``vdim`` (of its value), ``eps``, ``scale`` (on the scores), ``bias`` (q, k and v projections have
    bias vectors), ``rot`` ({base, dims, scaling} or None: the first ``dims`` values of every head are rotated, value i
    paired with i + dims / 2; see ``rotary_frequencies`` for ``scaling``), ``window`` (> 0: a row reads its last
    ``window`` keys, itself included; older pages are given back), ``softcap`` (> 0: scores become cap * tanh(s / cap)),
    ``weights`` ("softmax", the default, or "sigmoid": a key's weight is sigmoid(score + b_h) with a learned number per
    head, not normalised over the keys), ``tensor_names``.

    Every head of q and of k is RMS-normed over its ``dim`` values with one weight vector for all heads, before the
    rotation.  One kernel sums the projection, adds the biases, norms, rotates and writes the pages; the attention is
    the engine's paged attention for changed scores (window, cap and sigmoid weights are arguments of its kernels)."""

    graph_safe = True

    def __init__(self, params, weights, ctx) -> None:
        super().__init__(params, weights, ctx)
        p = params
        self.n_q, self.n_kv, self.dk, self.dv = int(p["heads"]), int(p["kv_heads"]), int(p["dim"]), int(p["vdim"])
        self.scale, self.eps = float(p["scale"]), float(p["eps"])
        self.window, self.softcap = int(p.get("window", 0)), float(p.get("softcap", 0.0))
        self.sigmoid = self._weights_kind(p) == "sigmoid"
        if self.n_q % self.n_kv:
            raise ops.KernelError(f"attention: {self.n_q} query heads do not divide into {self.n_kv} groups")
        rot = p.get("rot") or {"dims": 0, "base": 1.0}
        if int(rot["dims"]) % 2 or int(rot["dims"]) > self.dk:
            raise ops.KernelError(f"attention: {rot['dims']} rotated values of {self.dk}")
        freq, self.rot_factor = rotary_frequencies(rot) if int(rot["dims"]) else (torch.zeros(0, dtype=torch.float64), 1.0)
        self.freq = freq.to(torch.float64).contiguous().to(ctx.device)
        names = {**_HEAD_NORM_NAMES, **p.get("tensor_names", {})}
        roles = ("q", "k", "v")
        self.in_weight = torch.cat([weights[names[role]] for role in roles], dim=0).contiguous()
        self.in_bias = (torch.cat([weights[names[role] + names["bias_suffix"]].to(torch.float32) for role in roles]).contiguous()
                        if p.get("bias", False) else None)
        self.q_norm = weights[names["q_norm"]].to(torch.float32).contiguous()
        self.k_norm = weights[names["k_norm"]].to(torch.float32).contiguous()
        self.head_bias = weights[names["head_bias"]].to(torch.float32).contiguous() if self.sigmoid else None
        self.out_weight = weights[names["out"]].contiguous()

    @staticmethod
    def _weights_kind(params) -> str:
        kind = params.get("weights", "softmax")
        if kind not in ("softmax", "sigmoid"):
            raise ops.KernelError(f"attention: weights {kind!r} must be softmax or sigmoid")
        return kind

    @classmethod
    def expected_tensors(cls, params, hidden_size):
        p = params
        n_q, n_kv, dk, dv = int(p["heads"]), int(p["kv_heads"]), int(p["dim"]), int(p["vdim"])
        names = {**_HEAD_NORM_NAMES, **p.get("tensor_names", {})}
        out = {names["q"]: TensorSpec((n_q * dk, hidden_size)), names["k"]: TensorSpec((n_kv * dk, hidden_size)),
               names["v"]: TensorSpec((n_kv * dv, hidden_size)), names["out"]: TensorSpec((hidden_size, n_q * dv)),
               names["q_norm"]: TensorSpec((dk,), "norm"), names["k_norm"]: TensorSpec((dk,), "norm")}
        if p.get("bias", False):
            for role in ("q", "k", "v"):
                out[names[role] + names["bias_suffix"]] = TensorSpec((out[names[role]].shape[0],), "bias")
        if cls._weights_kind(p) == "sigmoid":
            out[names["head_bias"]] = TensorSpec((n_q,), "bias")
        return out

    @classmethod
    def cache_requirement(cls, params, hidden_size):
        dk, dv = int(params["dim"]), int(params["vdim"])
        return PagedKV(int(params["kv_heads"]), dk, int(params.get("window", 0)), 0 if dv == dk else dv)

    def _on_tcgen05(self, segment_counts, page_size=None) -> bool:
        """Long prompt portions of the sigmoid-weighted form without a window run on the tcgen05 kernel."""
        if not self.sigmoid or self.window > 0:
            return False
        if not prompt_shape_for_tcgen05(self.ctx.dtype, self.dk, self.dv, segment_counts):
            return False
        return page_size is None or ops.attention_tc_supported(self.dk, self.n_q, self.n_kv, page_size, self.ctx.dtype)

    def launch_signature(self, segment_counts):
        return ("tcgen05",) if self._on_tcgen05(segment_counts) else ()

    def inner(self, proj, offset, step, cache, out, scale):
        pages = cache
        tokens = out.shape[0]
        q = torch.empty((tokens, self.n_q, self.dk), dtype=out.dtype, device=out.device)
        ops.head_norm_rope_kv_write(proj, self.in_bias, self.q_norm, self.k_norm, self.eps, pages.slot_mapping,
                                    step.positions, self.freq, self.rot_factor, q, pages.keys, pages.values, self.n_q,
                                    self.n_kv, self.dk, self.dv, offset=offset)
        attended = torch.empty((tokens, self.n_q, self.dv), dtype=out.dtype, device=out.device)
        if (not step.decode_only and step.segments
                and self._on_tcgen05([segment.count for segment in step.segments], pages.keys.shape[2])):
            ops.attention_sigmoid_tc(q, pages.keys, pages.values, attended, pages.block_tables, step.segment_start,
                                     step.segment_first_position, self.scale, self.head_bias, self.softcap)
        else:
            ops.attention_scored(q, pages.keys, pages.values, attended, pages.block_tables, step.segment_of_token,
                                 step.positions, self.scale, segment_start=step.segment_start,
                                 segment_first_position=step.segment_first_position, window=self.window, cap=self.softcap,
                                 head_bias=self.head_bias)
        ops.head_gate_scale(attended, None, out, scale, step.segment_of_token)


_SSD_NAMES = {"in": "in", "conv": "conv", "conv_bias": "conv.b", "dt_bias": "dt_bias", "a_log": "A_log", "skip": "D",
              "norm": "norm", "out": "o"}


@register_mixer("grouped_state_space")
class GroupedStateSpace(BranchMixer):
    """params: ``heads``, ``vdim`` (channels of a head; inner = heads * vdim), ``state`` (N, rows of a head's state),
    ``groups`` (head h reads the B and C of group h // (heads / groups)), ``conv`` (taps), ``norm_groups`` (equal parts of
    the inner width that the output norm takes one by one), ``eps``, ``tensor_names``.

    A state-space scan with one decay per head and token (the duality form).  W_in x = [z (inner) | u (inner) | B (groups *
    N) | C (groups * N) | dt (heads)]; [u | B | C] pass a short causal convolution per channel (with bias) and SiLU;
    dt <- softplus(dt + dt_bias) without a clamp; per head
        S <- exp(-exp(A_log_h) dt) S + dt B u^T      (S is [N, vdim]),        y = S^T C + D_h u;
    the output is W_out (rmsnorm_in_parts(y * silu(z)) * w): the gate comes before the norm.  Kept per request, in
    float32: S [heads, N, vdim] and the last ``conv - 1`` rows of [u | B | C] before the convolution.  Step sizes, decays
    and the state are float32.  The scan is the engine's matrix-memory scan with a keep and a take factor per token and
    head, its keys and queries shared by the heads of a group."""

    graph_safe = True

    def __init__(self, params, weights, ctx) -> None:
        super().__init__(params, weights, ctx)
        p = params
        self.heads, self.vdim, self.states, self.groups = int(p["heads"]), int(p["vdim"]), int(p["state"]), int(p["groups"])
        self.taps, self.norm_groups, self.eps = int(p["conv"]), int(p.get("norm_groups", 1)), float(p["eps"])
        self.inner_width = self.heads * self.vdim
        self.channels = self.inner_width + 2 * self.groups * self.states
        if self.heads % self.groups or self.inner_width % self.norm_groups:
            raise ops.KernelError(f"state space: {self.heads} heads, {self.groups} groups, {self.norm_groups} norm parts")
        names = {**_SSD_NAMES, **p.get("tensor_names", {})}
        self.in_weight = weights[names["in"]].contiguous()
        self.conv_weight = weights[names["conv"]].to(torch.float32).contiguous()
        self.conv_bias = weights[names["conv_bias"]].to(torch.float32).contiguous()
        self.dt_bias = weights[names["dt_bias"]].to(torch.float32).contiguous()
        self.a_log = weights[names["a_log"]].to(torch.float32).contiguous()
        self.skip = weights[names["skip"]].to(torch.float32).contiguous()
        self.norm_weight = weights[names["norm"]].to(torch.float32).contiguous()
        self.out_weight = weights[names["out"]].contiguous()

    @classmethod
    def expected_tensors(cls, params, hidden_size):
        p = params
        heads, vdim, states, groups, taps = int(p["heads"]), int(p["vdim"]), int(p["state"]), int(p["groups"]), int(p["conv"])
        inner, channels = heads * vdim, heads * vdim + 2 * groups * states
        names = {**_SSD_NAMES, **p.get("tensor_names", {})}
        return {names["in"]: TensorSpec((inner + channels + heads, hidden_size)),
                names["conv"]: TensorSpec((channels, taps), "filter"), names["conv_bias"]: TensorSpec((channels,), "bias"),
                names["dt_bias"]: TensorSpec((heads,), "bias"), names["a_log"]: TensorSpec((heads,), "bias"),
                names["skip"]: TensorSpec((heads,), "norm"), names["norm"]: TensorSpec((inner,), "norm"),
                names["out"]: TensorSpec((hidden_size, inner))}

    @classmethod
    def cache_requirement(cls, params, hidden_size):
        heads, vdim, states, groups, taps = (int(params[key]) for key in ("heads", "vdim", "state", "groups", "conv"))
        channels = heads * vdim + 2 * groups * states
        return (RequestState((heads, states, vdim), "float32"), RequestState((max(taps - 1, 0), channels), "float32"))

    def inner(self, proj, offset, step, cache, out, scale):
        state, window = cache.parts[0].state, cache.parts[1].state
        tokens = out.shape[0]
        inner = self.inner_width
        u = torch.empty((tokens, self.channels), dtype=out.dtype, device=out.device)
        ops.short_conv_act(proj, offset + inner, self.conv_weight, self.conv_bias, window, step, u, "silu")
        if self.taps > 1:
            ops.short_conv_state(proj, offset + inner, self.channels, self.taps, window, step)
        keep, take = ops.ssd_gates(proj, offset + inner + self.channels, self.dt_bias, self.a_log)
        read = torch.empty((tokens, inner), dtype=torch.float32, device=out.device)
        b_off = inner
        c_off = inner + self.groups * self.states
        ops.token_decay_scan(u, c_off, b_off, 0, keep, take, 1.0, state, step.segment_start, step.segment_state_slot,
                             read, self.heads, self.states, self.vdim, qk_share=self.heads // self.groups)
        ops.gated_group_rmsnorm(read, proj, offset, self.norm_weight, self.eps, out, self.norm_groups, gate_first=True,
                                gate_activation="silu", scale=scale, skip=self.skip, skip_source=u, skip_offset=0,
                                segment_of_token=step.segment_of_token)


@register_mixer("parallel_mixers")
class ParallelMixers(Mixer):
    """params: ``branches``: a list of {"kind" (a registered mixer of the ``BranchMixer`` form), "params", "prefix" (of
    its tensors after this part's), "scale"}; ``float32_output`` (the output product leaves float32 sums whatever the
    compute dtype: for layers that add this output to another branch's before the residual takes it).

    y = sum_b scale_b * branch_b(x): every branch reads the same x.  The branches' input matrices are stacked into
    one product and their output matrices laid side by side, each branch writing scale_b times its activations into
    its columns of one tensor, so that the weighted sum is the one output product.  Each branch keeps what it
    keeps alone; this part's requirement is the branches' needs in a row."""

    graph_safe = True

    def __init__(self, params, weights, ctx) -> None:
        super().__init__(params, weights, ctx)
        self.branches, self.scales, self.needs = [], [], []
        self.float32_output = bool(params.get("float32_output", False))
        for branch in params["branches"]:
            cls = MIXERS.get(branch["kind"])
            if not issubclass(cls, BranchMixer):
                raise ops.KernelError(f"parallel mixers: {branch['kind']!r} cannot share its products with a sibling")
            prefix = branch["prefix"]
            local = {name[len(prefix):]: tensor for name, tensor in weights.items() if name.startswith(prefix)}
            self.branches.append(cls(branch["params"], local, ctx))
            self.scales.append(float(branch.get("scale", 1.0)))
            self.needs.append(len(cache_needs(cls.cache_requirement(branch["params"], ctx.hidden_size))))
        if not all(branch.graph_safe for branch in self.branches):
            self.graph_safe = False
        self.in_weight = torch.cat([branch.in_weight for branch in self.branches], dim=0).contiguous()
        pad = -self.in_weight.shape[0] % 16
        if pad:
            self.in_weight = torch.cat([self.in_weight, self.in_weight.new_zeros((pad, self.in_weight.shape[1]))]).contiguous()
        self.out_weight = torch.cat([branch.out_weight for branch in self.branches], dim=1).contiguous()
        self.in_offsets, self.mid_offsets = [0], [0]
        for branch in self.branches:
            self.in_offsets.append(self.in_offsets[-1] + branch.in_weight.shape[0])
            self.mid_offsets.append(self.mid_offsets[-1] + branch.out_weight.shape[1])
            branch.in_weight = branch.out_weight = None      # held once, stacked

    @classmethod
    def expected_tensors(cls, params, hidden_size):
        out = {}
        for branch in params["branches"]:
            declared = MIXERS.get(branch["kind"]).expected_tensors(branch["params"], hidden_size)
            out.update({branch["prefix"] + local: tensor for local, tensor in declared.items()})
        return out

    @classmethod
    def cache_requirement(cls, params, hidden_size):
        needs = ()
        for branch in params["branches"]:
            needs += cache_needs(MIXERS.get(branch["kind"]).cache_requirement(branch["params"], hidden_size))
        return needs or None

    def launch_signature(self, segment_counts):
        return tuple(answer for branch in self.branches for answer in branch.launch_signature(segment_counts))

    def forward(self, x, step, cache):
        proj = input_projection(x, self.in_weight)
        mid = torch.empty((x.shape[0], self.mid_offsets[-1]), dtype=x.dtype, device=x.device)
        first = 0
        for index, branch in enumerate(self.branches):
            view = mid[:, self.mid_offsets[index]:self.mid_offsets[index + 1]]
            branch.inner(proj, self.in_offsets[index], step, cache_for(cache, self.needs[index], first), view,
                         self.scales[index])
            first += self.needs[index]
        return linear_sums(mid, self.out_weight) if self.float32_output else linear_partials(mid, self.out_weight)
