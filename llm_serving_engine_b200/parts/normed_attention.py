"""Grouped-query attention with normed heads and learned changes to its scores or weights."""
from __future__ import annotations

import os

import torch

from ..kernels import ops
from ..weights.tensor_spec import TensorSpec
from .base import Mixer, PagedKV, register_mixer
from .linear import linear_partials

# Rows of the longest portion from which a step's attention runs on the tcgen05 kernel (tiles of 128 rows of one head),
# when the portions are also long on average; LSE_SCORED_TCGEN05=0 keeps every step on the mma.sync kernel.
TCGEN05_MIN_ROWS = 128
TCGEN05_MIN_ROWS_PER_REQUEST = 64
TCGEN05 = os.environ.get("LSE_SCORED_TCGEN05", "1") != "0"


def prompt_shape_for_tcgen05(dtype, dk: int, dv: int, segment_counts: list[int]) -> bool:
    """Whether a step of these portions, with heads of these sizes, is one for ``ops.attention_scored_tc``: bfloat16, keys
    and values of one size that is 64 or 128, a portion of at least 128 rows, portions long on average (a single token
    would take a tile of 128 rows)."""
    if not TCGEN05 or dtype != torch.bfloat16 or dk != dv or dk not in (64, 128) or not segment_counts:
        return False
    return (max(segment_counts) >= TCGEN05_MIN_ROWS
            and sum(segment_counts) >= TCGEN05_MIN_ROWS_PER_REQUEST * len(segment_counts))

_DEFAULT_NAMES = {"q": "q", "k": "k", "v": "v", "out": "o", "q_norm": "q.norm", "k_norm": "k.norm", "r1": "r1", "r2": "r2",
                  "sink": "sink", "mix": "talk", "gate": "g", "bias_suffix": ".b"}


@register_mixer("normed_attention")
class NormedAttention(Mixer):
    """params: ``heads``, ``kv_heads`` (query head h uses key/value head h // (heads / kv_heads)), ``dim`` (size of a
    head's query and key), ``vdim`` (of its value), ``scale`` (on the scores), ``eps`` (of the head norms), and the
    switches
      ``bias``             q, k, v and the output projection have biases (tensor name + ``bias_suffix``);
      ``distance_penalty`` s_ij -= r1_h ln(1 + r2_h (i - j)), learned numbers per head (``r1``, ``r2``);
      ``sink``             exp(sink_h), a learned number per head, joins the softmax's denominator;
      ``head_mixing``      the heads' softmax weights are mixed, w'_h = sum_g M[h, g] w_g (``mix`` [heads, heads]),
                           before head h applies them to the values of its own key/value head;
      ``gate``             the concatenated heads are multiplied by sigmoid(W_g x) before the output projection;
      ``own_cache``        false: no key/value tensors; the layer reads the pages of another layer
                           (``LayerSpec.cache_from``) with its own queries;
    and ``tensor_names``.  Queries and keys are RMS-normed per head with one weight [dim] shared by the heads; there
    is no rotation: positions enter through the distance penalty or not at all.

    Prompt steps with a portion of 128 rows and more, heads of 64 or 128, run on the tcgen05 kernel
    (``ops.attention_scored_tc``).  Other shapes that the mma.sync kernel takes (bfloat16, keys and values of one size that is 32, 48, 64, 96 or 128) run
    there, prompt portions as tiles of rows and few rows with their keys split into chunks; the rest, and float32, on
    the general kernel.

    One stacked product gives [q | k | v | gate]; one kernel norms the heads, adds the biases and writes keys and
    values into the pages; the attention kernel applies penalty and sink; with mixing it leaves head g's weights
    applied to every key/value head's values in float32, and a small kernel takes the mixed sums and the gate."""

    graph_safe = True

    def __init__(self, params, weights, ctx) -> None:
        super().__init__(params, weights, ctx)
        p = params
        self.n_q, self.n_kv = int(p["heads"]), int(p["kv_heads"])
        self.dk, self.dv = int(p["dim"]), int(p["vdim"])
        self.scale, self.eps = float(p["scale"]), float(p["eps"])
        self.own_cache = bool(p.get("own_cache", True))
        if self.n_q % self.n_kv:
            raise ops.KernelError(f"attention: {self.n_q} query heads do not divide into {self.n_kv} groups")
        names = {**_DEFAULT_NAMES, **p.get("tensor_names", {})}
        suffix = names["bias_suffix"]
        biased = bool(p.get("bias", False))
        stacked, biases = [weights[names["q"]]], [weights[names["q"] + suffix]] if biased else []
        if self.own_cache:
            stacked += [weights[names["k"]], weights[names["v"]]]
            if biased:
                biases += [weights[names["k"] + suffix], weights[names["v"] + suffix]]
        self.gate_offset = -1
        if p.get("gate", False):
            self.gate_offset = sum(w.shape[0] for w in stacked)
            stacked.append(weights[names["gate"]])
        self.in_weight = torch.cat(stacked, dim=0).contiguous()
        self.in_bias = torch.cat([b.float() for b in biases]).contiguous() if biased else None
        self.q_norm = weights[names["q_norm"]].float().contiguous()
        self.k_norm = weights[names["k_norm"]].float().contiguous() if self.own_cache else None
        penalty = bool(p.get("distance_penalty", False))
        self.r1 = weights[names["r1"]].float().contiguous() if penalty else None
        self.r2 = weights[names["r2"]].float().contiguous() if penalty else None
        self.sink = weights[names["sink"]].float().contiguous() if p.get("sink", False) else None
        self.mix = weights[names["mix"]].float().contiguous() if p.get("head_mixing", False) else None
        self.out_weight = weights[names["out"]].contiguous()
        self.output_bias = weights[names["out"] + suffix].float().contiguous() if biased else None

    @classmethod
    def expected_tensors(cls, params, hidden_size):
        p = params
        n_q, n_kv, dk, dv = int(p["heads"]), int(p["kv_heads"]), int(p["dim"]), int(p["vdim"])
        names = {**_DEFAULT_NAMES, **p.get("tensor_names", {})}
        suffix = names["bias_suffix"]
        out = {names["q"]: TensorSpec((n_q * dk, hidden_size)), names["q_norm"]: TensorSpec((dk,), "norm"),
               names["out"]: TensorSpec((hidden_size, n_q * dv))}
        if p.get("own_cache", True):
            out[names["k"]] = TensorSpec((n_kv * dk, hidden_size))
            out[names["v"]] = TensorSpec((n_kv * dv, hidden_size))
            out[names["k_norm"]] = TensorSpec((dk,), "norm")
        if p.get("bias", False):
            for name in ("q", "k", "v", "out") if p.get("own_cache", True) else ("q", "out"):
                out[names[name] + suffix] = TensorSpec((out[names[name]].shape[0],), "bias")
        if p.get("distance_penalty", False):
            out[names["r1"]] = TensorSpec((n_q,), "positive")
            out[names["r2"]] = TensorSpec((n_q,), "positive")
        if p.get("sink", False):
            out[names["sink"]] = TensorSpec((n_q,), "bias")
        if p.get("head_mixing", False):
            out[names["mix"]] = TensorSpec((n_q, n_q), "mixing")
        if p.get("gate", False):
            out[names["gate"]] = TensorSpec((n_q * dv, hidden_size))
        return out

    @classmethod
    def cache_requirement(cls, params, hidden_size):
        dk, dv = int(params["dim"]), int(params["vdim"])
        return PagedKV(int(params["kv_heads"]), dk, 0, 0 if dv == dk else dv)

    def _on_tcgen05(self, segment_counts: list[int], page_size: int | None = None) -> bool:
        """Whether a step of this shape takes the tcgen05 kernel: bfloat16, heads of 64 or 128 (keys and values alike), a
        portion of at least 128 rows, portions long on average (a single token would take a tile of 128 rows)."""
        if not prompt_shape_for_tcgen05(self.ctx.dtype, self.dk, self.dv, segment_counts):
            return False
        if self.mix is not None and self.n_kv > 1 and not ops.head_mix_gate_stages(self.n_q, self.n_kv, self.dv):
            return False
        return page_size is None or ops.attention_tc_supported(self.dk, self.n_q, self.n_kv, page_size, self.ctx.dtype)

    def launch_signature(self, segment_counts):
        return ("tcgen05",) if self._on_tcgen05(segment_counts) else ()

    def forward(self, x, step, cache):
        tokens = x.shape[0]
        proj = linear_partials(x, self.in_weight)
        q = torch.empty((tokens, self.n_q, self.dk), dtype=x.dtype, device=x.device)
        ops.head_norm_kv_write(proj, self.in_bias, self.q_norm, self.k_norm, self.eps, cache.slot_mapping, q,
                               cache.keys, cache.values, self.n_q, self.n_kv if self.own_cache else 0, self.dk, self.dv)
        attended = torch.empty((tokens, self.n_q * self.dv), dtype=x.dtype, device=x.device)
        tcgen05 = (not step.decode_only and step.segments
                   and self._on_tcgen05([segment.count for segment in step.segments], cache.keys.shape[2]))
        if self.mix is None and self.gate_offset < 0:
            if tcgen05:
                ops.attention_scored_tc(q, cache.keys, cache.values, attended.view(tokens, self.n_q, self.dv),
                                        cache.block_tables, step.segment_start, step.segment_first_position, self.scale,
                                        self.r1, self.r2, self.sink)
            else:
                ops.attention_scored(q, cache.keys, cache.values, attended.view(tokens, self.n_q, self.dv), cache.block_tables,
                                     step.segment_of_token, step.positions, self.scale, self.r1, self.r2, self.sink,
                                     segment_start=step.segment_start, segment_first_position=step.segment_first_position)
        else:
            cross = self.mix is not None and self.n_kv > 1
            wide = torch.empty((tokens, self.n_q, self.n_kv if cross else 1, self.dv),
                               dtype=torch.bfloat16 if tcgen05 else torch.float32, device=x.device)
            if tcgen05:
                ops.attention_scored_tc(q, cache.keys, cache.values, wide, cache.block_tables, step.segment_start,
                                        step.segment_first_position, self.scale, self.r1, self.r2, self.sink, cross=cross)
            else:
                ops.attention_scored(q, cache.keys, cache.values, wide, cache.block_tables, step.segment_of_token,
                                     step.positions, self.scale, self.r1, self.r2, self.sink, cross=cross,
                                     segment_start=step.segment_start, segment_first_position=step.segment_first_position)
            gate_bias = None
            if self.gate_offset >= 0 and self.in_bias is not None and self.in_bias.shape[0] > self.gate_offset:
                gate_bias = self.in_bias[self.gate_offset:]
            ops.head_mix_gate(wide, self.mix, proj if self.gate_offset >= 0 else None, max(self.gate_offset, 0), gate_bias,
                              step.segment_of_token, attended, self.n_q, self.n_kv, self.dv)
        return linear_partials(attended, self.out_weight)
