"""The arrangement of the parts in a layer."""
from __future__ import annotations

import torch

from ..weights.tensor_spec import TensorSpec
from .base import NORMS, Block, ResidualStream, register_block
from .linear import stack_sums


@register_block("prenorm_residual")
class PreNormResidualBlock(Block):
    """h = h + mixer(norm1(h)); h = h + feed_forward(norm2(h))
    (reference ``src/llmserve/model.py:199-201,233-234``).  Each branch output
    stays pending in the stream; the next norm adds it to the float32 residual."""

    graph_safe = True

    def forward(self, stream: ResidualStream, step, cache) -> None:
        x = self.mixer_norm.forward(stream)
        stream.delta = self.mixer.forward(x, step, cache)
        x = self.feed_forward_norm.forward(stream)
        stream.delta = self.feed_forward.forward(x)


@register_block("residual_streams")
class ResidualStreamsBlock(Block):
    """Pre-norm residual layer whose residual is kept in ``streams`` copies (hyper-connections) and whose branch
    outputs are scaled.

    params: ``streams`` (copies of the residual, the model's), ``residual_mult`` (a constant on every branch output),
    ``layer_scale`` (a learned vector ``ls<q>`` on the output of branch q), ``hyper`` (learned tables ``hc<q>.in``
    [streams], ``hc<q>.out`` [streams], ``hc<q>.mix`` [streams, streams] of branch q), ``feed_forward`` (false: the
    layer has the mixer branch only).  For branch q (1: mixer, 2: feed-forward), over the copies x_1 .. x_S:
        u = sum_s in[s] x_s;  y = branch(norm(u));  x_t <- sum_s mix[s, t] x_s + residual_mult * out[t] * ls * y
    (without ``hyper``: in, out are ones and mix the identity; S = 1 gives x <- x + residual_mult * ls * y).
    The update is left pending in the stream; the next norm's kernel applies it together with its own read."""

    graph_safe = True

    def __init__(self, params, mixer_norm, mixer, feed_forward_norm, feed_forward, weights=None, ctx=None) -> None:
        super().__init__(params, mixer_norm, mixer, feed_forward_norm, feed_forward)
        weights = weights or {}
        self.mult = float(params.get("residual_mult", 1.0))
        self.streams = int(params.get("streams", 1))
        self.tables = {}
        for name in self.expected_tensors(params, 0):
            self.tables[name] = weights[name].to(torch.float32).contiguous()

    @classmethod
    def expected_tensors(cls, params, hidden_size):
        streams = int(params.get("streams", 1))
        out = {}
        for branch in (1, 2) if params.get("feed_forward", True) else (1,):
            if params.get("layer_scale", False):
                out[f"ls{branch}"] = TensorSpec((hidden_size,), "norm")
            if params.get("hyper", False):
                out[f"hc{branch}.in"] = TensorSpec((streams,), "norm")
                out[f"hc{branch}.out"] = TensorSpec((streams,), "norm")
                out[f"hc{branch}.mix"] = TensorSpec((streams, streams), "mixing")
        return out

    def _branch(self, stream: ResidualStream, number: int, norm, run) -> None:
        stream.read = self.tables.get(f"hc{number}.in")
        x = norm.forward(stream)           # applies what the branch before left pending, then reads
        stream.delta = run(x)
        stream.delta_mult = self.mult
        stream.delta_scale = self.tables.get(f"ls{number}")
        stream.mix = self.tables.get(f"hc{number}.mix")
        stream.write = self.tables.get(f"hc{number}.out")

    def forward(self, stream: ResidualStream, step, cache) -> None:
        self._branch(stream, 1, self.mixer_norm, lambda x: self.mixer.forward(x, step, cache))
        if self.feed_forward is not None:
            self._branch(stream, 2, self.feed_forward_norm, self.feed_forward.forward)


@register_block("postnorm_residual")
class PostNormResidualBlock(Block):
    """h = norm1(alpha h + mixer(h)); h = norm2(alpha h + feed_forward(h)): the branches read the residual itself,
    the norm comes after the sum (alpha is the norms' ``residual_mult``).  The residual is kept in float32 and, beside
    it, in the compute dtype as ``stream.hidden``, the branches' input; a layer may have no feed-forward."""

    graph_safe = True

    def forward(self, stream: ResidualStream, step, cache) -> None:
        if stream.hidden is None:    # the model's embedding left float32 rows only
            stream.hidden = (stream.residual if stream.residual.dtype == self.mixer.ctx.dtype
                             else stream.residual.to(self.mixer.ctx.dtype))
        stream.delta = self.mixer.forward(stream.hidden, step, cache)
        stream.delta_bias = self.mixer.output_bias
        x = self.mixer_norm.forward(stream)
        if self.feed_forward is not None:
            stream.delta = self.feed_forward.forward(x)
            stream.delta_row_scale = self.feed_forward.row_scale
            self.feed_forward_norm.forward(stream)


@register_block("sandwich_residual")
class SandwichResidualBlock(Block):
    """h = h + after1(mixer(before1(h))); h = h + after2(feed_forward(before2(h))): a norm before and a norm after every
    branch.  The norms before are the layer's ``mixer_norm`` and ``feed_forward_norm``; the norms after belong to the
    arrangement: params ``after_norm`` ({"kind", "params"}: a registered norm, built once per branch) and
    ``after_prefixes`` ({"mixer": ..., "feed_forward": ...}: their tensors' prefixes after the layer's).  A branch's
    output stays pending in the stream together with its norm (``stream.delta_norm``); the next norm before applies
    both in its one launch.  A layer may have no feed-forward."""

    graph_safe = True

    def __init__(self, params, mixer_norm, mixer, feed_forward_norm, feed_forward, weights=None, ctx=None) -> None:
        super().__init__(params, mixer_norm, mixer, feed_forward_norm, feed_forward)
        weights = weights or {}
        spec, prefixes = params["after_norm"], params["after_prefixes"]
        cls = NORMS.get(spec["kind"])

        def build(prefix: str):
            local = {name[len(prefix):]: tensor for name, tensor in weights.items() if name.startswith(prefix)}
            return cls(spec["params"], local, ctx)

        self.mixer_after = build(prefixes["mixer"])
        self.feed_forward_after = build(prefixes["feed_forward"]) if feed_forward is not None else None

    @classmethod
    def expected_tensors(cls, params, hidden_size):
        spec, prefixes = params["after_norm"], params["after_prefixes"]
        declared = NORMS.get(spec["kind"]).expected_tensors(spec["params"], hidden_size)
        roles = ("mixer", "feed_forward") if params.get("feed_forward", True) else ("mixer",)
        return {prefixes[role] + local: tensor for role in roles for local, tensor in declared.items()}

    def parts(self) -> list:
        return super().parts() + [part for part in (self.mixer_after, self.feed_forward_after) if part is not None]

    def forward(self, stream: ResidualStream, step, cache) -> None:
        x = self.mixer_norm.forward(stream)
        stream.delta = self.mixer.forward(x, step, cache)
        stream.delta_norm = self.mixer_after
        if self.feed_forward is not None:
            x = self.feed_forward_norm.forward(stream)
            stream.delta = self.feed_forward.forward(x)
            stream.delta_norm = self.feed_forward_after


@register_block("parallel_residual")
class ParallelResidualBlock(Block):
    """n = norm(h); h = h + mixer(n) + feed_forward(n): one norm, both sublayers read its output, and the residual takes
    their sum.  The two outputs stay pending in the stream as one float32 stack of sums (each sublayer's partial sums
    one after the other), which the next norm adds up in float32 before the residual is touched.  A layer may have no
    feed-forward; a feed-forward norm is not used."""

    graph_safe = True

    def forward(self, stream: ResidualStream, step, cache) -> None:
        x = self.mixer_norm.forward(stream)
        mixed = self.mixer.forward(x, step, cache)
        if self.feed_forward is None:
            stream.delta = mixed
        else:
            stream.delta = stack_sums(mixed, self.feed_forward.forward(x))
