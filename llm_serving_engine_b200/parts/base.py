"""Interfaces of the parts a decoder layer is put together from, and their registries.

A part is built from ``params`` (its sizes and constants, taken from the
configuration), ``weights`` (its own tensors, by their local names) and a
``BuildContext``.  No part knows which model it is in.

* ``Norm``:            ``forward(stream, rows=None) -> x``  (adds the pending branch
                       output to the float32 residual, returns the normalised rows)
* ``PositionEncoding``: ``encode_and_store(...)`` (rotates queries and keys and
                       writes keys and values into the layer's cache pages)
* ``Mixer``:           ``forward(x, step, cache) -> y`` over the step's flat rows
                       (y is [T, H], or a float32 stack of partial sums [P, T, H]
                       that the next norm adds up; ``reduce_partials`` gives [T, H]),
                       reading and writing its layer's cache; ``cache_requirement``
                       says what it needs (pages of keys and values, or a
                       fixed-size state per request, or nothing, or a tuple of
                       several such needs: pages and a state, two states)
* ``FeedForward``:     ``forward(x) -> y``, row-local
* ``Block``:           the arrangement of the four in a layer:
                       ``forward(stream, step, cache)``

Each class also has ``expected_tensors(params, hidden_size)``: local tensor name
-> ``TensorSpec``; the loader and the random-weights mode are driven by it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

import torch

from ..weights.tensor_spec import TensorSpec


@dataclass(frozen=True)
class BuildContext:
    dtype: torch.dtype            # compute dtype: torch.bfloat16 or torch.float32
    device: torch.device
    hidden_size: int
    layer_index: int
    max_position_embeddings: int


@dataclass(frozen=True)
class PagedKV:
    """The mixer keeps keys and values of every token in pages.  ``window`` > 0:
    only the last ``window`` keys are read, older pages are given back.
    ``value_dim`` > 0: a value has this size instead of ``head_dim`` (keys and values then lie in two tensors)."""

    num_kv_heads: int
    head_dim: int
    window: int = 0
    value_dim: int = 0


@dataclass(frozen=True)
class PagedLatent:
    """The mixer keeps one row of ``width`` values per token in pages (a latent from which keys and
    values of all heads are made, and whatever else of a key is shared by the heads).  ``window`` as
    for ``PagedKV``."""

    width: int
    window: int = 0


@dataclass(frozen=True)
class RequestState:
    """The mixer keeps a state of fixed size per request: a tensor of ``shape``
    and ``dtype`` ("float32" or "bfloat16"), zeroed when the request is created."""

    shape: tuple[int, ...]
    dtype: str = "float32"


class ResidualStream:
    """The hidden state between parts: the float32 residual [T, H] and the output
    of the last branch, not yet added (the next norm adds it in float32).

    A model may keep the residual in ``copies`` copies side by side ([T, copies * H]) and scale what a
    branch adds: ``delta_mult`` (a constant) and ``delta_scale`` (float32 [H], or None) multiply the
    pending output; ``mix`` (float32 [copies, copies], indexed [from, to], or None for the identity) and
    ``write`` (float32 [copies], or None for ones) say how the copies are mixed and how much of the
    output each receives when it is added; ``read`` (float32 [copies], or None for ones) are the
    weights with which the next branch reads the copies.  The norm that adds the pending output
    applies all of it (``Norm.forward``)."""

    __slots__ = ("residual", "delta", "copies", "delta_mult", "delta_scale", "mix", "write", "read", "hidden",
                 "delta_bias", "delta_row_scale", "delta_norm")

    def __init__(self, residual: torch.Tensor, delta: torch.Tensor | None = None, copies: int = 1) -> None:
        self.residual = residual
        self.delta = delta
        self.copies = copies
        self.delta_mult = 1.0
        self.delta_scale = None
        self.mix = None
        self.write = None
        self.read = None
        # For models that normalise AFTER the sum (the residual itself is what the branches read): the residual in
        # the compute dtype, kept up to date by the embedding and by every norm (the residual tensor itself in
        # float32), and a bias (float32 [H]) that belongs to the pending output.
        self.hidden = None
        self.delta_bias = None
        self.delta_row_scale = None   # float32 [T] c: c_t times the branch's input row belongs to the pending output too
        self.delta_norm = None        # a Norm that the pending output passes before it is added (a layer that norms after a branch too)

    @property
    def plain(self) -> bool:
        """One copy, and the pending output is added as it is."""
        return (self.copies == 1 and self.delta_mult == 1.0 and self.delta_scale is None and self.mix is None
                and self.write is None and self.read is None)


class Part:
    # True when the part only launches work whose shape depends on the number of rows and reads
    # everything else (positions, segments, tables, routing decisions) from device memory, without
    # waiting for the device: a step made of such parts can be captured in a CUDA graph and
    # replayed with other contents.  A model is captured only if every part of it says so.
    graph_safe = False

    def __init__(self, params: dict[str, Any], weights: dict[str, torch.Tensor], ctx: BuildContext) -> None:
        self.params = params
        self.ctx = ctx

    @classmethod
    def expected_tensors(cls, params: dict[str, Any], hidden_size: int) -> dict[str, TensorSpec]:
        return {}


class Norm(Part):
    def forward(self, stream: ResidualStream, rows: torch.Tensor | None = None) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    def encode_and_store(self, qkv, bias, step, cache, q_out, n_q, n_kv, head_dim) -> None:
        raise NotImplementedError


class Mixer(Part):
    output_bias = None     # float32 [H]: a bias of the output projection, left to the norm that adds the output

    @classmethod
    def cache_requirement(cls, params: dict[str, Any], hidden_size: int):
        """``PagedKV``, ``PagedLatent``, ``RequestState`` or ``None``; or a tuple of these, when the mixer keeps several
        things (pages and a state, two states of different shapes): ``forward`` then finds them, in the tuple's
        order, in ``cache.parts``."""
        return None

    def forward(self, x: torch.Tensor, step, cache) -> torch.Tensor:
        raise NotImplementedError

    def launch_signature(self, segment_counts: list[int]) -> tuple:
        """What of a step's shape, beyond its numbers of rows and requests, decides which kernels ``forward``
        launches (``segment_counts``: tokens of each request in the step).  Steps with different signatures
        are captured in CUDA graphs of their own; ``forward`` must choose by the same rule."""
        return ()


def cache_needs(requirement) -> tuple:
    """A mixer's cache requirement as a tuple of single needs (empty for none)."""
    if requirement is None:
        return ()
    return tuple(requirement) if isinstance(requirement, tuple) else (requirement,)


def cache_for(cache, needs: int, first: int = 0):
    """What a mixer with ``needs`` single needs gets when its needs are members ``first`` .. of a larger tuple (a mixer
    built from several): the member itself for one need, a view whose ``parts`` are the members for several, None for
    none."""
    if needs == 0:
        return None
    members = cache.parts[first:first + needs]
    if needs == 1:
        return members[0]
    view = type(cache)()
    view.parts = members
    return view


class FeedForward(Part):
    row_scale = None       # set by forward: float32 [T] c, when c_t x_t is part of the output and left to the next norm

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class Block:
    graph_safe = False     # as for ``Part``: the arrangement itself launches nothing that depends on the step's contents

    def __init__(self, params, mixer_norm: Norm, mixer: Mixer, feed_forward_norm: Norm | None,
                 feed_forward: FeedForward | None, weights: dict | None = None, ctx: BuildContext | None = None) -> None:
        self.params = params
        self.mixer_norm, self.mixer = mixer_norm, mixer
        self.feed_forward_norm, self.feed_forward = feed_forward_norm, feed_forward   # both None: a layer without one

    @classmethod
    def expected_tensors(cls, params: dict[str, Any], hidden_size: int) -> dict[str, TensorSpec]:
        """Tensors of the arrangement itself (scales, mixing weights), by their names after the layer's prefix."""
        return {}

    def parts(self) -> list:
        """Every part this block runs (a mixer's position encoding included)."""
        found = [part for part in (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward)
                 if part is not None]
        position = getattr(self.mixer, "position", None)
        if position is not None:
            found.append(position)
        return found

    def forward(self, stream: ResidualStream, step, cache) -> None:
        raise NotImplementedError


@dataclass
class _Registry:
    what: str
    entries: dict[str, type] = field(default_factory=dict)

    def register(self, name: str, cls: type | None = None):
        if cls is None:
            def decorator(inner: type) -> type:
                self.entries[name] = inner
                return inner
            return decorator
        self.entries[name] = cls
        return cls

    def get(self, name: str) -> type:
        try:
            return self.entries[name]
        except KeyError:
            raise KeyError(f"unknown {self.what} {name!r}; registered: {sorted(self.entries)}") from None


MIXERS = _Registry("mixer")
FEED_FORWARDS = _Registry("feed-forward")
NORMS = _Registry("norm")
POSITION_ENCODINGS = _Registry("position encoding")
BLOCKS = _Registry("block")

register_mixer = MIXERS.register
register_feed_forward = FEED_FORWARDS.register
register_norm = NORMS.register
register_position_encoding = POSITION_ENCODINGS.register
register_block = BLOCKS.register
