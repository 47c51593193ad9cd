"""Typed ``config.json`` of the Tufevik design.

Tufevik is a decoder that lists its layers one by one.  Every layer norms before and after each of its two branches
(x <- x + after(branch(before(x)))) with a tanh norm, tanh(alpha x) * w + b, that takes no statistics.  A layer's token
mixer is ``mlstm`` (a matrix memory with exponential gates and a running maximum, kept per request) or ``parallel``
(the weighted sum of ``left``, a grouped-query attention whose q, k and v pass short causal convolutions, with one
norm over all of q and one over all of k, partly rotated heads with stretched frequencies and a gate per head, and
``right``, a selective state-space scan); its feed-forward is dense (relu-gated), a mixture of experts whose weights
are the softmax over the chosen logits, or absent.  The output head is the embedding table.

Keys: ``architecture`` ("Tufevik"), ``vocab``, ``width``, ``embedding.scale``, ``norm.eps``, ``layers`` (a list of
``{"type", "mixer", "mlp"}``; mlstm mixer: ``heads``, ``dim``, ``vdim``, ``gate_cap``; parallel mixer: ``left {heads,
kv_heads, dim, vdim, conv, scale, rot {base, dims, scaling {factor, original, fast, slow}}}``, ``right {inner, state,
dt_rank, conv}``, ``left_scale``, ``right_scale``; mlp: ``kind`` "dense" with ``ff``, or "moe" with ``router {experts,
top}`` and ``expert {ff}``, or null).  ``max_position_embeddings`` is this engine's own optional key (the design has no
limit of its own; the cache manager wants one for its tables).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from .model_config import ConfigError

MIXER_TYPES = ("mlstm", "parallel")
_MIXER_KEYS = {
    "mlstm": ("heads", "dim", "vdim", "gate_cap"),
    "parallel": ("left", "right", "left_scale", "right_scale"),
}
_LEFT_KEYS = ("heads", "kv_heads", "dim", "vdim", "conv", "scale", "rot")
_RIGHT_KEYS = ("inner", "state", "dt_rank", "conv")


@dataclass(frozen=True)
class TufevikConfig:
    vocab: int
    width: int
    layers: tuple
    norm_eps: float
    embedding_scale: float = 1.0
    max_position_embeddings: int = 131_072

    def __post_init__(self) -> None:
        if self.vocab <= 0 or self.width <= 0 or not self.layers:
            raise ConfigError("vocab, width and the number of layers must be positive")
        if not self.norm_eps > 0:
            raise ConfigError("norm.eps must be positive")
        for index, layer in enumerate(self.layers):
            kind = layer.get("type")
            if kind not in MIXER_TYPES:
                raise ConfigError(f"layer {index}: unknown type {kind!r}; known: {list(MIXER_TYPES)}")
            mixer = layer.get("mixer") or {}
            missing = [key for key in _MIXER_KEYS[kind] if key not in mixer]
            if missing:
                raise ConfigError(f"layer {index} ({kind}): mixer lacks {missing}")
            if kind == "mlstm":
                if not float(mixer["gate_cap"]) > 0:
                    raise ConfigError(f"layer {index}: gate_cap must be positive")
            else:
                left, right = mixer["left"], mixer["right"]
                missing = [f"left.{key}" for key in _LEFT_KEYS if key not in left]
                missing += [f"right.{key}" for key in _RIGHT_KEYS if key not in right]
                if missing:
                    raise ConfigError(f"layer {index} (parallel): mixer lacks {missing}")
                if int(left["heads"]) % int(left["kv_heads"]):
                    raise ConfigError(f"layer {index}: left.heads must be a multiple of left.kv_heads")
                rot = left["rot"]
                if int(rot["dims"]) % 2 or int(rot["dims"]) > int(left["dim"]):
                    raise ConfigError(f"layer {index}: rot.dims must be even and at most left.dim")
                if int(left["conv"]) < 1 or int(right["conv"]) < 1:
                    raise ConfigError(f"layer {index}: a convolution has at least one tap")
            mlp = layer.get("mlp")
            if mlp is not None:
                if mlp.get("kind") == "dense":
                    if int(mlp.get("ff", 0)) <= 0:
                        raise ConfigError(f"layer {index}: a dense feed-forward needs ff")
                elif mlp.get("kind") == "moe":
                    router = mlp.get("router") or {}
                    if "experts" not in router or "top" not in router or "ff" not in (mlp.get("expert") or {}):
                        raise ConfigError(f"layer {index}: the mixture lacks router.experts, router.top or expert.ff")
                    if not 0 < int(router["top"]) <= int(router["experts"]):
                        raise ConfigError(f"layer {index}: router.top must lie in 1 .. experts")
                else:
                    raise ConfigError(f"layer {index}: mlp.kind must be 'dense' or 'moe', got {mlp.get('kind')!r}")

    @classmethod
    def from_dict(cls, values: dict[str, Any]) -> "TufevikConfig":
        missing = [key for key in ("vocab", "width", "layers", "norm") if key not in values]
        if missing:
            raise ConfigError(f"config.json lacks required keys: {missing}")
        if "eps" not in values["norm"]:
            raise ConfigError("config.json lacks norm.eps")
        return cls(vocab=int(values["vocab"]), width=int(values["width"]), layers=tuple(values["layers"]),
                   norm_eps=float(values["norm"]["eps"]),
                   embedding_scale=float((values.get("embedding") or {}).get("scale", 1.0)),
                   max_position_embeddings=int(values.get("max_position_embeddings", 131_072)))
