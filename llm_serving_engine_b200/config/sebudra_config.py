"""Typed ``config.json`` of the Sebudra design.

Sebudra is a decoder that lists its layers one by one.  A layer norms once and runs both of its sublayers on that one
normed input: n = rmsnorm(x), x <- x + mixer(n) + feed_forward(n).  A layer's token mixer is ``parallel`` (the weighted
sum of ``left``, a sliding-window softmax attention with biased projections, an RMS norm per head of q and k and a
rotation of the first values of every head with stretched frequencies, and ``right``, a state-space scan with one decay
per head and token, grouped B and C, a gate before a norm taken in parts), ``attention`` (causal, capped scores, every
key weighted by the sigmoid of its score plus a learned number per head, no normalisation over the keys) or ``gla``
(a matrix memory whose rows decay by a learned factor per key channel and token); its feed-forward is dense (clamped,
swish-gated), a mixture of squared-relu experts (sigmoid scores, a correction on the choice only, the choice confined to
the best groups of experts, weights renormalised and scaled, a gated shared expert), or absent.  A layer with
``weights_of: j`` runs with layer j's tensors and a cache of its own.  The output head is a matrix of its own.

Keys: ``architecture`` ("Sebudra"), ``vocab``, ``width``, ``embedding.scale``, ``norm.eps``, ``layers`` (a list of
``{"type", "mixer", "mlp", "weights_of"?}``; parallel mixer: ``left {heads, kv_heads, dim, vdim, scale, mask {size},
rot {base, dims, scaling {factor, original, fast, slow}}}``, ``right {heads, vdim, state, groups, conv, norm_groups}``,
``left_scale``, ``right_scale``; attention mixer: ``heads, kv_heads, dim, vdim, scale, softcap, rot {base, dims}``; gla
mixer: ``heads, dim, vdim, tau``; mlp: ``kind`` "dense" with ``ff`` and ``limit``, or "moe" with ``router {experts, top,
scale, groups {count, keep}}``, ``expert {ff}`` and ``shared {ff}``, or null).  The rank of a gla layer's decay map is the
first dimension of its ``mix.a1`` tensor; without a checkpoint it is read from the mixer's ``rank`` key.
``max_position_embeddings`` is this engine's own optional key (the design has no limit of its own; the cache manager
wants one for its tables).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from .model_config import ConfigError

MIXER_TYPES = ("parallel", "attention", "gla")
_ATTENTION_KEYS = ("heads", "kv_heads", "dim", "vdim", "scale")
_MIXER_KEYS = {
    "parallel": ("left", "right", "left_scale", "right_scale"),
    "attention": _ATTENTION_KEYS,
    "gla": ("heads", "dim", "vdim", "tau"),
}
_RIGHT_KEYS = ("heads", "vdim", "state", "groups", "conv")


def _check_attention(where: str, mixer: dict) -> None:
    missing = [key for key in _ATTENTION_KEYS if key not in mixer]
    if missing:
        raise ConfigError(f"{where}: the attention lacks {missing}")
    if int(mixer["heads"]) % int(mixer["kv_heads"]):
        raise ConfigError(f"{where}: heads must be a multiple of kv_heads")
    rot = mixer.get("rot")
    if rot and (int(rot["dims"]) % 2 or int(rot["dims"]) > int(mixer["dim"])):
        raise ConfigError(f"{where}: rot.dims must be even and at most dim")


@dataclass(frozen=True)
class SebudraConfig:
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
            source = layer.get("weights_of")
            if source is not None:
                if not 0 <= int(source) < len(self.layers) or self.layers[int(source)].get("weights_of") is not None:
                    raise ConfigError(f"layer {index}: weights_of must name a layer that has tensors of its own")
                if self.layers[int(source)].get("type") != kind:
                    raise ConfigError(f"layer {index}: weights_of names a layer of another type")
            mixer = layer.get("mixer") or {}
            missing = [key for key in _MIXER_KEYS[kind] if key not in mixer]
            if missing:
                raise ConfigError(f"layer {index} ({kind}): mixer lacks {missing}")
            if kind == "parallel":
                _check_attention(f"layer {index} (parallel, left)", mixer["left"])
                right = mixer["right"]
                missing = [f"right.{key}" for key in _RIGHT_KEYS if key not in right]
                if missing:
                    raise ConfigError(f"layer {index} (parallel): mixer lacks {missing}")
                if int(right["heads"]) % int(right["groups"]) or int(right["conv"]) < 1:
                    raise ConfigError(f"layer {index}: right.heads must be a multiple of right.groups, right.conv at least 1")
                if (int(right["heads"]) * int(right["vdim"])) % int(right.get("norm_groups", 1)):
                    raise ConfigError(f"layer {index}: right.norm_groups must divide heads * vdim")
            elif kind == "attention":
                _check_attention(f"layer {index} (attention)", mixer)
            elif source is None and int(mixer.get("rank", 0)) <= 0:
                raise ConfigError(f"layer {index} (gla): the decay map's rank is neither in the checkpoint nor in mixer.rank")
            mlp = layer.get("mlp")
            if mlp is not None:
                if mlp.get("kind") == "dense":
                    if int(mlp.get("ff", 0)) <= 0 or not float(mlp.get("limit", 0.0)) > 0:
                        raise ConfigError(f"layer {index}: a dense feed-forward needs ff and a positive limit")
                elif mlp.get("kind") == "moe":
                    router = mlp.get("router") or {}
                    if "experts" not in router or "top" not in router or "ff" not in (mlp.get("expert") or {}):
                        raise ConfigError(f"layer {index}: the mixture lacks router.experts, router.top or expert.ff")
                    if not 0 < int(router["top"]) <= int(router["experts"]):
                        raise ConfigError(f"layer {index}: router.top must lie in 1 .. experts")
                    groups = router.get("groups")
                    if groups:
                        count, keep = int(groups["count"]), int(groups["keep"])
                        if count <= 0 or int(router["experts"]) % count or not 0 < keep <= count:
                            raise ConfigError(f"layer {index}: router.groups must divide the experts, keep in 1 .. count")
                        if keep * (int(router["experts"]) // count) < int(router["top"]):
                            raise ConfigError(f"layer {index}: the kept groups hold fewer experts than router.top")
                else:
                    raise ConfigError(f"layer {index}: mlp.kind must be 'dense' or 'moe', got {mlp.get('kind')!r}")

    @classmethod
    def from_dict(cls, values: dict[str, Any], tensor_shapes: dict | None = None) -> "SebudraConfig":
        missing = [key for key in ("vocab", "width", "layers", "norm") if key not in values]
        if missing:
            raise ConfigError(f"config.json lacks required keys: {missing}")
        if "eps" not in values["norm"]:
            raise ConfigError("config.json lacks norm.eps")
        layers = []
        for index, layer in enumerate(values["layers"]):
            if layer.get("type") == "gla" and layer.get("weights_of") is None and tensor_shapes is not None:
                shape = tensor_shapes.get(f"l{index}.mix.a1")     # a size that only the tensor gives
                if shape is not None:
                    layer = {**layer, "mixer": {**layer["mixer"], "rank": int(shape[0])}}
            layers.append(layer)
        return cls(vocab=int(values["vocab"]), width=int(values["width"]), layers=tuple(layers),
                   norm_eps=float(values["norm"]["eps"]),
                   embedding_scale=float((values.get("embedding") or {}).get("scale", 1.0)),
                   max_position_embeddings=int(values.get("max_position_embeddings", 131_072)))
