"""The Tufevik design as a ``ModelSpec`` (``config/tufevik_config.py`` describes the design and its keys).

Tensor names: ``embed`` (also the output head), ``final.norm``; for layer i ``l<i>.norm1``, ``l<i>.norm1b`` (before and
after the mixer), ``l<i>.norm2``, ``l<i>.norm2b`` (around the feed-forward), each with ``.b`` and ``.alpha``;
``l<i>.mix.*`` (mlstm: ``q k v g o norm i i.b f f.b``; parallel: ``left.{q k v g o q.norm k.norm q.conv k.conv v.conv}``
and ``right.{in conv conv.b x dt dt.b A_log D o}``) and ``l<i>.mlp.*`` (dense: ``gate up down``; mixture: ``router
router.b e<j>.{gate,up,down}``).  Every mechanism is a registered part with its constants as parameters:
``sandwich_residual`` (block), ``dynamic_tanh`` (every norm), ``mlstm``, ``parallel_mixers`` over
``conv_rotary_attention`` and ``selective_state_space``, ``gated_mlp`` with relu, ``routed_experts``; the embedding's
constant is a field of the ``ModelSpec``.
"""
from __future__ import annotations

from ..config.model_config import LayerSpec, ModelSpec, PartSpec
from ..config.registry import register_architecture
from ..config.tufevik_config import TufevikConfig

_NORM_PARAMS = {"weight_name": ""}     # the norms' tensors are named without a suffix: the part's prefix is the whole name


def _mixer_spec(kind: str, mixer: dict, eps: float) -> PartSpec:
    if kind == "mlstm":
        return PartSpec("mlstm", {"heads": int(mixer["heads"]), "dim": int(mixer["dim"]), "vdim": int(mixer["vdim"]),
                                  "gate_cap": float(mixer["gate_cap"]), "eps": eps})
    left, right = mixer["left"], mixer["right"]
    attention = {"heads": int(left["heads"]), "kv_heads": int(left["kv_heads"]), "dim": int(left["dim"]),
                 "vdim": int(left["vdim"]), "conv": int(left["conv"]), "scale": float(left["scale"]), "eps": eps,
                 "rot": left["rot"], "gate": True}
    scan = {"inner": int(right["inner"]), "state": int(right["state"]), "dt_rank": int(right["dt_rank"]),
            "conv": int(right["conv"])}
    return PartSpec("parallel_mixers", {"branches": [
        {"kind": "conv_rotary_attention", "params": attention, "prefix": "left.", "scale": float(mixer["left_scale"])},
        {"kind": "selective_state_space", "params": scan, "prefix": "right.", "scale": float(mixer["right_scale"])}]})


def _feed_forward_spec(mlp: dict) -> PartSpec:
    if mlp["kind"] == "dense":
        return PartSpec("gated_mlp", {"intermediate_size": int(mlp["ff"]), "activation": "relu",
                                      "tensor_names": {"gate": "gate", "up": "up", "down": "down"}})
    return PartSpec("routed_experts", {
        "experts": int(mlp["router"]["experts"]), "top": int(mlp["router"]["top"]), "ff": int(mlp["expert"]["ff"]),
        "correction": False, "router_bias": True, "weights": "softmax_chosen", "activation": "silu", "shared": None})


def build_tufevik_spec(config: TufevikConfig) -> ModelSpec:
    norm = PartSpec("dynamic_tanh", dict(_NORM_PARAMS))
    layers = []
    for index, entry in enumerate(config.layers):
        mlp = entry.get("mlp")
        block = PartSpec("sandwich_residual", {
            "tensor_prefixes": {"mixer_norm": "norm1", "mixer": "mix.", "feed_forward_norm": "norm2", "feed_forward": "mlp."},
            "after_norm": {"kind": "dynamic_tanh", "params": dict(_NORM_PARAMS)},
            "after_prefixes": {"mixer": "norm1b", "feed_forward": "norm2b"}, "feed_forward": mlp is not None})
        layers.append(LayerSpec(
            prefix=f"l{index}.", block=block, mixer=_mixer_spec(entry["type"], entry["mixer"], config.norm_eps),
            feed_forward=None if mlp is None else _feed_forward_spec(mlp),
            mixer_norm=norm, feed_forward_norm=None if mlp is None else norm))
    return ModelSpec(
        architecture="Tufevik", vocab_size=config.vocab, hidden_size=config.width, layers=tuple(layers),
        order=tuple(range(len(layers))), final_norm=norm, embedding_name="embed", final_norm_prefix="final.norm",
        lm_head_name="head", tie_word_embeddings=True, max_position_embeddings=config.max_position_embeddings,
        embedding_scale=config.embedding_scale)


register_architecture("Tufevik", TufevikConfig, build_tufevik_spec, model_types=("tufevik",))
