"""The Sebudra design as a ``ModelSpec`` (``config/sebudra_config.py`` describes the design and its keys).

Tensor names: ``embed``, ``head``, ``final.norm``; for layer i ``l<i>.norm1``; ``l<i>.mix.*`` (parallel: ``left.{q k v o
q.b k.b v.b q.norm k.norm}`` and ``right.{in conv conv.b dt_bias A_log D norm o}``; attention: ``q k v o q.norm k.norm
pb``; gla: ``q k v g o norm a1 a2 a2.b``) and ``l<i>.mlp.*`` (dense: ``gate up down``; mixture: ``router correction
e<j>.{up,down} shared.{up,down,sg}``).  A layer with ``weights_of`` has no tensors: it is the named layer run once more
(``ModelSpec.order`` names that layer again; every run has a cache of its own).  Every mechanism is a registered part
with its constants as parameters: ``parallel_residual`` (block), ``rmsnorm``, ``parallel_mixers`` over
``head_norm_rotary_attention`` and ``grouped_state_space``, ``head_norm_rotary_attention`` alone with sigmoid weights,
``channel_decay_linear_attention``, ``gated_mlp`` with the clamped swish, ``routed_experts`` with sigmoid scores; the
embedding's constant is a field of the ``ModelSpec``.
"""
from __future__ import annotations

from ..config.model_config import LayerSpec, ModelSpec, PartSpec
from ..config.registry import register_architecture
from ..config.sebudra_config import SebudraConfig


def _attention_params(mixer: dict, eps: float, **more) -> dict:
    return {"heads": int(mixer["heads"]), "kv_heads": int(mixer["kv_heads"]), "dim": int(mixer["dim"]),
            "vdim": int(mixer["vdim"]), "scale": float(mixer["scale"]), "eps": eps, "rot": mixer.get("rot"), **more}


def _mixer_spec(kind: str, mixer: dict, eps: float) -> PartSpec:
    if kind == "attention":
        return PartSpec("head_norm_rotary_attention", _attention_params(
            mixer, eps, bias=False, weights="sigmoid", softcap=float(mixer.get("softcap", 0.0)),
            window=int((mixer.get("mask") or {}).get("size", 0))))
    if kind == "gla":
        return PartSpec("channel_decay_linear_attention", {
            "heads": int(mixer["heads"]), "dim": int(mixer["dim"]), "vdim": int(mixer["vdim"]), "tau": float(mixer["tau"]),
            "rank": int(mixer["rank"]), "eps": eps})
    left, right = mixer["left"], mixer["right"]
    attention = _attention_params(left, eps, bias=True, weights="softmax", softcap=float(left.get("softcap", 0.0)),
                                  window=int((left.get("mask") or {}).get("size", 0)))
    scan = {"heads": int(right["heads"]), "vdim": int(right["vdim"]), "state": int(right["state"]),
            "groups": int(right["groups"]), "conv": int(right["conv"]), "norm_groups": int(right.get("norm_groups", 1)),
            "eps": eps}
    return PartSpec("parallel_mixers", {"float32_output": True, "branches": [
        {"kind": "head_norm_rotary_attention", "params": attention, "prefix": "left.", "scale": float(mixer["left_scale"])},
        {"kind": "grouped_state_space", "params": scan, "prefix": "right.", "scale": float(mixer["right_scale"])}]})


def _feed_forward_spec(mlp: dict) -> PartSpec:
    if mlp["kind"] == "dense":
        return PartSpec("gated_mlp", {"intermediate_size": int(mlp["ff"]), "activation": "clamped_swish",
                                      "limit": float(mlp["limit"]), "float32_output": True,
                                      "tensor_names": {"gate": "gate", "up": "up", "down": "down"}})
    router, shared = mlp["router"], mlp.get("shared")
    return PartSpec("routed_experts", {
        "experts": int(router["experts"]), "top": int(router["top"]), "ff": int(mlp["expert"]["ff"]),
        "correction": True, "scores": "sigmoid", "groups": router.get("groups"),
        "router_scale": float(router.get("scale", 1.0)), "activation": "squared_relu",
        "shared": {"ff": int(shared["ff"])} if shared else None})


def build_sebudra_spec(config: SebudraConfig) -> ModelSpec:
    norm = PartSpec("rmsnorm", {"eps": config.norm_eps, "weight_name": ""})
    layers, place, order = [], {}, []
    for index, entry in enumerate(config.layers):
        source = entry.get("weights_of")
        if source is not None:
            order.append(int(source))      # resolved to the place in ``layers`` below
            continue
        mlp = entry.get("mlp")
        block = PartSpec("parallel_residual", {
            "tensor_prefixes": {"mixer_norm": "norm1", "mixer": "mix.", "feed_forward": "mlp."}})
        place[index] = len(layers)
        order.append(index)
        layers.append(LayerSpec(
            prefix=f"l{index}.", block=block, mixer=_mixer_spec(entry["type"], entry["mixer"], config.norm_eps),
            feed_forward=None if mlp is None else _feed_forward_spec(mlp),
            mixer_norm=norm, feed_forward_norm=None))
    return ModelSpec(
        architecture="Sebudra", vocab_size=config.vocab, hidden_size=config.width, layers=tuple(layers),
        order=tuple(place[index] for index in order), final_norm=norm, embedding_name="embed",
        final_norm_prefix="final.norm", lm_head_name="head", tie_word_embeddings=False,
        max_position_embeddings=config.max_position_embeddings, embedding_scale=config.embedding_scale)


register_architecture("Sebudra", SebudraConfig, build_sebudra_spec, model_types=("sebudra",))
