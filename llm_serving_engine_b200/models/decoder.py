"""The generic decoder: embedding, blocks run in the order the description gives,
final norm and LM head on the wanted rows only.  Built from a ``ModelSpec``; it
does not know which architecture it serves."""
from __future__ import annotations

import torch

from ..config.model_config import LayerSpec, ModelSpec, PartSpec
from ..kernels import ops
from ..parts.base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, BuildContext, ResidualStream)
from ..parts.linear import linear
from ..weights.tensor_spec import TensorSpec

_PART_ROLES = ("mixer_norm", "mixer", "feed_forward_norm", "feed_forward")


def _layer_part_prefixes(layer: LayerSpec) -> dict[str, str]:
    """Full tensor prefix of each part of a layer: the layer's own prefix followed by the part's,
    which the architecture's builder gives in ``block.params["tensor_prefixes"]`` (a role that is
    not named there is called by its role: ``mixer.``, ``feed_forward_norm.`` and so on)."""
    names = dict(layer.block.params.get("tensor_prefixes", {}))
    return {role: layer.prefix + names.get(role, role + ".") for role in _PART_ROLES}


def _layer_parts(layer: LayerSpec) -> list[tuple[str, type, PartSpec] | None]:
    """(tensor prefix, class, description) of the four parts of a layer, in the order a block is built from;
    None for the feed-forward and its norm of a layer that has none, and for a norm that the arrangement does without."""
    prefixes = _layer_part_prefixes(layer)
    found = [
        (prefixes["mixer_norm"], NORMS.get(layer.mixer_norm.kind), layer.mixer_norm),
        (prefixes["mixer"], MIXERS.get(layer.mixer.kind), layer.mixer),
    ]
    if layer.feed_forward is None:
        return found + [None, None]
    norm = layer.feed_forward_norm     # None: an arrangement whose feed-forward reads the mixer's norm
    return found + [
        None if norm is None else (prefixes["feed_forward_norm"], NORMS.get(norm.kind), norm),
        (prefixes["feed_forward"], FEED_FORWARDS.get(layer.feed_forward.kind), layer.feed_forward),
    ]


def _block_tensors(layer: LayerSpec, hidden_size: int) -> dict[str, TensorSpec]:
    """Tensors of the layer's arrangement itself, by their names after the layer's prefix (none for the blocks
    that registered before ``Block.expected_tensors`` existed)."""
    declare = getattr(BLOCKS.get(layer.block.kind), "expected_tensors", None)
    return declare(layer.block.params, hidden_size) if declare else {}


def expected_tensors(spec: ModelSpec) -> dict[str, TensorSpec]:
    """Every tensor the model reads from the checkpoint, by its full name."""
    out: dict[str, TensorSpec] = {spec.embedding_name: TensorSpec((spec.vocab_size, spec.hidden_size))}
    for layer in spec.layers:
        for entry in _layer_parts(layer):
            if entry is None:
                continue
            prefix, cls, part = entry
            for local, tensor in cls.expected_tensors(part.params, spec.hidden_size).items():
                out[prefix + local] = tensor
        for local, tensor in _block_tensors(layer, spec.hidden_size).items():
            out[layer.prefix + local] = tensor
    if spec.position_table_name:
        out[spec.position_table_name] = TensorSpec((spec.max_position_embeddings, spec.hidden_size))
    norm_cls = NORMS.get(spec.final_norm.kind)
    for local, tensor in norm_cls.expected_tensors(spec.final_norm.params, spec.hidden_size).items():
        out[spec.final_norm_prefix + local] = tensor
    if not spec.tie_word_embeddings:
        out[spec.lm_head_name] = TensorSpec((spec.vocab_size, spec.hidden_size))
    return out


def cache_requirements(spec: ModelSpec) -> list:
    """What each entry of ``spec.order`` keeps between steps.

    The list runs along ``order``, not along ``layers``: a layer that is named twice
    runs twice with the same weights, and each run has a cache of its own.  An entry
    is ``PagedKV``, ``RequestState`` or ``None`` (from the mixer), or an int: the
    position in ``order`` whose cache this run reads (``LayerSpec.cache_from`` names a
    layer; its first run is meant, and it must come earlier in the order).
    """
    from ..config.model_config import ConfigError

    first_run: dict[int, int] = {}
    out = []
    for position, index in enumerate(spec.order):
        layer = spec.layers[index]
        if layer.cache_from is not None:
            if layer.cache_from not in first_run:
                raise ConfigError(f"layer {index} reads the cache of layer {layer.cache_from}, which has not run before it")
            out.append(first_run[layer.cache_from])
        else:
            out.append(MIXERS.get(layer.mixer.kind).cache_requirement(layer.mixer.params, spec.hidden_size))
        first_run.setdefault(index, position)
    return out


class DecoderModel:
    def __init__(self, spec: ModelSpec, weights: dict[str, torch.Tensor], dtype: torch.dtype, device) -> None:
        self.spec = spec
        self.dtype = dtype
        self.device = torch.device(device)
        self.embedding = weights[spec.embedding_name].contiguous()
        self.lm_head = self.embedding if spec.tie_word_embeddings else weights[spec.lm_head_name].contiguous()
        self.position_table = weights[spec.position_table_name].contiguous() if spec.position_table_name else None
        self.blocks = []
        for index, layer in enumerate(spec.layers):
            ctx = BuildContext(dtype, self.device, spec.hidden_size, index, spec.max_position_embeddings)
            built = []
            for entry in _layer_parts(layer):
                if entry is None:
                    built.append(None)
                    continue
                prefix, cls, part = entry
                local = {name[len(prefix):]: tensor for name, tensor in weights.items() if name.startswith(prefix)}
                built.append(cls(part.params, local, ctx))
            block_cls = BLOCKS.get(layer.block.kind)
            own = {local: weights[layer.prefix + local] for local in _block_tensors(layer, spec.hidden_size)}
            if own:
                self.blocks.append(block_cls(layer.block.params, *built, weights=own, ctx=ctx))
            else:
                self.blocks.append(block_cls(layer.block.params, *built))
        ctx = BuildContext(dtype, self.device, spec.hidden_size, -1, spec.max_position_embeddings)
        prefix = spec.final_norm_prefix
        local = {name[len(prefix):]: tensor for name, tensor in weights.items() if name.startswith(prefix)}
        self.final_norm = NORMS.get(spec.final_norm.kind)(spec.final_norm.params, local, ctx)
        self.layer_hook = None   # for inspection: called as hook(position in the order, stream) after every layer run

    @property
    def graph_safe(self) -> bool:
        """Whether a step of this model can be captured in a CUDA graph: every block, every part of
        every block (mixer, its position encoding, feed-forward, both norms) and the final norm say so."""
        for block in self.blocks:
            if not getattr(block, "graph_safe", False):
                return False
            if not all(getattr(part, "graph_safe", False) for part in block.parts()):
                return False
        return bool(getattr(self.final_norm, "graph_safe", False))

    def launch_signature(self, segment_counts: list[int]) -> tuple:
        """The mixers' answers to ``Mixer.launch_signature`` for a step of this shape (each distinct answer once)."""
        answers = {block.mixer.launch_signature(segment_counts) for block in self.blocks}
        return tuple(sorted(answer for answer in answers if answer))

    @property
    def vocab_size(self) -> int:
        return self.spec.vocab_size

    def weight_bytes_per_step(self) -> int:
        """Bytes of weights a step reads once: every matrix of every layer run, and
        the LM head (the embedding rows that a step gathers are not counted)."""
        total = self.lm_head.numel() * self.lm_head.element_size()
        for index in self.spec.order:
            block = self.blocks[index]
            for part in (block.mixer, block.feed_forward, block.mixer_norm, block.feed_forward_norm):
                if part is None:
                    continue
                held: dict[int, int] = {}     # a part may keep views of a matrix beside it: every storage counts once
                for value in vars(part).values():
                    if isinstance(value, torch.Tensor) and value.dim() >= 1 and value.is_floating_point():
                        key = value.untyped_storage().data_ptr()
                        held[key] = max(held.get(key, 0), value.numel() * value.element_size())
                total += sum(held.values())
        return total

    def forward(self, step, caches) -> torch.Tensor:
        """Run the step's rows through the layers and return float32 logits
        [number of wanted rows, vocab] (an empty tensor when nothing is wanted)."""
        tokens = step.num_tokens
        copies = self.spec.residual_streams
        residual = torch.empty((tokens, copies * self.spec.hidden_size), dtype=torch.float32, device=self.device)
        if self.position_table is not None:
            if copies != 1:
                raise ops.KernelError("a position table comes with one copy of the residual")
            hidden = residual if self.dtype == torch.float32 else torch.empty_like(residual, dtype=self.dtype)
            ops.embedding_positions(self.embedding, self.position_table, step.token_ids, step.positions,
                                    self.spec.embedding_scale, residual, None if hidden is residual else hidden)
            stream = ResidualStream(residual, copies=copies)
            stream.hidden = hidden
        else:
            # every copy starts as the embedding
            ops.embedding(self.embedding, step.token_ids, residual, copies, scale=self.spec.embedding_scale)
            stream = ResidualStream(residual, copies=copies)
        for position, index in enumerate(self.spec.order):   # caches run along the order
            self.blocks[index].forward(stream, step, caches[position])
            if self.layer_hook is not None:
                self.layer_hook(position, stream)
        if step.num_wanted == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=self.device)
        stream.read = None     # the head reads the sum of the copies
        x = self.final_norm.forward(stream, rows=step.want_rows)
        logits = linear(x, self.lm_head, out_dtype=torch.float32)
        if self.spec.logit_scale != 1.0:
            logits.mul_(self.spec.logit_scale)
        if self.spec.logit_softcap > 0.0:
            ops.softcap(logits, self.spec.logit_softcap)
        return logits
