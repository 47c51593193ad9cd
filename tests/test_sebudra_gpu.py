"""The Sebudra design through the engine against the plain implementation (``tests/plain/sebudra_plain.py``): every mixer
alone and together, layers that run with another layer's tensors, whole prompts, decoding through pages and states,
portions down to two tokens, mixed batches with pages and slots that are used again, other sizes, both precisions,
greedy generation through ``LLMEngine``; and the kernels of its mechanisms alone, with inputs made so that a lost key, a
window that is one token off, a group that should have been shut out or a state that is not carried shows."""
import json
import random
import tempfile
from pathlib import Path
from types import SimpleNamespace

import pytest
import torch

import helpers
from plain import sebudra_plain as plain

pytestmark = pytest.mark.gpu


def moe(experts=6, top=2, ff=40, count=3, keep=2, scale=1.25, shared=48):
    router = {"experts": experts, "top": top, "scale": scale}
    if count:
        router["groups"] = {"count": count, "keep": keep}
    out = {"kind": "moe", "router": router, "expert": {"ff": ff}}
    if shared:
        out["shared"] = {"ff": shared}
    return out


def dense(ff=88, limit=1.75):
    return {"kind": "dense", "ff": ff, "limit": limit}


def side_by_side(heads=4, kv_heads=2, dim=16, vdim=24, window=11, scale=None, rot_dims=8, base=10000.0, factor=3.0,
                 original=64, fast=8.0, slow=1.0, ssm_heads=4, ssm_vdim=12, state=8, groups=2, conv=4, norm_groups=2,
                 left_scale=0.7, right_scale=1.2, mlp="default", **more):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": window},
            "scale": scale if scale is not None else 1.5 / dim ** 0.5,
            "rot": {"base": base, "dims": rot_dims,
                    "scaling": {"factor": factor, "original": original, "fast": fast, "slow": slow}}}
    right = {"heads": ssm_heads, "vdim": ssm_vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}
    return {"type": "parallel", "mlp": dense() if mlp == "default" else mlp,
            "mixer": {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale}, **more}


def sigmoid_attention(heads=4, kv_heads=2, dim=16, vdim=16, scale=None, softcap=5.0, rot_dims=16, base=5000.0, mlp="default",
                      **more):
    return {"type": "attention", "mlp": moe() if mlp == "default" else mlp,
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "softcap": softcap,
                      "scale": scale if scale is not None else 2.0 / dim ** 0.5, "rot": {"base": base, "dims": rot_dims}}, **more}


def memory(heads=3, dim=16, vdim=24, tau=8.0, rank=4, mlp="default", **more):
    return {"type": "gla", "mlp": dense() if mlp == "default" else mlp,
            "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "rank": rank}, **more}


def again(layer: dict, source: int) -> dict:
    """The entry of a layer that runs with layer ``source``'s tensors: the same entry, and ``weights_of``."""
    return {**layer, "weights_of": source}


def model(layers, width=64, vocab=211, embed_scale=3.0, eps=1e-5, positions=2048):
    return {"architecture": "Sebudra", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": eps},
            "embedding": {"scale": embed_scale}, "max_position_embeddings": positions}


_FIRST, _SECOND = side_by_side(), sigmoid_attention()
CONFIGS = {
    "side_by_side_only": model([side_by_side(), side_by_side(heads=6, kv_heads=3, dim=8, vdim=8, window=5, mlp=None, conv=2),
                                side_by_side(heads=2, kv_heads=1, dim=32, vdim=16, rot_dims=32, window=64, mlp=moe())]),
    "sigmoid_only": model([sigmoid_attention(), sigmoid_attention(heads=6, kv_heads=6, dim=8, vdim=24, rot_dims=4, mlp=None),
                           sigmoid_attention(heads=2, kv_heads=1, dim=32, vdim=16, softcap=1.5, mlp=dense())]),
    "memory_only": model([memory(), memory(heads=2, dim=32, vdim=32, mlp=None), memory(heads=4, dim=8, vdim=16, tau=2.0, mlp=moe())]),
    # every kind, and two layers that run a second time with the first run's tensors and a cache of their own
    "all_kinds": model([_FIRST, _SECOND, memory(), again(_FIRST, 0), sigmoid_attention(mlp=dense()), again(_SECOND, 1),
                        memory(heads=2, dim=64, vdim=16, mlp=moe(experts=8, top=3, count=4, keep=2))], width=80),
    # head sizes that the tensor-core kernels take in bfloat16 (the windowed attention and single tokens on mma.sync, long
    # prompt portions of the sigmoid-weighted attention on tcgen05); no router, so that no row of a long bfloat16 run
    # rests on a close call between two experts
    "tensor_core_sizes": model([side_by_side(heads=4, kv_heads=2, dim=64, vdim=64, window=100, rot_dims=32, ssm_heads=4, ssm_vdim=32,
                                             state=64),
                                sigmoid_attention(heads=4, kv_heads=2, dim=64, vdim=64, rot_dims=64, mlp=dense(ff=120)),
                                memory(heads=2, dim=64, vdim=64),
                                sigmoid_attention(heads=2, kv_heads=1, dim=128, vdim=128, rot_dims=64, mlp=dense())], width=128),
    # values that many models make equal or one: one head, one key/value head per query head, a window of one token and
    # a window wider than any prompt, every dimension rotated, a stretch factor of one, branches unscaled, one group and
    # a group per head, one norm part, one tap, one state row, tau one, one expert chosen, groups that shut nothing out,
    # a single group, one expert in all, no shared expert, a cap that caps nothing, an embedding constant of one
    "equal_or_one": model([side_by_side(heads=1, kv_heads=1, dim=32, vdim=32, window=1, scale=1.0, rot_dims=32, factor=1.0,
                                        ssm_heads=1, ssm_vdim=32, state=1, groups=1, conv=1, norm_groups=1, left_scale=1.0,
                                        right_scale=1.0, mlp=moe(experts=4, top=1, count=4, keep=4, scale=1.0, shared=0)),
                           sigmoid_attention(heads=1, kv_heads=1, dim=32, vdim=32, scale=1.0, softcap=1000.0, rot_dims=32,
                                             mlp=moe(experts=1, top=1, count=1, keep=1, ff=64)),
                           memory(heads=1, dim=32, vdim=32, tau=1.0, rank=1, mlp=moe(experts=4, top=2, count=0)),
                           side_by_side(heads=3, kv_heads=3, dim=16, vdim=16, rot_dims=2, window=4096, ssm_heads=3,
                                        ssm_vdim=16, groups=3, norm_groups=3, mlp=None)],
                          width=64, embed_scale=1.0),
    # sizes that no vector load or few-rows product takes; nine query heads on three key/value heads; keys and values of
    # different sizes; more taps than most; a rotated part of a few values; a state of 23 rows; a memory head wider than
    # 32 rows; groups of one expert
    "odd_sizes": model([side_by_side(heads=9, kv_heads=3, dim=20, vdim=12, window=23, rot_dims=6, ssm_heads=6, ssm_vdim=7,
                                     state=23, groups=3, conv=5, norm_groups=3, mlp=moe(experts=7, top=3, ff=18, count=7, keep=4, shared=10)),
                        memory(heads=5, dim=12, vdim=28, rank=3, mlp=None),
                        sigmoid_attention(heads=5, kv_heads=1, dim=12, vdim=28, rot_dims=12, softcap=2.5, mlp=dense(ff=50, limit=0.7)),
                        memory(heads=1, dim=72, vdim=5, tau=3.0, rank=7, mlp=dense(ff=34, limit=1.1)),
                        side_by_side(heads=5, kv_heads=5, dim=12, vdim=28, window=7, rot_dims=12, base=77.0, factor=2.5,
                                     original=40, fast=4.0, slow=0.5, ssm_heads=2, ssm_vdim=35, state=3, groups=1, conv=3,
                                     norm_groups=5, mlp=moe(experts=9, top=4, ff=14, count=3, keep=2, scale=0.5))],
                       width=102, vocab=333),
}
# float32: the recurrences pass rounding on from token to token.  A lost key, a window that is one token off or a state
# that is not carried moves a row by a hundredth and more.
RMS_LIMIT = {"float32": 3.0e-4, "bfloat16": 1.0e-1}
_MODELS: dict = {}


def folder_of(name: str):
    if name not in _MODELS:
        holder = tempfile.TemporaryDirectory(prefix=f"sebudra_{name}_")
        plain.write_model(holder.name, CONFIGS[name], seed=61 + len(_MODELS))
        _MODELS[name] = (holder, Path(holder.name), plain.load_folder(holder.name))
    return _MODELS[name][1]


def reference(name: str, tokens):
    folder_of(name)
    config, weights = _MODELS[name][2]
    return plain.forward_full(config, weights, tokens).to(torch.float32)


def replay(name: str, dtype: str, steps, max_tokens: int, page: int = 16, max_requests: int = 4):
    from llm_serving_engine_b200.engine.trace_replay import replay as run

    with tempfile.TemporaryDirectory(prefix="sebudra_out_") as out:
        run(folder_of(name), dtype, out, max_tokens, [json.dumps(step) for step in steps], block_size=page,
            max_requests=max_requests)
        return helpers.collect(steps, Path(out))


def compare(name, dtype, requests, got, what):
    """Row error over logit size, per position.  float32: every row within the limit.  bfloat16: a router's choice
    between two almost equal scores may fall the other way than in the plain implementation, which moves that row by
    more than rounding does: up to one row in thirty may pass the limit, none by more than four times."""
    over = rows = 0
    for rid, tokens in requests.items():
        want = reference(name, tokens)
        assert got[rid].shape == want.shape, f"{what}: {rid}: shape {tuple(got[rid].shape)} against {tuple(want.shape)}"
        centred = want - want.mean(-1, keepdim=True)
        per_row = (got[rid] - want).double().pow(2).mean(-1).sqrt() / centred.double().pow(2).mean().sqrt()
        worst = float(per_row.max())
        hard = RMS_LIMIT[dtype] * (4.0 if dtype == "bfloat16" else 1.0)
        assert worst <= hard, (f"{what}: {name} {dtype} request {rid}: row error / logit size {worst:.2e} at position "
                               f"{int(per_row.argmax())}, first above the limit {int((per_row > hard).nonzero()[0])}")
        over += int((per_row > RMS_LIMIT[dtype]).sum())
        rows += per_row.shape[0]
    assert over <= rows // 30, f"{what}: {name} {dtype}: {over} of {rows} rows above {RMS_LIMIT[dtype]:.0e}"


def some_requests(name, lengths, seed=5):
    rng = random.Random(seed)
    vocab = CONFIGS[name]["vocab"]
    return {f"r{index}": helpers.random_tokens(rng, vocab, length) for index, length in enumerate(lengths)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_whole_prompts(name, dtype):
    requests = some_requests(name, [1, 2, 17, 70])
    got = replay(name, dtype, helpers.trace_whole(requests), helpers.max_tokens_for(requests))
    compare(name, dtype, requests, got, "whole")


@pytest.mark.parametrize("name", ["all_kinds", "odd_sizes", "equal_or_one"])
def test_every_layer_against_the_plain_layers(name):
    """The float32 residual after every layer run, through the engine's own step function."""
    from llm_serving_engine_b200.cache.manager import CacheManager
    from llm_serving_engine_b200.config import CacheConfig
    from llm_serving_engine_b200.engine.step import StepEntry, StepRunner
    from llm_serving_engine_b200.models import cache_requirements, load_model
    from llm_serving_engine_b200.parts.linear import reduce_partials

    tokens = some_requests(name, [45], seed=2)["r0"]
    engine_model = load_model(folder_of(name), dtype="float32")
    cache = CacheManager(cache_requirements(engine_model.spec), CacheConfig(block_size=8, num_blocks=16), engine_model.dtype,
                         engine_model.device, engine_model.spec.max_position_embeddings, num_state_slots=2)
    runner = StepRunner(engine_model, cache, 64, 2, use_graphs=False)
    seen = []

    def after_layer(position, stream):
        """A layer's output is still pending (the next layer's norm adds it): add it to a copy."""
        residual = stream.residual.clone()
        if stream.delta is not None:
            residual += reduce_partials(stream.delta)
        seen.append(residual.cpu())

    engine_model.layer_hook = after_layer
    cache.create("a")
    runner.run([StepEntry("a", tokens, [])])
    config, weights = _MODELS[name][2]
    want = plain.forward_layers(config, weights, tokens)[1:]
    assert len(seen) == len(want)
    for index, (got, expected) in enumerate(zip(seen, want)):
        assert float((got - expected).abs().max()) <= 5e-5 * float(expected.abs().max()), f"layer {index}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_prompt_then_token_by_token(name, dtype):
    """Decoding reads the pages, windows and states that the prompt step left (single tokens are replayed from a
    captured graph); a prompt of one token and of fewer tokens than a convolution has taps are among them, and the
    attention windows pass over decoded tokens."""
    requests = some_requests(name, [40, 9, 3, 25], seed=6)
    got = replay(name, dtype, helpers.trace_tail_decode(requests, tail=24), helpers.max_tokens_for(requests))
    compare(name, dtype, requests, got, "tail decoded")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["all_kinds", "odd_sizes"])
def test_portions_of_changing_size(name, dtype):
    """Portions shorter than the convolutions' windows and than the attention windows, portions that end on a page's
    and a chunk's border, one token at a time between longer ones."""
    requests = some_requests(name, [150, 33], seed=7)
    for sizes in ((7, 2, 13, 3, 2, 31, 5, 16, 2, 64, 17), (2,), (16, 16, 1, 15, 17), (1, 2, 3, 1, 1, 64, 63)):
        got = replay(name, dtype, helpers.trace_portions(requests, sizes), helpers.max_tokens_for(requests))
        compare(name, dtype, requests, got, f"portions {sizes}")


def test_a_long_prompt_is_scanned_in_chunks_and_in_portions_alike():
    """A prompt long enough for the chunked form of the scans (chunks side by side, a carry between them), whole and in
    portions that cut chunks anywhere."""
    for name, dtype in (("all_kinds", "float32"), ("memory_only", "float32"), ("odd_sizes", "float32"),
                        ("tensor_core_sizes", "bfloat16"), ("tensor_core_sizes", "float32")):
        requests = some_requests(name, [413], seed=13)
        whole = replay(name, dtype, helpers.trace_whole(requests), 448)
        compare(name, dtype, requests, whole, "long whole")
        cut = replay(name, dtype, helpers.trace_portions(requests, (130, 1, 199, 65, 2)), 448)
        compare(name, dtype, requests, cut, "long in portions")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("page", [16, 8])
def test_mixed_batches_reuse_pages_and_slots(dtype, page):
    """Nine requests through four slots and a pool sized for the live ones only: a page's old rows must not be read
    (the windowed layers give pages back while a request runs), and a slot's states and convolution windows must start
    from zero for the request that takes it next."""
    requests = some_requests("all_kinds", [61, 5, 90, 33, 2, 47, 130, 18, 64], seed=8)
    steps, peak = helpers.trace_mixed(requests, seed=3, max_live=4)
    got = replay("all_kinds", dtype, steps, peak, page=page)
    compare("all_kinds", dtype, requests, got, "mixed")


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_long_portions_beside_single_tokens_on_the_tensor_cores(dtype):
    """Steps in which a portion of 128 rows and more stands beside other portions and single decoded tokens, with head
    sizes that the tensor-core kernels take: in bfloat16 the sigmoid-weighted layers then run on tcgen05 (a single token
    takes a tile of its own there) and the windowed ones on mma.sync; pages and slots are used again by a fourth request."""
    name = "tensor_core_sizes"
    requests = some_requests(name, [156, 150, 270, 140], seed=21)
    a, b, c, d = (requests[f"r{index}"] for index in range(4))

    def entry(rid, tokens, first, count):
        return {"id": rid, "tokens": tokens[first:first + count], "want": list(range(count))}

    steps = [
        {"step": 0, "entries": [entry("r0", a, 0, 150), entry("r1", b, 0, 3)], "end": []},
        {"step": 1, "entries": [entry("r0", a, 150, 1), entry("r1", b, 3, 140), entry("r2", c, 0, 130)], "end": []},
        {"step": 2, "entries": [entry("r0", a, 151, 1), entry("r1", b, 143, 1), entry("r2", c, 130, 135)], "end": []},
        {"step": 3, "entries": [entry("r0", a, 152, 4), entry("r1", b, 144, 6), entry("r2", c, 265, 1)], "end": ["r0", "r1"]},
        {"step": 4, "entries": [entry("r2", c, 266, 1), entry("r3", d, 0, 128)], "end": []},
        {"step": 5, "entries": [entry("r2", c, 267, 3), entry("r3", d, 128, 12)], "end": ["r2", "r3"]},
    ]
    got = replay(name, dtype, steps, 640)
    compare(name, dtype, requests, got, "long portions beside single tokens")


def test_a_batch_gives_what_each_request_gives_alone():
    for name in ("all_kinds", "odd_sizes"):
        requests = some_requests(name, [37, 12, 80, 5], seed=9)
        steps, peak = helpers.trace_mixed(requests, seed=4, max_live=4)
        together = replay(name, "float32", steps, peak)
        for rid, tokens in requests.items():
            alone = replay(name, "float32", helpers.trace_whole({rid: tokens}), helpers.max_tokens_for({rid: tokens}))
            assert float((together[rid] - alone[rid]).abs().max()) <= 2e-5 * float(alone[rid].abs().max())


def test_long_decoding_crosses_key_chunks_and_many_pages():
    """600 single tokens after a short prompt: the keys pass the borders of tiles, chunks and many pages, the windows
    slide over hundreds of decoded tokens, and the recurrent states are carried six hundred times."""
    requests = some_requests("all_kinds", [610], seed=10)
    got = replay("all_kinds", "float32", helpers.trace_tail_decode(requests, tail=600), 640)
    compare("all_kinds", "float32", requests, got, "long decoding")


def test_greedy_generation_through_the_engine_and_its_scheduler():
    """More requests than the scheduler keeps live, prompts cut into portions: every request's greedy tokens equal
    the plain implementation's (float32; a request whose top two logits are closer than the arithmetic's noise is
    skipped from that token on)."""
    from llm_serving_engine_b200.config import CacheConfig, SchedulerConfig
    from llm_serving_engine_b200.engine.llm_engine import LLMEngine
    from llm_serving_engine_b200.models import load_model
    from llm_serving_engine_b200.sampling.sampler import GenerationConfig

    name = "all_kinds"
    engine = LLMEngine(load_model(folder_of(name), dtype="float32"), None,
                       cache_config=CacheConfig(block_size=16, num_blocks=40),
                       scheduler_config=SchedulerConfig(max_batch_size=3, max_tokens_per_step=48), prefill_chunk_size=20)
    prompts = list(some_requests(name, [30, 7, 55, 2, 19, 41], seed=12).values())
    new_tokens = 12
    produced = engine.generate_many(prompts, GenerationConfig(max_new_tokens=new_tokens, temperature=0.0))
    for prompt, tokens in zip(prompts, produced):
        assert len(tokens) == new_tokens
        logits = reference(name, prompt + tokens)
        for index, token in enumerate(tokens):
            row = logits[len(prompt) + index - 1]
            top = torch.topk(row, 2).values
            if float(top[0] - top[1]) < 1e-3 * float(row.abs().max()):
                break
            assert int(row.argmax()) == token, f"token {index} of a {len(prompt)}-token prompt"


# ------------------------------------------------------------------ architectures drawn at random
def _divisors(n):
    return [d for d in range(1, n + 1) if n % d == 0]


def _drawn_attention(rng, windowed):
    kv_heads, group = rng.choice([1, 2, 3]), rng.choice([1, 2, 3, 4])
    dim = rng.choice([16, 24, 32, 48, 64, 96, 128])
    vdim = dim if rng.random() < 0.5 else rng.choice([8, 16, 40, 48, 64])
    rot = {"base": rng.choice([100.0, 10000.0, 1000000.0]),
           "dims": rng.choice([d for d in (2, 4, 8, 16, dim // 2, dim) if d <= dim and d % 2 == 0])}
    if rng.random() < (0.8 if windowed else 0.3):
        rot["scaling"] = {"factor": rng.choice([1.0, 2.0, 3.0, 8.0]), "original": rng.choice([32, 64, 256]),
                          "fast": rng.choice([4.0, 8.0, 16.0]), "slow": rng.choice([0.5, 1.0])}
    mixer = {"heads": kv_heads * group, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
             "scale": rng.choice([1.0, 1.5, 2.0]) / dim ** 0.5, "rot": rot}
    if windowed:
        mixer["mask"] = {"size": rng.choice([1, 3, 16, 17, 33, 64, 100, 500])}
    else:
        mixer["softcap"] = rng.choice([1.0, 5.0, 20.0, 100.0])
    return mixer


def _drawn_feed_forward(rng):
    draw = rng.random()
    if draw < 0.15:
        return None
    if draw < 0.55:
        return dense(ff=rng.choice([24, 50, 88, 128]), limit=rng.choice([0.7, 1.75, 7.0]))
    experts = rng.choice([2, 4, 6, 8, 12])
    if rng.random() < 0.7:
        count = rng.choice(_divisors(experts))
        keep = rng.randint(1, count)
        top = rng.randint(1, keep * (experts // count))
    else:
        count, keep, top = 0, 0, rng.randint(1, experts)
    return moe(experts=experts, top=top, ff=rng.choice([8, 18, 40, 64]), count=count, keep=keep,
               scale=rng.choice([1.0, 1.25, 2.5]), shared=rng.choice([0, 8, 24, 48]))


def _drawn_layer(rng):
    kind = rng.choice(["parallel", "attention", "gla"])
    if kind == "parallel":
        heads, vdim = rng.choice([1, 2, 4, 6, 8]), rng.choice([4, 8, 12, 48, 64])
        right = {"heads": heads, "vdim": vdim, "state": rng.choice([1, 2, 8, 16, 32, 64, 128]), "groups": rng.choice(_divisors(heads)),
                 "conv": rng.choice([1, 2, 3, 4, 5]), "norm_groups": rng.choice([d for d in _divisors(heads * vdim) if d <= 8])}
        mixer = {"left": _drawn_attention(rng, True), "right": right, "left_scale": rng.choice([0.3, 1.0, 1.7]),
                 "right_scale": rng.choice([0.4, 1.0, 1.3])}
    elif kind == "attention":
        mixer = _drawn_attention(rng, False)
    else:
        mixer = {"heads": rng.choice([1, 2, 3, 6]), "dim": rng.choice([8, 16, 32, 64, 96]), "vdim": rng.choice([8, 24, 64, 100]),
                 "tau": rng.choice([1.0, 4.0, 8.0]), "rank": rng.choice([1, 4, 8])}
    return {"type": kind, "mixer": mixer, "mlp": _drawn_feed_forward(rng)}


def _drawn_model(rng):
    """Two to five layers of any kinds in any order with sizes drawn one by one, and up to two more that run an earlier
    layer again on its tensors."""
    own = [_drawn_layer(rng) for _ in range(rng.randint(2, 5))]
    layers = [(layer, None) for layer in own]
    for _ in range(rng.randint(0, 2)):
        source = rng.randrange(len(own))
        place = rng.randint([index for index, (layer, of) in enumerate(layers) if layer is own[source] and of is None][0] + 1, len(layers))
        layers.insert(place, (own[source], source))
    entries = []
    for layer, of in layers:
        if of is None:
            entries.append(layer)
        else:     # the index of the source among all entries, which the insertions have moved
            entries.append(again(layer, [index for index, (other, other_of) in enumerate(layers) if other is layer and other_of is None][0]))
    return model(entries, width=rng.choice([48, 64, 96, 120, 256]), vocab=rng.choice([97, 300, 501]),
                 embed_scale=rng.choice([1.0, 3.0, 9.0]), eps=rng.choice([1e-5, 1e-6]))


@pytest.mark.parametrize("seed", range(10))
def test_architectures_drawn_at_random(seed):
    """Kinds, order, sizes and constants drawn at random, four requests whole, in portions of drawn sizes, with decoded
    tails and in mixed batches through four slots, in float32 against the plain implementation (a router's close call
    would decide a bfloat16 row, so the draw is compared where rounding does not reach it)."""
    rng = random.Random(1000 + seed)
    config = _drawn_model(rng)
    name = f"drawn_{seed}"
    CONFIGS[name] = config
    try:
        requests = {f"r{index}": helpers.random_tokens(rng, config["vocab"], count)
                    for index, count in enumerate([rng.randint(1, 40), rng.randint(100, 300), rng.randint(30, 150), rng.randint(2, 70)])}
        sizes = tuple(rng.choice([1, 2, 3, 7, 16, 33, 64, 130]) for _ in range(6))
        peak = helpers.max_tokens_for(requests)
        compare(name, "float32", requests, replay(name, "float32", helpers.trace_whole(requests), peak), f"whole {config['layers']}")
        compare(name, "float32", requests, replay(name, "float32", helpers.trace_portions(requests, sizes), peak), f"portions {sizes}")
        compare(name, "float32", requests, replay(name, "float32", helpers.trace_tail_decode(requests, tail=20), peak), "tail decoded")
        steps, live = helpers.trace_mixed(requests, seed=seed, max_live=4)
        compare(name, "float32", requests, replay(name, "float32", steps, live), "mixed")
    finally:
        CONFIGS.pop(name, None)
        _MODELS.pop(name, None)


# ------------------------------------------------------------------ the mechanisms' kernels alone
def _step(lengths, first_positions=None, slots=None):
    """The step's tensors that the kernels read, for requests of ``lengths`` rows laid one after the other."""
    first_positions = first_positions or [0] * len(lengths)
    slots = slots if slots is not None else list(range(len(lengths)))
    seg, pos, start = [], [], [0]
    for index, (count, first) in enumerate(zip(lengths, first_positions)):
        seg += [index] * count
        pos += list(range(first, first + count))
        start.append(start[-1] + count)
    as_int = lambda values: torch.tensor(values, dtype=torch.int32, device="cuda")
    return SimpleNamespace(segment_of_token=as_int(seg), positions=as_int(pos), segment_start=as_int(start),
                           segment_first_position=as_int(first_positions), segment_state_slot=as_int(slots))


def _cuts(total, sizes):
    """(first row, rows) of the portions of ``sizes``, repeated until ``total`` rows are spent."""
    out, at, index = [], 0, 0
    while at < total:
        size = min(sizes[index % len(sizes)], total - at)
        out.append((at, size))
        at, index = at + size, index + 1
    return out


def _paged_attention(q, k, v, cuts, page, dtype, **changes):
    """q [T, H, d], k [T, G, d], v [T, G, e] of one request through the paged attention in the portions ``cuts``: the
    keys and values are written to pages scattered in a pool whose other rows hold NaN."""
    from llm_serving_engine_b200.kernels import ops

    total, n_q, dk = q.shape
    n_kv, dv = k.shape[1], v.shape[2]
    pages = -(-total // page)
    order = torch.randperm(pages + 4, generator=torch.Generator().manual_seed(total + page))[:pages].to(torch.int32)
    keys = torch.full((pages + 4, n_kv, page, dk), float("nan"), dtype=dtype, device="cuda")
    values = torch.full((pages + 4, n_kv, page, dv), float("nan"), dtype=dtype, device="cuda")
    out = []
    for at, count in cuts:
        step = _step([count], [at])
        places = torch.arange(at, at + count)
        where, offset = order[places // page].long().cuda(), (places % page).cuda()
        keys[where, :, offset] = k[at:at + count].to(dtype).cuda()
        values[where, :, offset] = v[at:at + count].to(dtype).cuda()
        attended = torch.empty(count, n_q, dv, dtype=dtype, device="cuda")
        ops.attention_scored(q[at:at + count].to(dtype).cuda().contiguous(), keys, values, attended, order.view(1, -1).cuda(),
                             step.segment_of_token, step.positions, changes["scale"],
                             segment_start=step.segment_start, segment_first_position=step.segment_first_position,
                             window=changes.get("window", 0), cap=changes.get("cap", 0.0),
                             head_bias=changes["head_bias"].cuda() if changes.get("head_bias") is not None else None)
        out.append(attended.float().cpu())
    return torch.cat(out)


def _plain_attention(q, k, v, scale, window=0, cap=0.0, head_bias=None):
    total = q.shape[0]
    scores = plain.key_scores(q.double(), k.double(), scale)
    if cap > 0:
        scores = cap * torch.tanh(scores / cap)
    distance = torch.arange(total)[:, None] - torch.arange(total)[None, :]
    seen = (distance >= 0) & ((distance < window) if window > 0 else True)
    if head_bias is None:
        weights = torch.softmax(scores.masked_fill(~seen, float("-inf")), dim=-1)
    else:
        weights = torch.sigmoid(scores + head_bias.double()[:, None, None]) * seen
    return plain.apply_weights(weights, v.double()).view(total, q.shape[1], v.shape[2])


# head sizes that the general kernel takes (keys and values of different sizes) and that the tensor-core kernel takes in bfloat16
_HEAD_SIZES = [(4, 2, 24, 40), (4, 2, 64, 64), (6, 2, 48, 48), (8, 1, 128, 128), (4, 2, 96, 96), (3, 1, 32, 32)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", _HEAD_SIZES)
@pytest.mark.parametrize("window", [1, 7, 40, 256, 300])
def test_a_window_ends_where_it_should(dtype, window, sizes):
    """One key far stronger than the others sits just inside and just outside the last row's window (and the rows before
    it see it or not by their own windows), at page and chunk borders; the rows come whole, as a prompt and a single
    token, and in portions of two."""
    torch.manual_seed(11)
    (n_q, n_kv, dk, dv), context, page = sizes, 330, 16
    scale = 1.5 / dk ** 0.5
    for back in (window - 1, window, window + 1, 0):       # the strong key's distance from the last row
        special = context - 1 - back
        if special < 0:
            continue
        q, k, v = (torch.randn(context, n, d).to(dtype).float() for n, d in ((n_q, dk), (n_kv, dk), (n_kv, dv)))
        k[special, 0] = 3.0 * q[context - 1, 1]       # head 1 of the last row finds it, if its window reaches it
        v[special, 0] = 5.0
        want = _plain_attention(q, k, v, scale, window=window)
        inside = back < window
        assert (float(want[-1, 1].mean()) > 4.0) == inside
        for cuts in ([(0, context)], [(0, context - 1), (context - 1, 1)], _cuts(context, (2,)) if back == window else None):
            if cuts is None:
                continue
            got = _paged_attention(q, k, v, cuts, page, dtype, scale=scale, window=window)
            limit = 3e-5 if dtype == torch.float32 else 3e-2
            error = (got.double() - want).abs()
            assert float(error.max()) <= limit * max(1.0, float(want.abs().max())), (back, len(cuts), int(error.amax((1, 2)).argmax()))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [(6, 2, 16, 24), (6, 2, 64, 64), (6, 3, 32, 32), (6, 1, 128, 128), (6, 3, 96, 96), (6, 2, 48, 48)])
def test_sigmoid_weights_are_not_normalised_and_find_a_far_key(dtype, sizes):
    """Weights sigmoid(capped score + a number per head): the output grows with the number of keys (a softmax's would
    not), the cap bounds what one key can weigh, and one far key with a large score and a large value shows at the
    borders of pages, tiles and chunks, in prompts, single tokens and portions of two."""
    torch.manual_seed(12)
    (n_q, n_kv, dk, dv), context, page, cap = sizes, 300, 16, 4.0
    scale = 2.0 / dk ** 0.5
    head_bias = torch.tensor([-6.0, -2.0, 0.0, 1.0, -4.0, -3.0])
    for special in (0, 1, 15, 16, 17, 31, 32, 255, 256, 257, 297, 298):
        q, k, v = (torch.randn(context, n, d).to(dtype).float() for n, d in ((n_q, dk), (n_kv, dk), (n_kv, dv)))
        k[special, 0] = 4.0 * q[context - 1, 0]       # head 0 (bias -6): only this key weighs much
        v[special, 0] = 9.0
        want = _plain_attention(q, k, v, scale, cap=cap, head_bias=head_bias)
        assert float(want[-1, 0].mean()) > 0.1 * 9.0 * float(torch.sigmoid(torch.tensor(cap - 6.0)))
        total = _plain_attention(q, k, torch.ones_like(v), scale, cap=cap, head_bias=head_bias)      # the weights' sums
        assert float(total[-1, 3].mean()) > 100.0 > 12.0 > float(total[9, 3].mean()) > 3.0      # a softmax's would be one
        for cuts in ([(0, context)], [(0, context - 1), (context - 1, 1)], _cuts(context, (2,)) if special in (16, 257) else None):
            if cuts is None:
                continue
            got = _paged_attention(q, k, v, cuts, page, dtype, scale=scale, cap=cap, head_bias=head_bias)
            limit = 3e-5 if dtype == torch.float32 else 3e-2
            error = (got.double() - want).abs()
            assert float(error.max()) <= limit * max(1.0, float(want.abs().max())), (special, len(cuts))


@pytest.mark.parametrize("sizes", [(6, 2, 64, 64), (4, 1, 128, 128)])
def test_sigmoid_weights_on_the_tcgen05_kernel(sizes):
    """Long prompt portions on the 5th-generation tensor cores: three requests in a step (portions of 128 rows and more
    behind prefixes of several lengths), a cap and none, against the plain weights; the kernel reports no wait that gave up."""
    from llm_serving_engine_b200.kernels import ops

    torch.manual_seed(13)
    (n_q, n_kv, dk, dv), page = sizes, 16
    scale = 2.0 / dk ** 0.5
    head_bias = torch.linspace(-5.0, 0.5, n_q)
    lengths, firsts = [300, 129, 700], [0, 40, 333]        # rows of the step, keys before them
    for cap in (3.0, 0.0):
        pool = sum(-(-(first + count) // page) for first, count in zip(firsts, lengths)) + 3
        keys = torch.full((pool, n_kv, page, dk), float("nan"), dtype=torch.bfloat16, device="cuda")
        values = torch.full((pool, n_kv, page, dv), float("nan"), dtype=torch.bfloat16, device="cuda")
        order = torch.randperm(pool, generator=torch.Generator().manual_seed(5)).to(torch.int32)
        width = max(-(-(first + count) // page) for first, count in zip(firsts, lengths))
        tables = torch.zeros(len(lengths), width, dtype=torch.int32)
        rows, wants, used = [], [], 0
        for index, (first, count) in enumerate(zip(firsts, lengths)):
            total = first + count
            q, k, v = (torch.randn(total, n, d).to(torch.bfloat16).float() for n, d in ((n_q, dk), (n_kv, dk), (n_kv, dv)))
            k[3, 0] = 4.0 * q[total - 1, 0]
            v[3, 0] = 9.0
            pages = -(-total // page)
            tables[index, :pages] = order[used:used + pages]
            places = torch.arange(total)
            where, offset = order[used + places // page].long().cuda(), (places % page).cuda()
            keys[where, :, offset] = k.to(torch.bfloat16).cuda()
            values[where, :, offset] = v.to(torch.bfloat16).cuda()
            used += pages
            rows.append(q[first:])
            wants.append(_plain_attention(q, k, v, scale, cap=cap, head_bias=head_bias)[first:])
        step = _step(lengths, firsts)
        out = torch.empty(sum(lengths), n_q, dv, dtype=torch.bfloat16, device="cuda")
        ops.attention_sigmoid_tc(torch.cat(rows).to(torch.bfloat16).cuda().contiguous(), keys, values, out, tables.cuda(),
                                 step.segment_start, step.segment_first_position, scale, head_bias.cuda(), cap)
        assert ops.attention_tc_status() == 0
        want = torch.cat(wants)
        error = (out.float().cpu().double() - want).abs()
        assert float(error.max()) <= 3e-2 * max(1.0, float(want.abs().max())), (cap, int(error.amax((1, 2)).argmax()))


def test_heads_are_normed_one_by_one_then_rotated_far_from_the_start():
    """Biases, an RMS norm per head with one weight for all heads, then the rotation of a head's first values, at
    positions beyond thirty thousand, with frequencies that are stretched, not stretched and in between; the projection
    arrives whole, as a stack of partial sums, and behind other columns."""
    from llm_serving_engine_b200.kernels import ops
    from llm_serving_engine_b200.parts.latent_attention import rotary_frequencies

    torch.manual_seed(9)
    n_q, n_kv, dk, dv, eps, count, offset = 3, 1, 32, 8, 1e-6, 6, 5
    channels = (n_q + n_kv) * dk + n_kv * dv
    q_norm, k_norm, bias = torch.rand(dk) + 0.5, torch.rand(dk) + 0.5, torch.randn(channels)
    for dims, scaling in ((32, {"factor": 8.0, "original": 512, "fast": 32.0, "slow": 1.0}), (6, {"factor": 1.0, "original": 64, "fast": 2.0, "slow": 1.0}),
                          (16, {"factor": 2.5, "original": 4096, "fast": 4.0, "slow": 0.25}), (0, None)):
        rot = {"base": 50000.0, "dims": dims, "scaling": scaling}
        freq, factor = rotary_frequencies(rot) if dims else (torch.zeros(0, dtype=torch.float64), 1.0)
        keys = torch.zeros(3000, n_kv, 16, dk, device="cuda")
        values = torch.zeros(3000, n_kv, 16, dv, device="cuda")
        for first in (0, 31000):
            wide = torch.randn(count, offset + channels + 3)
            proj = wide[:, offset:offset + channels]
            step = _step([count], [first])
            slots = torch.arange(first, first + count, dtype=torch.int32, device="cuda")
            with_bias = proj.double() + bias.double()
            want = plain.rms(with_bias[:, :n_q * dk].view(count, n_q, dk), eps) * q_norm.double()
            want_k = plain.rms(with_bias[:, n_q * dk:(n_q + n_kv) * dk].view(count, n_kv, dk), eps) * k_norm.double()
            if dims:
                cos, sin = plain.rotary_table(rot, first + count)
                cos, sin = cos[first:], sin[first:]
                want, want_k = plain.rotate_half(want, cos, sin, dims), plain.rotate_half(want_k, cos, sin, dims)
            for form in ("whole", "stack"):
                given = wide.cuda() if form == "whole" else torch.stack([wide * 0.25, wide * 0.75]).cuda().contiguous()
                q = torch.empty(count, n_q, dk, device="cuda")
                ops.head_norm_rope_kv_write(given, bias.cuda(), q_norm.cuda(), k_norm.cuda(), eps, slots, step.positions,
                                            freq.to(torch.float64).contiguous().cuda(), factor, q, keys, values, n_q, n_kv, dk, dv,
                                            offset=offset)
                assert float((q.cpu().double() - want).abs().max()) <= 2e-5, (dims, first, form)
                written = keys.view(-1, n_kv, 16, dk)[first // 16:(first + count) // 16 + 1].transpose(1, 2).reshape(-1, n_kv, dk)
                assert float((written[first % 16:first % 16 + count].cpu().double() - want_k).abs().max()) <= 2e-5, (dims, first)
                stored = values.view(-1, n_kv, 16, dv)[first // 16:(first + count) // 16 + 1].transpose(1, 2).reshape(-1, n_kv * dv)
                assert float((stored[first % 16:first % 16 + count].cpu().double() - with_bias[:, (n_q + n_kv) * dk:]).abs().max()) <= 2e-6


@pytest.mark.parametrize("heads,vdim,states,groups", [(4, 12, 8, 2), (6, 7, 23, 3), (2, 64, 128, 1), (3, 16, 1, 3), (8, 32, 16, 8)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_state_space_scan_with_a_decay_per_head(heads, vdim, states, groups, dtype):
    """Step sizes from tiny to large, B and C shared by the heads of a group, whole, in chunks side by side and in
    portions down to one row, two requests in a step with slots of their own; then the skip, the gate before the norm
    and the norm in parts, written into a column range with the branch's weight."""
    from llm_serving_engine_b200.kernels import ops

    torch.manual_seed(7)
    total, inner, eps, scale = 203, heads * vdim, 1e-5, 0.75
    channels = inner + 2 * groups * states
    parts = groups if inner % groups == 0 else 1
    u = torch.randn(2, total, channels).to(dtype).float()                   # [x | B | C] behind the convolution
    proj = torch.randn(2, total, 3 + inner + heads)                          # some columns, z, then dt
    proj[:, :, -heads:] = proj[:, :, -heads:] * 3.0 - 1.0
    dt_bias, a_log, skip, weight = torch.randn(heads), torch.randn(heads), torch.rand(heads) + 0.5, torch.rand(inner) + 0.5
    want = []
    for r in (0, 1):
        x = u[r, :, :inner].double().view(total, heads, vdim)
        b = u[r, :, inner:inner + groups * states].double().view(total, groups, states).repeat_interleave(heads // groups, dim=1)
        c = u[r, :, inner + groups * states:].double().view(total, groups, states).repeat_interleave(heads // groups, dim=1)
        dt = torch.nn.functional.softplus(proj[r, :, -heads:].double() + dt_bias.double())
        y = plain.state_space_scan(x, dt, torch.exp(a_log.double()), b, c, skip.double()).reshape(total, inner)
        y = y * torch.nn.functional.silu(proj[r, :, 3:3 + inner].double())
        want.append(plain.rms(y.view(total, parts, inner // parts), eps).reshape(total, inner) * weight.double() * scale)
    for sizes, chunked in (((total,), True), ((total,), False), ((64, 1, 2, 65, 1, 1, 3), None), ((2,), None)):
        state = torch.zeros(3, heads, states, vdim, device="cuda")
        state[1] = 5.0       # another request's state
        got = [[], []]
        for first, count in _cuts(total, sizes):
            step = _step([count, count], [first, first], slots=[2, 0])
            pick = lambda t: torch.cat([t[0, first:first + count], t[1, first:first + count]]).cuda().contiguous()
            rows, inputs = pick(proj), pick(u).to(dtype)
            keep, take = ops.ssd_gates(rows, 3 + inner, dt_bias.cuda(), a_log.cuda())
            read = torch.empty(2 * count, inner, device="cuda")
            ops.token_decay_scan(inputs, inner + groups * states, inner, 0, keep, take, 1.0, state, step.segment_start,
                                 step.segment_state_slot, read, heads, states, vdim, qk_share=heads // groups, chunked=chunked)
            wide = torch.zeros(2 * count, inner + 4, dtype=dtype, device="cuda")      # the output is a column range
            ops.gated_group_rmsnorm(read, rows, 3, weight.cuda(), eps, wide[:, 4:], parts, gate_first=True, gate_activation="silu",
                                    scale=scale, skip=skip.cuda(), skip_source=inputs, skip_offset=0,
                                    segment_of_token=step.segment_of_token)
            assert float(wide[:, :4].float().abs().max()) == 0.0
            got[0].append(wide[:count, 4:].float().cpu())
            got[1].append(wide[count:, 4:].float().cpu())
        limit = 5e-5 if dtype == torch.float32 else 1.5e-2
        for r in (0, 1):
            error = (torch.cat(got[r]).double() - want[r]).abs()
            assert float(error.max()) <= limit * float(want[r].abs().max()), (sizes, chunked, r, int(error.max(1).values.argmax()))
        assert float((state[1] - 5.0).abs().max()) == 0.0


@pytest.mark.parametrize("heads,dim,vdim", [(3, 16, 24), (1, 72, 5), (2, 128, 128), (4, 8, 33), (6, 32, 64)])
def test_matrix_memory_with_a_decay_per_key_channel(heads, dim, vdim):
    """Decays from nearly one to nearly zero, different in every channel, whole, in chunks side by side and in portions
    down to one row, the state carried between them; then the norm per head and the gate behind it."""
    from llm_serving_engine_b200.kernels import ops

    torch.manual_seed(6)
    total, tau, eps = 203, 4.0, 1e-5
    qk, val = heads * dim, heads * vdim
    proj = torch.randn(2, total, 2 * qk + 2 * val)
    z = torch.randn(2, total, qk) * 4.0 + 2.0
    z[0, :, 0] = 30.0                       # a channel that forgets nothing ...
    z[0, :, 1] = -30.0                      # ... and one that keeps nothing
    bias, weight = torch.randn(qk), torch.rand(vdim) + 0.5
    want = []
    for r in (0, 1):
        p = proj[r].double()
        q = p[:, :qk].view(total, heads, dim) * dim ** -0.5
        k = p[:, qk:2 * qk].view(total, heads, dim)
        v = p[:, 2 * qk:2 * qk + val].view(total, heads, vdim)
        keep = torch.sigmoid(z[r].double() + bias.double()).pow(1.0 / tau).view(total, heads, dim)
        o = plain.rms(plain.decayed_memory(q, k, v, keep), eps) * weight.double()
        want.append(o.reshape(total, val) * torch.nn.functional.silu(p[:, 2 * qk + val:]))
    for sizes, chunked in (((total,), True), ((total,), False), ((64, 1, 2, 65, 1, 1, 3), None), ((2,), None)):
        memory = torch.zeros(4, heads, dim, vdim, device="cuda")
        memory[1] = 3.0       # another request's state
        got = [[], []]
        for first, count in _cuts(total, sizes):
            step = _step([count, count], [first, first], slots=[2, 0])
            pick = lambda t: torch.cat([t[0, first:first + count], t[1, first:first + count]]).cuda().contiguous()
            rows = pick(proj)
            keep = ops.sigmoid_power(pick(z), 0, qk, bias.cuda(), tau)
            read = torch.empty(2 * count, val, device="cuda")
            ops.channel_decay_scan(rows, 0, qk, 2 * qk, keep, dim ** -0.5, memory, step.segment_start, step.segment_state_slot,
                                   read, heads, dim, vdim, chunked=chunked)
            out = torch.empty(2 * count, val, device="cuda")
            ops.gated_group_rmsnorm(read, rows, 2 * qk + val, weight.cuda(), eps, out, heads, gate_first=False,
                                    gate_activation="silu", segment_of_token=step.segment_of_token)
            got[0].append(out[:count].cpu())
            got[1].append(out[count:].cpu())
        for r in (0, 1):
            error = (torch.cat(got[r]).double() - want[r]).abs()
            assert float(error.max()) <= 3e-4 * float(want[r].abs().max()), (sizes, chunked, r, int(error.max(1).values.argmax()))
        assert float((memory[1] - 3.0).abs().max()) == 0.0


@pytest.mark.parametrize("experts,top,count,keep", [(8, 3, 4, 2), (6, 2, 3, 2), (7, 3, 7, 4), (4, 1, 4, 4), (1, 1, 1, 1), (12, 3, 0, 0),
                                                    (64, 6, 8, 2)])
def test_router_chooses_within_the_best_groups(experts, top, count, keep):
    """Sigmoid scores; the correction moves the choice and not the weights; an expert with a large score in a group
    that is shut out is not chosen, also when every choice score is negative; the weights of the chosen add up to the
    scale."""
    from llm_serving_engine_b200.kernels import ops

    torch.manual_seed(10)
    rows, scale = 60, 1.5
    logits = torch.randn(rows, experts + 3) * 2
    correction = torch.randn(experts) * 0.5
    correction[0] -= 3.0          # some choice scores are negative
    if rows > 30:
        logits[30:, :experts] -= 6.0     # rows whose scores are all tiny: corrected scores below zero throughout
    w = {"p.router": torch.eye(experts, dtype=torch.float64), "p.correction": correction.double()}
    router = {"experts": experts, "top": top, "scale": scale}
    if count:
        router["groups"] = {"count": count, "keep": keep}
    chosen_want, weights_want = plain.route(logits[:, :experts].double(), w, "p.", router)
    chosen = torch.empty(rows, top, dtype=torch.int32, device="cuda")
    weights, _, gate = ops.moe_route_sigmoid(logits.cuda(), correction.cuda(), experts, top, count, keep, scale,
                                             shared_gate=True, chosen=chosen)
    assert torch.equal(chosen.cpu().long().sort(dim=1).values, chosen_want.sort(dim=1).values)
    want = torch.zeros(rows, experts, dtype=torch.float64).scatter(1, chosen_want, weights_want)
    assert float((weights.cpu().double() - want).abs().max()) <= 2e-6
    assert float((weights.sum(1).cpu() - scale).abs().max()) <= 1e-5
    assert float((gate.cpu().double() - torch.sigmoid(logits[:, experts].double())).abs().max()) <= 1e-6
    if count and keep < top and experts // count > 1:      # the largest score of a row often lies in a group that is shut out: it must not be chosen
        per = experts // count
        plainly = (torch.sigmoid(logits[:, :experts].double()) + correction.double()).topk(top, dim=-1).indices
        assert not torch.equal(plainly.sort(dim=1).values, chosen_want.sort(dim=1).values)
        assert all(len({int(e) // per for e in row}) <= keep for row in chosen.cpu())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_experts_without_a_gate_and_the_clamped_dense_form(dtype):
    from llm_serving_engine_b200.kernels import ops

    torch.manual_seed(3)
    rows, experts, ff, shared_ff = 9, 3, 16, 24
    inter = experts * ff + shared_ff
    up = (torch.randn(rows, inter) * 2).to(dtype)
    weights = torch.rand(rows, experts)
    weights[:, 1] = 0.0
    gate = torch.rand(rows)
    out = torch.empty(rows, inter, dtype=dtype, device="cuda")
    ops.moe_gated_act(up.cuda(), weights.cuda(), gate.cuda(), out, experts, ff, shared_ff, 0.0, 0.0, activation="squared_relu")
    factor = torch.cat([weights.repeat_interleave(ff, dim=1), gate[:, None].expand(rows, shared_ff)], dim=1)
    want = torch.relu(up.double()).pow(2) * factor.double()
    limit = 1e-6 if dtype == torch.float32 else 1e-2
    assert float((out.float().cpu().double() - want).abs().max()) <= limit * float(want.abs().max())
    for inter, cap in ((40, 2.0), (37, 0.7)):
        gate_up = (torch.randn(rows, 2 * inter) * 3).to(dtype)
        out = torch.empty(rows, inter, dtype=dtype, device="cuda")
        ops.silu_mul(gate_up.cuda(), out, "clamped_swish", cap)
        g = gate_up[:, :inter].double().clamp(max=cap)
        u = gate_up[:, inter:].double().clamp(-cap, cap)
        want = g * torch.sigmoid(1.702 * g) * (u + 1.0)
        assert float((out.float().cpu().double() - want).abs().max()) <= limit * float(want.abs().max())


def test_command_line_generates_from_a_model_folder_and_from_the_stand_in():
    """``bin/llmserve generate`` on a folder of the design (the class comes from config.json): the greedy tokens are the
    plain implementation's; and on the random stand-in of the design."""
    import os
    import subprocess
    import sys

    root = str(Path(__file__).resolve().parent.parent)
    env = dict(os.environ, PYTHONPATH=root)
    name, prompt, count = "all_kinds", [5, 17, 3, 150, 99, 42, 7], 8
    out = subprocess.run([sys.executable, os.path.join(root, "bin", "llmserve"), "generate", "--model", str(folder_of(name)),
                          "--dtype", "float32", "--prompt-ids", " ".join(map(str, prompt)), "--max-new-tokens", str(count)],
                         capture_output=True, text=True, env=env, timeout=600)
    assert out.returncode == 0, out.stderr
    tokens = json.loads(out.stdout.strip().splitlines()[-1])["output_ids"]
    assert len(tokens) == count
    logits = reference(name, prompt + tokens)
    for index, token in enumerate(tokens):
        row = logits[len(prompt) + index - 1]
        top = torch.topk(row, 2).values
        if float(top[0] - top[1]) < 1e-3 * float(row.abs().max()):
            break
        assert int(row.argmax()) == token, f"token {index}"
    out = subprocess.run([sys.executable, os.path.join(root, "bin", "llmserve"), "generate", "--random", "sebudra",
                          "--prompt-ids", "5 17 3 250 99", "--max-new-tokens", "6"],
                         capture_output=True, text=True, env=env, timeout=600)
    assert out.returncode == 0, out.stderr
    assert len(json.loads(out.stdout.strip().splitlines()[-1])["output_ids"]) == 6
