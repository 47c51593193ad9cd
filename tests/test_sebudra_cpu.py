"""Host-side pieces of the Sebudra design: configuration, description, tensor names, layers that run with another layer's
tensors, a size that only a tensor's shape gives, cache needs and slots, the plain implementation's pieces against each
other."""
import math

import pytest
import torch

from plain import sebudra_plain as plain


def small_config(**changes):
    mlp = {"kind": "moe", "router": {"experts": 6, "top": 2, "scale": 1.25, "groups": {"count": 3, "keep": 2}},
           "expert": {"ff": 24}, "shared": {"ff": 16}}
    left = {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 12, "scale": 0.3, "mask": {"size": 9},
            "rot": {"base": 500.0, "dims": 4, "scaling": {"factor": 3.0, "original": 64, "fast": 8.0, "slow": 1.0}}}
    right = {"heads": 4, "vdim": 10, "state": 6, "groups": 2, "conv": 3, "norm_groups": 2}
    first = {"type": "parallel", "mlp": {"kind": "dense", "ff": 56, "limit": 1.5},
             "mixer": {"left": left, "right": right, "left_scale": 0.7, "right_scale": 1.3}}
    config = {
        "architecture": "Sebudra", "vocab": 97, "width": 48, "norm": {"eps": 1e-5}, "embedding": {"scale": 4.0},
        "layers": [
            first,
            {"type": "attention", "mlp": mlp, "mixer": {"heads": 3, "kv_heads": 1, "dim": 8, "vdim": 8, "scale": 0.35,
                                                         "softcap": 20.0, "rot": {"base": 100.0, "dims": 8}}},
            {"type": "gla", "mlp": None, "mixer": {"heads": 2, "dim": 16, "vdim": 12, "tau": 8.0, "rank": 5}},
            dict(first, weights_of=0),
        ],
    }
    config.update(changes)
    return config


def test_the_description_names_the_tensors_that_the_design_has():
    from llm_serving_engine_b200.config import load_config
    from llm_serving_engine_b200.models import cache_requirements, expected_tensors
    from llm_serving_engine_b200.parts import PagedKV, RequestState

    config = small_config()
    entry, typed, spec = load_config(config)
    assert entry.name == "Sebudra" and spec.embedding_scale == 4.0 and not spec.tie_word_embeddings
    expected = {name: tuple(item.shape) for name, item in expected_tensors(spec).items()}
    assert expected == {name: shape for name, (shape, _) in plain.tensor_shapes(config).items()}
    assert not any(name.startswith("l3.") for name in expected)       # the fourth layer has no tensors of its own
    assert spec.order == (0, 1, 2, 0) and len(spec.layers) == 3
    assert spec.layers[2].feed_forward is None and spec.layers[0].feed_forward.params["activation"] == "clamped_swish"
    assert all(layer.block.kind == "parallel_residual" and layer.feed_forward_norm is None for layer in spec.layers)
    mixture = spec.layers[1].feed_forward.params
    assert mixture["scores"] == "sigmoid" and mixture["groups"] == {"count": 3, "keep": 2} and mixture["router_scale"] == 1.25
    branches = spec.layers[0].mixer.params["branches"]
    assert [b["scale"] for b in branches] == [0.7, 1.3] and branches[0]["params"]["window"] == 9
    assert spec.layers[1].mixer.params["weights"] == "sigmoid" and spec.layers[1].mixer.params["window"] == 0
    needs = cache_requirements(spec)
    side_by_side = (PagedKV(2, 8, 9, 12), RequestState((4, 6, 10)), RequestState((2, 40 + 2 * 2 * 6)))
    assert needs[0] == side_by_side and needs[3] == side_by_side      # the second run keeps a cache of its own
    assert needs[1] == PagedKV(1, 8, 0, 0) and needs[2] == RequestState((2, 16, 12))


def test_a_size_that_only_a_tensor_gives_is_read_from_the_checkpoint(tmp_path):
    """The rank of a decay map is in no key of the design's own: with a checkpoint beside config.json it is the first
    dimension of the layer's ``mix.a1``."""
    from llm_serving_engine_b200.config import load_config

    config = small_config()
    weights = plain.random_weights(config, seed=3)
    del config["layers"][2]["mixer"]["rank"]
    plain.write_model(tmp_path, config, seed=0, weights=weights)
    _, typed, spec = load_config(tmp_path)
    assert spec.layers[2].mixer.params["rank"] == 5
    from llm_serving_engine_b200.config.model_config import ConfigError

    with pytest.raises(ConfigError, match="rank"):
        load_config(config)


@pytest.mark.parametrize("change,message", [
    ({"layers": [{"type": "other", "mixer": {}}]}, "unknown type"),
    ({"layers": [{"type": "gla", "mixer": {"heads": 2}, "mlp": None}]}, "lacks"),
    ({"layers": [{"type": "parallel", "mixer": {"left": {}, "right": {}, "left_scale": 1, "right_scale": 1}}]}, "lacks"),
    ({"layers": [{"type": "gla", "mixer": {"heads": 2, "dim": 4, "vdim": 4, "tau": 2.0, "rank": 2}, "mlp": None, "weights_of": 0}]},
     "weights_of"),
    ({"layers": [{"type": "gla", "mixer": {"heads": 2, "dim": 4, "vdim": 4, "tau": 2.0, "rank": 2},
                  "mlp": {"kind": "moe", "router": {"experts": 6, "top": 3, "groups": {"count": 3, "keep": 1}}, "expert": {"ff": 8}}}]},
     "fewer experts"),
    ({"norm": {}}, "norm.eps"),
    ({"vocab": 0}, "positive"),
])
def test_a_configuration_that_cannot_run_is_refused_with_the_reason(change, message):
    from llm_serving_engine_b200.config import load_config
    from llm_serving_engine_b200.config.model_config import ConfigError

    with pytest.raises(ConfigError, match=message):
        load_config(small_config(**change))


def test_every_run_of_a_layer_gets_pages_and_states_of_its_own():
    """The layer that runs twice: two views with pages of their own in the windowed group and states of their own, one
    slot per request for all of them; the states of a slot are zeroed when it is taken again."""
    from llm_serving_engine_b200.cache.manager import CacheManager
    from llm_serving_engine_b200.config import CacheConfig, load_config
    from llm_serving_engine_b200.models import cache_requirements

    _, _, spec = load_config(small_config())
    cache = CacheManager(cache_requirements(spec), CacheConfig(block_size=4, num_blocks=6), torch.float32, "cpu", 64,
                         num_state_slots=2)
    first, second = cache.layer_view(0), cache.layer_view(3)
    assert first.parts[0].keys.shape == (6, 2, 4, 8) and first.parts[0].values.shape == (6, 2, 4, 12)
    assert first.parts[0].keys.data_ptr() != second.parts[0].keys.data_ptr()
    assert first.parts[1].state.shape == (2, 4, 6, 10) and first.parts[2].state.shape == (2, 2, 64)
    assert first.parts[1].state.data_ptr() != second.parts[1].state.data_ptr()
    assert cache.layer_view(2).state.shape == (2, 2, 16, 12)
    taken = cache.create("a")
    cache.reserve("a", 9)
    second.parts[1].state[taken.state_slot].fill_(3.0)
    cache.layer_view(2).state[taken.state_slot].fill_(5.0)
    cache.create("b")
    cache.free("a")
    again = cache.create("c")
    assert again.state_slot == taken.state_slot
    assert float(second.parts[1].state[again.state_slot].abs().max()) == 0.0
    assert float(cache.layer_view(2).state[again.state_slot].abs().max()) == 0.0


def test_the_plain_recurrences_agree_with_their_closed_forms():
    torch.manual_seed(1)
    count, heads, n, e = 17, 2, 3, 4
    x = torch.randn(count, heads, e, dtype=torch.float64)
    b, c = torch.randn(count, heads, n, dtype=torch.float64), torch.randn(count, heads, n, dtype=torch.float64)
    dt, rate = torch.rand(count, heads, dtype=torch.float64) + 0.1, torch.rand(heads, dtype=torch.float64) + 0.2
    skip = torch.randn(heads, dtype=torch.float64)
    got = plain.state_space_scan(x, dt, rate, b, c, skip)
    for t in (0, 5, 16):
        for h in range(heads):
            want = skip[h] * x[t, h]
            for s in range(t + 1):
                weight = torch.exp(-rate[h] * dt[s + 1:t + 1, h].sum()) * dt[s, h] * (b[s, h] @ c[t, h])
                want = want + weight * x[s, h]
            assert torch.allclose(got[t, h], want, rtol=1e-9, atol=1e-12)
    q, k = torch.randn(count, heads, n, dtype=torch.float64), torch.randn(count, heads, n, dtype=torch.float64)
    keep = torch.rand(count, heads, n, dtype=torch.float64)
    got = plain.decayed_memory(q, k, x, keep)
    for t in (0, 6, 16):
        for h in range(heads):
            want = torch.zeros(e, dtype=torch.float64)
            for s in range(t + 1):
                want = want + ((keep[s + 1:t + 1, h].prod(0) * k[s, h]) @ q[t, h]) * x[s, h]
            assert torch.allclose(got[t, h], want, rtol=1e-9, atol=1e-12)


def test_the_window_the_cap_and_the_unnormalised_weights_of_the_plain_attentions():
    torch.manual_seed(2)
    config = small_config()
    weights = {name: tensor.double() for name, tensor in plain.random_weights(config, seed=4).items()}
    h = torch.randn(30, 48, dtype=torch.float64)
    left = config["layers"][0]["mixer"]["left"]
    whole = plain.window_attention(h, weights, "l0.mix.left.", left, 1e-5)
    tail = plain.window_attention(h[12:], weights, "l0.mix.left.", left, 1e-5)
    # a row's output depends on the last `size` rows only, up to the rotation, which is relative: rows beyond the window
    # of the cut sequence's rows agree with the whole sequence's
    assert torch.allclose(whole[12 + 8:], tail[8:], atol=1e-9)
    assert not torch.allclose(whole[12 + 7], tail[7], atol=1e-6)
    mixer = config["layers"][1]["mixer"]
    once = plain.sigmoid_attention(h, weights, "l1.mix.", mixer, 1e-5)
    assert once.shape == (30, 48)
    capped = dict(mixer, softcap=1e-3)       # every score nearly zero: every visible key weighs sigmoid(pb)
    out = plain.sigmoid_attention(h, weights, "l1.mix.", capped, 1e-5)
    v = (h @ weights["l1.mix.v"].t()).view(30, 1, 8)
    share = torch.sigmoid(weights["l1.mix.pb"])
    want = torch.stack([torch.cat([share[head] * v[:t + 1, 0].sum(0) for head in range(3)]) for t in range(30)])
    assert torch.allclose(out, want @ weights["l1.mix.o"].t(), atol=2e-2 * float(want.abs().max()))


def test_the_plain_router_keeps_to_the_best_groups():
    torch.manual_seed(3)
    router = {"experts": 6, "top": 2, "scale": 1.25, "groups": {"count": 3, "keep": 1}}
    w = {"router": torch.eye(6, dtype=torch.float64), "correction": torch.tensor([0.0, 0.0, 0.0, 0.0, 0.3, 0.3], dtype=torch.float64)}
    logits = torch.tensor([[4.0, -4.0, 1.0, 1.2, 0.9, 1.0]], dtype=torch.float64)
    chosen, weights = plain.route(logits, w, "", router)
    # group 0 holds the largest score but sums to less than group 2 with its corrections; group 2 is the one kept
    assert sorted(chosen[0].tolist()) == [4, 5]
    scores = torch.sigmoid(logits[0, 4:])
    assert torch.allclose(weights[0].sort().values, (scores / scores.sum() * 1.25).sort().values)
    assert math.isclose(float(weights.sum()), 1.25, rel_tol=1e-12)


def test_the_command_line_has_a_stand_in_of_the_design():
    from llm_serving_engine_b200.cli import tiny_config
    from llm_serving_engine_b200.config import load_config

    _, _, spec = load_config(tiny_config(300, "sebudra"))
    assert spec.architecture == "Sebudra" and spec.vocab_size == 300 and len(spec.layers) == 3 and spec.order == (0, 1, 2, 0)
    assert [layer.mixer.kind for layer in spec.layers] == ["parallel_mixers", "head_norm_rotary_attention",
                                                           "channel_decay_linear_attention"]
