"""Host-side pieces of the Tufevik design: configuration, description, tensor names, cache needs and slots, the plain
implementation's pieces against each other."""
import pytest
import torch

from plain import tufevik_plain as plain


def small_config(**changes):
    mlp = {"kind": "moe", "router": {"experts": 3, "top": 2}, "expert": {"ff": 24}}
    left = {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 12, "conv": 3, "scale": 0.3,
            "rot": {"base": 500.0, "dims": 4, "scaling": {"factor": 3.0, "original": 64, "fast": 8.0, "slow": 1.0}}}
    right = {"inner": 40, "state": 6, "dt_rank": 5, "conv": 2}
    config = {
        "architecture": "Tufevik", "vocab": 97, "width": 48, "norm": {"eps": 1e-5}, "embedding": {"scale": 0.25},
        "layers": [
            {"type": "parallel", "mlp": mlp, "mixer": {"left": left, "right": right, "left_scale": 0.7, "right_scale": 1.3}},
            {"type": "mlstm", "mlp": None, "mixer": {"heads": 3, "dim": 8, "vdim": 10, "gate_cap": 12.0}},
            {"type": "mlstm", "mlp": {"kind": "dense", "ff": 56}, "mixer": {"heads": 2, "dim": 16, "vdim": 16, "gate_cap": 9.0}},
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
    assert entry.name == "Tufevik" and spec.embedding_scale == 0.25 and spec.tie_word_embeddings
    expected = {name: tuple(item.shape) for name, item in expected_tensors(spec).items()}
    assert expected == plain.tensor_shapes(config)
    assert spec.layers[1].feed_forward is None and spec.layers[2].feed_forward.params["activation"] == "relu"
    assert spec.layers[0].feed_forward.params["weights"] == "softmax_chosen"
    branches = spec.layers[0].mixer.params["branches"]
    assert [b["scale"] for b in branches] == [0.7, 1.3] and branches[0]["params"]["conv"] == 3
    needs = cache_requirements(spec)
    assert needs[0] == (PagedKV(2, 8, 0, 12), RequestState((2, 4 * 8 + 2 * 8 + 2 * 12)), RequestState((40, 6)),
                        RequestState((1, 40)))
    assert needs[1] == (RequestState((3, 8, 11)), RequestState((3,)))


@pytest.mark.parametrize("change,message", [
    ({"layers": [{"type": "other", "mixer": {}}]}, "unknown type"),
    ({"layers": [{"type": "mlstm", "mixer": {"heads": 2}, "mlp": None}]}, "lacks"),
    ({"layers": [{"type": "parallel", "mixer": {"left": {}, "right": {}, "left_scale": 1, "right_scale": 1}}]}, "lacks"),
    ({"norm": {}}, "norm.eps"),
    ({"vocab": 0}, "positive"),
])
def test_a_configuration_that_cannot_run_is_refused_with_the_reason(change, message):
    from llm_serving_engine_b200.config import load_config
    from llm_serving_engine_b200.config.model_config import ConfigError

    with pytest.raises(ConfigError, match=message):
        load_config(small_config(**change))


def test_a_mixer_with_several_needs_gets_a_view_per_need_and_one_slot():
    """Pages and three states for the parallel layer, two states for a matrix memory; a request takes one slot for all
    of them, the states of a slot are zeroed when it is taken again, pages go back."""
    from llm_serving_engine_b200.cache.manager import CacheManager
    from llm_serving_engine_b200.config import CacheConfig, load_config
    from llm_serving_engine_b200.models import cache_requirements

    _, _, spec = load_config(small_config())
    cache = CacheManager(cache_requirements(spec), CacheConfig(block_size=4, num_blocks=6), torch.float32, "cpu", 64,
                         num_state_slots=2)
    view = cache.layer_view(0)
    assert [part.group for part in view.parts] == [0, -1, -1, -1]
    assert view.parts[0].keys.shape == (6, 2, 4, 8) and view.parts[0].values.shape == (6, 2, 4, 12)
    assert view.parts[1].state.shape == (2, 2, 72) and view.parts[2].state.shape == (2, 40, 6)
    memory = cache.layer_view(1)
    assert memory.parts[0].state.shape == (2, 3, 8, 11) and memory.parts[1].state.shape == (2, 3)
    first = cache.create("a")
    cache.reserve("a", 9)
    memory.parts[0].state[first.state_slot].fill_(3.0)
    view.parts[2].state[first.state_slot].fill_(5.0)
    assert cache.free_pages() == [3]
    cache.create("b")
    cache.free("a")
    assert cache.free_pages() == [6]
    again = cache.create("c")
    assert again.state_slot == first.state_slot
    assert float(memory.parts[0].state[again.state_slot].abs().max()) == 0.0
    assert float(view.parts[2].state[again.state_slot].abs().max()) == 0.0


def test_the_plain_pieces_agree_with_each_other():
    """The recurrences of the plain implementation do not depend on where a sequence is cut when their state is
    carried: the matrix memory against its closed form, the convolution against a shifted sum."""
    torch.manual_seed(1)
    count, heads, d, e = 19, 2, 4, 5
    q, k = torch.randn(count, heads, d, dtype=torch.float64), torch.randn(count, heads, d, dtype=torch.float64)
    v = torch.randn(count, heads, e, dtype=torch.float64)
    i, f = torch.randn(count, heads, dtype=torch.float64) * 2, -torch.rand(count, heads, dtype=torch.float64)
    got = plain.mlstm_recurrence(q, k, v, i, f)
    # closed form: weights exp(i_s + sum_{r>s} f_r), the maximum taken off, the floor exp(-m)
    for t in (0, 7, 18):
        for h in range(heads):
            logs = torch.stack([i[s, h] + f[s + 1:t + 1, h].sum() for s in range(t + 1)])
            m = torch.maximum(logs.max(), f[:t + 1, h].sum())      # the maximum that starts at zero decays with f
            weights = torch.exp(logs - m)
            memory = torch.einsum("s,sd,se->de", weights, k[:t + 1, h], v[:t + 1, h])
            normaliser = torch.einsum("s,sd->d", weights, k[:t + 1, h])
            want = memory.t() @ q[t, h] / (torch.maximum((normaliser @ q[t, h]).abs(), torch.exp(-m)) + 1e-6)
            assert torch.allclose(got[t, h], want, rtol=1e-9, atol=1e-12)
    u, taps = torch.randn(11, 3, dtype=torch.float64), torch.randn(3, 4, dtype=torch.float64)
    y = plain.causal_conv(u, taps)
    assert torch.allclose(y[0], taps[:, 3] * u[0]) and torch.allclose(y[5], sum(taps[:, j] * u[5 - 3 + j] for j in range(4)))


def test_the_softmax_over_the_chosen_logits_only():
    torch.manual_seed(2)
    h = torch.randn(6, 8, dtype=torch.float64)
    w = {"router": torch.randn(5, 8, dtype=torch.float64), "router.b": torch.randn(5, dtype=torch.float64)}
    chosen, weights = plain.route(h, w, "", 3)
    logits = h @ w["router"].t() + w["router.b"]
    assert torch.allclose(weights.sum(-1), torch.ones(6, dtype=torch.float64))
    for t in range(6):
        assert set(chosen[t].tolist()) == set(logits[t].argsort(descending=True)[:3].tolist())
        assert torch.allclose(weights[t], torch.softmax(logits[t][chosen[t]], dim=-1))


def test_the_command_line_has_a_stand_in_of_the_design():
    from llm_serving_engine_b200.cli import tiny_config
    from llm_serving_engine_b200.config import load_config

    _, _, spec = load_config(tiny_config(300, "tufevik"))
    assert spec.architecture == "Tufevik" and spec.vocab_size == 300 and len(spec.layers) == 3
    assert [layer.mixer.kind for layer in spec.layers] == ["mlstm", "parallel_mixers", "mlstm"]
