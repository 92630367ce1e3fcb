"""Host-side pieces of the Fororax design: configuration, description, tensor names, cache needs, the plain
implementation against itself."""
import pytest
import torch

from plain import fororax_plain as plain


def small_config(**changes):
    mlp = {"kind": "moe", "router": {"experts": 3, "identity": 2, "top": 2}, "expert": {"ff": 24, "limit": 0.5},
           "shared": {"ff": 16, "limit": 1.5}}
    config = {
        "architecture": "Fororax", "vocab": 97, "width": 48, "max_positions": 128, "norm": {"eps": 1e-5},
        "postln_alpha": 1.5, "embedding": {"scale": 0.25}, "logit_softcap": 8.0,
        "layers": [
            {"type": "attention_2", "mlp": mlp, "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 12, "scale": 0.3}},
            {"type": "attention", "mlp": None, "mixer": {"heads": 2, "kv_heads": 1, "dim": 16, "vdim": 16, "scale": 0.25}},
            {"type": "attention", "mlp": dict(mlp, shared=None),
             "mixer": {"heads": 3, "kv_heads": 1, "dim": 16, "vdim": 16, "scale": 0.25, "kv_from": 1}},
        ],
    }
    config.update(changes)
    return config


def test_the_description_names_the_tensors_that_the_design_has():
    from llm_serving_engine_b200.config import load_config
    from llm_serving_engine_b200.models import cache_requirements, expected_tensors
    from llm_serving_engine_b200.parts import PagedKV

    config = small_config()
    entry, typed, spec = load_config(config)
    assert entry.name == "Fororax" and typed.postln_alpha == 1.5 and spec.embedding_scale == 0.25
    assert spec.logit_softcap == 8.0 and spec.position_table_name == "pos" and not spec.tie_word_embeddings
    expected = {name: tuple(item.shape) for name, item in expected_tensors(spec).items()}
    assert expected == plain.tensor_shapes(config)
    assert spec.layers[1].feed_forward is None and spec.layers[2].cache_from == 1
    assert spec.layers[0].mixer.params["sink"] and not spec.layers[1].mixer.params["sink"]
    assert spec.layers[1].mixer.params["distance_penalty"] and not spec.layers[2].mixer.params["own_cache"]
    assert cache_requirements(spec) == [PagedKV(2, 8, 0, 12), PagedKV(1, 16, 0, 0), 1]


def test_the_correction_follows_the_tensors_where_there_are_some():
    from llm_serving_engine_b200.config import FororaxConfig

    assert FororaxConfig.from_dict(small_config()).router_correction
    assert not FororaxConfig.from_dict(small_config(), tensor_names=frozenset({"l0.mlp.router"})).router_correction
    assert FororaxConfig.from_dict(small_config(), tensor_names=frozenset({"l0.mlp.correction"})).router_correction


def _broken(index, **mixer):
    config = small_config()
    config["layers"][index]["mixer"].update(mixer)
    return {"layers": config["layers"]}


@pytest.mark.parametrize("change,message", [
    ({"layers": [{"type": "other", "mixer": {}}]}, "unknown type"),
    ({"layers": [{"type": "attention", "mixer": {"heads": 2}, "mlp": None}]}, "lacks"),
    (_broken(0, heads=3), "multiple"),
    (_broken(2, kv_from=2), "earlier"),
    (_broken(2, vdim=8), "same"),
    (_broken(0, kv_from=0), "only attention"),
    ({"norm": {}}, "eps"),
])
def test_configurations_that_cannot_run_are_refused(change, message):
    from llm_serving_engine_b200.config import ConfigError, load_config

    with pytest.raises(ConfigError, match=message):
        load_config(small_config(**change))


def test_keys_and_values_of_different_sizes_get_their_own_tensors():
    from llm_serving_engine_b200.cache import CacheManager
    from llm_serving_engine_b200.config import CacheConfig, load_config
    from llm_serving_engine_b200.models import cache_requirements

    _, _, spec = load_config(small_config())
    cache = CacheManager(cache_requirements(spec), CacheConfig(block_size=8, num_blocks=6), torch.float32, "cpu", 128,
                         num_state_slots=2)
    assert [tuple(group.storage.shape) for group in cache.groups] == [(1, 1, 6, 2, 8, 8), (1, 2, 6, 1, 8, 16)]
    first, second, reader = cache.layer_view(0), cache.layer_view(1), cache.layer_view(2)
    assert tuple(first.keys.shape) == (6, 2, 8, 8) and tuple(first.values.shape) == (6, 2, 8, 12)
    assert tuple(second.keys.shape) == tuple(second.values.shape) == (6, 1, 8, 16)
    assert reader.keys.data_ptr() == second.keys.data_ptr() and reader.values.data_ptr() == second.values.data_ptr()
    assert cache.kv_bytes_per_token() == (2 * (8 + 12) + 1 * (16 + 16)) * 4
    cache.create("a")
    cache.reserve("a", 20)
    assert cache.free_pages() == [3, 3]
    cache.free("a")
    assert cache.free_pages() == [6, 6]


def test_random_weights_of_the_design_are_usable():
    """The random-weights mode draws the penalty's constants positive (a negative one would put a negative number
    under the logarithm at some distance)."""
    from llm_serving_engine_b200.config import load_config
    from llm_serving_engine_b200.models import expected_tensors
    from llm_serving_engine_b200.weights.random_init import random_weights

    _, _, spec = load_config(small_config())
    weights = random_weights(expected_tensors(spec), seed=4)
    assert float(weights["l1.mix.r1"].min()) > 0 and float(weights["l2.mix.r2"].min()) > 0
    assert weights["l0.mix.talk"].shape == (4, 4) and weights["pos"].shape == (128, 48)


def test_the_plain_pieces_agree_with_each_other():
    """The plain implementation against simpler forms of its own pieces: the mixing of the heads' weights equals a
    mix of the heads' outputs over the same values; a sink of minus infinity is no sink; the distance penalty is
    zero at distance zero; a mixture whose router picks only identity experts returns the scaled input."""
    torch.manual_seed(0)
    q, k, v = torch.randn(9, 4, 8, dtype=torch.float64), torch.randn(9, 2, 8, dtype=torch.float64), torch.randn(9, 2, 5, dtype=torch.float64)
    weights = plain.softmax_with_sink(plain.causal_scores(q, k, 0.4), torch.full((4,), -1e30, dtype=torch.float64))
    assert torch.allclose(weights, torch.softmax(plain.causal_scores(q, k, 0.4), -1))
    assert torch.allclose(weights.sum(-1), torch.ones(4, 9, dtype=torch.float64))
    table = torch.randn(4, 4, dtype=torch.float64)
    mixed = plain.apply_weights(plain.mix_heads(weights, table), v).view(9, 4, 5)
    per_group = torch.einsum("hij,jgd->ihgd", weights, v)                   # head h's weights on group g's values
    for head in range(4):
        want = sum(table[head, other] * per_group[:, other, head // 2] for other in range(4))
        assert torch.allclose(mixed[:, head], want)
    penalty = plain.distance_penalty(6, torch.tensor([0.5, 2.0], dtype=torch.float64), torch.tensor([1.0, 0.1], dtype=torch.float64))
    assert float(penalty.diagonal(dim1=1, dim2=2).abs().max()) == 0.0 and float(penalty[1, 5, 0]) == pytest.approx(2.0 * 0.4054651081)
    x = torch.randn(3, 8, dtype=torch.float64)
    mlp = {"router": {"experts": 1, "identity": 2, "top": 2}, "expert": {"ff": 4, "limit": 1.0}}
    w = {"m.router": torch.randn(3, 8, dtype=torch.float64), "m.correction": torch.tensor([-10.0, 0.0, 0.0], dtype=torch.float64)}
    for name, shape in (("gate", (4, 8)), ("up", (4, 8)), ("down", (8, 4))):
        w["m.e0." + name] = torch.randn(shape, dtype=torch.float64)
    scores = torch.softmax(x @ w["m.router"].t(), -1)
    assert torch.allclose(plain.mixture(x, w, "m.", mlp), x * scores[:, 1:].sum(-1, keepdim=True))


def test_the_command_line_has_a_stand_in_of_the_design():
    from llm_serving_engine_b200.cli import tiny_config
    from llm_serving_engine_b200.config import load_config

    _, _, spec = load_config(tiny_config(300, "fororax"))
    assert spec.architecture == "Fororax" and spec.vocab_size == 300 and len(spec.layers) == 3
