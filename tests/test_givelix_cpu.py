"""Host-side pieces of the Givelix design: configuration, description, tensor names, cache needs, frequencies."""
import pytest
import torch

from plain import givelix_plain as plain


def small_config(**changes):
    rot = {"base": 10000.0, "dims": 8}
    config = {
        "architecture": "Givelix", "vocab": 97, "width": 48, "norm": {"eps": 1e-5}, "residual_mult": 0.25, "streams": 2,
        "logit_scale": 2.0,
        "layers": [
            {"type": "latent_attention", "mlp": {"kind": "dense", "ff": 64},
             "mixer": {"heads": 2, "dim": 8, "rot_dim": 8, "vdim": 12, "kv_rank": 20, "q_rank": 16, "scale": 0.25, "rot": rot}},
            {"type": "lightning", "mlp": None, "mixer": {"heads": 3, "dim": 8, "vdim": 4, "decay": [0.5, 0.9, 0.99]}},
            {"type": "latent_attention", "mlp": None,
             "mixer": {"heads": 1, "dim": 4, "rot_dim": 8, "vdim": 4, "kv_rank": 20, "q_rank": 8, "scale": 0.3, "rot": rot, "kv_from": 0}},
            {"type": "latent_attention_2", "mlp": {"kind": "dense", "ff": 32},
             "mixer": {"heads": 2, "dim": 8, "rot_dim": 4, "vdim": 8, "kv_rank": 12, "scale": 0.3,
                       "rot": {"base": 100.0, "dims": 4, "scaling": {"factor": 2.0, "original": 32, "fast": 4.0, "slow": 1.0}}}},
        ],
    }
    config.update(changes)
    return config


def test_the_description_names_the_tensors_that_the_design_has():
    from llm_serving_engine_b200.config import load_config
    from llm_serving_engine_b200.models import cache_requirements, expected_tensors
    from llm_serving_engine_b200.parts import PagedLatent, RequestState

    config = small_config()
    entry, typed, spec = load_config(config)
    assert entry.name == "Givelix" and typed.hyper_connections and spec.residual_streams == 2 and spec.logit_scale == 2.0
    expected = {name: tuple(item.shape) for name, item in expected_tensors(spec).items()}
    assert expected == plain.tensor_shapes(config)
    assert spec.layers[1].feed_forward is None and spec.layers[2].cache_from == 0
    needs = cache_requirements(spec)
    assert needs == [PagedLatent(28), RequestState((3, 8, 4), "float32"), 0, PagedLatent(16)]


def test_streams_and_scales_follow_the_file_or_the_tensors():
    from llm_serving_engine_b200.config import GivelixConfig, load_config
    from llm_serving_engine_b200.models import expected_tensors

    plain_config = small_config()
    del plain_config["streams"]
    _, typed, spec = load_config(plain_config)
    assert typed.streams == 1 and not typed.hyper_connections
    assert not any(".hc" in name for name in expected_tensors(spec))
    # a checkpoint's tensor names decide where the file is silent
    typed = GivelixConfig.from_dict(small_config(), tensor_names=frozenset({"l0.hc1.in"}))
    assert typed.hyper_connections and not typed.layer_scale


@pytest.mark.parametrize("change,message", [
    ({"streams": 9}, "streams"),
    ({"layers": [{"type": "other", "mixer": {}}]}, "unknown type"),
    ({"layers": [{"type": "lightning", "mixer": {"heads": 2, "dim": 4, "vdim": 4, "decay": [0.5]}, "mlp": None}]}, "decays"),
    ({"layers": [{"type": "latent_attention_2", "mlp": None,
                  "mixer": {"heads": 1, "dim": 4, "rot_dim": 4, "vdim": 4, "kv_rank": 4, "scale": 1.0, "rot": {"base": 10.0, "dims": 6}}}]},
     "rot.dims"),
])
def test_configurations_that_cannot_run_are_refused(change, message):
    from llm_serving_engine_b200.config import ConfigError, load_config

    with pytest.raises(ConfigError, match=message):
        load_config(small_config(**change))


def test_a_layer_may_read_only_an_earlier_cache_of_its_own_shape():
    from llm_serving_engine_b200.config import ConfigError, load_config

    config = small_config()
    config["layers"][2]["mixer"]["kv_rank"] = 24
    with pytest.raises(ConfigError, match="kv_from|same"):
        load_config(config)


def test_scaled_frequencies_equal_the_plain_ones():
    from llm_serving_engine_b200.parts.latent_attention import rotary_frequencies

    for rot in ({"base": 500.0, "dims": 16},
                {"base": 10000.0, "dims": 32, "scaling": {"factor": 8.0, "original": 128, "fast": 16.0, "slow": 2.0}},
                {"base": 100.0, "dims": 4, "scaling": {"factor": 2.0, "original": 32, "fast": 4.0, "slow": 1.0}}):
        ours, factor = rotary_frequencies(rot)
        theirs, their_factor = plain.rotary_frequencies(rot)
        assert torch.equal(ours, theirs) and factor == their_factor


def test_latent_rows_get_pages_and_states_get_slots():
    from llm_serving_engine_b200.cache import CacheManager
    from llm_serving_engine_b200.config import CacheConfig, load_config
    from llm_serving_engine_b200.models import cache_requirements

    _, _, spec = load_config(small_config())
    cache = CacheManager(cache_requirements(spec), CacheConfig(block_size=8, num_blocks=6), torch.float32, "cpu", 64,
                         num_state_slots=2)
    assert [tuple(group.storage.shape) for group in cache.groups] == [(1, 1, 6, 8, 28), (1, 1, 6, 8, 16)]
    assert cache.layer_view(2).keys.data_ptr() == cache.layer_view(0).keys.data_ptr()      # the reader sees layer 0's rows
    assert tuple(cache.layer_view(1).state.shape) == (2, 3, 8, 4) and cache.layer_view(0).values is None
    first = cache.create("a")
    cache.layer_view(1).state[first.state_slot].fill_(3.0)
    cache.reserve("a", 20)
    assert cache.free_pages() == [3, 3]
    cache.free("a")
    cache.create("b")
    again = cache.create("c")
    assert again.state_slot == first.state_slot and float(cache.layer_view(1).state[again.state_slot].abs().max()) == 0.0
    saved = cache.snapshot_states()
    cache.layer_view(1).state.fill_(1.0)
    cache.restore_states(saved)
    assert float(cache.layer_view(1).state.abs().max()) == 0.0


def test_the_command_line_has_a_stand_in_of_the_design():
    from llm_serving_engine_b200.cli import tiny_config
    from llm_serving_engine_b200.config import load_config

    _, _, spec = load_config(tiny_config(300, "givelix"))
    assert spec.architecture == "Givelix" and spec.vocab_size == 300 and len(spec.layers) == 4
