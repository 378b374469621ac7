"""Doderax without a GPU: configuration -> model description, tensor names and shapes, what the cache manager is
asked for and how a window with kept first tokens gives pages back; fixed points of the plain implementation."""

import math

import pytest
import torch

import plain_doderax as plain
from doderax_configs import ALL, DODERAX_X, DODERAX_Y, make_folder

from libmir_b200.cache import CacheManager
from libmir_b200.config.spec import CacheBundle, FixedState, PagedKv, bundle_requirements, split_requirement
from libmir_b200.errors import ConfigError
from libmir_b200.models.decoder import DecoderModel
from libmir_b200.parts.base import BuildEnv
from libmir_b200.registry import architecture_of, build_spec
from libmir_b200.weights import catalog_shapes, parameter_specs


def test_the_class_is_chosen_by_the_configuration():
    assert architecture_of(DODERAX_X) == "Doderax"
    assert architecture_of({"architectures": ["LlamaForCausalLM"]}) == "LlamaForCausalLM"
    with pytest.raises(ConfigError):
        architecture_of({"width": 3})


def test_description_and_tensor_names():
    spec = build_spec(DODERAX_X, None)
    kinds = [layer.mixer.kind for layer in spec.layers]
    assert kinds == ["side_by_side", "gated_delta_rule", "gated_delta_rule", "side_by_side"]
    assert all(layer.arrangement == "parallel" and layer.feed_forward_norm is None for layer in spec.layers)
    assert spec.layers[2].feed_forward is None and spec.layers[1].feed_forward.intermediate_size == 128
    left = dict(spec.layers[0].mixer.branches)["left"]
    assert (left.window, left.keep_first, left.value_dim, left.head_dim, left.position.rotary_dim) == (20, 3, 48, 32, 16)
    assert spec.head.scale == 0.5 and spec.embedding.pairs.buckets == 97 and spec.layers[0].mixer_norm.offset == 1.0
    shapes = {name: tuple(param.shape) for name, param in parameter_specs(DODERAX_X).items()}
    assert shapes["embed"] == (211, 96) and shapes["bigram"] == (98, 96) and shapes["final.norm"] == (96,)
    assert shapes["l0.norm1"] == (96,) and shapes["l0.mix.left.q"] == (128, 96) and shapes["l0.mix.left.v"] == (96, 96)
    assert shapes["l0.mix.left.o"] == (96, 192) and shapes["l0.mix.left.out"] == (96,)
    assert shapes["l0.mix.right.q.conv"] == (48, 3) and shapes["l0.mix.right.a"] == (4, 96)
    assert shapes["l0.mix.right.dt_bias"] == (4,) and shapes["l0.mix.right.g"] == (64, 96)
    assert shapes["l1.mix.a2"] == (120, 16) and shapes["l1.mix.dt_bias"] == (120,) and shapes["l1.mix.g2"] == (72, 16)
    assert shapes["l1.mix.A_log"] == (3,) and shapes["l1.mix.norm"] == (24,) and shapes["l1.mlp.up"] == (128, 96)
    assert "l2.mlp.up" not in shapes and "bigram" not in parameter_specs(DODERAX_Y)


def test_ranks_come_from_the_stored_tensors(tmp_path):
    folder = make_folder(tmp_path, DODERAX_Y, seed=1, dtype="float32")
    catalog = dict(catalog_shapes(folder))
    catalog["l1.mix.a1"], catalog["l1.mix.g1"] = (5, 64), (9, 64)
    spec = build_spec(DODERAX_Y, catalog)
    assert (spec.layers[1].mixer.decay_rank, spec.layers[1].mixer.gate_rank) == (5, 9)


@pytest.mark.parametrize("change,text", [
    (lambda c: c["layers"][0].update(type="mamba"), "type"),
    (lambda c: c["layers"][1]["mlp"].update(kind="routed"), "kind"),
    (lambda c: c["layers"][1]["mixer"].pop("conv"), "conv"),
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(heads=3), "multiple"),
])
def test_what_the_configuration_lacks_is_said(change, text):
    import copy
    config = copy.deepcopy(DODERAX_X)
    change(config)
    with pytest.raises(ConfigError, match=text):
        build_spec(config, None)


def test_cache_needs_pages_and_two_states_per_recurrent_mixer():
    spec = build_spec(DODERAX_X, None)
    model = DecoderModel(spec, BuildEnv(torch.float32, torch.device("meta")))
    plan = model.cache_plan()
    first = plan[0].requirement
    assert isinstance(first, CacheBundle) and first.paged == PagedKv(2, 32, 20, 48, 3)
    assert first.states == (FixedState((4, 16, 24)), FixedState((2, 2 * 48 + 64)))
    assert split_requirement(plan[1].requirement) == (None, (FixedState((3, 24, 40)), FixedState((3, 2 * 120 + 72))))
    manager = CacheManager(plan, 8, 30, 2)
    assert len(manager.groups) == 2 and sorted(manager.state_entries) == [0, 1, 2, 3]
    assert all(isinstance(states, tuple) and len(states) == 2 for states in manager.state_entries.values())
    assert bundle_requirements([None, FixedState((3,))]) == FixedState((3,))
    with pytest.raises(ConfigError):
        bundle_requirements([PagedKv(1, 8), PagedKv(1, 8)])


@pytest.mark.parametrize("page,window,keep", [(8, 9, 20), (4, 6, 1), (16, 16, 16), (8, 20, 0)])
def test_a_window_gives_pages_back_but_for_the_kept_first_tokens(page, window, keep):
    from types import SimpleNamespace
    plan = [SimpleNamespace(entry=0, requirement=PagedKv(1, 8, window, None, keep), source=0, writes=True)]
    manager = CacheManager(plan, page, 64, 2)
    sequence = manager.admit("a")
    length = 0
    for count in (3, 1, 30, 1, 1, 17, 2, 40, 1):
        manager.grow(sequence, length + count)
        length += count
        manager.commit(sequence, length, list(range(count)))
        table = sequence.tables[0]
        for position in range(length):
            needed = position < keep or position > length - window      # a later query (>= length) may still see it
            if needed:
                assert table[position // page] >= 0, f"the page of position {position} was given back at length {length}"
        held = sum(1 for p in table if p >= 0)
        assert held <= -(-keep // page) + window // page + 2
        manager.check()
    assert sequence.last_token == 0
    manager.release("a")
    assert manager.groups[0].pool.free == 64


def test_plain_pieces():
    assert plain.token_pair_rows([4, 9, 9], 7, 3, 5) == [7, (4 * 3 + 9 * 5) % 7, (9 * 3 + 9 * 5) % 7]
    mask = plain.visible(6, 2, 1)
    assert mask[5].tolist() == [True, False, False, False, True, True] and mask[1].tolist() == [True, True] + [False] * 4
    x = torch.arange(6, dtype=torch.float64).reshape(3, 2)
    taps = torch.tensor([[1.0, 10.0], [0.0, 1.0]], dtype=torch.float64)
    want = plain.silu(torch.tensor([[0.0, 1.0], [20.0, 3.0], [42.0, 5.0]], dtype=torch.float64))
    assert torch.allclose(plain.short_conv_silu(x, taps), want)
    # with decay 1, beta 1 and orthonormal keys the delta rule stores each value under its key and reads it back
    d = 4
    keys = torch.eye(d, dtype=torch.float64)[:, None, :]
    values = torch.randn(d, 1, 3, dtype=torch.float64)
    read = plain.delta_rule(keys, keys, values, torch.ones(d, 1, dtype=torch.float64), torch.ones(d, 1, d, dtype=torch.float64))
    assert torch.allclose(read, values * d ** -0.5, atol=1e-5)
    assert math.isclose(float(plain.gelu_tanh(torch.tensor(1.0, dtype=torch.float64))), 0.8411919906082768, rel_tol=1e-12)


@pytest.mark.parametrize("name", sorted(ALL))
def test_a_written_folder_is_read_back_and_runs_in_the_plain_implementation(tmp_path, name):
    folder = make_folder(tmp_path, ALL[name], seed=2, dtype="bfloat16")
    config, weights = plain.read_model(folder)
    steps = []
    logits = plain.forward(config, weights, [1, 5, 5, 2, 9, 0, 3], steps)
    assert logits.shape == (7, ALL[name]["vocab"]) and torch.isfinite(logits).all() and len(steps) == len(config["layers"])
    assert float(logits.std()) > 0.05
