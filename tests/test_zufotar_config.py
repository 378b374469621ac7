"""Zufotar without a GPU: configuration -> model description, the order of layer runs, tensor names and shapes, what
the cache manager is asked for; the rotation table against the plain implementation; fixed points of the plain
implementation itself."""

import copy
import math

import pytest
import torch

import plain_zufotar as plain
from zufotar_configs import ALL, ZUFOTAR_A, ZUFOTAR_B, ZUFOTAR_C, make_folder, random_config

from libmir_b200.cache import CacheManager
from libmir_b200.config.spec import CacheBundle, FixedState, PagedKv, YarnScaling
from libmir_b200.errors import ConfigError
from libmir_b200.models.decoder import DecoderModel
from libmir_b200.parts.base import BuildEnv
from libmir_b200.parts.rope import inverse_frequencies, yarn_magnitude
from libmir_b200.registry import architecture_of, build_spec
from libmir_b200.weights import catalog_shapes, parameter_specs


def test_the_class_is_chosen_by_the_configuration():
    assert architecture_of(ZUFOTAR_A) == "Zufotar"
    assert build_spec(ZUFOTAR_A, None).architecture == "Zufotar"


def test_description_and_tensor_names():
    spec = build_spec(ZUFOTAR_A, None)
    assert [layer.mixer.kind for layer in spec.layers] == ["wkv", "latent_attention", "wkv", "latent_attention"]
    assert all(layer.arrangement == "parallel" for layer in spec.layers)
    assert spec.layers[2].feed_forward is None and spec.layers[2].feed_forward_norm is None
    assert spec.layers[1].feed_forward.activation == "gelu_erf" and spec.layers[1].feed_forward_norm is not None
    experts = spec.layers[0].feed_forward
    assert (experts.experts, experts.top, experts.groups, experts.keep_groups, experts.scale, experts.shared_size) == \
        (6, 2, 2, 1, 1.7, 24)
    attention = spec.layers[1].mixer
    assert (attention.heads, attention.head_dim, attention.rotary_dim, attention.value_dim, attention.q_rank,
            attention.kv_rank) == (4, 24, 8, 40, 48, 56)
    assert attention.position.layout == "interleaved" and attention.position.scaling == YarnScaling(4.0, 64.0, 16.0, 2.0)
    assert spec.layers[3].mixer.position.scaling is None
    assert spec.head.tied and spec.head.softcap == 9.0 and spec.embedding.multiplier == 1.5
    shapes = {name: tuple(param.shape) for name, param in parameter_specs(ZUFOTAR_A).items()}
    assert shapes["embed"] == (211, 96) and shapes["loop.step"] == (3, 96) and shapes["final.norm"] == (96,)
    assert shapes["l0.norm1"] == (96,) and shapes["l0.norm2"] == (96,) and "l2.norm2" not in shapes
    assert shapes["l0.mix.mu.w"] == (96,) and shapes["l0.mix.r"] == (96, 96) and shapes["l0.mix.w1"] == (5, 96)
    assert shapes["l0.mix.w2"] == (96, 5) and shapes["l0.mix.u"] == (3, 32) and shapes["l0.mix.norm"] == (96,)
    assert shapes["l1.mix.dq"] == (48, 96) and shapes["l1.mix.uq"] == (4 * 32, 48) and shapes["l1.mix.dkv"] == (64, 96)
    assert shapes["l1.mix.dkv.norm"] == (56,) and shapes["l1.mix.uk"] == (96, 56) and shapes["l1.mix.uv"] == (160, 56)
    assert shapes["l1.mix.g"] == (160, 96) and shapes["l1.mix.o"] == (96, 160) and shapes["l1.mlp.up"] == (160, 96)
    assert shapes["l0.mlp.router"] == (6, 96) and shapes["l0.mlp.correction"] == (6,)
    assert shapes["l0.mlp.e5.gate"] == (40, 96) and shapes["l0.mlp.e5.down"] == (96, 40)
    assert shapes["l0.mlp.shared.up"] == (24, 96) and shapes["l0.mlp.shared.sg"] == (1, 96)
    assert "l3.mlp.shared.sg" not in shapes and "head" not in shapes
    assert "loop.step" not in parameter_specs(ZUFOTAR_C)


def test_the_order_of_layer_runs_follows_the_loop():
    runs = lambda config: [(entry.layer, entry.opens_pass) for entry in build_spec(config, None).schedule]
    assert runs(ZUFOTAR_A) == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (1, 2), (2, None), (3, None)]
    assert runs(ZUFOTAR_B) == [(0, 0), (1, None)]
    assert runs(ZUFOTAR_C) == [(0, None), (1, None), (2, None)]
    for name, config in ALL.items():
        assert runs(config) == plain.layer_order(config), name
    rng = __import__("numpy").random.default_rng(1)
    for _ in range(20):
        config = random_config(rng)
        assert runs(config) == plain.layer_order(config)


def test_every_run_of_a_layer_has_a_cache_or_state_of_its_own():
    spec = build_spec(ZUFOTAR_A, None)
    model = DecoderModel(spec, BuildEnv(torch.float32, torch.device("cpu")))
    plan = model.cache_plan()
    assert all(item.source == item.entry and item.writes for item in plan)
    assert plan[1].requirement == PagedKv(1, 64, None, 0) and plan[3].requirement == plan[1].requirement
    assert plan[0].requirement == CacheBundle(None, (FixedState((3, 32, 32)), FixedState((96,))))
    manager = CacheManager(plan, page_size=8, num_pages=10, max_requests=2)
    assert [len(group.entries) for group in manager.groups] == [3, 1]        # three passes of layer 1; layer 3
    assert sorted(manager.state_entries) == [0, 2, 4, 6]
    assert manager.groups[0].requirement.elements_per_token == 64             # one vector per token, no value rows


def test_the_decay_rank_comes_from_the_stored_tensor(tmp_path):
    folder = make_folder(tmp_path, ZUFOTAR_B, seed=1, dtype="float32")
    catalog = dict(catalog_shapes(folder))
    assert build_spec(ZUFOTAR_B, catalog).layers[1].mixer.decay_rank == 1
    catalog["l1.mix.w1"] = (9, 64)
    assert build_spec(ZUFOTAR_B, catalog).layers[1].mixer.decay_rank == 9


@pytest.mark.parametrize("change,text", [
    (lambda c: c["layers"][0].update(type="mamba"), "type"),
    (lambda c: c["layers"][1]["mlp"].update(kind="routed"), "kind"),
    (lambda c: c["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=4), "rot.dims"),
    (lambda c: c["loop"].update(stop=9), "loop"),
    (lambda c: c.pop("width"), "width"),
])
def test_configuration_errors_name_what_is_wrong(change, text):
    config = copy.deepcopy(ZUFOTAR_A)
    change(config)
    with pytest.raises(ConfigError) as error:
        build_spec(config, None)
    assert text in str(error.value)


@pytest.mark.parametrize("dims,base,scaling", [(8, 10000.0, (4.0, 64, 16.0, 2.0)), (16, 1000000.0, (2.0, 512, 32.0, 1.0)),
                                               (32, 500.0, (16.0, 32, 32.0, 1.0)), (2, 50.0, (1.0, 16, 8.0, 2.0)),
                                               (6, 250000.0, None)])
def test_rotation_table_against_the_plain_implementation(dims, base, scaling):
    rot = {"dims": dims, "base": base}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    want, magnitude = plain.rotary_table(rot)
    yarn = YarnScaling(*map(float, scaling)) if scaling else None
    got = inverse_frequencies(dims, base, yarn)
    assert torch.allclose(got.double(), want, rtol=1e-6, atol=0)
    assert math.isclose(yarn_magnitude(yarn), magnitude, rel_tol=1e-12)


def test_plain_implementation_fixed_points():
    # no scaling: the plain table; a factor of 1 changes nothing; the ramp runs from kept (0) to stretched (1)
    freq, magnitude = plain.rotary_table({"dims": 4, "base": 100.0})
    assert torch.allclose(freq, torch.tensor([1.0, 0.1], dtype=torch.float64)) and magnitude == 1.0
    same, one = plain.rotary_table({"dims": 4, "base": 100.0, "scaling": {"factor": 1.0, "original": 64, "fast": 8.0, "slow": 1.0}})
    assert torch.allclose(same, freq) and one == 1.0
    # interleaved pairs: position 0 turns nothing; at position 1 the first pair (frequency 1) turns by one radian
    x = torch.tensor([[3.0, 4.0, 5.0]], dtype=torch.float64)
    assert torch.equal(plain.rotate_interleaved(x, torch.tensor([0]), {"dims": 2, "base": 7.0}), x)
    turned = plain.rotate_interleaved(x, torch.tensor([1]), {"dims": 2, "base": 7.0})[0]
    assert math.isclose(float(turned[0]), 3.0 * math.cos(1.0) - 4.0 * math.sin(1.0), rel_tol=1e-12)
    assert math.isclose(float(turned[1]), 4.0 * math.cos(1.0) + 3.0 * math.sin(1.0), rel_tol=1e-12) and turned[2] == 5.0
    # the router: the kept group wins although the best single expert lies in the other
    weights = {"m.router": torch.zeros(4, 2, dtype=torch.float64), "m.correction": torch.tensor([0.9, -0.9, 0.5, 0.45], dtype=torch.float64)}
    chosen, share = plain.route(torch.ones(1, 2, dtype=torch.float64), weights, "m.",
                                {"experts": 4, "top": 2, "scale": 3.0, "groups": {"count": 2, "keep": 1}})
    assert sorted(chosen[0].tolist()) == [2, 3] and math.isclose(float(share.sum()), 3.0, rel_tol=1e-12)
    # wkv: one token, the state starts at zero, so the read-out is the bonus term alone
    heads, dim, width = 1, 2, 2
    w = {"p.mu." + n: torch.zeros(width, dtype=torch.float64) for n in "rkvgw"}
    eye = torch.eye(2, dtype=torch.float64)
    w.update({"p.r": eye, "p.k": eye, "p.v": eye, "p.g": eye, "p.o": eye, "p.w1": torch.zeros(1, 2, dtype=torch.float64),
              "p.w2": torch.zeros(2, 1, dtype=torch.float64), "p.w0": torch.zeros(2, dtype=torch.float64),
              "p.u": torch.tensor([[2.0, 0.0]], dtype=torch.float64), "p.norm": torch.ones(2, dtype=torch.float64)})
    h = torch.tensor([[1.0, 3.0]], dtype=torch.float64)
    out = plain.wkv(h, w, "p.", {"heads": heads, "dim": dim}, 0.0)
    o = torch.tensor([2.0 * 1.0, 2.0 * 3.0])                                 # (r . (u * k)) v = 2 * v
    want = o / torch.sqrt((o * o).mean()) * plain.silu(h[0])
    assert torch.allclose(out[0], want.double())
