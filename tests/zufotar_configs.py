"""Tiny Zufotar configurations for the tests, and model folders with weights that make every mechanism matter.
The configurations differ from one another in every size, in the order and kinds of layers, in the loop, the router's
groups and constants; some take values that make two sizes equal or 1, some leave optional keys out."""

from __future__ import annotations

from pathlib import Path

import torch


def _rot(dims, base, scaling=None):
    rot = {"dims": dims, "base": base}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return rot


def _latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, base=10000.0, scaling=None):
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
             "scale": scale}
    if rot_dim:
        mixer["rot"] = _rot(rot_dim, base, scaling)
    return {"type": "latent_attention", "mixer": mixer}


def _wkv(heads, dim, rank):
    return {"type": "wkv", "mixer": {"heads": heads, "dim": dim, "decay_rank": rank}}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(experts, top, ff, groups=None, scale=1.0, shared=0):
    router = {"experts": experts, "top": top, "scale": scale}
    if groups:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    mlp = {"kind": "moe", "expert": {"ff": ff}, "router": router}
    if shared:
        mlp["shared"] = {"ff": shared}
    return mlp


def _layer(mixer, mlp):
    return dict(mixer, mlp=mlp)


ZUFOTAR_A = {   # a loop in the middle, three passes; value heads wider than key heads; groups of three experts
    "architecture": "Zufotar", "vocab": 211, "width": 96, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.5},
    "logit_softcap": 9.0, "loop": {"start": 1, "stop": 3, "times": 3},
    "layers": [
        _layer(_wkv(3, 32, 5), _moe(6, 2, 40, groups=(2, 1), scale=1.7, shared=24)),
        _layer(_latent(4, 24, 8, 40, 48, 56, 0.2, base=10000.0, scaling=(4.0, 64, 16.0, 2.0)), _dense(160)),
        _layer(_wkv(2, 48, 12), None),
        _layer(_latent(3, 32, 16, 16, 24, 40, 0.17, base=500.0), _moe(8, 3, 24, groups=(4, 3), scale=1.0)),
    ],
}

ZUFOTAR_B = {   # sizes that are equal or 1: one head, one expert chosen, one group, one pass, no cap, no scaling
    "architecture": "Zufotar", "vocab": 130, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0},
    "loop": {"start": 0, "stop": 2, "times": 1},
    "layers": [
        _layer(_latent(1, 16, 2, 16, 16, 16, 0.25, base=100.0), _moe(2, 1, 64, shared=64)),
        _layer(_wkv(1, 64, 1), _dense(64)),
    ],
}

ZUFOTAR_C = {   # no loop at all, a width and head sizes that are no multiples of 8, many experts without a shared one
    "architecture": "Zufotar", "vocab": 150, "width": 100, "norm": {"eps": 1e-5}, "logit_softcap": 30.0,
    "layers": [
        _layer(_latent(5, 12, 6, 20, 30, 44, 0.3, base=250000.0, scaling=(2.0, 40, 8.0, 1.0)), _moe(12, 4, 36, groups=(3, 2), scale=2.5)),
        _layer(_wkv(5, 20, 7), _moe(4, 4, 20, scale=0.5, shared=52)),
        _layer(_latent(2, 40, 0, 24, 64, 72, 0.15), None),
    ],
}

ZUFOTAR_D = {   # the whole model is the loop; heads of 128 channels; every expert in a group of its own
    "architecture": "Zufotar", "vocab": 97, "width": 128, "norm": {"eps": 1e-6}, "embedding": {"scale": 0.25},
    "logit_softcap": 5.0, "loop": {"start": 0, "stop": 2, "times": 2},
    "layers": [
        _layer(_wkv(1, 128, 16), _moe(5, 2, 48, groups=(5, 3), scale=1.0, shared=16)),
        _layer(_latent(2, 64, 32, 64, 96, 128, 0.1, base=1000000.0, scaling=(8.0, 32, 32.0, 1.0)), _dense(200)),
    ],
}

ALL = {"A": ZUFOTAR_A, "B": ZUFOTAR_B, "C": ZUFOTAR_C, "D": ZUFOTAR_D}
PAGE_SIZES = {"A": 8, "B": 16, "C": 4, "D": 16}


def make_folder(tmp_path, config: dict, seed: int, dtype: str, sharpen: float = 12.0) -> Path:
    """config.json + model.safetensors.  The random weights of the package's writer are rescaled so that decays,
    blends, gates, norm weights, router scores and attention scores are far from their neutral values: a lost state,
    a blend with the wrong token, a missed key, a wrong expert or a dropped pass then changes the logits well beyond
    the tolerances."""
    from libmir_b200.weights import load_tensor, read_catalog, write_file, write_model_folder
    folder = write_model_folder(Path(tmp_path), config, seed=seed, dtype=dtype)
    tensors = {name: load_tensor(entry) for name, entry in read_catalog(folder).items()}
    generator = torch.Generator().manual_seed(seed + 1000)
    normal = lambda shape, deviation: torch.randn(shape, generator=generator) * deviation
    for name, tensor in list(tensors.items()):
        kind = tensor.dtype
        parts = name.split(".")
        last = parts[-1]
        if ".mu." in name:
            new = torch.rand(tensor.shape, generator=generator)
        elif last in ("norm", "norm1", "norm2") or name == "final.norm":
            new = 1.0 + normal(tensor.shape, 0.25)
        elif last == "w0":
            new = normal(tensor.shape, 1.0) - 0.5
        elif last == "u":
            new = normal(tensor.shape, 0.5)
        elif last == "correction":
            new = normal(tensor.shape, 0.3)
        elif last == "router":
            new = tensor.float() * 6.0
        elif last == "sg":
            new = tensor.float() * 10.0
        elif name == "loop.step":
            new = normal(tensor.shape, 0.2)
        elif name == "embed":
            new = tensor.float() * 10.0
        elif last in ("uq", "uk"):
            new = tensor.float() * sharpen
        elif last == "dkv":
            new = tensor.float() * 6.0
        elif ".mix." in name and last in ("r", "k", "v", "w1", "w2"):
            new = tensor.float() * 5.0
        elif ".mix." in name and last == "g":
            new = tensor.float() * 10.0
        elif last in ("gate", "up"):
            new = tensor.float() * 5.0
        elif last in ("o", "down"):
            new = tensor.float() * 2.0
        else:
            continue
        tensors[name] = new.to(kind)
    write_file(folder / "model.safetensors", tensors)
    return folder


def random_config(rng) -> dict:
    """A configuration drawn at random: any layer order, head counts and widths that are no multiples of 8 (or of 4),
    ranks from 1 on, with and without rotation, scaling, loop, cap, shared expert, groups and feed-forward."""
    def latent():
        dim = int(rng.choice([4, 12, 16, 20, 24, 40, 64]))
        rot_dim = int(rng.choice([0, 2, 6, 8, 16, 32]))
        scaling = None
        if rot_dim and rng.random() < 0.7:
            scaling = (float(rng.choice([1.0, 2.0, 4.0, 16.0])), int(rng.choice([16, 64, 512])), float(rng.choice([8.0, 32.0])),
                       float(rng.choice([1.0, 2.0])))
        return _latent(int(rng.integers(1, 7)), dim, rot_dim, int(rng.choice([4, 6, 8, 12, 24, 40, 96])),
                       int(rng.choice([3, 8, 20, 48, 64])), int(rng.choice([5, 8, 24, 56, 64, 100])),
                       float(rng.uniform(0.05, 0.4)), float(rng.choice([50.0, 10000.0, 1000000.0])), scaling)

    def feed_forward():
        draw = rng.random()
        if draw < 0.2:
            return None
        if draw < 0.45:
            return _dense(int(rng.choice([40, 64, 100, 130])))
        groups = int(rng.choice([1, 2, 3, 4]))
        per_group = int(rng.integers(1, 5))
        keep = int(rng.integers(1, groups + 1))
        top = int(rng.integers(1, keep * per_group + 1))
        return _moe(groups * per_group, top, int(rng.choice([8, 20, 36, 64])), (groups, keep) if rng.random() < 0.8 or groups > 1 else None,
                    float(rng.uniform(0.5, 3.0)), int(rng.choice([0, 12, 40])))

    layers = []
    for _ in range(int(rng.integers(1, 5))):
        mixer = latent() if rng.random() < 0.5 else _wkv(int(rng.integers(1, 6)), int(rng.choice([4, 12, 20, 32, 36, 64, 100, 128])),
                                                         int(rng.integers(1, 21)))
        layers.append(_layer(mixer, feed_forward()))
    config = {"architecture": "Zufotar", "vocab": int(rng.integers(30, 300)), "width": int(rng.choice([48, 52, 64, 72, 100, 136, 50])),
              "norm": {"eps": float(rng.choice([1e-5, 1e-6, 1e-4]))}, "layers": layers}
    if rng.random() < 0.7:
        config["embedding"] = {"scale": float(rng.uniform(0.2, 3.0))}
    if rng.random() < 0.7:
        config["logit_softcap"] = float(rng.uniform(4.0, 40.0))
    if rng.random() < 0.75:
        start = int(rng.integers(0, len(layers)))
        stop = int(rng.integers(start + 1, len(layers) + 1))
        config["loop"] = {"start": start, "stop": stop, "times": int(rng.integers(1, 4))}
    return config
