"""Tiny Doderax configurations for the tests, and model folders with weights that make every mechanism matter.
The configurations differ from one another in every size, in the order and kinds of layers, in windows, kept
first tokens, taps, ranks and constants; some take values that make two sizes equal or 1."""

from __future__ import annotations

from pathlib import Path

import torch


def _left(heads, kv_heads, dim, vdim, scale, rot=None, mask=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot:
        mixer["rot"] = {"dims": rot[0], "base": rot[1]}
    if mask:
        mixer["mask"] = {"size": mask[0], "keep_first": mask[1]}
    return mixer


def _right(heads, kv_heads, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def _layer(kind, mixer, ff):
    return {"type": kind, "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


DODERAX_X = {   # mixed layers; value heads wider than key heads; a window with kept first tokens; key heads of 24 and 40
    "architecture": "Doderax", "vocab": 211, "width": 96, "logit_scale": 0.5, "norm": {"eps": 1e-6},
    "embedding": {"bigram": {"buckets": 97, "mul_prev": 31, "mul_cur": 7}},
    "layers": [
        _layer("parallel", {"left": _left(4, 2, 32, 48, 0.2, rot=(16, 10000.0), mask=(20, 3)),
                            "right": _right(4, 2, 24, 16, 3)}, 160),
        _layer("channel_delta", _right(3, 3, 40, 24, 4), 128),
        _layer("channel_delta", _right(4, 1, 32, 8, 2), 0),
        _layer("parallel", {"left": _left(2, 1, 64, 64, 0.125, rot=(64, 500.0), mask=(33, 0)),
                            "right": _right(2, 2, 64, 40, 4)}, 104),
    ],
}

DODERAX_Y = {   # sizes that are equal or 1: one head, one tap, no window, no pair table, no logit scale, no feed-forward
    "architecture": "Doderax", "vocab": 130, "width": 64, "norm": {"eps": 1e-5},
    "layers": [
        _layer("parallel", {"left": _left(2, 2, 16, 16, 0.25, rot=(8, 100.0)), "right": _right(1, 1, 32, 32, 1)}, 0),
        _layer("channel_delta", _right(1, 1, 8, 64, 4), 64),
        _layer("parallel", {"left": _left(1, 1, 24, 8, 0.3, mask=(5, 1)), "right": _right(2, 1, 16, 16, 5)}, 72),
    ],
}

DODERAX_Z = {   # a window shorter than a page beside kept tokens that span pages; a key head of 200 channels
    "architecture": "Doderax", "vocab": 150, "width": 80, "logit_scale": 2.0, "norm": {"eps": 1e-5},
    "embedding": {"bigram": {"buckets": 64, "mul_prev": 5, "mul_cur": 11}},
    "layers": [
        _layer("parallel", {"left": _left(3, 3, 40, 24, 0.16, rot=(20, 250.0), mask=(9, 20)),
                            "right": _right(2, 2, 200, 8, 4)}, 96),
        _layer("parallel", {"left": _left(6, 2, 16, 32, 0.25, rot=(16, 10000.0), mask=(64, 2)),
                            "right": _right(6, 3, 16, 16, 2)}, 0),
    ],
}

DODERAX_W = {   # key and value heads of 64 and of 128 with kept first tokens: in bfloat16 the tensor-core tile kernel
    "architecture": "Doderax", "vocab": 180, "width": 128, "logit_scale": 1.5, "norm": {"eps": 1e-6},
    "embedding": {"bigram": {"buckets": 50, "mul_prev": 3, "mul_cur": 1}},
    "layers": [
        _layer("parallel", {"left": _left(4, 2, 64, 64, 0.125, rot=(32, 10000.0), mask=(70, 5)),
                            "right": _right(2, 1, 32, 64, 4)}, 192),
        _layer("channel_delta", _right(2, 2, 128, 16, 3), 0),
        _layer("parallel", {"left": _left(2, 1, 128, 128, 0.09, rot=(128, 1000.0), mask=(40, 66)),
                            "right": _right(4, 4, 16, 32, 2)}, 160),
    ],
}

DODERAX_V = {   # recurrent layers only (no pages at all), a width that is no multiple of 8, seven taps, five heads
    "architecture": "Doderax", "vocab": 97, "width": 100, "logit_scale": 0.75, "norm": {"eps": 1e-5},
    "embedding": {"bigram": {"buckets": 31, "mul_prev": 1, "mul_cur": 2}},
    "layers": [
        _layer("channel_delta", _right(5, 5, 48, 20, 7), 120),
        _layer("channel_delta", _right(2, 1, 72, 36, 3), 0),
    ],
}

DODERAX_U = {   # attention heads whose widths are no multiples of 8 (keys 20, values 12, 6 rotated); a rank of 3
    "architecture": "Doderax", "vocab": 120, "width": 72, "logit_scale": 1.0, "norm": {"eps": 1e-5},
    "layers": [
        _layer("parallel", {"left": _left(4, 2, 20, 12, 0.22, rot=(6, 77.0), mask=(11, 2)),
                            "right": _right(2, 2, 12, 10, 2)}, 80),
        _layer("channel_delta", dict(_right(3, 1, 20, 4, 4), decay_rank=3, gate_rank=5), 0),
    ],
}

ALL = {"U": DODERAX_U, "V": DODERAX_V, "W": DODERAX_W, "X": DODERAX_X, "Y": DODERAX_Y, "Z": DODERAX_Z}
PAGE_SIZES = {"U": 4, "V": 16, "W": 16, "X": 8, "Y": 16, "Z": 8}


def make_folder(tmp_path, config: dict, seed: int, dtype: str, sharpen: float = 4.0) -> Path:
    """config.json + model.safetensors.  The random weights of the package's writer are rescaled so that decays,
    gates, convolutions, norm weights and attention scores are far from their neutral values: a lost state, a tap
    read from the wrong token, a window one token off or a missing kept token then changes the logits well beyond
    the tolerances."""
    from libmir_b200.weights import load_tensor, read_catalog, write_file, write_model_folder
    folder = write_model_folder(Path(tmp_path), config, seed=seed, dtype=dtype)
    tensors = {name: load_tensor(entry) for name, entry in read_catalog(folder).items()}
    generator = torch.Generator().manual_seed(seed + 1000)
    normal = lambda shape, deviation: torch.randn(shape, generator=generator) * deviation
    for name, tensor in list(tensors.items()):
        kind = tensor.dtype
        last = name.rsplit(".", 1)[-1]
        if name.endswith(".conv"):
            new = normal(tensor.shape, 0.6)
        elif last == "A_log":
            new = torch.rand(tensor.shape, generator=generator) * 2.0 - 1.5
        elif last == "dt_bias":
            new = normal(tensor.shape, 1.0)
        elif last in ("norm", "out"):
            new = 1.0 + normal(tensor.shape, 0.25)
        elif last == "norm1" or name == "final.norm":
            new = normal(tensor.shape, 0.25)
        elif last in ("a", "b", "a1", "a2", "g1", "g2"):
            new = tensor.float() * 3.0
        elif last in ("q", "k") and ".left." in name:
            new = tensor.float() * sharpen
        elif last in ("o", "down"):
            new = tensor.float() * 2.0
        elif name == "head":
            new = tensor.float() * 5.0
        else:
            continue
        tensors[name] = new.to(kind)
    write_file(folder / "model.safetensors", tensors)
    return folder


def random_config(rng) -> dict:
    """A configuration drawn at random: any layer order, heads and groups, head widths that are no multiples of 8 (or
    of 4), one to six taps, ranks from 1 on, windows shorter than a page, more kept tokens than the window holds, with
    and without rotation, window, pair table, logit scale and feed-forward."""
    def delta(channel):
        kv_heads = int(rng.integers(1, 4))
        mixer = _right(kv_heads * int(rng.integers(1, 4)), kv_heads, int(rng.choice([4, 12, 16, 20, 36, 44, 64, 100, 130])),
                       int(rng.choice([1, 6, 8, 10, 24, 33, 70])), int(rng.integers(1, 7)))
        if channel:
            mixer.update(decay_rank=int(rng.integers(1, 21)), gate_rank=int(rng.integers(1, 21)))
        return mixer

    def attention():
        kv_heads = int(rng.integers(1, 4))
        dim = int(rng.choice([8, 12, 16, 20, 24, 40, 64, 128]))
        vdim = dim if rng.random() < 0.4 else int(rng.choice([4, 6, 8, 12, 24, 40, 96]))
        rot = (int(rng.choice(list(range(2, dim + 1, 2)))), float(rng.choice([50.0, 10000.0, 250000.0]))) if rng.random() < 0.8 else None
        mask = (int(rng.integers(1, 60)), int(rng.integers(0, 40))) if rng.random() < 0.85 else None
        return _left(kv_heads * int(rng.integers(1, 5)), kv_heads, dim, vdim, float(rng.uniform(0.05, 0.4)), rot, mask)

    layers = []
    for _ in range(int(rng.integers(1, 5))):
        ff = int(rng.choice([40, 64, 100, 130])) if rng.random() < 0.7 else 0
        if rng.random() < 0.5:
            layers.append(_layer("channel_delta", delta(True), ff))
        else:
            layers.append(_layer("parallel", {"left": attention(), "right": delta(False)}, ff))
    config = {"architecture": "Doderax", "vocab": int(rng.integers(30, 300)), "width": int(rng.choice([48, 52, 64, 72, 100, 136, 50])),
              "norm": {"eps": float(rng.choice([1e-5, 1e-6, 1e-4]))}, "layers": layers}
    if rng.random() < 0.7:
        config["logit_scale"] = float(rng.uniform(0.2, 3.0))
    if rng.random() < 0.7:
        config["embedding"] = {"bigram": {"buckets": int(rng.integers(2, 200)), "mul_prev": int(rng.integers(1, 1000)),
                                          "mul_cur": int(rng.integers(1, 1000))}}
    return config
