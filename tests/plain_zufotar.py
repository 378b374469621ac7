"""A plain, slow implementation of the Zufotar design in float64: whole sequences, no cache, no batching, one
function per mechanism.  It shares no code with the package and is what the engine is compared with.

Notation: n tokens, width w.  Weights are stored [out, in] and applied as W x; a row vector x of a token is
multiplied as x @ W.T.
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import numpy as np
import torch

F64 = torch.float64


# ------------------------------------------------------------------------------ reading a model folder
def read_model(folder):
    """(config, {name: float64 tensor}) of a folder with config.json and model.safetensors."""
    folder = Path(folder)
    config = json.loads((folder / "config.json").read_text())
    raw = (folder / "model.safetensors").read_bytes()
    size = int.from_bytes(raw[:8], "little")
    header = json.loads(raw[8:8 + size])
    body = raw[8 + size:]
    weights = {}
    for name, entry in header.items():
        if name == "__metadata__":
            continue
        begin, end = entry["data_offsets"]
        data = body[begin:end]
        if entry["dtype"] == "BF16":
            bits = np.frombuffer(data, dtype=np.uint16).astype(np.uint32) << 16
            values = torch.from_numpy(bits.view(np.float32).copy())
        elif entry["dtype"] == "F32":
            values = torch.from_numpy(np.frombuffer(data, dtype=np.float32).copy())
        elif entry["dtype"] == "I32":
            values = torch.from_numpy(np.frombuffer(data, dtype=np.int32).copy())
        else:
            raise ValueError(f"{name}: dtype {entry['dtype']}")
        weights[name] = values.reshape(entry["shape"]).to(F64)
    return config, weights


# ------------------------------------------------------------------------------ small pieces
def unit_rms(x, eps):
    """x divided by its root mean square over the last axis, eps inside the root."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def gelu_erf(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def silu(z):
    return z / (1.0 + torch.exp(-z))


def sigmoid(z):
    return 1.0 / (1.0 + torch.exp(-z))


# ------------------------------------------------------------------------------ rotation
def rotary_table(rot):
    """(frequencies [dims / 2], factor on cos and sin) of a `rot` table {dims, base, scaling?}."""
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    scaling = rot.get("scaling")
    if not scaling:
        return freq, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def turns_to_dim(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    low = max(math.floor(turns_to_dim(float(scaling["fast"]))), 0)
    high = min(math.ceil(turns_to_dim(float(scaling["slow"]))), dims - 1)
    ramp = torch.tensor([min(max((i - low) / max(high - low, 0.001), 0.0), 1.0) for i in range(half)], dtype=F64)
    return freq / factor * ramp + freq * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_interleaved(x, positions, rot):
    """x [n, ..., d]: the first rot.dims of the last axis rotated in pairs (2i, 2i + 1) by position * frequency."""
    freq, magnitude = rotary_table(rot)
    dims = int(rot["dims"])
    angles = positions.to(F64)[:, None] * freq[None, :]                       # [n, dims / 2]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    cos, sin = (torch.cos(angles) * magnitude).reshape(shape), (torch.sin(angles) * magnitude).reshape(shape)
    out = x.clone()
    even, odd = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = even * cos - odd * sin
    out[..., 1:dims:2] = odd * cos + even * sin
    return out


# ------------------------------------------------------------------------------ mixers
def latent_attention(h, weights, prefix, mixer, eps):
    """Attention whose queries and keys / values come through low-rank latents; h [n, w]."""
    n = h.shape[0]
    heads, dim, vdim, rank = (int(mixer[k]) for k in ("heads", "dim", "vdim", "kv_rank"))
    rot_dim = int(mixer.get("rot_dim", 0))
    w = lambda name: weights[prefix + name]
    positions = torch.arange(n)
    latent_q = unit_rms(h @ w("dq").T, eps) * w("dq.norm")
    q = (latent_q @ w("uq").T).reshape(n, heads, dim + rot_dim)
    down = h @ w("dkv").T
    latent = unit_rms(down[:, :rank], eps) * w("dkv.norm")
    q_plain, q_rot, k_rot = q[..., :dim], q[..., dim:], down[:, rank:]        # k_rot [n, rot_dim]: one for all heads
    if rot_dim:
        q_rot, k_rot = rotate_interleaved(q_rot, positions, mixer["rot"]), rotate_interleaved(k_rot, positions, mixer["rot"])
    k_plain = (latent @ w("uk").T).reshape(n, heads, dim)
    v = (latent @ w("uv").T).reshape(n, heads, vdim)
    scores = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihd,jd->hij", q_rot, k_rot)) * float(mixer["scale"])
    hidden = torch.triu(torch.ones(n, n, dtype=torch.bool), diagonal=1)
    scores = scores.masked_fill(hidden[None], float("-inf"))
    mixed = torch.einsum("hij,jhd->ihd", torch.softmax(scores, dim=-1), v).reshape(n, heads * vdim)
    return (mixed * sigmoid(h @ w("g").T)) @ w("o").T


def wkv(h, weights, prefix, mixer, eps):
    """Time mixing with a matrix state per head and a decay per head and key channel; h [n, w]."""
    n = h.shape[0]
    heads, dim = int(mixer["heads"]), int(mixer["dim"])
    w = lambda name: weights[prefix + name]
    before = torch.cat([torch.zeros(1, h.shape[1], dtype=F64), h[:-1]], dim=0)
    mix = lambda name: h + (before - h) * w("mu." + name)
    r = (mix("r") @ w("r").T).reshape(n, heads, dim)
    k = (mix("k") @ w("k").T).reshape(n, heads, dim)
    v = (mix("v") @ w("v").T).reshape(n, heads, dim)
    gate = silu(mix("g") @ w("g").T)
    decay = torch.exp(-torch.exp(torch.tanh(mix("w") @ w("w1").T) @ w("w2").T + w("w0"))).reshape(n, heads, dim)
    bonus = w("u").reshape(heads, dim)
    state = torch.zeros(heads, dim, dim, dtype=F64)                           # [head, key channel, value channel]
    out = torch.zeros(n, heads, dim, dtype=F64)
    for t in range(n):
        outer = k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hkv,hk->hv", state + bonus[:, :, None] * outer, r[t])
        state = decay[t][:, :, None] * state + outer
    out = unit_rms(out, eps).reshape(n, heads * dim) * w("norm")
    return (out * gate) @ w("o").T


# ------------------------------------------------------------------------------ feed-forwards
def dense_mlp(h, weights, prefix):
    return gelu_erf(h @ weights[prefix + "up"].T) @ weights[prefix + "down"].T


def gated_expert(h, weights, prefix):
    return (silu(h @ weights[prefix + "gate"].T) * (h @ weights[prefix + "up"].T)) @ weights[prefix + "down"].T


def route(h, weights, prefix, router):
    """(chosen experts [n, top], their weights [n, top]) of every token."""
    experts, top = int(router["experts"]), int(router["top"])
    groups = router.get("groups") or {"count": 1, "keep": 1}
    count, keep = int(groups["count"]), int(groups["keep"])
    scores = sigmoid(h @ weights[prefix + "router"].T)
    choice = scores + weights[prefix + "correction"]
    per_group = experts // count
    grouped = choice.reshape(-1, count, per_group)
    group_score = grouped.topk(min(2, per_group), dim=-1).values.sum(dim=-1)
    kept = group_score.topk(keep, dim=-1).indices
    allowed = torch.zeros(h.shape[0], count, dtype=torch.bool)
    allowed.scatter_(1, kept, True)
    allowed = allowed[:, :, None].expand(-1, -1, per_group).reshape(-1, experts)
    chosen = choice.masked_fill(~allowed, float("-inf")).topk(top, dim=-1).indices
    picked = scores.gather(1, chosen)
    return chosen, picked / (picked.sum(dim=-1, keepdim=True) + 1e-20) * float(router["scale"])


def mixture(h, weights, prefix, mlp):
    chosen, share = route(h, weights, prefix, mlp["router"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for expert, weight in zip(chosen[t].tolist(), share[t].tolist()):
            out[t] += weight * gated_expert(h[t:t + 1], weights, f"{prefix}e{expert}.")[0]
    if mlp.get("shared"):
        out = out + gated_expert(h, weights, prefix + "shared.") * sigmoid(h @ weights[prefix + "shared.sg"].T)
    return out


# ------------------------------------------------------------------------------ the model
def layer_order(config):
    """[(layer, number of the pass it opens or None)] in the order the layers run."""
    count = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, None) for i in range(count)]
    start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    order = [(i, None) for i in range(start)]
    for t in range(times):
        order += [(i, t if i == start else None) for i in range(start, stop)]
    return order + [(i, None) for i in range(stop, count)]


def layer(x, index, config, weights):
    spec = config["layers"][index]
    eps = float(config["norm"]["eps"])
    prefix = f"l{index}."
    h1 = unit_rms(x, eps) * weights[prefix + "norm1"]
    if spec["type"] == "latent_attention":
        mixed = latent_attention(h1, weights, prefix + "mix.", spec["mixer"], eps)
    elif spec["type"] == "wkv":
        mixed = wkv(h1, weights, prefix + "mix.", spec["mixer"], eps)
    else:
        raise ValueError(spec["type"])
    mlp = spec.get("mlp")
    if mlp is None:
        return x + mixed
    h2 = unit_rms(x, eps) * weights[prefix + "norm2"]
    fed = dense_mlp(h2, weights, prefix + "mlp.") if mlp["kind"] == "dense" else mixture(h2, weights, prefix + "mlp.", mlp)
    return x + (mixed + fed)


def forward(config, weights, ids, trace=None):
    """Logits [n, vocab] of one sequence; `trace`, a list, receives the residual stream after every layer run."""
    ids = torch.as_tensor(ids, dtype=torch.long)
    embedded = weights["embed"][ids] * float((config.get("embedding") or {}).get("scale", 1.0))
    x = embedded
    for index, opens in layer_order(config):
        if opens is not None:
            if opens > 0:
                x = x + embedded
            x = x + weights["loop.step"][opens]
        x = layer(x, index, config, weights)
        if trace is not None:
            trace.append(x.clone())
    x = unit_rms(x, float(config["norm"]["eps"])) * weights["final.norm"]
    logits = x @ weights["embed"].T
    cap = config.get("logit_softcap")
    return cap * torch.tanh(logits / cap) if cap else logits
