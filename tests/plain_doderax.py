"""A plain, slow implementation of the Doderax design in float64: whole sequences, no cache, no batching, one
function per mechanism.  It shares no code with the package and is what the engine is compared with.

Notation: n tokens, width w; a mixer with H value heads of width e, G key heads of width d (value head i reads key
head i // (H / G)); weights are stored [out, in] and applied as W x.
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


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z / (1.0 + torch.exp(-z))


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def token_pair_rows(ids, buckets, mul_previous, mul_current):
    """Row of the pair table for every token: a hash of the token and the one before; the last row for the first."""
    rows = [buckets]
    for before, current in zip(ids[:-1], ids[1:]):
        rows.append((before * mul_previous + current * mul_current) % buckets)
    return rows


def short_conv_silu(x, taps_weight):
    """x [n, c], taps_weight [c, taps] with the current token's tap in the last column; zeros before the start."""
    n, taps = x.shape[0], taps_weight.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, x.shape[1], dtype=x.dtype), x], dim=0)
    total = torch.zeros_like(x)
    for tap in range(taps):
        total = total + padded[tap:tap + n] * taps_weight[:, tap]
    return silu(total)


def rotate_half_pairs(x, positions, rotary, base):
    """x [n, heads, d]: dimension i < rotary / 2 is paired with i + rotary / 2, angle = position * base^(-2i / rotary);
    dimensions from `rotary` on pass unchanged."""
    half = rotary // 2
    if half == 0:
        return x
    frequency = torch.tensor([base ** (-2.0 * i / rotary) for i in range(half)], dtype=F64)
    angle = positions.to(F64)[:, None, None] * frequency
    cosine, sine = torch.cos(angle), torch.sin(angle)
    first, second = x[..., :half], x[..., half:rotary]
    return torch.cat([first * cosine - second * sine, second * cosine + first * sine, x[..., rotary:]], dim=-1)


def visible(n, window, keep_first):
    """[n, n] mask: query i sees key j iff j <= i and (no window, or i - j < window, or j < keep_first)."""
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    mask = j <= i
    if window is not None:
        mask = mask & ((i - j < window) | (j < keep_first))
    return mask


def softmax_attention(q, k, v, scale, window, keep_first):
    """q [n, H, d], k [n, G, d], v [n, G, e] -> [n, H, e]."""
    n, heads = q.shape[0], q.shape[1]
    group = heads // k.shape[1]
    mask = visible(n, window, keep_first)
    out = torch.zeros(n, heads, v.shape[2], dtype=F64)
    for head in range(heads):
        scores = (q[:, head] @ k[:, head // group].T) * scale
        scores = scores.masked_fill(~mask, -math.inf)
        out[:, head] = torch.softmax(scores, dim=-1) @ v[:, head // group]
    return out


def delta_rule(q, k, v, beta, decay):
    """q, k [n, G, d] (not yet unit vectors), v [n, H, e], beta [n, H], decay [n, H, d] -> o [n, H, e].
    Per head: S <- diag(decay) S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q."""
    n, heads, e = v.shape
    d = q.shape[2]
    group = heads // q.shape[1]
    q = q / torch.sqrt((q * q).sum(dim=-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(dim=-1, keepdim=True) + 1e-6)
    out = torch.zeros(n, heads, e, dtype=F64)
    for head in range(heads):
        state = torch.zeros(d, e, dtype=F64)
        for t in range(n):
            key, query = k[t, head // group], q[t, head // group]
            state = decay[t, head][:, None] * state
            write = beta[t, head] * (v[t, head] - state.T @ key)
            state = state + torch.outer(key, write)
            out[t, head] = state.T @ query
    return out


# ------------------------------------------------------------------------------ mixers
def attention_mixer(h, w, prefix, m):
    n = h.shape[0]
    heads, groups, d, e = m["heads"], m["kv_heads"], m["dim"], m.get("vdim", m["dim"])
    positions = torch.arange(n)
    q = (h @ w[prefix + "q"].T).reshape(n, heads, d)
    k = (h @ w[prefix + "k"].T).reshape(n, groups, d)
    v = (h @ w[prefix + "v"].T).reshape(n, groups, e)
    rot = m.get("rot")
    if rot:
        q = rotate_half_pairs(q, positions, rot["dims"], rot["base"])
        k = rotate_half_pairs(k, positions, rot["dims"], rot["base"])
    mask = m.get("mask") or {}
    window = mask.get("size") or None
    mixed = softmax_attention(q, k, v, m["scale"], window, mask.get("keep_first", 0))
    return mixed.reshape(n, heads * e) @ w[prefix + "o"].T


def delta_mixer(h, w, prefix, m, eps, per_channel):
    n = h.shape[0]
    heads, groups, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = short_conv_silu(h @ w[prefix + "q"].T, w[prefix + "q.conv"]).reshape(n, groups, d)
    k = short_conv_silu(h @ w[prefix + "k"].T, w[prefix + "k.conv"]).reshape(n, groups, d)
    v = short_conv_silu(h @ w[prefix + "v"].T, w[prefix + "v.conv"]).reshape(n, heads, e)
    beta = torch.sigmoid(h @ w[prefix + "b"].T)
    rate = torch.exp(w[prefix + "A_log"])
    if per_channel:
        raw = ((h @ w[prefix + "a1"].T) @ w[prefix + "a2"].T + w[prefix + "dt_bias"]).reshape(n, heads, d)
        decay = torch.exp(-rate[None, :, None] * softplus(raw))
        gate = torch.sigmoid((h @ w[prefix + "g1"].T) @ w[prefix + "g2"].T).reshape(n, heads, e)
    else:
        raw = h @ w[prefix + "a"].T + w[prefix + "dt_bias"]
        decay = torch.exp(-rate[None, :] * softplus(raw))[:, :, None].expand(n, heads, d)
        gate = silu(h @ w[prefix + "g"].T).reshape(n, heads, e)
    read = delta_rule(q, k, v, beta, decay)
    mixed = unit_rms(read, eps) * w[prefix + "norm"] * gate
    return mixed.reshape(n, heads * e) @ w[prefix + "o"].T


def side_by_side(outputs, weights, eps):
    """Half the sum of the branch outputs, each divided by its root mean square over the width and weighted."""
    return 0.5 * sum(unit_rms(out, eps) * weight for out, weight in zip(outputs, weights))


# ------------------------------------------------------------------------------ the model
def forward(config, w, ids, residual_after_layers=None):
    """Logits [n, vocab] of one whole sequence."""
    eps = config["norm"]["eps"]
    x = w["embed"][torch.tensor(ids)]
    pairs = (config.get("embedding") or {}).get("bigram")
    if pairs:
        rows = token_pair_rows(list(ids), pairs["buckets"], pairs["mul_prev"], pairs["mul_cur"])
        x = x + w["bigram"][torch.tensor(rows)]
    for index, layer in enumerate(config["layers"]):
        prefix = f"l{index}."
        h = unit_rms(x, eps) * (1.0 + w[prefix + "norm1"])
        if layer["type"] == "parallel":
            left = attention_mixer(h, w, prefix + "mix.left.", layer["mixer"]["left"])
            right = delta_mixer(h, w, prefix + "mix.right.", layer["mixer"]["right"], eps, False)
            mixed = side_by_side([left, right], [w[prefix + "mix.left.out"], w[prefix + "mix.right.out"]], eps)
        elif layer["type"] == "channel_delta":
            mixed = delta_mixer(h, w, prefix + "mix.", layer["mixer"], eps, True)
        else:
            raise ValueError(layer["type"])
        branch = mixed
        if layer.get("mlp"):
            branch = branch + gelu_tanh(h @ w[prefix + "mlp.up"].T) @ w[prefix + "mlp.down"].T
        x = x + branch
        if residual_after_layers is not None:
            residual_after_layers.append(x.clone())
    x = unit_rms(x, eps) * (1.0 + w["final.norm"])
    return (x @ w["head"].T) * config.get("logit_scale", 1.0)


def greedy(config, w, prompt, count):
    """`count` tokens chosen greedily after the prompt (ties to the lowest id), recomputing the whole sequence."""
    ids = list(prompt)
    for _ in range(count):
        logits = forward(config, w, ids)[-1]
        ids.append(int(torch.argmax(logits)))
    return ids[len(prompt):]
