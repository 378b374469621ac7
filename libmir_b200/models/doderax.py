"""Doderax: a decoder whose layers are `parallel` in arrangement (one norm, mixer and feed-forward both read it)
and whose mixers are recurrent: config.json -> ModelSpec.

config.json:
    architecture  "Doderax"
    vocab, width, logit_scale, norm.eps
    embedding.bigram {buckets, mul_prev, mul_cur}     a second embedding table over pairs of tokens (tensor `bigram`)
    layers[i]     {type, mixer, mlp}; tensors of layer i start with "l<i>."
        type "channel_delta"  mixer {heads, kv_heads, dim, vdim, conv}: the gated delta rule with one decay per head
                              and key channel (low-rank a1, a2) and a sigmoid gate (low-rank g1, g2); the two ranks
                              are the shapes of `a1` and `g1`
        type "parallel"       mixer {left, right}: softmax attention (heads, kv_heads, dim, vdim, scale, rot {dims,
                              base}, mask {size, keep_first}) beside the gated delta rule with one decay per head and
                              a silu gate (heads, kv_heads, dim, vdim, conv); half the sum of the two outputs, each
                              RMS-normed over the width with `left.out` / `right.out`
        mlp       {kind "dense", ff} (up, tanh GELU, down) or null
Norm weights are stored around zero (the norm multiplies by 1 + w); the norms inside mixers have plain weights.
Tensor names: embed, bigram, l<i>.norm1, l<i>.mix.*, l<i>.mlp.{up,down}, final.norm, head.
"""

from __future__ import annotations

from typing import Mapping, Optional

from ..config.spec import (EmbeddingSpec, GatedDeltaRuleSpec, GeluMlpSpec, HeadSpec, LayerSpec, ModelSpec, RmsNormSpec,
                           RotarySpec, ScheduleEntry, SideBySideSpec, SoftmaxAttentionSpec, TokenPairsSpec)
from ..errors import ConfigError
from ..registry import register_architecture

LAYER_NAMES = {"mixer_norm": "norm1", "mixer": "mix.", "feed_forward": "mlp."}
ATTENTION_NAMES = (("q_proj.weight", "q"), ("k_proj.weight", "k"), ("v_proj.weight", "v"), ("o_proj.weight", "o"))
DEFAULT_RANK = 16            # of the low-rank pairs, when neither a checkpoint nor the configuration says


def _need(table: Mapping, key: str, where: str):
    if not isinstance(table, Mapping) or key not in table:
        raise ConfigError(f"Doderax config: {where} needs `{key}`")
    return table[key]


def _rank(catalog, name: str, mixer: Mapping, key: str) -> int:
    if catalog is not None and name in catalog:
        return int(catalog[name][0])
    return int(mixer.get(key, DEFAULT_RANK))


def _delta(mixer: Mapping, width: int, eps: float, where: str, channel: bool, catalog, prefix: str) -> GatedDeltaRuleSpec:
    sizes = {key: int(_need(mixer, key, where)) for key in ("heads", "kv_heads", "dim", "vdim", "conv")}
    if sizes["heads"] % sizes["kv_heads"]:
        raise ConfigError(f"Doderax config: {where}: heads must be a multiple of kv_heads")
    return GatedDeltaRuleSpec(
        hidden_size=width, heads=sizes["heads"], kv_heads=sizes["kv_heads"], key_dim=sizes["dim"],
        value_dim=sizes["vdim"], conv_taps=sizes["conv"], norm_eps=eps,
        decay="channel" if channel else "head", decay_rank=_rank(catalog, prefix + "a1", mixer, "decay_rank") if channel else 0,
        gate="sigmoid" if channel else "silu", gate_rank=_rank(catalog, prefix + "g1", mixer, "gate_rank") if channel else 0)


def _attention(mixer: Mapping, width: int, where: str) -> SoftmaxAttentionSpec:
    heads, kv_heads, dim = (int(_need(mixer, key, where)) for key in ("heads", "kv_heads", "dim"))
    if heads % kv_heads:
        raise ConfigError(f"Doderax config: {where}: heads must be a multiple of kv_heads")
    position = None
    rot = mixer.get("rot")
    if rot:
        position = RotarySpec(head_dim=dim, rotary_dim=int(_need(rot, "dims", where + ".rot")),
                              theta=float(_need(rot, "base", where + ".rot")))
    mask = mixer.get("mask") or {}
    window = int(mask["size"]) if mask.get("size") else None
    return SoftmaxAttentionSpec(
        hidden_size=width, heads=heads, kv_heads=kv_heads, head_dim=dim, scale=float(_need(mixer, "scale", where)),
        window=window, keep_first=int(mask.get("keep_first", 0)) if window is not None else 0, position=position,
        value_head_dim=int(mixer.get("vdim", dim)), names=ATTENTION_NAMES)


def build(config: Mapping, catalog: Optional[Mapping[str, tuple]] = None) -> ModelSpec:
    width, vocab = int(_need(config, "width", "the model")), int(_need(config, "vocab", "the model"))
    eps = float(_need(_need(config, "norm", "the model"), "eps", "norm"))
    layers = []
    for index, layer in enumerate(_need(config, "layers", "the model")):
        where = f"layers[{index}]"
        prefix = f"l{index}."
        kind, mixer = _need(layer, "type", where), _need(layer, "mixer", where)
        if kind == "channel_delta":
            mixer_spec = _delta(mixer, width, eps, where, True, catalog, prefix + "mix.")
        elif kind == "parallel":
            left = _attention(_need(mixer, "left", where), width, where + ".left")
            right = _delta(_need(mixer, "right", where), width, eps, where + ".right", False, catalog, prefix + "mix.right.")
            mixer_spec = SideBySideSpec(hidden_size=width, branches=(("left", left), ("right", right)), eps=eps, scale=0.5)
        else:
            raise ConfigError(f"Doderax config: {where} has type {kind!r}; known: channel_delta, parallel")
        mlp = layer.get("mlp")
        feed_forward = None
        if mlp is not None:
            if mlp.get("kind") != "dense":
                raise ConfigError(f"Doderax config: {where}.mlp has kind {mlp.get('kind')!r}; known: dense")
            feed_forward = GeluMlpSpec(hidden_size=width, intermediate_size=int(_need(mlp, "ff", where + ".mlp")))
        layers.append(LayerSpec(prefix=prefix, mixer=mixer_spec, feed_forward=feed_forward,
                                mixer_norm=RmsNormSpec(size=width, eps=eps, offset=1.0, tensor=""),
                                feed_forward_norm=None, names=LAYER_NAMES, arrangement="parallel"))
    pairs = None
    bigram = (config.get("embedding") or {}).get("bigram")
    if bigram:
        pairs = TokenPairsSpec("bigram", int(_need(bigram, "buckets", "embedding.bigram")),
                               int(_need(bigram, "mul_prev", "embedding.bigram")),
                               int(_need(bigram, "mul_cur", "embedding.bigram")))
    return ModelSpec(
        architecture="Doderax", hidden_size=width, vocab_size=vocab,
        max_positions=int(config.get("max_positions", 1 << 30)),
        embedding=EmbeddingSpec("embed", vocab, width, 1.0, pairs),
        layers=tuple(layers), schedule=tuple(ScheduleEntry(layer=i) for i in range(len(layers))),
        final_norm=RmsNormSpec(size=width, eps=eps, offset=1.0, tensor=""), final_norm_name="final.norm",
        head=HeadSpec("head", vocab, width, tied=False, scale=float(config.get("logit_scale", 1.0))),
    )


register_architecture("Doderax", build)
