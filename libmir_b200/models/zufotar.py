"""Zufotar: a decoder whose layers add a mixer and a feed-forward, each behind a norm of its own, to the same
residual (x += mixer(norm1(x)) + ff(norm2(x))), with latent attention and wkv mixers, dense or routed feed-forwards,
and a run of layers that is repeated with the same weights: config.json -> ModelSpec.

config.json:
    architecture  "Zufotar"
    vocab, width, norm.eps, embedding.scale, logit_softcap
    layers[i]     {type, mixer, mlp}; tensors of layer i start with "l<i>."
        type "latent_attention"  mixer {heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, rot {dims, base, scaling
                                 {factor, original, fast, slow}}}: queries and keys / values through low-rank latents,
                                 interleaved rotation with YaRN scaling on the rot_dim part, an output gate
        type "wkv"               mixer {heads, dim}: time mixing with a matrix state per head; the rank of the decay's
                                 low-rank pair is the shape of `w1`
        mlp       {kind "dense", ff} (up, exact GELU, down), {kind "moe", expert {ff}, router {experts, top, scale,
                  groups {count, keep}}, shared {ff}} or null
    loop          {start, stop, times}: layers start .. stop - 1 run `times` times in a row, every pass with a cache
                  or state of its own; tensor `loop.step` [times, width]
Tensor names: embed (also the output head), loop.step, l<i>.norm1, l<i>.norm2, l<i>.mix.*, l<i>.mlp.*, final.norm.
"""

from __future__ import annotations

from typing import Mapping, Optional

from ..config.spec import (EmbeddingSpec, GeluMlpSpec, HeadSpec, LatentAttentionSpec, LayerSpec, LoopSpec, ModelSpec,
                           RmsNormSpec, RotarySpec, RoutedExpertsSpec, ScheduleEntry, WkvSpec, YarnScaling)
from ..errors import ConfigError
from ..registry import register_architecture

LAYER_NAMES = {"mixer_norm": "norm1", "feed_forward_norm": "norm2", "mixer": "mix.", "feed_forward": "mlp."}
DEFAULT_DECAY_RANK = 16      # of the decay's low-rank pair, when no checkpoint is at hand to take it from


def _need(table, key: str, where: str):
    if not isinstance(table, Mapping) or key not in table:
        raise ConfigError(f"Zufotar config: {where} needs `{key}`")
    return table[key]


def _rotation(mixer: Mapping, rotary_dim: int, where: str) -> Optional[RotarySpec]:
    rot = mixer.get("rot")
    if not rot or not rotary_dim:
        return None
    dims = int(_need(rot, "dims", where + ".rot"))
    if dims != rotary_dim:
        raise ConfigError(f"Zufotar config: {where}: rot.dims {dims} must equal rot_dim {rotary_dim}")
    scaling = rot.get("scaling")
    yarn = None
    if scaling:
        yarn = YarnScaling(*(float(_need(scaling, key, where + ".rot.scaling"))
                             for key in ("factor", "original", "fast", "slow")))
    return RotarySpec(head_dim=rotary_dim, rotary_dim=rotary_dim, theta=float(_need(rot, "base", where + ".rot")),
                      scaling=yarn, layout="interleaved")


def _latent_attention(mixer: Mapping, width: int, eps: float, where: str) -> LatentAttentionSpec:
    sizes = {key: int(_need(mixer, key, where)) for key in ("heads", "dim", "vdim", "q_rank", "kv_rank")}
    rotary_dim = int(mixer.get("rot_dim", 0))
    return LatentAttentionSpec(
        hidden_size=width, heads=sizes["heads"], head_dim=sizes["dim"], rotary_dim=rotary_dim, value_dim=sizes["vdim"],
        q_rank=sizes["q_rank"], kv_rank=sizes["kv_rank"], scale=float(_need(mixer, "scale", where)), norm_eps=eps,
        gate=True, position=_rotation(mixer, rotary_dim, where))


def _wkv(mixer: Mapping, width: int, eps: float, where: str, catalog, prefix: str) -> WkvSpec:
    name = prefix + "w1"
    rank = int(catalog[name][0]) if catalog is not None and name in catalog else int(mixer.get("decay_rank", DEFAULT_DECAY_RANK))
    return WkvSpec(hidden_size=width, heads=int(_need(mixer, "heads", where)), head_dim=int(_need(mixer, "dim", where)),
                   decay_rank=rank, norm_eps=eps)


def _feed_forward(mlp: Mapping, width: int, where: str):
    kind = mlp.get("kind")
    if kind == "dense":
        return GeluMlpSpec(hidden_size=width, intermediate_size=int(_need(mlp, "ff", where)), activation="gelu_erf")
    if kind == "moe":
        router = _need(mlp, "router", where)
        groups = router.get("groups") or {}
        shared = mlp.get("shared") or {}
        return RoutedExpertsSpec(
            hidden_size=width, expert_size=int(_need(_need(mlp, "expert", where), "ff", where + ".expert")),
            experts=int(_need(router, "experts", where + ".router")), top=int(_need(router, "top", where + ".router")),
            groups=int(groups.get("count", 1)), keep_groups=int(groups.get("keep", groups.get("count", 1))),
            scale=float(router.get("scale", 1.0)), correction=True, shared_size=int(shared.get("ff", 0)),
            shared_gate=True)
    raise ConfigError(f"Zufotar config: {where} has kind {kind!r}; known: dense, moe")


def build(config: Mapping, catalog: Optional[Mapping[str, tuple]] = None) -> ModelSpec:
    width, vocab = int(_need(config, "width", "the model")), int(_need(config, "vocab", "the model"))
    eps = float(_need(_need(config, "norm", "the model"), "eps", "norm"))
    layers = []
    for index, layer in enumerate(_need(config, "layers", "the model")):
        where = f"layers[{index}]"
        prefix = f"l{index}."
        kind, mixer = _need(layer, "type", where), _need(layer, "mixer", where)
        if kind == "latent_attention":
            mixer_spec = _latent_attention(mixer, width, eps, where)
        elif kind == "wkv":
            mixer_spec = _wkv(mixer, width, eps, where, catalog, prefix + "mix.")
        else:
            raise ConfigError(f"Zufotar config: {where} has type {kind!r}; known: latent_attention, wkv")
        mlp = layer.get("mlp")
        feed_forward = _feed_forward(mlp, width, where + ".mlp") if mlp is not None else None
        norm = RmsNormSpec(size=width, eps=eps, offset=0.0, tensor="")
        layers.append(LayerSpec(prefix=prefix, mixer=mixer_spec, feed_forward=feed_forward, mixer_norm=norm,
                                feed_forward_norm=norm if feed_forward is not None else None, names=LAYER_NAMES,
                                arrangement="parallel"))
    count = len(layers)
    loop_config = config.get("loop")
    loop = None
    if loop_config:
        start, stop, times = (int(_need(loop_config, key, "loop")) for key in ("start", "stop", "times"))
        if not 0 <= start <= stop <= count or times < 1:
            raise ConfigError(f"Zufotar config: loop {start}..{stop} x {times} does not fit {count} layers")
        schedule = [ScheduleEntry(layer=i) for i in range(start)]
        for number in range(times):
            schedule += [ScheduleEntry(layer=i, opens_pass=number if i == start else None) for i in range(start, stop)]
        schedule += [ScheduleEntry(layer=i) for i in range(stop, count)]
        loop = LoopSpec(passes=times, step_tensor="loop.step", add_embedding=True)
    else:
        schedule = [ScheduleEntry(layer=i) for i in range(count)]
    cap = config.get("logit_softcap")
    return ModelSpec(
        architecture="Zufotar", hidden_size=width, vocab_size=vocab,
        max_positions=int(config.get("max_positions", 1 << 30)),
        embedding=EmbeddingSpec("embed", vocab, width, float((config.get("embedding") or {}).get("scale", 1.0))),
        layers=tuple(layers), schedule=tuple(schedule),
        final_norm=RmsNormSpec(size=width, eps=eps, offset=0.0, tensor=""), final_norm_name="final.norm",
        head=HeadSpec("embed", vocab, width, tied=True, softcap=float(cap) if cap else None), loop=loop,
    )


register_architecture("Zufotar", build)
