"""The Mogevik decoder as a `ModelSpec`.

Every layer is the "parallel" arrangement (one layer norm whose output the mixer and the feed-forward
both read) around one of two mixers (a recurrent block with a real-gated linear recurrent unit, or
attention with a penalty on distance, a sliding window and an output gate) and a routed feed-forward
with identity experts and a gated shared expert, or none.  The embedding's rows are multiplied by a
constant; the output head is the embedding table itself.  A run of layers may be looped: it is scheduled
`times` times with the same weights, every pass with a cache and state of its own, and a "loop_add"
junction in front of each pass.

Tensor names: `embed`, `final.norm`, `loop.step`, and per layer i `l<i>.norm1`, `l<i>.mix.*`, `l<i>.mlp.*`.
"""
from __future__ import annotations

from ..registry import ARCHITECTURES
from ..spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .mogevik import MogevikConfig

SLOPE_POWER = 8.0        # slope of head h: 2^(-8 (h + 1) / heads)
LRU_DECAY = 8.0          # log a = -8 r softplus(lam)


def _norm(width: int, eps: float, name: str) -> PartSpec:
    return PartSpec("layernorm", dict(width=width, eps=eps), aliases={"weight": name})


def _mixer(c: MogevikConfig, kind: str, m: dict, prefix: str) -> PartSpec:
    if kind == "rglru":
        return PartSpec("rglru", dict(hidden_size=c.width, width=m["width"], blocks=m["blocks"], conv=m["conv"],
                                      decay=LRU_DECAY), prefix=prefix)
    return PartSpec("distance_attention",
                    dict(hidden_size=c.width, num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"],
                         v_dim=m["vdim"], scale=m["scale"], window=m["window"], slope_power=SLOPE_POWER, bias=True,
                         gate=True), prefix=prefix)


def describe_mogevik(c: MogevikConfig) -> ModelSpec:
    W = c.width
    layers = []
    for i, layer in enumerate(c.layers):
        p = f"l{i}."
        ffn = None
        if layer.mlp is not None:
            r = layer.mlp
            ffn = PartSpec("routed_mlp", dict(hidden_size=W, intermediate_size=r.ff, experts=r.experts, identity=r.identity,
                                              top=r.top, groups=r.groups, keep_groups=r.keep, shared_ff=r.shared_ff,
                                              shared_gate=True, correction=True), prefix=p + "mlp.")
        layers.append(LayerSpec("parallel", _norm(W, c.eps, p + "norm1"), _mixer(c, layer.type, layer.mixer, p + "mix."),
                                None, ffn))
    n = len(layers)
    junctions = []
    if c.loop_times:
        junctions.append(PartSpec("loop_add", dict(width=W, passes=c.loop_times), prefix="loop."))
        schedule = [ScheduleEntry(i) for i in range(c.loop_start)]
        for t in range(c.loop_times):
            for i in range(c.loop_start, c.loop_stop):
                first = i == c.loop_start
                schedule.append(ScheduleEntry(i, junction=0 if first else None, junction_arg=t if first else 0))
        schedule += [ScheduleEntry(i) for i in range(c.loop_stop, n)]
    else:
        schedule = [ScheduleEntry(i) for i in range(n)]
    return ModelSpec(
        hidden_size=W, vocab_size=c.vocab, max_positions=c.max_context,
        embedding=PartSpec("embedding", dict(vocab_size=c.vocab, width=W, scale=c.embedding_scale), aliases={"weight": "embed"}),
        layers=layers, schedule=schedule, final_norm=_norm(W, c.eps, "final.norm"),
        lm_head=PartSpec("lm_head", dict(vocab_size=c.vocab, width=W), aliases={"weight": "embed"}),
        stop_token_ids=tuple(c.eos_token_id), junctions=junctions)


def _register() -> None:
    from . import Architecture
    ARCHITECTURES.register("Mogevik", Architecture("Mogevik", MogevikConfig.from_dict, describe_mogevik), replace=True)


_register()
