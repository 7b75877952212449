"""The Gevonex decoder as a `ModelSpec`.

Every layer is the "shift_gated" arrangement (dynamic-tanh norms, a token shift in front of
the mixer, a learned gate on each sublayer's result) around one of three mixers (minGRU,
Mamba-2, attention over a cached latent with a sink) and a dense GELU feed-forward or none.
A run of layers may be looped: it is scheduled `times` times with the same weights, every
pass with a cache and state of its own, and a "loop_input" junction in front of each pass.
The head's logits go through a soft cap.

Tensor names: `embed`, `head`, `final.norm[.b|.alpha]`, `loop.in`, `loop.step`, and per layer i
`l<i>.norm1|norm2[.b|.alpha]`, `l<i>.shift`, `l<i>.rg1|rg2[.b]`, `l<i>.mix.*`, `l<i>.mlp.up|down`.
"""
from __future__ import annotations

from ..registry import ARCHITECTURES
from ..spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .gevonex import GevonexConfig


def _norm(width: int, name: str) -> PartSpec:
    # the weight is stored under the norm's own name, its companions beside it
    return PartSpec("dyt", dict(width=width), prefix=name + ".", aliases={"weight": name})


def _mixer(c: GevonexConfig, kind: str, sizes: dict, prefix: str) -> PartSpec:
    if kind == "mingru":
        return PartSpec("mingru", dict(hidden_size=c.width, width=sizes["width"]), prefix=prefix)
    if kind == "mamba2":
        return PartSpec("mamba2", dict(hidden_size=c.width, eps=c.eps, **sizes), prefix=prefix)
    return PartSpec("latent_attention", dict(hidden_size=c.width, eps=c.eps, window=0, **sizes), prefix=prefix)


def describe_gevonex(c: GevonexConfig) -> ModelSpec:
    W = c.width
    layers = []
    for i, layer in enumerate(c.layers):
        p = f"l{i}."
        extras = {"shift": PartSpec("token_shift", dict(width=W), aliases={"mu": p + "shift"}),
                  "mixer_gate": PartSpec("residual_gate", dict(width=W), aliases={"weight": p + "rg1", "bias": p + "rg1.b"})}
        ffn_norm = ffn = None
        if layer.mlp is not None:
            ffn_norm = _norm(W, p + "norm2")
            ffn = PartSpec("dense_mlp", dict(hidden_size=W, intermediate_size=layer.mlp["ff"], activation="gelu_tanh"),
                           prefix=p + "mlp.")
            extras["ffn_gate"] = PartSpec("residual_gate", dict(width=W), aliases={"weight": p + "rg2", "bias": p + "rg2.b"})
        layers.append(LayerSpec("shift_gated", _norm(W, p + "norm1"), _mixer(c, layer.type, layer.mixer, p + "mix."),
                                ffn_norm, ffn, extras))
    n = len(layers)
    junctions = []
    if c.loop_times:
        junctions.append(PartSpec("loop_input", dict(width=W, passes=c.loop_times), prefix="loop."))
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
        embedding=PartSpec("embedding", dict(vocab_size=c.vocab, width=W), aliases={"weight": "embed"}),
        layers=layers, schedule=schedule, final_norm=_norm(W, "final.norm"),
        lm_head=PartSpec("lm_head", dict(vocab_size=c.vocab, width=W, softcap=c.logit_softcap or None),
                         aliases={"weight": "head"}),
        stop_token_ids=tuple(c.eos_token_id), junctions=junctions)


def _register() -> None:
    from . import Architecture
    ARCHITECTURES.register("Gevonex", Architecture("Gevonex", GevonexConfig.from_dict, describe_gevonex), replace=True)


_register()
