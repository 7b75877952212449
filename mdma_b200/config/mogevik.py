"""Typed configuration of the Mogevik decoder, read from config.json.

Keys: `vocab`, `width`, `embedding.scale`, `norm.eps`, `layers` (a list; each entry has `type`, the
mixer kind, `mixer`, its sizes, and `mlp`, the feed-forward's description or null), `loop` (`start`,
`stop`, `times`: layers start..stop-1 run `times` times in a row; absent or null: no loop).

Mixers: `rglru` {`width`, `blocks`, `conv`}; `attention` {`heads`, `kv_heads`, `dim`, `vdim`, `scale`,
`mask`: {`size`} (absent or null: every earlier token is seen)}.
Feed-forward: {`kind`: "moe", `expert`: {`ff`}, `router`: {`experts`, `top`, `identity`, `groups`:
{`count`, `keep`}}, `shared`: {`ff`} or null}.

Every size and every constant that can differ between models comes from here.  A layer kind or a
feed-forward kind the engine does not know rejects the file (it would change what is computed); other
keys it does not know are named in a warning and left alone.
"""
from __future__ import annotations

import math
import sys
from dataclasses import dataclass
from typing import Optional

from .llama import ConfigError

_TOP_KEYS = {"architecture", "architectures", "model_type", "torch_dtype", "dtype", "vocab", "width", "layers", "loop",
             "norm", "embedding", "eos_token_id", "max_context"}
_MIXER_KEYS = {"rglru": {"width", "blocks", "conv"},
               "attention": {"heads", "kv_heads", "dim", "vdim", "scale", "mask"}}
DEFAULT_CONTEXT = 1 << 17        # positions enter only as distances: the design has no limit of its own


def _positive_int(where: str, v) -> int:
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"{where} must be a positive integer, got {v!r}")
    return v


def _count(where: str, v) -> int:
    if isinstance(v, bool) or not isinstance(v, int) or v < 0:
        raise ConfigError(f"{where} must be a non-negative integer, got {v!r}")
    return v


def _number(where: str, v) -> float:
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(v):
        raise ConfigError(f"{where} must be a finite number, got {v!r}")
    return float(v)


def _warn_unknown(where: str, have, known) -> None:
    unknown = sorted(set(have) - set(known))
    if unknown:
        print(f"[mdma_b200] {where} has keys the Mogevik reader does not know and leaves alone: {unknown}", file=sys.stderr)


@dataclass(frozen=True)
class MogevikRouted:
    """A routed feed-forward: `experts` experts of `ff` + `identity` identity experts, `top` per token, in
    `groups` groups of which `keep` can be chosen from, and a shared expert of `shared_ff` (0: none)."""
    ff: int
    experts: int
    identity: int
    top: int
    groups: int
    keep: int
    shared_ff: int


@dataclass(frozen=True)
class MogevikLayer:
    type: str
    mixer: dict                   # rglru: width, blocks, conv; attention: heads, kv_heads, dim, vdim, scale, window
    mlp: Optional[MogevikRouted]


@dataclass(frozen=True)
class MogevikConfig:
    vocab: int
    width: int
    layers: tuple
    eps: float
    embedding_scale: float = 1.0
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 0           # 0: no loop
    eos_token_id: tuple = ()
    max_context: int = DEFAULT_CONTEXT

    @classmethod
    def from_dict(cls, raw: dict) -> "MogevikConfig":
        _warn_unknown("config.json", raw, _TOP_KEYS)
        for key in ("vocab", "width", "layers", "norm"):
            if key not in raw:
                raise ConfigError(f"config.json lacks {key!r}")
        vocab, width = _positive_int("vocab", raw["vocab"]), _positive_int("width", raw["width"])
        norm = raw["norm"]
        if not isinstance(norm, dict) or "eps" not in norm:
            raise ConfigError("`norm` must be {\"eps\": number}")
        eps = _number("norm.eps", norm["eps"])
        if eps < 0:
            raise ConfigError(f"norm.eps must be >= 0, got {eps!r}")
        scale = 1.0
        emb = raw.get("embedding")
        if emb is not None:
            if not isinstance(emb, dict):
                raise ConfigError("`embedding` must be an object")
            _warn_unknown("embedding", emb, {"scale"})
            if emb.get("scale") is not None:
                scale = _number("embedding.scale", emb["scale"])
        if not isinstance(raw["layers"], list) or not raw["layers"]:
            raise ConfigError("`layers` must be a list with at least one layer")
        layers = tuple(cls._layer(f"layers[{i}]", entry) for i, entry in enumerate(raw["layers"]))
        start = stop = times = 0
        loop = raw.get("loop")
        if loop is not None:
            if not isinstance(loop, dict) or not {"start", "stop", "times"} <= set(loop):
                raise ConfigError("`loop` must be null or have `start`, `stop` and `times`")
            start, stop, times = (_count(f"loop.{k}", loop[k]) for k in ("start", "stop", "times"))
            if not (0 <= start < stop <= len(layers)) or times < 1:
                raise ConfigError(f"loop {loop} does not name a run of the {len(layers)} layers at least once")
        eos = raw.get("eos_token_id", ())
        eos = (eos,) if isinstance(eos, int) else tuple(eos or ())
        max_context = _positive_int("max_context", raw.get("max_context", DEFAULT_CONTEXT))
        return cls(vocab, width, layers, eps, scale, start, stop, times, eos, max_context)

    @staticmethod
    def _layer(where: str, entry) -> MogevikLayer:
        if not isinstance(entry, dict) or "type" not in entry or "mixer" not in entry:
            raise ConfigError(f"{where} must have `type`, `mixer` and `mlp`")
        _warn_unknown(where, entry, {"type", "mixer", "mlp"})
        kind, raw = entry["type"], entry["mixer"]
        if kind not in _MIXER_KEYS:
            raise ConfigError(f"{where}.type {kind!r} is not implemented (have {sorted(_MIXER_KEYS)})")
        if not isinstance(raw, dict):
            raise ConfigError(f"{where}.mixer must be an object")
        _warn_unknown(f"{where}.mixer", raw, _MIXER_KEYS[kind])
        if kind == "rglru":
            mixer = {k: _positive_int(f"{where}.mixer.{k}", raw.get(k)) for k in ("width", "blocks", "conv")}
            if mixer["width"] % mixer["blocks"]:
                raise ConfigError(f"{where}: {mixer['width']} channels do not divide into {mixer['blocks']} blocks")
        else:
            mixer = {k: _positive_int(f"{where}.mixer.{k}", raw.get(k)) for k in ("heads", "dim")}
            mixer["kv_heads"] = _positive_int(f"{where}.mixer.kv_heads", raw.get("kv_heads", mixer["heads"]))
            mixer["vdim"] = _positive_int(f"{where}.mixer.vdim", raw.get("vdim", mixer["dim"]))
            mixer["scale"] = _number(f"{where}.mixer.scale", raw.get("scale", mixer["dim"] ** -0.5))
            if mixer["heads"] % mixer["kv_heads"]:
                raise ConfigError(f"{where}: {mixer['heads']} heads do not divide over {mixer['kv_heads']} kv heads")
            mask = raw.get("mask")
            mixer["window"] = 0
            if mask is not None:
                if not isinstance(mask, dict):
                    raise ConfigError(f"{where}.mixer.mask must be an object or null")
                _warn_unknown(f"{where}.mixer.mask", mask, {"size"})
                if mask.get("size") is not None:
                    mixer["window"] = _positive_int(f"{where}.mixer.mask.size", mask["size"])
        return MogevikLayer(kind, mixer, MogevikConfig._mlp(f"{where}.mlp", entry.get("mlp")))

    @staticmethod
    def _mlp(where: str, raw) -> Optional[MogevikRouted]:
        if raw is None:
            return None
        if not isinstance(raw, dict) or raw.get("kind") != "moe":
            raise ConfigError(f"{where} must be null or a feed-forward of kind 'moe'")
        _warn_unknown(where, raw, {"kind", "expert", "router", "shared"})
        expert, router = raw.get("expert"), raw.get("router")
        if not isinstance(expert, dict) or not isinstance(router, dict):
            raise ConfigError(f"{where} must have `expert` and `router`")
        _warn_unknown(f"{where}.router", router, {"experts", "top", "identity", "groups"})
        ff = _positive_int(f"{where}.expert.ff", expert.get("ff"))
        experts = _count(f"{where}.router.experts", router.get("experts"))
        identity = _count(f"{where}.router.identity", router.get("identity") or 0)
        top = _positive_int(f"{where}.router.top", router.get("top"))
        n_routed = experts + identity
        if not 0 < top <= n_routed:
            raise ConfigError(f"{where}: top {top} of {n_routed} routed outputs")
        count = keep = 1
        groups = router.get("groups")
        if groups is not None:
            if not isinstance(groups, dict):
                raise ConfigError(f"{where}.router.groups must be an object or null")
            count = _positive_int(f"{where}.router.groups.count", groups.get("count"))
            keep = _positive_int(f"{where}.router.groups.keep", groups.get("keep", count))
            if n_routed % count or keep > count:
                raise ConfigError(f"{where}: {n_routed} routed outputs do not form {count} groups of which {keep} are kept")
        shared_ff = 0
        shared = raw.get("shared")
        if shared is not None:
            if not isinstance(shared, dict):
                raise ConfigError(f"{where}.shared must be an object or null")
            shared_ff = _positive_int(f"{where}.shared.ff", shared.get("ff"))
        return MogevikRouted(ff, experts, identity, top, count, keep, shared_ff)
