"""Typed configuration of the Gevonex decoder, read from config.json.

Keys: `vocab`, `width`, `layers` (a list; each entry has `type`, the mixer kind, `mixer`,
its sizes, and `mlp`, the feed-forward's sizes or null), `loop` (`start`, `stop`, `times`:
layers start..stop-1 run `times` times in a row; absent or null: no loop), `norm.eps`,
`logit_softcap` (absent, null or 0: none).  Every size and every constant that can differ
between models comes from here.  A layer kind, a feed-forward kind or a mixer key the engine does
not know rejects the file (it would change what is computed); a top-level key it does not know
is named in a warning and otherwise left alone (tensors it would call for fail the weight check).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional

from .llama import ConfigError

_TOP_KEYS = {"architecture", "architectures", "model_type", "torch_dtype", "dtype", "vocab", "width", "layers",
             "loop", "norm", "logit_softcap", "eos_token_id", "max_context"}
_MIXER_KEYS = {
    "mingru": {"width"},
    "mamba2": {"heads", "vdim", "state", "groups", "norm_groups", "conv"},
    "latent_attention": {"heads", "dim", "vdim", "kv_rank", "scale"},
}
DEFAULT_CONTEXT = 1 << 17        # the design has no positions, so no limit of its own; engines size their cache below this


def _positive_int(where: str, v) -> int:
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"{where} must be a positive integer, got {v!r}")
    return v


@dataclass(frozen=True)
class GevonexLayer:
    type: str
    mixer: dict
    mlp: Optional[dict]           # {"kind": "dense", "ff": n} or None


@dataclass(frozen=True)
class GevonexConfig:
    vocab: int
    width: int
    layers: tuple
    eps: float
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 0           # 0: no loop
    logit_softcap: float = 0.0
    eos_token_id: tuple = ()
    max_context: int = DEFAULT_CONTEXT

    @classmethod
    def from_dict(cls, raw: dict) -> "GevonexConfig":
        unknown = sorted(set(raw) - _TOP_KEYS)
        if unknown:
            import sys
            print(f"[mdma_b200] config.json has keys the Gevonex reader does not know and leaves alone: {unknown}",
                  file=sys.stderr)
        for key in ("vocab", "width", "layers", "norm"):
            if key not in raw:
                raise ConfigError(f"config.json lacks {key!r}")
        vocab, width = _positive_int("vocab", raw["vocab"]), _positive_int("width", raw["width"])
        norm = raw["norm"]
        if not isinstance(norm, dict) or set(norm) != {"eps"}:
            raise ConfigError("`norm` must be {\"eps\": number}")
        eps = norm["eps"]
        if isinstance(eps, bool) or not isinstance(eps, (int, float)) or not math.isfinite(eps) or eps < 0:
            raise ConfigError(f"norm.eps must be a finite number >= 0, got {eps!r}")
        if not isinstance(raw["layers"], list) or not raw["layers"]:
            raise ConfigError("`layers` must be a list with at least one layer")
        layers = []
        for i, entry in enumerate(raw["layers"]):
            where = f"layers[{i}]"
            if not isinstance(entry, dict) or set(entry) - {"type", "mixer", "mlp"} or "type" not in entry or "mixer" not in entry:
                raise ConfigError(f"{where} must have `type`, `mixer` and `mlp`")
            kind = entry["type"]
            if kind not in _MIXER_KEYS:
                raise ConfigError(f"{where}.type {kind!r} is not implemented (have {sorted(_MIXER_KEYS)})")
            mixer = entry["mixer"]
            if not isinstance(mixer, dict) or set(mixer) != _MIXER_KEYS[kind]:
                raise ConfigError(f"{where}.mixer must have exactly the keys {sorted(_MIXER_KEYS[kind])}")
            for k, v in mixer.items():
                if k == "scale":
                    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(v):
                        raise ConfigError(f"{where}.mixer.scale must be a finite number")
                else:
                    _positive_int(f"{where}.mixer.{k}", v)
            if kind == "mamba2":
                if mixer["heads"] % mixer["groups"]:
                    raise ConfigError(f"{where}: {mixer['heads']} heads do not divide over {mixer['groups']} groups")
                if (mixer["heads"] * mixer["vdim"]) % mixer["norm_groups"]:
                    raise ConfigError(f"{where}: heads*vdim does not divide into {mixer['norm_groups']} norm parts")
            mlp = entry.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or set(mlp) != {"kind", "ff"}:
                    raise ConfigError(f"{where}.mlp must be null or have `kind` and `ff`")
                if mlp["kind"] != "dense":
                    raise ConfigError(f"{where}.mlp.kind {mlp['kind']!r} is not implemented (only 'dense')")
                _positive_int(f"{where}.mlp.ff", mlp["ff"])
            layers.append(GevonexLayer(kind, dict(mixer), dict(mlp) if mlp is not None else None))
        start = stop = times = 0
        loop = raw.get("loop")
        if loop is not None:
            if not isinstance(loop, dict) or set(loop) != {"start", "stop", "times"}:
                raise ConfigError("`loop` must be null or have `start`, `stop` and `times`")
            start, stop, times = loop["start"], loop["stop"], loop["times"]
            for k, v in loop.items():
                if isinstance(v, bool) or not isinstance(v, int) or v < 0:
                    raise ConfigError(f"loop.{k} must be a non-negative integer, got {v!r}")
            if not (0 <= start < stop <= len(layers)) or times < 1:
                raise ConfigError(f"loop {loop} does not name a run of the {len(layers)} layers at least once")
        cap = raw.get("logit_softcap") or 0.0
        if isinstance(cap, bool) or not isinstance(cap, (int, float)) or not math.isfinite(cap) or cap < 0:
            raise ConfigError(f"logit_softcap must be a positive number or null, got {cap!r}")
        eos = raw.get("eos_token_id", ())
        eos = (eos,) if isinstance(eos, int) else tuple(eos or ())
        max_context = _positive_int("max_context", raw.get("max_context", DEFAULT_CONTEXT))
        return cls(vocab, width, tuple(layers), float(eps), start, stop, times, float(cap), eos, max_context)
