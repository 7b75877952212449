"""Small Mogevik configurations and weights for the tests.  The sizes differ from one another in every
respect.  Weights are made here, tensor kind by tensor kind, so that every mechanism carries signal:
gates are not all half open, decays span slow and fast channels, the router's softmax is peaked, its
correction changes who is chosen, and the shared expert's gate is not constant."""
import json
import os
import tempfile

import torch


def _moe(ff, experts, top, identity=0, groups=None, shared=None):
    router = {"experts": experts, "top": top, "identity": identity}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": router, "shared": None if shared is None else {"ff": shared}}


def _attn(heads, kv_heads, dim, vdim, scale, window):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
            "mask": None if window is None else {"size": window}}


def _layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


# a loop in the middle with three passes over a recurrent and an attention layer; grouped queries with value heads
# wider than key heads; a window that is no multiple of anything; groups of which half are kept; a layer without a
# feed-forward; a layer whose router has no groups, no identity experts, no shared expert and takes one expert
CFG_A = {
    "architecture": "Mogevik", "vocab": 97, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 4.0},
    "loop": {"start": 1, "stop": 3, "times": 3},
    "layers": [
        _layer("attention", _attn(4, 4, 8, 8, 0.35, 20), _moe(24, 5, 1)),
        _layer("rglru", {"width": 80, "blocks": 5, "conv": 3}, _moe(40, 6, 3, identity=2, groups=(4, 2), shared=56)),
        _layer("attention", _attn(6, 2, 16, 24, 0.25, 37), None),
        _layer("rglru", {"width": 48, "blocks": 1, "conv": 2}, _moe(16, 3, 2, identity=3, groups=(3, 2), shared=8)),
    ],
}

# no loop; a width that is no multiple of 8 (no tensor-core product takes it); one kv head for all query heads;
# key heads wider than value heads; no window at all; a convolution of one tap and one of five; every group kept
CFG_B = {
    "architecture": "Mogevik", "vocab": 53, "width": 36, "norm": {"eps": 1e-6}, "embedding": {"scale": 3.0},
    "layers": [
        _layer("rglru", {"width": 36, "blocks": 3, "conv": 1}, _moe(20, 4, 2, identity=4, groups=(2, 2), shared=12)),
        _layer("attention", _attn(5, 1, 12, 4, 0.3, None), _moe(28, 7, 4, identity=1, groups=(4, 3))),
        _layer("rglru", {"width": 60, "blocks": 4, "conv": 5}, None),
    ],
}

# sizes the tensor-core products take (multiples of 16); one pass of a loop over the first layers; a window of
# exactly one page; as many identity experts as experts; only identity experts beside one expert
CFG_C = {
    "architecture": "Mogevik", "vocab": 160, "width": 128, "norm": {"eps": 1e-5}, "embedding": {"scale": 5.5},
    "loop": {"start": 0, "stop": 2, "times": 1},
    "layers": [
        _layer("attention", _attn(8, 2, 32, 64, 0.18, 64), _moe(64, 8, 4, identity=8, groups=(4, 3), shared=96)),
        _layer("rglru", {"width": 192, "blocks": 4, "conv": 4}, _moe(48, 1, 2, identity=3, shared=32)),
        _layer("attention", _attn(2, 2, 64, 64, 0.12, 150), _moe(80, 16, 6, groups=(8, 4))),
    ],
}

# recurrent layers only (no cache group at all), looped twice from the start; attention only (no state at all)
CFG_D = {
    "architecture": "Mogevik", "vocab": 61, "width": 48, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0},
    "loop": {"start": 0, "stop": 2, "times": 2},
    "layers": [
        _layer("rglru", {"width": 64, "blocks": 2, "conv": 4}, _moe(32, 4, 2, identity=2, groups=(3, 1), shared=24)),
        _layer("rglru", {"width": 40, "blocks": 8, "conv": 2}, None),
    ],
}
CFG_E = {
    "architecture": "Mogevik", "vocab": 70, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0},
    "layers": [
        _layer("attention", _attn(2, 1, 24, 40, 0.2, 9), _moe(32, 9, 3, identity=3, groups=(6, 4), shared=16)),
        _layer("attention", _attn(12, 4, 16, 16, 0.3, 300), None),
    ],
}


def make_tensors(cfg, seed):
    """name -> float32 tensor, for every tensor the architecture declares."""
    from mdma_b200.config import load_config
    from mdma_b200.engine.model import expected_tensors
    arch, typed = load_config(cfg)
    g = torch.Generator().manual_seed(seed)
    rn = lambda *shape: torch.randn(tuple(shape), generator=g)
    ru = lambda lo, hi, *shape: lo + (hi - lo) * torch.rand(tuple(shape), generator=g)
    out = {}
    for name, ts in expected_tensors(arch.describe(typed)).items():
        shape = tuple(ts.shape)
        last = name.split(".")[-1]
        if name == "embed":
            t = rn(*shape) * (1.6 / shape[1] ** 0.5)          # also the output head: logits of deviation ~1.6
        elif name == "loop.step":
            t = rn(*shape) * 0.5
        elif last == "norm1" or name == "final.norm":
            t = 1.0 + 0.25 * rn(*shape)
        elif last == "lam":
            t = ru(-7.0, 0.5, *shape)                         # slow channels (a unit step keeps 0.99) and fast ones
        elif last == "correction":
            t = 0.08 * rn(*shape)                             # of the size of the scores themselves
        elif last == "router":
            t = rn(*shape) * (2.5 / shape[1] ** 0.5)          # a peaked softmax
        elif last == "sg":
            t = rn(*shape) * (2.0 / shape[1] ** 0.5)
        elif last == "b":                                     # projection, gate and convolution biases
            t = 0.5 * rn(*shape)
        elif last == "conv":
            t = 0.6 * rn(*shape)
        elif last in ("ra", "ri"):
            t = rn(*shape) * (1.5 / shape[2] ** 0.5)
        elif len(shape) == 2:
            t = rn(*shape) * (1.3 / shape[1] ** 0.5)
        else:
            raise AssertionError(f"no recipe for {name} {shape}")
        out[name] = t.to(torch.float32)
    return out


def make_model(cfg, seed, dtype=torch.float32, root=None):
    """Write a folder (config.json + model.safetensors in `dtype`); returns (dir, tensors as stored, in float32)."""
    from mdma_b200.weights import write_safetensors
    d = tempfile.mkdtemp(prefix="mogevik_tiny_", dir=root)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    tensors = {n: t.to(dtype) for n, t in make_tensors(cfg, seed).items()}
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    return d, {n: t.float() for n, t in tensors.items()}
