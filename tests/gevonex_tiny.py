"""Small Gevonex configurations and weights for the tests.  The sizes differ from one another
in every respect; none repeats a size combination of a released model.  Weights are made here,
tensor kind by tensor kind, so that every mechanism carries signal: gates are not all half open,
decays differ per head, sinks take real probability mass, shifts mix a good part of the row before."""
import json
import os
import tempfile

import torch


def _layer(kind, mixer, ff):
    return {"type": kind, "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


# a loop in the middle (a layer before it, one after), three passes; a layer without feed-forward;
# groups and norm parts that are not 1; query, value and latent sizes all different; a recurrent width
# that is not the model's
CFG_A = {
    "architecture": "Gevonex", "vocab": 97, "width": 64, "norm": {"eps": 1e-5}, "logit_softcap": 9.0,
    "loop": {"start": 1, "stop": 3, "times": 3},
    "layers": [
        _layer("mamba2", {"heads": 4, "vdim": 8, "state": 16, "groups": 2, "norm_groups": 2, "conv": 3}, 96),
        _layer("latent_attention", {"heads": 3, "dim": 16, "vdim": 24, "kv_rank": 40, "scale": 0.3}, None),
        _layer("mingru", {"width": 80}, 72),
        _layer("latent_attention", {"heads": 2, "dim": 8, "vdim": 8, "kv_rank": 16, "scale": 0.5}, 64),
    ],
}

# no loop, no soft cap; a width that is no multiple of 8 (no tensor-core product takes it);
# a convolution of two taps and one of five; a state size that is no power of two
CFG_B = {
    "architecture": "Gevonex", "vocab": 53, "width": 36, "norm": {"eps": 1e-6}, "logit_softcap": None,
    "layers": [
        _layer("mingru", {"width": 36}, 50),
        _layer("mamba2", {"heads": 3, "vdim": 12, "state": 24, "groups": 3, "norm_groups": 1, "conv": 2}, None),
        _layer("latent_attention", {"heads": 5, "dim": 12, "vdim": 4, "kv_rank": 20, "scale": 0.25}, 44),
        _layer("mamba2", {"heads": 2, "vdim": 20, "state": 8, "groups": 1, "norm_groups": 4, "conv": 5}, 36),
    ],
}

# sizes the tensor-core products take (multiples of 16), one pass of a loop over the first layers
CFG_C = {
    "architecture": "Gevonex", "vocab": 160, "width": 128, "norm": {"eps": 1e-5}, "logit_softcap": 20.0,
    "loop": {"start": 0, "stop": 2, "times": 1},
    "layers": [
        _layer("latent_attention", {"heads": 4, "dim": 32, "vdim": 16, "kv_rank": 64, "scale": 0.2}, 192),
        _layer("mamba2", {"heads": 4, "vdim": 32, "state": 64, "groups": 1, "norm_groups": 2, "conv": 4}, 128),
        _layer("mingru", {"width": 192}, 256),
    ],
}


# no attention at all (no cache group), and attention only (state only for the token shift); a latent wider than
# the tensor-core attention kernels take, so the plain kernel serves it in both engines
CFG_D = {
    "architecture": "Gevonex", "vocab": 61, "width": 48, "norm": {"eps": 1e-5}, "logit_softcap": 12.0,
    "loop": {"start": 0, "stop": 1, "times": 2},
    "layers": [
        _layer("mingru", {"width": 64}, 48),
        _layer("mamba2", {"heads": 2, "vdim": 16, "state": 40, "groups": 2, "norm_groups": 2, "conv": 3}, 80),
    ],
}
CFG_E = {
    "architecture": "Gevonex", "vocab": 70, "width": 64, "norm": {"eps": 1e-5}, "logit_softcap": 25.0,
    "layers": [
        _layer("latent_attention", {"heads": 2, "dim": 24, "vdim": 40, "kv_rank": 144, "scale": 0.15}, 64),
        _layer("latent_attention", {"heads": 4, "dim": 16, "vdim": 16, "kv_rank": 48, "scale": 0.3}, None),
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
        if name in ("embed",):
            t = rn(*shape)
        elif name == "head":
            t = rn(*shape) * (2.0 / shape[1] ** 0.5)
        elif name == "loop.in":
            t = rn(*shape) * (1.2 / shape[1] ** 0.5)
            t[:, :shape[0]] += 0.7 * torch.eye(shape[0])          # the stream mostly goes through
        elif name == "loop.step":
            t = rn(*shape) * 0.5
        elif last == "alpha":
            t = ru(0.4, 1.3)
        elif last in ("norm1", "norm2") or name == "final.norm" or name.endswith("mix.norm") or name.endswith("dkv.norm"):
            t = 1.0 + 0.25 * rn(*shape)
        elif last == "b" and len(shape) == 1 and ("norm" in name.split(".")[-2]):
            t = 0.1 * rn(*shape)
        elif last == "shift":
            t = ru(0.05, 0.95, *shape)
        elif last == "b":                        # gate and projection biases, the convolution's
            t = 0.8 * rn(*shape)
        elif last == "conv":
            t = 0.6 * rn(*shape)
        elif last == "dt_bias":
            t = ru(-4.0, 0.5, *shape)
        elif last == "A_log":
            t = ru(-1.5, 1.5, *shape)
        elif last == "D":
            t = 1.0 + 0.3 * rn(*shape)
        elif last == "sink":
            t = 1.5 * rn(*shape) + 0.5
        elif len(shape) == 2:
            t = rn(*shape) * (1.3 / shape[1] ** 0.5)
        else:
            raise AssertionError(f"no recipe for {name} {shape}")
        out[name] = t.to(torch.float32)
    return out


def make_model(cfg, seed, dtype=torch.float32, root=None):
    """Write a folder (config.json + model.safetensors in `dtype`); returns (dir, tensors as stored, in float32)."""
    from mdma_b200.weights import write_safetensors
    d = tempfile.mkdtemp(prefix="gevonex_tiny_", dir=root)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    tensors = {n: t.to(dtype) for n, t in make_tensors(cfg, seed).items()}
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    return d, {n: t.float() for n, t in tensors.items()}
