"""The Gevonex decoder written out plainly: whole sequences, float64, no cache, one
function per mechanism, token-by-token loops where the design has a recurrence.
Shares nothing with the library; the tests compare the engine with this."""
import math

import torch


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def rms_unit(x, eps):
    """x divided by its root mean square over the last axis (eps inside the root)."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def dyt(x, w, b, alpha):
    """Dynamic tanh: no statistics of x at all."""
    return torch.tanh(alpha * x) * w + b


def token_shift(h, mu):
    """h_t + (h_(t-1) - h_t) * mu, with h_(-1) = 0; the previous token's h is the one before the shift."""
    prev = torch.cat([torch.zeros_like(h[:1]), h[:-1]], dim=0)
    return h + (prev - h) * mu


def mingru(h, W, p):
    z = torch.sigmoid(h @ W[p + "z"].t() + W[p + "z.b"])
    u = h @ W[p + "x"].t() + W[p + "x.b"]
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    g = silu(h @ W[p + "g"].t())
    s = torch.zeros_like(u[0])
    out = []
    for t in range(h.shape[0]):
        s = (1.0 - z[t]) * s + z[t] * cand[t]
        out.append(s * g[t])
    return torch.stack(out) @ W[p + "o"].t()


def causal_conv(u, w, b):
    """u [T, C]; w [C, taps], the last column multiplies the current token; zeros before the start."""
    T, C = u.shape
    taps = w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=u.dtype), u], dim=0)
    out = torch.zeros_like(u)
    for j in range(taps):
        out = out + padded[j:j + T] * w[:, j]
    return out + b


def mamba2(h, W, p, m, eps):
    heads, vd, N, G, ng = m["heads"], m["vdim"], m["state"], m["groups"], m["norm_groups"]
    inner = heads * vd
    T = h.shape[0]
    proj = h @ W[p + "in"].t()
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, W[p + "conv"], W[p + "conv.b"]))
    x = xbc[:, :inner].reshape(T, heads, vd)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = torch.nn.functional.softplus(dt + W[p + "dt_bias"], threshold=1e9)
    rate = torch.exp(W[p + "A_log"])
    S = torch.zeros(heads, N, vd, dtype=h.dtype)
    y = torch.zeros(T, heads, vd, dtype=h.dtype)
    per = heads // G
    for t in range(T):
        for hd in range(heads):
            g = hd // per
            S[hd] = torch.exp(-rate[hd] * dt[t, hd]) * S[hd] + dt[t, hd] * torch.outer(B[t, g], x[t, hd])
            y[t, hd] = S[hd].t() @ C[t, g] + W[p + "D"][hd] * x[t, hd]
    y = y.reshape(T, inner) * silu(z)
    y = rms_unit(y.reshape(T, ng, inner // ng), eps).reshape(T, inner) * W[p + "norm"]
    return y @ W[p + "o"].t()


def latent_attention(h, W, p, m, eps):
    H, d, vd, R = m["heads"], m["dim"], m["vdim"], m["kv_rank"]
    T = h.shape[0]
    q = (h @ W[p + "q"].t()).reshape(T, H, d)
    c = rms_unit(h @ W[p + "dkv"].t(), eps) * W[p + "dkv.norm"]
    k = (c @ W[p + "uk"].t()).reshape(T, H, d)
    v = (c @ W[p + "uv"].t()).reshape(T, H, vd)
    out = torch.zeros(T, H, vd, dtype=h.dtype)
    for hd in range(H):
        s = (q[:, hd] @ k[:, hd].t()) * m["scale"]
        s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
        top = torch.maximum(s.max(dim=-1, keepdim=True).values, W[p + "sink"][hd])
        e = torch.exp(s - top)
        denom = e.sum(dim=-1, keepdim=True) + torch.exp(W[p + "sink"][hd] - top)   # the sink: no key, no value
        out[:, hd] = (e / denom) @ v[:, hd]
    return out.reshape(T, H * vd) @ W[p + "o"].t()


def dense_mlp(h, W, p):
    return gelu_tanh(h @ W[p + "up"].t()) @ W[p + "down"].t()


MIXERS = {"mingru": lambda h, W, p, m, eps: mingru(h, W, p),
          "mamba2": mamba2, "latent_attention": latent_attention}


def layer(x, W, i, spec, eps):
    p = f"l{i}."
    h = dyt(x, W[p + "norm1"], W[p + "norm1.b"], W[p + "norm1.alpha"])
    gate = torch.sigmoid(h @ W[p + "rg1"].t() + W[p + "rg1.b"])
    mixed = MIXERS[spec["type"]](token_shift(h, W[p + "shift"]), W, p + "mix.", spec["mixer"], eps)
    x = x + gate * mixed
    if spec.get("mlp") is not None:
        h = dyt(x, W[p + "norm2"], W[p + "norm2.b"], W[p + "norm2.alpha"])
        gate = torch.sigmoid(h @ W[p + "rg2"].t() + W[p + "rg2.b"])
        x = x + gate * dense_mlp(h, W, p + "mlp.")
    return x


def layer_runs(cfg):
    """The order in which layers run: [(layer, pass number or None when no pass starts there)]."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    runs = [(i, None) for i in range(start)]
    for t in range(times):
        runs += [(i, t if i == start else None) for i in range(start, stop)]
    return runs + [(i, None) for i in range(stop, n)]


def forward(cfg, W, ids, trace=None):
    """Logits [T, vocab] of one sequence; `trace` (a list) receives the residual stream after every layer run."""
    W = {k: v.double() for k, v in W.items()}
    eps = cfg["norm"]["eps"]
    x = W["embed"][torch.tensor(ids)]
    x0 = x
    for i, t in layer_runs(cfg):
        if t is not None:
            x = torch.cat([x, x0], dim=-1) @ W["loop.in"].t() + W["loop.step"][t]
        x = layer(x, W, i, cfg["layers"][i], eps)
        if trace is not None:
            trace.append(x.clone())
    h = dyt(x, W["final.norm"], W["final.norm.b"], W["final.norm.alpha"])
    logits = h @ W["head"].t()
    cap = cfg.get("logit_softcap")
    return cap * torch.tanh(logits / cap) if cap else logits
