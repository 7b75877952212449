"""A plain statement of the Mogevik decoder in float64: whole sequences, no cache, no batches, one
function per mechanism, written from the equations and sharing nothing with the engine.

Notation: x [T, W] the residual stream of one sequence, positions 0..T-1; W[name] the tensors.
"""
import math

import torch

F64 = torch.float64


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def layer_norm(x, w, eps):
    """(x - mean) / sqrt(var + eps) * w; var = mean of squared deviations; no bias."""
    mean = x.mean(-1, keepdim=True)
    var = ((x - mean) ** 2).mean(-1, keepdim=True)
    return (x - mean) / torch.sqrt(var + eps) * w


def causal_conv(x, w, b):
    """out[t, c] = b[c] + sum_j w[c, j] x[t - (taps-1) + j, c]; zeros before the start; the last tap is the current row."""
    T, C = x.shape
    taps = w.shape[1]
    out = b.expand(T, C).clone()
    for t in range(T):
        for j in range(taps):
            src = t - (taps - 1) + j
            if src >= 0:
                out[t] += w[:, j] * x[src]
    return out


def rglru(h, W, p, sizes, decay=8.0):
    """The recurrent block: y = gelu(Wy h + by); u = conv(Wx h + bx); per block of channels r, i = sigmoid(R u + b);
    log a = -decay r softplus(lam); S = a S + sqrt(1 - a^2) i u from S = 0; out = Wo (S * y)."""
    width, blocks = sizes["width"], sizes["blocks"]
    T = h.shape[0]
    y = gelu_tanh(h @ W[p + "y"].T + W[p + "y.b"])
    u = causal_conv(h @ W[p + "x"].T + W[p + "x.b"], W[p + "conv"], W[p + "conv.b"])
    n = width // blocks
    r, i = torch.empty_like(u), torch.empty_like(u)
    for b in range(blocks):
        part = u[:, b * n:(b + 1) * n]
        r[:, b * n:(b + 1) * n] = torch.sigmoid(part @ W[p + "ra"][b].T + W[p + "ra.b"][b])
        i[:, b * n:(b + 1) * n] = torch.sigmoid(part @ W[p + "ri"][b].T + W[p + "ri.b"][b])
    log_a = -decay * r * torch.nn.functional.softplus(W[p + "lam"])
    a = torch.exp(log_a)
    S = torch.zeros(width, dtype=h.dtype)
    rows = []
    for t in range(T):
        S = a[t] * S + torch.sqrt(-torch.expm1(2.0 * log_a[t])) * i[t] * u[t]
        rows.append(S)
    return (torch.stack(rows) * y) @ W[p + "o"].T


def distance_attention(h, W, p, sizes, slope_power=8.0):
    """softmax over the keys j with 0 <= i - j < window of (q.k) scale - slope_h (i - j), slope_h = 2^(-power (h+1) / H);
    heads concatenated, times sigmoid(Wg h), through Wo."""
    H, G, D, V = sizes["heads"], sizes["kv_heads"], sizes["dim"], sizes["vdim"]
    window = (sizes.get("mask") or {}).get("size") or 0
    T = h.shape[0]
    q = (h @ W[p + "q"].T + W[p + "q.b"]).view(T, H, D)
    k = (h @ W[p + "k"].T + W[p + "k.b"]).view(T, G, D)
    v = (h @ W[p + "v"].T + W[p + "v.b"]).view(T, G, V)
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for head in range(H):
        g = head // (H // G)
        slope = 2.0 ** (-slope_power * (head + 1) / H)
        for i in range(T):
            lo = max(0, i + 1 - window) if window else 0
            js = torch.arange(lo, i + 1)
            score = (k[lo:i + 1, g] @ q[i, head]) * sizes["scale"] - slope * (i - js).to(h.dtype)
            out[i, head] = torch.softmax(score, 0) @ v[lo:i + 1, g]
    return (out.reshape(T, H * V) * torch.sigmoid(h @ W[p + "g"].T)) @ W[p + "o"].T


_margins = None      # while a list: every call of `route` appends, per token, how close its choice was (see `forward`)


def route(h, W, p, router):
    """(chosen [T, top], weights [T, top], scores s [T, n]) of the router."""
    n = router["experts"] + (router.get("identity") or 0)
    s = torch.softmax(h @ W[p + "router"].T, -1)
    c = s + W[p + "correction"]
    groups = router.get("groups")
    if groups and groups["keep"] < groups["count"]:
        per = n // groups["count"]
        for t in range(h.shape[0]):
            scores = [float(c[t, g * per:(g + 1) * per].max()) for g in range(groups["count"])]
            kept = sorted(range(groups["count"]), key=lambda g: (-scores[g], g))[:groups["keep"]]
            for g in range(groups["count"]):
                if g not in kept:
                    c[t, g * per:(g + 1) * per] = float("-inf")
    chosen = torch.empty(h.shape[0], router["top"], dtype=torch.long)
    margin = torch.full((h.shape[0],), float("inf"), dtype=h.dtype)
    for t in range(h.shape[0]):
        order = sorted(range(n), key=lambda e: (-float(c[t, e]), e))
        chosen[t] = torch.tensor(order[:router["top"]])
        if router["top"] < n and float(c[t, order[router["top"]]]) > float("-inf"):
            margin[t] = c[t, order[router["top"] - 1]] - c[t, order[router["top"]]]      # last chosen against first left out
    if groups and groups["keep"] < groups["count"]:
        per = n // groups["count"]
        gs = (s + W[p + "correction"]).view(-1, groups["count"], per).max(-1).values.sort(-1, descending=True).values
        margin = torch.minimum(margin, gs[:, groups["keep"] - 1] - gs[:, groups["keep"]])   # last kept group against the next
    if _margins is not None:
        _margins.append(margin)
    picked = s.gather(1, chosen)
    return chosen, picked / (picked.sum(-1, keepdim=True) + 1e-20), s


def gated_ffn(h, W, p):
    return (silu(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def routed_ffn(h, W, p, mlp):
    router = mlp["router"]
    chosen, weights, _ = route(h, W, p, router)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(router["top"]):
            e = int(chosen[t, j])
            y = h[t] if e >= router["experts"] else gated_ffn(h[t:t + 1], W, f"{p}e{e}.")[0]      # identity experts return h
            out[t] += weights[t, j] * y
    if mlp.get("shared"):
        out = out + torch.sigmoid(h @ W[p + "shared.sg"].T) * gated_ffn(h, W, p + "shared.")
    return out


def schedule(cfg):
    """[(layer, pass number if a pass starts here else None)]"""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    runs = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        runs += [(i, t if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return runs + [(i, None) for i in range(loop["stop"], n)]


def forward(cfg, tensors, ids, trace=None, skip=None, margins=None):
    """Logits [T, vocab] of one sequence.  `trace`: a list that receives the residual stream after every run of a
    layer.  `skip`: the name of one mechanism to leave out (tests use it to show that each one matters).  `margins`: a
    list that receives ONE tensor [T]: per token, the smallest distance by which any router of any run decided (between
    the last expert chosen and the first left out, and between the last group kept and the next)."""
    global _margins
    W = {k: v.to(F64) for k, v in tensors.items()}
    _margins = [] if margins is not None else None
    eps = cfg["norm"]["eps"]
    x = W["embed"][torch.tensor(ids)] * (1.0 if skip == "embedding_scale" else (cfg.get("embedding") or {}).get("scale", 1.0))
    x0 = x.clone()
    for i, t in schedule(cfg):
        if t is not None:
            if t > 0 and skip != "loop_embedding":
                x = x + x0
            if skip != "loop_step":
                x = x + W["loop.step"][t]
        layer, p = cfg["layers"][i], f"l{i}."
        h = layer_norm(x, W[p + "norm1"], eps)
        if layer["type"] == "rglru":
            mix = rglru(h, W, p + "mix.", layer["mixer"])
        else:
            sizes = dict(layer["mixer"])
            if skip == "window":
                sizes["mask"] = None
            mix = distance_attention(h, W, p + "mix.", sizes, 0.0 if skip == "slopes" else 8.0)
        ff = 0.0
        if layer.get("mlp") is not None:
            mlp = layer["mlp"]
            if skip == "groups":
                mlp = dict(mlp, router=dict(mlp["router"], groups=None))
            if skip == "shared":
                mlp = dict(mlp, shared=None)
            ff = routed_ffn(h, W, p + "mlp.", mlp)
        x = x + (mix + ff)
        if trace is not None:
            trace.append(x.clone())
    if margins is not None:
        margins.append(torch.stack(_margins).min(0).values if _margins else torch.full((len(ids),), float("inf"), dtype=F64))
    _margins = None
    return layer_norm(x, W["final.norm"], eps) @ W["embed"].T
