"""Grouped-query attention whose positions enter as a penalty on distance (`distance_attention`).

q = Wq h + bq, k = Wk h + bk, v = Wv h + bv (the biases are optional); nothing is rotated.  A query at
position i of head h reads the keys j of its own sequence with 0 <= i - j < window (every j <= i
without a window):

    score = (q . k) * scale - slope_h * (i - j),    slope_h = 2^(-slope_power (h + 1) / heads),

an ordinary softmax over those keys in float, values of `v_dim` numbers a head (which may differ from
the keys' `head_dim`), kv head = q head // (heads / kv heads).  With `gate`, the concatenated heads are
multiplied element by element with sigmoid(Wg h) before the output product; the result times Wo^T is
added to the residual stream.  Heads, sizes, scale, window and the slopes' power are parameters
(`slope_power` 0: no penalty).

Keys and values go to the paged cache as they leave the projection.  In the serving engine, heads whose
keys and values have one size that the tensor-core attention kernels take run on those (the tcgen05
kernel for long steps, the mma.sync kernel between, the decode kernel for single tokens: the same
kernels as the other attention mixers, with the slopes as one more per-head parameter); the gate is
then a small kernel of its own.  Other geometries run on this mixer's CUDA-core kernels, which take
keys and values of different sizes and apply the gate themselves: one that stages a tile's keys and
values in shared memory (the serving engine), and one that keeps a warp per (token, head) and visits
keys in position order (the 32-bit engine, and geometries whose tile does not fit shared memory).
"""
from __future__ import annotations

import torch

from .. import ops
from ..cache import KVNeed
from ..registry import MIXERS
from ..spec import TensorSpec
from .base import Part
from .linear import Linear


@MIXERS.register("distance_attention")
class DistanceAttention(Part):
    graph_safe = True      # forward reads no host-side per-step values
    MAX_HEAD_DIM = 256     # the kernels' limit for keys and for values

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden = int(p["hidden_size"])
        self.n_heads, self.n_kv_heads = int(p["num_heads"]), int(p["num_kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.v_dim = int(p.get("v_dim") or self.head_dim)
        self.scale = float(p["scale"])
        self.window = int(p.get("window", 0) or 0)
        self.slope_power = float(p.get("slope_power", 8.0))
        self.bias = bool(p.get("bias", False))
        self.gate = bool(p.get("gate", False))
        if self.n_heads % self.n_kv_heads:
            raise ValueError(f"{self.n_heads} heads do not divide over {self.n_kv_heads} kv heads")
        self.q_width = self.n_heads * self.head_dim
        self.k_width = self.n_kv_heads * self.head_dim
        self.v_width = self.n_kv_heads * self.v_dim
        self.out_width = self.n_heads * self.v_dim
        self.row_width = self.q_width + self.k_width + self.v_width

    def check_limits(self, rt):
        if max(self.head_dim, self.v_dim) > self.MAX_HEAD_DIM:
            raise ValueError(f"head sizes {self.head_dim} / {self.v_dim} are beyond the attention kernels' limit of "
                             f"{self.MAX_HEAD_DIM}")

    def tensor_specs(self):
        specs = {"q": TensorSpec((self.q_width, self.hidden)), "k": TensorSpec((self.k_width, self.hidden)),
                 "v": TensorSpec((self.v_width, self.hidden))}
        if self.bias:
            for name in ("q", "k", "v"):
                specs[name + ".b"] = TensorSpec((specs[name].shape[0],), "vector", "normal")
        if self.gate:
            specs["g"] = TensorSpec((self.out_width, self.hidden))
        specs["o"] = TensorSpec((self.hidden, self.out_width))
        return specs

    def fused_tensors(self):
        fused = {"qkv": ("q", "k", "v")}          # one product for the three projections
        if self.bias:
            fused["qkv.b"] = ("q.b", "k.b", "v.b")
        return fused

    def device_tensors(self):
        return {"slopes": ((self.n_heads,), torch.float32), "slopes_log2": ((self.n_heads,), torch.float32)}

    def kv_need(self):
        return KVNeed(self.n_kv_heads, self.head_dim, self.window, v_dim=0 if self.v_dim == self.head_dim else self.v_dim)

    def state_need(self):
        return None

    def workspace(self):
        tag = f"{self.row_width}_{self.out_width}"
        return {f"dqkv_{tag}": (self.row_width, "act"), f"dgate_{tag}": (self.out_width, "act"),
                f"dout_{tag}": (self.out_width, "act")}

    def slope_values(self) -> torch.Tensor:
        """slope_h = 2^(-slope_power (h + 1) / heads), worked out in double and kept as float."""
        if self.slope_power == 0:
            return torch.zeros(self.n_heads, dtype=torch.float32)
        h = torch.arange(1, self.n_heads + 1, dtype=torch.float64)
        return torch.pow(torch.tensor(2.0, dtype=torch.float64), -self.slope_power * h / self.n_heads).to(torch.float32)

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        fused = tensors.get("qkv")
        if fused is None:
            fused = torch.cat([tensors["q"], tensors["k"], tensors["v"]], dim=0).contiguous()
        bias = None
        if self.bias:
            bias = tensors.get("qkv.b")
            if bias is None:
                bias = torch.cat([tensors["q.b"], tensors["k.b"], tensors["v.b"]]).contiguous()
        self.qkv = Linear(fused, rt, bias=bias)
        self.g = Linear(tensors["g"], rt) if self.gate else None
        self.o = Linear(tensors["o"], rt)
        self.slopes = rt.derived(self.slope_values())
        self.slopes_log2 = None
        self._fast_ok = False
        if rt.attention == "fast" and self.v_dim == self.head_dim:
            from .. import ops_tensor
            self._fast_ok = ops_tensor.attention_supported(self.n_heads, self.n_kv_heads, self.head_dim)
        if self._fast_ok:
            self.slopes_log2 = rt.derived((self.slope_values().double() * 1.4426950408889634).to(torch.float32))
        self._tiled_ok = ops.attention_distance_tiled_fits(self.n_heads, self.n_kv_heads, self.head_dim, self.v_dim)

    def forward(self, ctx, h, x, view, owns_cache=True):
        n = ctx.n_tokens
        tag = f"{self.row_width}_{self.out_width}"
        qkv = ctx.buf(f"dqkv_{tag}", self.row_width)
        out = ctx.buf(f"dout_{tag}", self.out_width)
        gate = None
        self.qkv.store(h, qkv, n)
        if self.g is not None:
            gate = ctx.buf(f"dgate_{tag}", self.out_width)
            self.g.store(h, gate, n)
        if owns_cache:
            ops.kv_store(qkv, self.q_width, self.q_width + self.k_width, self.k_width, self.v_width, ctx.tok_seq,
                         ctx.tok_pos, ctx.seq_slot, view.page_table, view.max_pages, view.page_size, view.k, view.v, n)
        if self._fast_ok:
            from .. import ops_tensor
            ops_tensor.attention(ctx, qkv, view, out, self.n_heads, self.n_kv_heads, self.head_dim, self.window, self.scale,
                                 st=self.rt.tc, slope_log2=self.slopes_log2)
            if gate is not None:
                ops.sigmoid_gate(out, gate, n)
            self.o.accumulate(out, x, n, defer=False)
            return
        # the serving engine stages keys and values per tile (also for single tokens: a block per sequence and kv head
        # reads them once for the whole group); the 32-bit engine visits keys in position order, one warp per (token, head)
        tiled = self._tiled_ok and qkv.dtype != torch.float32
        ops.attention_distance(qkv, view.k, view.v, ctx, view.page_table, view.max_pages, view.page_size, self.slopes,
                               gate, out, self.n_heads, self.n_kv_heads, self.head_dim, self.v_dim, self.window,
                               self.scale, tiled)
        self.o.accumulate(out, x, n, defer=False)

    def resident_tensors(self):
        return [t for t in (self.qkv.w, self.qkv.bias, self.g.w if self.g else None, self.o.w) if t is not None]
