"""Attention over a cached latent, without positions.

q = Wq h (heads x dim); c = rms_unit(Wdkv h) * w, `kv_rank` numbers, the only thing the
cache keeps of a token; per head k = Wuk c and v = Wuv c; a query at position p sees every
key up to p; score = (q . k) * scale; the softmax's denominator also holds exp(sink_h), a
learned number per head with no key and no value; the heads' results go through Wo.

Computed in the absorbed form: q'_h = Wuk,h^T q_h lives in the latent space, so that
score = q'_h . c and o_h = Wuv,h (sum_j p_j c_j); the cache is read as one shared head of
size kv_rank that serves as key and as value, whatever the number of heads.
"""
from __future__ import annotations

import dataclasses

import torch

from .. import ops
from ..cache import KVNeed
from ..registry import MIXERS
from ..spec import TensorSpec
from .base import Part
from .linear import Linear


class HeadwiseLinear:
    """out[:, h*N:(h+1)*N] = a[:, h*K:(h+1)*K] @ w[h].T for every head h; w is [heads, N, K].  Steps of
    many tokens (256 or more) run head by head on the tensor cores when the shapes allow, others as one
    launch on the CUDA cores."""

    TENSOR_TOKENS = 256       # below this a launch per head costs more than the CUDA-core launch for all heads

    def __init__(self, w: torch.Tensor, rt):
        self.w, self.rt = w, rt
        self.heads, self.n, self.k = w.shape
        self._tensor_ok = False
        if rt.gemm == "tensor" and w.dtype == torch.bfloat16:
            from .. import ops_tensor
            self._tensor_ok = ops_tensor.gemm_supported(self.n, self.k) and self.n % 8 == 0

    def run(self, a, out, m):
        if (self._tensor_ok and m >= self.TENSOR_TOKENS and a.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0
                and out.dtype == torch.bfloat16):
            from .. import ops_tensor
            for h in range(self.heads):
                ops_tensor.gemm(a[:, h * self.k:(h + 1) * self.k], self.w[h], out[:, h * self.n:(h + 1) * self.n],
                                ops.GEMM_STORE, None, m, st=self.rt.tc)
            return
        if self.rt.gemm == "tensor":
            from .. import ops_tensor
            ops_tensor.flush_pending(a.device, self.rt.tc)
        ops.gemm_simt_batched(a, self.w, out, m)


@MIXERS.register("latent_attention")
class LatentAttention(Part):
    graph_safe = True      # forward reads no host-side per-step values
    MAX_RANK = 1024        # the attention kernel's limit (csrc/latent_attention.cu)

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden = int(p["hidden_size"])
        self.n_heads, self.dim, self.vdim, self.rank = int(p["heads"]), int(p["dim"]), int(p["vdim"]), int(p["kv_rank"])
        self.scale, self.eps = float(p["scale"]), float(p["eps"])
        self.window = int(p.get("window", 0) or 0)
        # as the attention kernels and the engine's scratch plan see it: every head reads one shared head of the cache
        self.n_kv_heads, self.head_dim = 1, self.rank
        self.q_width, self.v_width, self.lat_width = self.n_heads * self.dim, self.n_heads * self.vdim, self.n_heads * self.rank

    def check_limits(self, rt):
        if self.rank > self.MAX_RANK:
            raise ValueError(f"kv_rank {self.rank} is beyond the attention kernel's limit of {self.MAX_RANK}")

    def tensor_specs(self):
        return {"q": TensorSpec((self.q_width, self.hidden)), "dkv": TensorSpec((self.rank, self.hidden)),
                "dkv.norm": TensorSpec((self.rank,), "vector"),
                "uk": TensorSpec((self.q_width, self.rank)), "uv": TensorSpec((self.v_width, self.rank)),
                "sink": TensorSpec((self.n_heads,), "vector", "zeros"), "o": TensorSpec((self.hidden, self.v_width))}

    def fused_tensors(self):
        return {"q_dkv": ("q", "dkv")}           # one product for the queries and the latent

    def device_tensors(self):
        # the keys' map per head, transposed, so that it is applied to the queries as an ordinary product
        # (counted at four bytes an element: the plan is made before the compute dtype is known to the part)
        return {"uk_t": ((self.n_heads, self.rank, self.dim), torch.float32),
                "sink_log2": ((self.n_heads,), torch.float32)}

    def kv_need(self):
        return KVNeed(1, self.rank, self.window, values=False)

    def state_need(self):
        return None

    def _names(self):
        tag = f"{self.n_heads}_{self.dim}_{self.vdim}_{self.rank}"
        return f"latent_proj_{tag}", f"latent_q_{tag}", f"latent_o_{tag}", f"latent_v_{tag}"

    def workspace(self):
        proj, q, o, v = self._names()
        return {proj: (self.q_width + self.rank, "act"), q: (self.lat_width, "act"), o: (self.lat_width, "act"),
                v: (self.v_width, "act")}

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        fused = tensors.get("q_dkv")
        if fused is None:
            fused = torch.cat([tensors["q"], tensors["dkv"]], dim=0).contiguous()
        self.q_dkv = Linear(fused, rt)
        self.o = Linear(tensors["o"], rt)
        self.latent_norm, self.sink = tensors["dkv.norm"], tensors["sink"]
        uk = self.uk = tensors["uk"]
        shape = (self.n_heads, self.rank, self.dim)
        uk_t = rt.alloc(shape, uk.dtype) if rt.alloc is not None else torch.empty(shape, dtype=uk.dtype, device=uk.device)
        uk_t.copy_(uk.view(self.n_heads, self.dim, self.rank).transpose(1, 2))
        self.absorb = HeadwiseLinear(uk_t, rt)
        # the tensor-core attention kernels work in powers of two: the sinks times log2(e), as floats
        self.sink_log2 = (rt.alloc((self.n_heads,), torch.float32) if rt.alloc is not None
                          else torch.empty(self.n_heads, dtype=torch.float32, device=uk.device))
        self.sink_log2.copy_(self.sink.float() * 1.4426950408889634)
        self._fast_ok = False
        if rt.attention == "fast":
            from .. import ops_tensor
            self._fast_ok = ops_tensor.attention_supported(self.n_heads, 1, self.rank) and self.scale > 0
        self.expand = HeadwiseLinear(tensors["uv"].view(self.n_heads, self.vdim, self.rank), rt)

    def forward(self, ctx, h, x, view, owns_cache=True):
        self._run(ctx, h, x, view, owns_cache, accumulate=True)

    def produce(self, ctx, h, out, view, owns_cache=True, defer=False):
        """`defer`: the last product may leave K-split partial sums of `out` for the caller's next kernel."""
        self._run(ctx, h, out, view, owns_cache, accumulate=False, defer=defer)

    def _run(self, ctx, h, target, view, owns_cache, accumulate, defer=False):
        n = ctx.n_tokens
        names = self._names()
        proj = ctx.buf(names[0], self.q_width + self.rank)
        q_lat, o_lat, v = ctx.buf(names[1], self.lat_width), ctx.buf(names[2], self.lat_width), ctx.buf(names[3], self.v_width)
        self.q_dkv.store(h, proj, n)
        if owns_cache:
            ops.latent_norm_store(proj, self.q_width, self.latent_norm, self.eps, self.rank, ctx.tok_seq, ctx.tok_pos,
                                  ctx.seq_slot, view.page_table, view.max_pages, view.page_size, view.k, n)
        self.absorb.run(proj, q_lat, n)
        if self._fast_ok:
            # the latent rows serve as the one key head and as the one value head
            from .. import ops_tensor
            ops_tensor.attention(ctx, q_lat, dataclasses.replace(view, v=view.k), o_lat, self.n_heads, 1, self.rank,
                                 self.window, self.scale, st=self.rt.tc, sink_log2=self.sink_log2)
        else:
            if self.rt.gemm == "tensor":
                from .. import ops_tensor
                ops_tensor.flush_pending(q_lat.device, self.rt.tc)
            ops.latent_attention(q_lat, view.k, self.sink, ctx.tok_seq, ctx.tok_pos, ctx.seq_slot, view.page_table,
                                 view.max_pages, view.page_size, o_lat, n, self.n_heads, self.rank, self.window, self.scale)
        self.expand.run(o_lat, v, n)
        if accumulate:
            self.o.accumulate(v, target, n, defer=False)
        else:
            self.o.store(v, target, n, defer=defer)

    def resident_tensors(self):
        return [self.q_dkv.w, self.o.w, self.latent_norm, self.sink, self.uk, self.expand.w]
