"""Mixers that carry fixed-size state from token to token instead of keys and values.

minGRU (`mingru`): a gated recurrence whose gates read the current token only,
    z = sigmoid(Wz h + bz),  u = Wx h + bx,  c = u + 1/2 (u >= 0) or sigmoid(u) (u < 0),
    S_t = (1 - z) S_(t-1) + z c,   out = Wo (S_t * silu(Wg h));  S has `width` numbers.

Mamba-2 (`mamba2`), the state-space-duality form: Win h = [z | x | B | C | dt] with
inner = heads * vdim, groups G and state size N; x, B, C go through a short causal
convolution per channel and silu; per head h (group h // (heads / G)),
    dt = softplus(dt + dt_bias),  S_t = exp(-exp(A_log) dt) S_(t-1) + dt B_t x_t^T,
    y_t = S_t^T C_t + D x_t;
y * silu(z) is divided by its root mean square in `norm_groups` equal parts, weighted and
sent through Wo.  State: S [heads, N, vdim] and the convolution's last taps-1 inputs.

RG-LRU (`rglru`), a recurrent block with a real-gated linear recurrent unit: two branches of
`width` channels, y = gelu_tanh(Wy h + by) and u = conv(Wx h + bx) (a short causal convolution per
channel, no activation); u is cut into `blocks` equal parts, and in part b
    r = sigmoid(Ra[b] u_b + ra_b),  i = sigmoid(Ri[b] u_b + ri_b)      (square matrices per part),
    log a = -decay r softplus(lam),  S_t = a S_(t-1) + sqrt(1 - a^2) (i u),  out = Wo (S_t * y).
State: S (`width` floats) and the convolution's last taps-1 inputs.  `decay` is 8 unless set.

The state is float, zero at a sequence's start, kept per slot by the cache; everything
that enters the recurrences is float in both engines (the projections write float rows).
Both offer `produce` (the result as float rows) beside the ordinary `forward`.
"""
from __future__ import annotations

import torch

from .. import ops
from ..cache import StateNeed
from ..registry import MIXERS
from ..spec import TensorSpec
from .base import Part
from .linear import Linear


class _StatefulMixer(Part):
    graph_safe = True      # forward reads no host-side per-step values

    def kv_need(self):
        return None

    def forward(self, ctx, h, x, view, owns_cache=True):
        self._run(ctx, h, x, view, accumulate=True)

    def produce(self, ctx, h, out, view, owns_cache=True, defer=False):
        """`defer`: the last product may leave K-split partial sums of `out` for the caller's next kernel."""
        self._run(ctx, h, out, view, accumulate=False, defer=defer)

    def _finish(self, proj, a, target, n, accumulate, defer=False):
        if accumulate:
            proj.accumulate(a, target, n, defer=False)
        else:
            proj.store(a, target, n, defer=defer)


@MIXERS.register("mingru")
class MinGRU(_StatefulMixer):
    CHUNKED_FROM = 128        # rows in the step's longest sequence from which the chunked scan is used

    def __init__(self, spec):
        super().__init__(spec)
        self.hidden, self.width = int(self.params["hidden_size"]), int(self.params["width"])

    def tensor_specs(self):
        w, h = self.width, self.hidden
        return {"z": TensorSpec((w, h)), "z.b": TensorSpec((w,), "vector", "normal"),
                "x": TensorSpec((w, h)), "x.b": TensorSpec((w,), "vector", "normal"),
                "g": TensorSpec((w, h)), "o": TensorSpec((h, w))}

    def fused_tensors(self):
        return {"zxg": ("z", "x", "g")}          # one product for the three projections

    def state_need(self):
        return StateNeed((self.width,), torch.float32)

    def workspace(self):
        return {f"mingru_p_{self.width}": (3 * self.width, "f32"), f"mingru_s_{self.width}": (self.width, "act")}

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        fused = tensors.get("zxg")
        if fused is None:
            fused = torch.cat([tensors["z"], tensors["x"], tensors["g"]], dim=0).contiguous()
        self.zxg = Linear(fused, rt)
        self.o = Linear(tensors["o"], rt)
        self.bz, self.bx = tensors["z.b"], tensors["x.b"]

    def _run(self, ctx, h, target, view, accumulate, defer=False):
        n, w = ctx.n_tokens, self.width
        p = ctx.buf(f"mingru_p_{w}", 3 * w, torch.float32)
        s = ctx.buf(f"mingru_s_{w}", w)
        self.zxg.store(h, p, n)
        # steps of many rows in the serving engine: runs of a sequence side by side; the 32-bit engine keeps the
        # row-by-row order, so that its results do not depend on how a prompt was cut
        chunked = ctx.max_new >= self.CHUNKED_FROM and s.dtype != torch.float32
        ops.mingru_scan(p, self.bz, self.bx, ctx.seq_start, ctx.seq_slot, view.state, s, ctx.n_seqs, w, chunked)
        self._finish(self.o, s, target, n, accumulate, defer)

    def resident_tensors(self):
        return [self.zxg.w, self.o.w, self.bz, self.bx]


@MIXERS.register("mamba2")
class Mamba2(_StatefulMixer):
    MAX_STATE, MAX_TAPS = 256, 16          # the scan kernel's and the convolution kernel's limits
    CHUNK_ROWS = 256                       # the serving engine walks prompts as runs of this many rows side by side

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden = int(p["hidden_size"])
        self.heads, self.vdim, self.n_state = int(p["heads"]), int(p["vdim"]), int(p["state"])
        self.groups, self.norm_groups, self.taps = int(p["groups"]), int(p["norm_groups"]), int(p["conv"])
        self.eps = float(p["eps"])
        self.inner = self.heads * self.vdim
        self.channels = self.inner + 2 * self.groups * self.n_state          # what the convolution sees
        self.proj_width = 2 * self.inner + 2 * self.groups * self.n_state + self.heads
        if self.heads % self.groups:
            raise ValueError(f"{self.heads} heads do not divide over {self.groups} groups")
        if self.inner % self.norm_groups:
            raise ValueError(f"{self.inner} columns do not divide into {self.norm_groups} norm parts")
        self.state_elements = self.heads * self.n_state * self.vdim
        self.state_floats = self.state_elements          # twice that in the 32-bit engine (see check_limits)
        self.wide_state = False
        self.conv_floats = (self.taps - 1) * self.channels

    def check_limits(self, rt):
        # The 32-bit engine keeps S, the step sizes and the decays in double: a decay over a long sequence is a product
        # of thousands of factors below one, and in float the roundings of that chain (not those of the matrix products)
        # are what its logits differ by from the exact ones (measured on a 1,100-token prompt: 7 times less error).
        # Asked here because this is where a part first learns the engine's dtype, before the memory plan is made.
        self.wide_state = rt.dtype == torch.float32
        self.state_floats = (2 if self.wide_state else 1) * self.state_elements
        if self.n_state > self.MAX_STATE:
            raise ValueError(f"state size {self.n_state} is beyond the scan kernel's limit of {self.MAX_STATE}")
        if not 1 <= self.taps <= self.MAX_TAPS:
            raise ValueError(f"a convolution of {self.taps} taps is outside the kernel's 1..{self.MAX_TAPS}")

    def tensor_specs(self):
        return {"in": TensorSpec((self.proj_width, self.hidden)),
                "conv": TensorSpec((self.channels, self.taps)),
                "conv.b": TensorSpec((self.channels,), "vector", "normal"),
                "dt_bias": TensorSpec((self.heads,), "vector", "normal"),
                "A_log": TensorSpec((self.heads,), "vector", "normal"),
                "D": TensorSpec((self.heads,), "vector", "ones"),
                "norm": TensorSpec((self.inner,), "vector"),
                "o": TensorSpec((self.hidden, self.inner))}

    def state_need(self):
        return StateNeed((self.state_floats + self.conv_floats,), torch.float32)

    def _names(self):
        tag = f"{self.proj_width}_{self.inner}_{self.n_state}"
        return f"mamba_proj_{tag}", f"mamba_conv_{tag}", f"mamba_y_{tag}", f"mamba_g_{tag}", f"mamba_runs_{tag}"

    def _run_columns(self) -> int:
        # scratch for the side-by-side runs: room for two runs' states (and decays) per CHUNK_ROWS rows of a step
        return -(-2 * (self.state_elements + self.heads) // self.CHUNK_ROWS)

    def workspace(self):
        proj, conv, y, g, runs = self._names()
        return {proj: (self.proj_width, "f32"), conv: (self.channels, "f32"), y: (self.inner, "f32"),
                g: (self.inner, "act"), runs: (self._run_columns(), "f32")}

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.w_in = Linear(tensors["in"], rt)
        self.o = Linear(tensors["o"], rt)
        self.conv_w, self.conv_b = tensors["conv"], tensors["conv.b"]
        self.dt_bias, self.a_log, self.d, self.norm = tensors["dt_bias"], tensors["A_log"], tensors["D"], tensors["norm"]

    def _run(self, ctx, h, target, view, accumulate, defer=False):
        n = ctx.n_tokens
        names = self._names()
        proj = ctx.buf(names[0], self.proj_width, torch.float32)
        conv = ctx.buf(names[1], self.channels, torch.float32)
        y = ctx.buf(names[2], self.inner, torch.float32)
        g = ctx.buf(names[3], self.inner)
        ssm_state = view.state[:, :self.state_floats]
        conv_state = view.state[:, self.state_floats:self.state_floats + self.conv_floats]
        self.w_in.store(h, proj, n)
        ops.causal_conv_silu(proj, self.inner, self.conv_w, self.conv_b, self.taps, self.channels, ctx.tok_seq,
                             ctx.seq_start, ctx.seq_slot, conv_state, conv, n, ctx.n_seqs)
        # steps of long prompts in the serving engine: runs of CHUNK_ROWS rows side by side, if the scratch holds
        # them (it does unless one long prompt comes with many short ones); else, and always in the 32-bit engine,
        # row by row
        chunk_rows, max_chunks, scratch = 0, 1, None
        if g.dtype != torch.float32 and ctx.max_new >= 2 * self.CHUNK_ROWS:
            runs = ctx.buf(names[4], self._run_columns(), torch.float32).view(-1)
            most = -(-ctx.max_new // self.CHUNK_ROWS)
            if ctx.n_seqs * most * (self.state_elements + self.heads) <= runs.numel():
                chunk_rows, max_chunks, scratch = self.CHUNK_ROWS, most, runs
        ops.mamba2_scan(conv, proj, self.proj_width - self.heads, self.dt_bias, self.a_log, self.d, ctx.seq_start,
                        ctx.seq_slot, ssm_state, y, ctx.n_seqs, self.heads, self.vdim, self.n_state, self.groups,
                        chunk_rows, max_chunks, scratch, self.wide_state)
        ops.gated_group_rmsnorm(y, proj[:, :self.inner], self.norm, g, n, self.norm_groups, self.eps)
        self._finish(self.o, g, target, n, accumulate, defer)

    def resident_tensors(self):
        return [self.w_in.w, self.o.w, self.conv_w, self.conv_b, self.dt_bias, self.a_log, self.d, self.norm]


@MIXERS.register("rglru")
class RGLRU(_StatefulMixer):
    MAX_TAPS = 16
    RUNS_FROM = 256           # rows in the step's longest sequence from which the side-by-side walk is used

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden, self.width = int(p["hidden_size"]), int(p["width"])
        self.blocks, self.taps = int(p["blocks"]), int(p["conv"])
        self.decay = float(p.get("decay", 8.0))
        if self.width % self.blocks:
            raise ValueError(f"{self.width} channels do not divide into {self.blocks} blocks")
        if not 1 <= self.taps <= self.MAX_TAPS:
            raise ValueError(f"a convolution of {self.taps} taps is outside the kernel's 1..{self.MAX_TAPS}")
        self.block_size = self.width // self.blocks
        self.conv_floats = (self.taps - 1) * self.width

    def tensor_specs(self):
        w, h, b, n = self.width, self.hidden, self.blocks, self.block_size
        vec = lambda: TensorSpec((w,), "vector", "normal")
        return {"y": TensorSpec((w, h)), "y.b": vec(), "x": TensorSpec((w, h)), "x.b": vec(),
                "conv": TensorSpec((w, self.taps)), "conv.b": vec(),
                "ra": TensorSpec((b, n, n)), "ra.b": TensorSpec((b, n), "vector", "normal"),
                "ri": TensorSpec((b, n, n)), "ri.b": TensorSpec((b, n), "vector", "normal"),
                "lam": vec(), "o": TensorSpec((h, w))}

    def fused_tensors(self):
        return {"yx": ("y", "x"), "yx.b": ("y.b", "x.b")}          # one product for the two branches

    def state_need(self):
        return StateNeed((self.width + self.conv_floats,), torch.float32)

    def workspace(self):
        w = self.width
        return {f"lru_p_{w}": (2 * w, "f32"), f"lru_u_{w}": (w, "f32"), f"lru_r_{w}": (w, "f32"),
                f"lru_i_{w}": (w, "f32"), f"lru_s_{w}": (w, "act")}

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        fused, bias = tensors.get("yx"), tensors.get("yx.b")
        if fused is None:
            fused = torch.cat([tensors["y"], tensors["x"]], dim=0).contiguous()
        if bias is None:
            bias = torch.cat([tensors["y.b"], tensors["x.b"]]).contiguous()
        self.yx = Linear(fused, rt, bias=bias)
        self.o = Linear(tensors["o"], rt)
        self.conv_w, self.conv_b = tensors["conv"], tensors["conv.b"]
        self.ra, self.ri = tensors["ra"], tensors["ri"]
        self.ra_b, self.ri_b = tensors["ra.b"].reshape(-1), tensors["ri.b"].reshape(-1)
        self.lam = tensors["lam"]

    def _run(self, ctx, h, target, view, accumulate, defer=False):
        n, w = ctx.n_tokens, self.width
        p = ctx.buf(f"lru_p_{w}", 2 * w, torch.float32)
        u = ctx.buf(f"lru_u_{w}", w, torch.float32)
        r = ctx.buf(f"lru_r_{w}", w, torch.float32)
        i = ctx.buf(f"lru_i_{w}", w, torch.float32)
        s = ctx.buf(f"lru_s_{w}", w)
        lru_state = view.state[:, :w]
        conv_state = view.state[:, w:w + self.conv_floats]
        self.yx.store(h, p, n)                            # [y | x] with their biases, float rows
        ops.causal_conv_silu(p, w, self.conv_w, self.conv_b, self.taps, w, ctx.tok_seq, ctx.seq_start, ctx.seq_slot,
                             conv_state, u, n, ctx.n_seqs, silu=False)
        # the gates' block-diagonal products read the float rows; float sums on the CUDA cores in both engines
        ops.gemm_simt_batched(u, self.ra, r, n)
        ops.gemm_simt_batched(u, self.ri, i, n)
        # long prompts in the serving engine: runs of a sequence side by side; the 32-bit engine keeps the row-by-row
        # order, so that its results do not depend on how a prompt was cut
        runs = ctx.max_new >= self.RUNS_FROM and s.dtype != torch.float32
        ops.rglru_scan(r, i, u, p[:, :w], self.ra_b, self.ri_b, self.lam, self.decay, ctx.seq_start, ctx.seq_slot,
                       lru_state, s, ctx.n_seqs, w, runs)
        self._finish(self.o, s, target, n, accumulate, defer)

    def resident_tensors(self):
        return [self.yx.w, self.yx.bias, self.o.w, self.conv_w, self.conv_b, self.ra, self.ri, self.ra_b, self.ri_b, self.lam]
