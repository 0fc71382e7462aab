"""Attention whose softmax weights are mixed over the heads ("talking heads" behind the softmax), with a norm over the
whole query and key projections, rotation of part of each head, a sink in the softmax and an output gate.

Per row x, with H heads, G key/value heads (head h reads key/value head h // (H / G)), key size dk, value size dv:
    q = W_q x [H * dk],  k = W_k x [G * dk],  v = W_v x [G, dv]
    q <- q_norm * q * rsqrt(mean(q^2) + eps) over all H * dk entries at once; k likewise over its G * dk   (weights of that size)
    the first ``rot_dim`` entries of every head of q and k rotated by position (entry i with entry i + rot_dim / 2; cosines and
    sines times the position encoding's ``magnitude``)
    w_h(i, j) = exp(scale q_h(i) . k(j)) / (sum_{j' <= i} exp(scale q_h(i) . k(j')) + exp(sink_h))           causal
    w'_h = sum_g talk[h, g] w_g;    o_h(i) = sum_j w'_h(i, j) v_{kv(h)}(j)
    out = W_o (concat_h o_h * sigmoid(W_g x))
Mixing the weights and then applying them to head h's values equals mixing what each head's weights give on those
values: o_h = sum_g talk[h, g] a[g, kv(h)] with a[g, c] = sum_j w_g(i, j) v_c(j). So the cache keeps the G value heads of
a token side by side as one value head of G * dv entries, the framework's general attention kernels run every query head
over it (``v_share`` = G: all key heads read the one value head; results in fp32), and ``ops.talk_combine`` forms the
sums over g, the gate and the caller's scale in one launch. Scores, softmax, the sink, the mix and the gate are fp32 in
both precisions.

Tensor names below the part's prefix: q, k, v, g, o, q.norm, k.norm, talk, sink. ``talk`` False: no mixing (the identity);
``gate`` False: no output gate.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import CacheNeed, Mixer, register_mixer
from . import flex_plan
from .linear import linear

USE_TENSOR_CORES = True      # bf16 only; False sends bf16 through the plain kernel as well
MAX_VALUE_WIDTH = 1024       # what the general attention kernels take as one value head


class TalkingAttention(Mixer):
    capturable = True

    def __init__(self, params, dtype, device, position=None):
        super().__init__(params, dtype, device, position)
        p = params
        self.hidden = int(p["hidden_size"])
        self.H = int(p["num_heads"])
        self.G = int(p["num_kv_heads"])
        self.dk = int(p["head_dim"])
        self.dv = int(p.get("value_dim") or self.dk)
        self.scale = float(p["scale"])
        self.eps = float(p["eps"])
        self.window = p.get("window") or None
        self.talk = bool(p.get("talk", True))
        self.gate = bool(p.get("gate", True))
        self.has_sink = bool(p.get("sink", True))
        if self.H % self.G:
            raise ValueError(f"talking_attention: {self.H} heads are not a multiple of {self.G} kv heads")
        self.wide = self.G * self.dv                            # a token's values, all key/value heads side by side
        if self.dk > 640 or self.wide > MAX_VALUE_WIDTH:
            raise ValueError(f"talking_attention: key size {self.dk} or kv_heads * value size {self.wide} above {MAX_VALUE_WIDTH} "
                             "is not supported")
        rot = position.rotary() if position is not None else None
        if position is not None and rot is None:
            raise ValueError("talking_attention: the position encoding must give rotary frequencies")
        self.inv_freq, self.rot_dims = rot if rot is not None else (None, 0)
        self.rot_scale = float(getattr(position, "magnitude", 1.0)) if position is not None else 1.0
        self.nq, self.nk = self.H * self.dk, self.G * self.dk
        self.gate_off = self.nq + self.nk + self.wide
        self.head_width = self.H * self.dv
        self.proj_rows = -(-(self.gate_off + (self.head_width if self.gate else 0)) // 8) * 8
        self.w_in = self.output_weight = self.q_norm = self.k_norm = self.talk_w = self.sink = None

    def weight_shapes(self):
        s = {"q": (self.nq, self.hidden), "k": (self.nk, self.hidden), "v": (self.wide, self.hidden),
             "o": (self.hidden, self.head_width), "q.norm": (self.nq,), "k.norm": (self.nk,)}
        if self.gate:
            s["g"] = (self.head_width, self.hidden)
        if self.talk:
            s["talk"] = (self.H, self.H)
        if self.has_sink:
            s["sink"] = (self.H,)
        return s

    def keeps_dtype(self, name):
        return name in ("q.norm", "k.norm", "talk", "sink")

    def norm_like(self, name):
        return name in ("q.norm", "k.norm")

    def load_weights(self, t):
        parts = [t["q"], t["k"], t["v"]] + ([t["g"]] if self.gate else [])
        rows = sum(p.shape[0] for p in parts)
        if rows < self.proj_rows:
            parts.append(torch.zeros(self.proj_rows - rows, self.hidden, dtype=parts[0].dtype, device=parts[0].device))
        self.w_in = torch.cat(parts, 0).contiguous()
        self.output_weight = t["o"].contiguous()
        self.q_norm = t["q.norm"].float().contiguous()
        self.k_norm = t["k.norm"].float().contiguous()
        self.talk_w = (t["talk"].float() if self.talk else torch.eye(self.H, dtype=torch.float32, device=self.w_in.device)).contiguous()
        self.sink = t["sink"].float().contiguous() if self.has_sink else None

    def cache_need(self):
        # G key heads of dk; one value head that holds the G value heads of a token side by side
        return CacheNeed(self.G, self.dk, self.window, self.wide, 1)

    def streams_first(self, rows):
        return self.w_in if self.dtype == torch.bfloat16 and rows <= ops.SKINNY_MAX_ROWS else None

    def kernel_files(self, page_size):
        if self.dtype == torch.float32:
            return ("qk_prepare", "attention_general", "gemm_f32")
        return ("qk_prepare", "attention_flex" if self.uses_flex() else "attention_general", "gemm_skinny", "gemm_rows", "gemm_tc05")

    def uses_flex(self) -> bool:
        """On the tensor cores: bfloat16 and sizes in multiples of 8."""
        return (self.dtype == torch.bfloat16 and USE_TENSOR_CORES
                and ops.attn_flex_ok(self.H, self.G, self.dk, self.wide, True))

    def prepare(self, ctx, cache):
        if self.uses_flex() and cache.k is not None:
            flex_plan.plan(ctx, self.device, self.H, self.G, self.dk, self.wide, True, self.window)

    def forward_heads(self, x, ctx, cache, out, scale: float = 1.0):
        """The gated heads, times ``scale``, into ``out`` [T, H * dv] (a view with a row stride): everything but W_o."""
        T = x.shape[0]
        H, G, dk = self.H, self.G, self.dk
        u = ctx.buf("tattn_proj", (T, self.proj_rows), self.dtype)
        linear(x, self.w_in, u, ctx.status)
        writes = cache.writes
        ops.qk_prepare(u, self.q_norm, self.k_norm, self.eps, self.inv_freq, self.rot_dims, False, ctx.positions, ctx.row_seq,
                       cache.block_table, cache.k if writes else None, cache.v if writes else None, cache.page_size,
                       ctx.seq_slots, H, G, 1, dk, self.wide, status=ctx.status, whole=True, rot_scale=self.rot_scale)
        a = ctx.buf("tattn_all", (T, H * self.wide), torch.float32)
        q = u[:, :self.nq]
        if self.uses_flex():
            flex_plan.attend(flex_plan.plan(ctx, self.device, H, G, dk, self.wide, True, self.window), q, cache.k, cache.v,
                             cache.block_table, a, cache.page_size, ctx.seq_slots, H, G, dk, self.wide, self.scale, self.window,
                             sink=self.sink, status=ctx.status, v_share=G)
        else:
            ops.attention_general(q, cache.k, cache.v, cache.block_table, ctx.row_seq, ctx.positions, a, cache.page_size,
                                  ctx.seq_slots, H, G, dk, self.wide, self.scale, self.window or 0, sink=self.sink,
                                  status=ctx.status, v_share=G)
        gate = u[:, self.gate_off:self.gate_off + self.head_width] if self.gate else None
        ops.talk_combine(a, self.talk_w, gate, out, H, G, self.dv, scale)

    def forward(self, x, ctx, cache):
        T = x.shape[0]
        heads = ctx.buf("attn_out", (T, self.head_width), self.dtype)
        self.forward_heads(x, ctx, cache, heads)
        out = ctx.buf("delta", (T, self.hidden), self.dtype)
        linear(heads, self.output_weight, out, ctx.status)
        return out


register_mixer("talking_attention", TalkingAttention)
