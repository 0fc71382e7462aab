"""Time mixing with a decaying matrix state (the recurrence of RWKV-style mixers).

Per row x, with x' the row before it in the same sequence (zeros for the first), H heads of size n, C = H * n:
    every product s in (r, k, v, g, w) reads its own mix  x + (x' - x) * mu_s
    r, k, v = W_r, W_k, W_v of their mixes [H, n];   gate = silu(W_g mix_g)
    decay = exp(-exp(W_w2 tanh(W_w1 mix_w) + w0))                      per head and key channel, in (0, 1)
    o_t = (S + diag(u) k_t v_t^T)^T r_t;   S <- diag(decay_t) S + k_t v_t^T      per head; S is n x n, fp32, zero at the start
    o <- o * rsqrt(mean(o^2) + eps) per head, times ``norm`` [C], times gate;   out = W_o o
A request's state is one fp32 vector per slot: ``[S, head by head in the scan kernel's layout | the last row x]``; kernels
start a portion from it and leave the next portion's behind, so prompts can be cut anywhere and decoding is the same path
with one row. The decay with its logarithm and exponentials, the state, the read-out, its norm and the gate are fp32 in
both precisions; r, k, v enter the recurrence as fp32 copies of the products' results.

Tensor names below the part's prefix: mu.r, mu.k, mu.v, mu.g, mu.w, r, k, v, g, w1, w2, w0, u, norm, o.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Mixer, StateNeed, register_mixer
from .linear import linear, linear_batched

MIXES = ("r", "k", "v", "g", "w")


class TimeMix(Mixer):
    capturable = True

    def __init__(self, params, dtype, device, position=None):
        super().__init__(params, dtype, device, position)
        p = params
        self.hidden = int(p["hidden_size"])
        self.H = int(p["num_heads"])
        self.n = int(p["head_dim"])
        self.eps = float(p["eps"])
        self.rank = p.get("decay_rank")                       # None: the checkpoint's w1 says
        if self.n > 512:
            raise ValueError("time_mix: head sizes above 512 are not supported")
        self.C = self.H * self.n
        self.head_width = self.C
        self.prev_off = self.H * ops.decay_state_floats(self.n)       # the scan's part of the slot, then the last row
        self.mu = self.w = self.w1 = self.w2t = self.w0 = self.u = self.norm_w = self.output_weight = None

    def weight_shapes(self):
        d, C, L = self.hidden, self.C, -1 if self.rank is None else int(self.rank)
        s = {f"mu.{m}": (d,) for m in MIXES}
        s.update({"r": (C, d), "k": (C, d), "v": (C, d), "g": (C, d), "w1": (L, d), "w2": (C, L), "w0": (C,),
                  "u": (self.H, self.n), "norm": (C,), "o": (d, C)})
        return s

    def keeps_dtype(self, name):
        return name.startswith("mu.") or name in ("w0", "u", "norm")

    def norm_like(self, name):
        return name == "norm"

    def load_weights(self, t):
        f32 = lambda n: t[n].float().contiguous()
        self.mu = torch.stack([t[f"mu.{m}"].float() for m in MIXES]).contiguous()
        self.w = torch.stack([t[m] for m in ("r", "k", "v", "g")]).contiguous()      # [4, C, d]: one launch for decode rows
        L = t["w1"].shape[0]
        if t["w2"].shape[1] != L:
            raise ValueError(f"time_mix: w1 has {L} rows but w2 {t['w2'].shape[1]} columns")
        self.L = L
        self.L_pad = -(-L // 8) * 8                            # rows of 16-byte multiples for the products
        w1 = t["w1"]
        if self.L_pad > L:
            w1 = torch.cat([w1, torch.zeros(self.L_pad - L, self.hidden, dtype=w1.dtype, device=w1.device)], 0)
        self.w1 = w1.contiguous()
        self.w2t = t["w2"].float().t().contiguous()            # [L, C], fp32: the decay is 32-bit arithmetic throughout
        self.w0, self.u, self.norm_w = f32("w0"), f32("u"), f32("norm")
        self.output_weight = t["o"].contiguous()

    def state_need(self):
        return StateNeed((self.prev_off + self.hidden,), torch.float32)

    def streams_first(self, rows):
        return None

    def kernel_files(self, page_size):
        return ("time_mix", "delta_rule") + (("gemm_f32",) if self.dtype == torch.float32 else ("gemm_skinny", "gemm_rows", "gemm_tc05"))

    def forward_heads(self, x, ctx, cache, out, scale: float = 1.0):
        """The normalised, gated read-out, times ``scale``, into ``out`` [T, C] (a view with a row stride): everything but W_o."""
        T = x.shape[0]
        C, H, n = self.C, self.H, self.n
        state = cache.state
        mixes = ctx.buf("tmix_in", (len(MIXES), T, self.hidden), self.dtype)
        ops.shift_mix(x, self.mu, mixes, state, self.prev_off, ctx.positions, ctx.row_seq, ctx.q_start, ctx.slots,
                      ctx.seq_slots, status=ctx.status)
        proj = ctx.buf("tmix_proj", (4, T, C), self.dtype)
        linear_batched(mixes[:4], self.w, proj, ctx.status)
        z = ctx.buf("tmix_low", (T, self.L_pad), self.dtype)
        linear(mixes[4], self.w1, z, ctx.status)
        xs = ctx.buf("tmix_xs", (T, 4 * C), torch.float32)
        ops.time_mix_prepare(proj[0], proj[1], proj[2], z[:, :self.L], self.w2t, self.w0, xs)
        y = ctx.buf("tmix_y", (T, C), torch.float32)
        ops.decay_scan(xs, self.u, state, y, ctx.q_start, ctx.ctx_len, ctx.slots, ctx.seq_slots, H, n)
        ops.head_norm_gate(y, proj[3], self.norm_w, out, H, n, self.eps, post=scale)

    def forward(self, x, ctx, cache):
        T = x.shape[0]
        heads = ctx.buf("tmix_heads", (T, self.C), self.dtype)
        self.forward_heads(x, ctx, cache, heads)
        out = ctx.buf("delta", (T, self.hidden), self.dtype)
        linear(heads, self.output_weight, out, ctx.status)
        return out


register_mixer("time_mix", TimeMix)
