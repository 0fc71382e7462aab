"""Latent attention mixer: queries, keys and values go through low-rank latents, and the cache keeps only the
key/value latent and one rotated key part that all heads share.

Per row h_t, with H heads, per head ``dq`` plain and ``dr`` rotated query/key entries, value size ``dv``, latent
sizes ``q_rank`` and ``rk``:
    c_q = norm(W_dq h) * g_q                         q = W_uq c_q        laid out head by head as [dq plain | dr rotated]
    [l | r] = W_dkv h   (rk + dr rows)               c = norm(l) * g_kv        k_rot = rotate(r)   (one for all heads)
    key of head i at position j:    [W_uk,i c_j | k_rot_j]          value: W_uv,i c_j
    s_ij = scale * (q_plain,i . W_uk,i c_j + rotate(q_rot,i) . k_rot_j);   softmax over j <= t with exp(sink_i) once more
    in the denominator;   out = W_o [heads' sums of p_j W_uv,i c_j]
The up-projections of keys and values are never applied to the cache. Instead they move to the query side and
behind the attention ("absorbed"): q_lat,i = W_uk,i^T q_plain,i scores against c_j directly, and
sum_j p_j W_uv,i c_j = W_uv,i (sum_j p_j c_j). Attention then runs with one shared key "head" [c | k_rot] of rk + dr
entries whose first rk entries also serve as the value, for prompts and decoding alike, so a page holds
(rk + dr) numbers a token whatever the head count.

Long prompt portions in bfloat16 take the other way round, which costs a third of the arithmetic there (a head's
key and value are dq + dr and dv wide instead of rk + dr and rk): the cached latents of the portion's sequence, all
positions up to the portion's end (with a window: from the first position that the portion's first row still sees), are
copied out of the pages (``latent_gather``), expanded by two matrix products
into per-head keys [W_uk,i c | k_rot] and values W_uv,i c, and ordinary multi-head attention with the sink runs over
them with the whole queries. Which sequences of a step go which way is decided on the host in ``prepare`` (those
that bring at least ``EXPAND_MIN_ROWS`` rows); both ways compute the same function, up to rounding.

Options: ``q_rank`` None: the queries have no latent, q = W_q h (tensor ``q`` instead of dq, dq.norm, uq; its rows are stacked
on the key/value down-projection's, one product); ``q_rank`` "checkpoint": the query latent's size is that of the stored tensors; ``rot_scaling`` (a scaling rule of the rotary frequencies as ``parts/rotary.py``
takes it; the "yarn" rule also multiplies cosines and sines by its magnitude); ``rot_interleaved`` (pairs (2i, 2i + 1) instead of
(i, i + rot_dims / 2)); ``sink`` False; ``window``.

Tensor names below the part's prefix: dq, dq.norm, uq (or q), dkv, dkv.norm, uk, uv, sink, o.
"""
from __future__ import annotations

import math

import numpy as np
import torch

from ..csrc import ops
from . import flex_plan
from .base import CacheNeed, Mixer, register_mixer
from .linear import linear
from .rotary import rotary_inverse_frequencies


USE_TENSOR_CORES = True      # bf16 only; False sends bf16 through the plain kernel as well
EXPAND_MIN_ROWS = 32         # sequences that bring at least this many rows attend to keys and values expanded per head


class LatentAttention(Mixer):
    capturable = True

    def __init__(self, params, dtype, device, position=None):
        super().__init__(params, dtype, device, position)
        g = params
        self.hidden = int(g["hidden_size"])
        self.H = int(g["num_heads"])
        self.dq = int(g["head_dim"])             # plain (unrotated) part of a query/key head
        self.dr = int(g["rot_dim"])              # rotated part
        self.dv = int(g["value_dim"])
        self.rk = int(g["kv_rank"])
        self.q_latent = bool(g.get("q_rank"))                            # False: queries straight from the input
        self.q_rank = (-1 if g["q_rank"] == "checkpoint" else int(g["q_rank"])) if self.q_latent else None
        self.scale = float(g["scale"])
        self.eps = float(g["eps"])
        self.rot_dims = int(g.get("rot_dims", self.dr))       # how many of the dr entries are rotated
        self.window = g.get("window") or None
        self.has_sink = bool(g.get("sink", True))
        if self.rot_dims % 2 or not 0 <= self.rot_dims <= self.dr:
            raise ValueError(f"latent_attention: rot_dims {self.rot_dims} must be even and at most rot_dim {self.dr}")
        if self.rk + self.dr > 640:
            raise ValueError(f"latent_attention: kv_rank + rot_dim {self.rk + self.dr} above 640 is not supported")
        scaling = g.get("rot_scaling") or None
        self.interleaved = bool(g.get("rot_interleaved", False))
        self.inv_freq = rotary_inverse_frequencies(self.rot_dims, float(g["rot_base"]), scaling).to(device) \
            if self.rot_dims else torch.zeros(0, dtype=torch.float32, device=device)
        # what cosines and sines are multiplied by (the "yarn" rule)
        self.rot_scale = 0.1 * math.log(float(scaling["factor"])) + 1.0 if scaling and scaling.get("rope_type") == "yarn" else 1.0
        self.q_cols = self.q_rank if self.q_latent else self.H * (self.dq + self.dr)  # what the first product holds before [latent | key part]
        self.down = self.uq = self.ukT = self.uv = self.o = None
        self.q_norm = self.kv_norm = self.sink = None

    def weight_shapes(self):
        H = self.H
        shapes = {"dkv": (self.rk + self.dr, self.hidden), "dkv.norm": (self.rk,),
                  "uk": (H * self.dq, self.rk), "uv": (H * self.dv, self.rk),
                  "o": (self.hidden, H * self.dv)}
        if self.q_rank:
            shapes.update({"dq": (self.q_rank, self.hidden), "dq.norm": (self.q_rank,), "uq": (H * (self.dq + self.dr), self.q_rank)})
        else:
            shapes["q"] = (H * (self.dq + self.dr), self.hidden)
        if self.has_sink:
            shapes["sink"] = (H,)
        return shapes

    def keeps_dtype(self, name):
        return name in ("dq.norm", "dkv.norm", "sink")

    def norm_like(self, name):
        return name in ("dq.norm", "dkv.norm")

    def load_weights(self, t):
        H = self.H
        if self.q_latent:
            self.q_rank = self.q_cols = int(t["dq"].shape[0])
        self.down = torch.cat([t["dq"] if self.q_rank else t["q"], t["dkv"]], 0).contiguous()   # one product for both
        self.uq = t["uq"].contiguous() if self.q_rank else None
        # per head the key up-projection transposed, [rk, dq]: q_lat = q_plain @ W_uk,i as a product with rows of W^T
        self.ukT = t["uk"].view(H, self.dq, self.rk).transpose(1, 2).contiguous()
        self.uk = t["uk"].contiguous()                                        # as stored, for the expanded way
        self.uv = t["uv"].view(H, self.dv, self.rk).contiguous()
        self.o = t["o"].contiguous()
        self.q_norm = t["dq.norm"].contiguous() if self.q_rank else None
        self.kv_norm = t["dkv.norm"].float().contiguous()
        self.sink = t["sink"].float().contiguous() if self.has_sink else None

    def cache_need(self):
        return CacheNeed(1, self.rk + self.dr, self.window, 0)

    def streams_first(self, rows):
        return self.down if self.dtype == torch.bfloat16 and rows <= ops.SKINNY_MAX_ROWS else None

    def kernel_files(self, page_size):
        names = ("attention_general", "norm")
        return names + (("gemm_f32",) if self.dtype == torch.float32 else ("attention_flex", "gemm_heads", "gemm_skinny", "gemm_rows", "gemm_tc05"))

    def uses_flex(self) -> bool:
        """Attention on the tensor cores: bfloat16 and sizes in multiples of 8."""
        return USE_TENSOR_CORES and self.dtype == torch.bfloat16 and ops.attn_flex_ok(self.H, 1, self.rk + self.dr, self.rk, False)

    def expands(self) -> bool:
        return (self.uses_flex() and EXPAND_MIN_ROWS > 0
                and ops.attn_flex_ok(self.H, self.H, self.dq + self.dr, self.dv, True))

    def prepare(self, ctx, cache):
        if not self.uses_flex() or cache.k is None:
            return
        key = ("latent_expand", self.H, self.dq, self.dr, self.dv, self.rk, self.window)
        ex = ctx.plans.get(key)
        if ex is None:
            ex = ctx.plans[key] = self._plan_expanded(ctx)
        if not ex["all"]:
            flex_plan.plan(ctx, self.device, self.H, 1, self.rk + self.dr, self.rk, False, self.window, skip=ex["skip"])

    def _plan_expanded(self, ctx) -> dict:
        """Which sequences of the step attend the expanded way, where their gathered rows lie, and their work items."""
        none = {"skip": frozenset(), "all": False, "total": 0}
        if not self.expands() or ctx.seq_cap is not None:
            return none
        qs, cl = ctx.h_q_start, ctx.h_ctx_len
        chosen = [s for s in range(ctx.num_seqs) if int(qs[s + 1] - qs[s]) >= EXPAND_MIN_ROWS]
        if not chosen:
            return none
        per_item = ops.attn_flex_tokens(self.H, self.H)
        seqs, items, total = [], [], 0
        for e, s in enumerate(chosen):
            row0, n, end = int(qs[s]), int(qs[s + 1] - qs[s]), int(cl[s])
            # the first position that any row of the portion sees; positions count from there in the gathered rows
            first = max(0, end - n - self.window + 1) if self.window else 0
            keys = end - first
            seqs.append((s, total, keys, first))
            for b in range(0, n, per_item):
                items.append((e, row0 + b, min(per_item, n - b), keys - n + b))
            total += keys
        items.sort(key=lambda it: -(it[3] + it[2]))
        width = max(k for _, _, k, _ in seqs)
        tag = f"latent_exp_{self.H}_{self.dq}_{self.dr}_{self.dv}_{self.rk}"
        both = ctx.upload_ints(tag, np.concatenate([np.asarray(seqs, dtype=np.int32).reshape(-1),
                                                    np.asarray(items, dtype=np.int32).reshape(-1)]))
        seqs_d, items_d = both[:4 * len(seqs)].view(-1, 4), both[4 * len(seqs):].view(-1, 4)
        # the expanded rows are "pages" of one key: row j of sequence e is page first_row(e) + j
        table = ctx.buf(tag + "_table", (len(seqs), width), torch.int32)
        torch.add(seqs_d[:, 1:2], torch.arange(width, dtype=torch.int32, device=self.device).view(1, -1), out=table)
        return {"skip": frozenset(chosen), "all": len(chosen) == ctx.num_seqs, "total": total, "seqs": seqs_d,
                "items": items_d, "table": table, "width": width}

    def forward(self, x, ctx, cache):
        T = x.shape[0]
        H, dq, dr, dv, rk = self.H, self.dq, self.dr, self.dv, self.rk
        lat = ctx.buf("lat_down", (T, self.q_cols + rk + dr), self.dtype)
        linear(x, self.down, lat, ctx.status)
        if self.q_rank:
            cq = ctx.buf("lat_cq", (T, self.q_rank), self.dtype)
            ops.rmsnorm_rows(lat[:, :self.q_rank], self.q_norm, self.eps, cq)
            q = ctx.buf("lat_q", (T, H * (dq + dr)), self.dtype)
            linear(cq, self.uq, q, ctx.status)
        else:
            q = lat[:, :self.q_cols]
        ex = ctx.plans.get(("latent_expand", H, dq, dr, dv, rk, self.window)) if self.uses_flex() else None
        expanded = ex is not None and ex["total"] > 0
        absorbed = not (expanded and ex["all"])
        # queries against the cached latents: [W_uk,i^T q_plain,i | rotated part] per head
        q_full = ctx.buf("lat_qfull", (T, H * (rk + dr)), self.dtype)
        q_exp = ctx.buf("lat_qexp", (T, H * (dq + dr)), self.dtype) if expanded else None
        if not absorbed:
            pass
        elif ops.gemm_heads_ok(q, self.ukT, q_full, H, dq + dr, rk + dr):          # few rows: all heads in one launch
            ops.gemm_heads(q, self.ukT, q_full, dq + dr, rk + dr)
        else:
            for i in range(H):
                linear(q[:, i * (dq + dr): i * (dq + dr) + dq], self.ukT[i], q_full[:, i * (rk + dr): i * (rk + dr) + rk], ctx.status)
        ops.latent_prepare(lat[:, self.q_cols:], q, q_full, self.kv_norm, self.eps, self.inv_freq, self.rot_dims,
                           ctx.positions, ctx.row_seq, cache.block_table, cache.k if cache.writes else None,
                           cache.page_size, ctx.seq_slots, H, dq, dr, rk, status=ctx.status, q_exp=q_exp,
                           interleaved=self.interleaved, rot_scale=self.rot_scale)
        attn = ctx.buf("attn_out", (T, H * dv), self.dtype)
        if absorbed:
            self._attend_absorbed(q_full, attn, ctx, cache, ex["skip"] if expanded else frozenset())
        if expanded:
            self._attend_expanded(q_exp, attn, ctx, cache, ex)
        out = ctx.buf("delta", (T, self.hidden), self.dtype)
        linear(attn, self.o, out, ctx.status)
        return out

    def _attend_expanded(self, q_exp, attn, ctx, cache, ex):
        """Multi-head attention of the chosen sequences' rows over keys and values expanded from the gathered latents."""
        H, dq, dr, dv, rk = self.H, self.dq, self.dr, self.dv, self.rk
        n = ex["total"]
        dense = ctx.buf("lat_dense", (n, rk + dr), self.dtype)
        ops.latent_gather(cache.k, cache.block_table, ex["seqs"], ex["width"], dense, cache.page_size, ctx.seq_slots,
                          status=ctx.status)
        plain = ctx.buf("lat_kplain", (n, H * dq), self.dtype)
        linear(dense[:, :rk], self.uk, plain, ctx.status)
        values = ctx.buf("lat_values", (n, H * dv), self.dtype)
        linear(dense[:, :rk], self.uv.view(H * dv, rk), values, ctx.status)
        keys = ctx.buf("lat_keys", (n, H * (dq + dr)), self.dtype)
        ops.latent_expand_keys(plain, dense, keys, H, dq, dr, rk)
        ops.attn_flex(q_exp, keys.view(n, H, 1, dq + dr), values.view(n, H, 1, dv), ex["table"], ex["items"], attn, 1,
                      ex["table"].shape[0], H, H, dq + dr, dv, self.scale, self.window or 0, sink=self.sink, status=ctx.status)

    def _attend_absorbed(self, q_full, attn, ctx, cache, skip):
        T = q_full.shape[0]
        H, dr, dv, rk = self.H, self.dr, self.dv, self.rk
        o_lat = ctx.buf("lat_olat", (T, H * rk), self.dtype)
        if self.uses_flex():
            flex_plan.attend(flex_plan.plan(ctx, self.device, H, 1, rk + dr, rk, False, self.window, skip=skip), q_full, cache.k, None,
                             cache.block_table, o_lat, cache.page_size, ctx.seq_slots, H, 1, rk + dr, rk, self.scale,
                             self.window, sink=self.sink, status=ctx.status)
        else:
            ops.attention_general(q_full, cache.k, None, cache.block_table, ctx.row_seq, ctx.positions, o_lat, cache.page_size,
                                  ctx.seq_slots, H, 1, rk + dr, rk, self.scale, self.window or 0, sink=self.sink,
                                  status=ctx.status)
        if ops.gemm_heads_ok(o_lat, self.uv, attn, H, rk, dv):
            ops.gemm_heads(o_lat, self.uv, attn, rk, dv)
        else:
            for i in range(H):
                linear(o_lat[:, i * rk:(i + 1) * rk], self.uv[i], attn[:, i * dv:(i + 1) * dv], ctx.status)


register_mixer("latent_attention", LatentAttention)
