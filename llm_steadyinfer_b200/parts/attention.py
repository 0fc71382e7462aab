"""Attention mixer: grouped-query causal attention over the paged cache, optional window, optional learned bias by
distance, a value size that may differ from the key size.

Per row: q, k, v from one stacked projection [ (H + 2 KV) * hs, d ] (the reference stacks
them too, src/source/model/llama3.cpp:434-498, but then reads the output with the wrong row
stride, llama3.cpp:1009-1019; every consumer here takes the row stride); rotation of q and k
and the store of k, v into the sequence's pages; softmax(scale * q . K) V over cache
positions up to the row's own (llama3.cpp:1048-1067); output projection (llama3.cpp:1136-1140).

Options beyond the reference's block, all parameters of the part:
``value_dim``      size of a value head (default ``head_dim``); the cache then keeps values of that size.
``distance_bias``  ``{"max_distance": D, "buckets": B or None, "name": tensor}``: a learned table [B, heads] whose row
                   ``bucket(i - j)`` is added to the scaled score of query i and key j. Distances below B/2 have a
                   row each; the other B - B/2 rows share the distances from B/2 to D on a logarithmic scale:
                   ``bucket(n) = min(B - 1, B/2 + floor(log(n / (B/2)) / log(D / (B/2)) * (B - B/2)))``. B None: the
                   checkpoint's tensor says how many rows there are. At load the table is spread out by distance
                   (one row for every n up to D), which is what the kernels index.
``names``          checkpoint names of the four matrices, ``{"q": .., "k": .., "v": .., "o": ..}``.
``values_are_keys`` the layer has no value projection: head g's value at a position is its key there, so the cache keeps keys
                   alone and the kernels read the values out of the key pages (a ``value_dim`` below ``head_dim``: the key's first entries).
``distance_slopes`` ``{"base": b, "exponent": e}``: ``slope_h * (i - j)`` with ``slope_h = b^(e (h + 1) / heads)`` is taken off
                   the scaled score of query i and key j (a penalty in proportion to the distance, steeper for the first heads).
``query_temperature`` ``{"coef": c, "every": n}``: the query at position p is multiplied by ``1 + c ln(floor((p + 1) / n) + 1)``
                   (applied by the attention kernels to the row's scale, in fp32).
``output_gate``    name of a matrix [heads * value_dim, hidden]: the heads' results are multiplied entry by entry with
                   ``sigmoid(W_g x)`` before the output projection; its rows are stacked behind q, k, v in one product, and the
                   attention kernels apply the gate when they store their results.
With any option but ``names`` the mixer runs the general attention kernels (``attention_general.cu`` in 32-bit,
``attention_flex.cu`` on the tensor cores in bfloat16) instead of the rotary ones. Sequences that bring a full work item of
rows to a bfloat16 step go to the tcgen05 prompt kernel (``attention_tc05.cu``) where its layout fits (key size 64 or 128,
values of the same size or the keys themselves, no bias table): it takes slopes, temperature and gate as well.
"""
from __future__ import annotations

import math

import numpy as np
import torch

from ..csrc import ops
from .base import CacheNeed, Mixer, register_mixer
from . import flex_plan
from . import linear as linear_mod
from .linear import linear


USE_TENSOR_CORES = True      # bf16 only; False sends bf16 through the plain kernel as well
USE_TMA = True               # decode tiles by TMA where the layout allows
USE_TC05 = True              # prompt portions on tcgen05 where the layout allows
FUSE_ROPE = True             # few rows (decode): rotation and cache store in the epilogue of the q/k/v product
DECODE_BLOCKS_PER_SM = 2     # decode attention blocks that one multiprocessor holds at once
MAX_SPLITS = 32
MIN_TILES_PER_SPLIT = 2      # a split covers at least this many 64-key tiles


class Attention(Mixer):
    adds_into_residual = True

    def __init__(self, params, dtype, device, position=None):
        super().__init__(params, dtype, device, position)
        self.hidden = int(params["hidden_size"])
        self.H = int(params["num_heads"])
        self.KV = int(params["num_kv_heads"])
        self.hs = int(params["head_dim"])
        self.scale = float(params["scale"])
        self.window = params.get("window") or None
        if self.H % self.KV:
            raise ValueError(f"attention: {self.H} heads are not a multiple of {self.KV} kv heads")
        if self.hs > 256:
            raise ValueError(f"attention: head_dim {self.hs} above 256 is not supported")
        self.vs = int(params.get("value_dim") or self.hs)
        self.names = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight"}
        self.names.update(params.get("names") or {})
        self.bias_spec = params.get("distance_bias") or None
        if self.bias_spec is not None:
            self.bias_name = self.bias_spec.get("name", "distance_bias")
            self.bias_rows = self.bias_spec.get("buckets")
            self.bias_max = float(self.bias_spec["max_distance"])
        self.own_v = not bool(params.get("values_are_keys", False))
        if not self.own_v and self.vs > self.hs:
            raise ValueError(f"attention: values that are the keys have at most the keys' size {self.hs}, found value_dim {self.vs}")
        sl = params.get("distance_slopes") or None
        self.slopes = None               # fp32 [H] on the device
        if sl is not None:
            base, expo = float(sl["base"]), float(sl["exponent"])
            self.slopes = torch.tensor([base ** (expo * (h + 1) / self.H) for h in range(self.H)], dtype=torch.float64) \
                .to(torch.float32).to(device)
        qt = params.get("query_temperature") or None
        self.q_temp = None if qt is None else (float(qt["coef"]), qt["every"])
        self.gate_name = params.get("output_gate") or None
        self.general = (self.bias_spec is not None or self.vs != self.hs or not self.own_v or self.slopes is not None
                        or self.q_temp is not None or self.gate_name is not None)
        if self.general and position is not None:
            raise ValueError("attention: the general form (a distance bias, slopes, a value size of its own, values that are "
                             "the keys, a query temperature, an output gate) goes without a position encoding")
        # columns of the stacked projection: q, k, v (if the layer has values of its own), the gate (if it has one)
        self.kv_cols = self.KV * (self.hs + (self.vs if self.own_v else 0))
        self.gate_off = self.H * self.hs + self.kv_cols
        self.proj_cols = -(-(self.gate_off + (self.H * self.vs if self.gate_name else 0)) // 8) * 8 if self.general else 0
        self.dist_bias = None            # fp32 [distances, H], made at load
        self.qkv = None
        self.o = None

    def weight_shapes(self):
        n = self.names
        shapes = {n["q"]: (self.H * self.hs, self.hidden),
                  n["k"]: (self.KV * self.hs, self.hidden),
                  n["o"]: (self.hidden, self.H * self.vs)}
        if self.own_v:
            shapes[n["v"]] = (self.KV * self.vs, self.hidden)
        if self.gate_name:
            shapes[self.gate_name] = (self.H * self.vs, self.hidden)
        if self.bias_spec is not None:
            shapes[self.bias_name] = (self.bias_rows if self.bias_rows else -1, self.H)   # -1: as the checkpoint has it
        return shapes

    def keeps_dtype(self, name):
        return self.bias_spec is not None and name == self.bias_name

    def norm_like(self, name):
        return False

    def load_weights(self, tensors):
        n = self.names
        parts = [tensors[n["q"]], tensors[n["k"]]] + ([tensors[n["v"]]] if self.own_v else []) \
            + ([tensors[self.gate_name]] if self.gate_name else [])
        rows = sum(p.shape[0] for p in parts)
        if self.general and rows < self.proj_cols:           # rows of the product's result stay 16-byte aligned
            parts.append(torch.zeros(self.proj_cols - rows, self.hidden, dtype=parts[0].dtype, device=parts[0].device))
        self.qkv = torch.cat(parts, 0).contiguous()
        self.o = tensors[n["o"]].contiguous()
        if self.bias_spec is not None:
            self.dist_bias = spread_by_distance(tensors[self.bias_name].float(), self.bias_max)

    def cache_need(self):
        if not self.own_v:
            return CacheNeed(self.KV, self.hs, self.window, 0)
        return CacheNeed(self.KV, self.hs, self.window, None if self.vs == self.hs else self.vs)

    @property
    def capturable(self):
        """The step's work lists are made in ``prepare``; a position encoding applied through its
        unfused hook decides for itself."""
        return self.position is None or self.position.capturable

    def streams_first(self, rows):
        # few rows in bfloat16 go to the weight-streaming product, which reads every weight once
        return self.qkv if self.dtype == torch.bfloat16 and rows <= ops.SKINNY_MAX_ROWS else None

    def kernel_files(self, page_size):
        if self.general:
            return ("attention_general",) + (("attention_tc05", "attention_tma") if self.dtype == torch.bfloat16 and self.general_tc05_ok(page_size) else ()) + (
                ("gemm_f32",) if self.dtype == torch.float32 else ("attention_flex", "gemm_skinny", "gemm_rows", "gemm_tc05"))
        names = ["rope_kv"] + (["gemm_f32"] if self.dtype == torch.float32 else ["gemm_skinny", "gemm_rows", "gemm_tc05"])
        if not self.uses_tensor_cores():
            return tuple(names + ["attention_ref"])
        names.append("attention_mma")
        if self.hs in (64, 128) and page_size in (8, 16, 32, 64):        # the layouts the TMA-fed kernels take
            names += ["attention_tma"] * bool(USE_TMA) + ["attention_tc05"] * bool(USE_TC05)
        return tuple(names)

    def forward(self, x, ctx, cache, resid=None):
        if self.general:
            return self.forward_general(x, ctx, cache)
        T = x.shape[0]
        H, KV, hs = self.H, self.KV, self.hs
        qkv = ctx.buf("attn_qkv", (T, (H + 2 * KV) * hs), self.dtype)
        rot = self.position.rotary() if self.position is not None else None
        if (FUSE_ROPE and linear_mod.USE_SKINNY and rot is not None and rot[1] == hs and hs % 16 == 0
                and self.dtype == torch.bfloat16 and ops.gemm_skinny_ok(x, self.qkv, qkv)):
            # a decode step: one kernel for the projection, the rotation and the store into the pages
            ops.gemm_skinny_qkv_rope(x, self.qkv, qkv, ctx.positions, ctx.row_seq, rot[0], cache.block_table,
                                     cache.k if cache.writes else None, cache.v if cache.writes else None,
                                     cache.page_size, ctx.seq_slots, H, KV, hs, status=ctx.status)
            attn = ctx.buf("attn_out", (T, H * hs), self.dtype)
            self.attend(qkv[:, :H * hs], cache, ctx, attn)
            out = ctx.buf("delta", (T, self.hidden), self.dtype)
            linear(attn, self.o, out, ctx.status)
            return out
        linear(x, self.qkv, qkv, ctx.status)
        if self.position is not None and rot is None:
            q3 = qkv[:, :H * hs].view(T, H, hs)
            k3 = qkv[:, H * hs:(H + KV) * hs].view(T, KV, hs)
            self.position.apply(q3, k3, ctx)
        inv_freq, rot_dim = rot if rot is not None else (None, 0)
        ops.rope_kv_write(qkv, ctx.positions, ctx.row_seq, inv_freq, rot_dim, cache.block_table,
                          cache.k if cache.writes else None, cache.v if cache.writes else None,
                          cache.page_size, ctx.seq_slots, H, KV, hs, status=ctx.status)
        attn = ctx.buf("attn_out", (T, H * hs), self.dtype)
        self.attend(qkv[:, :H * hs], cache, ctx, attn)
        if resid is not None and linear_mod.linear_into_residual(attn, self.o, resid, ctx.status):
            return None                                   # the output projection added itself into the stream
        out = ctx.buf("delta", (T, self.hidden), self.dtype)
        linear(attn, self.o, out, ctx.status)
        return out

    def general_tc05_ok(self, page_size: int) -> bool:
        """The general form's long portions on the tcgen05 prompt kernel: its layouts, and nothing it does not know."""
        return (USE_TC05 and self.bias_spec is None and self.vs == self.hs and (self.q_temp is None or self.q_temp[0] >= 0)
                and ops.attn_portion_tc05_ok(self.H, self.KV, self.hs, page_size))

    def _plan_general_tc05(self, ctx, page_size: int) -> dict:
        """Which sequences of the step go to the tcgen05 prompt kernel (those that bring at least one full item of rows),
        and their work items; the others are the general tensor-core kernel's."""
        key = ("attention_general_tc05", self.H, self.KV, self.hs, self.window)
        got = ctx.plans.get(key)
        if got is not None:
            return got
        out = {"skip": frozenset(), "all": False, "items": None}
        if ctx.seq_cap is None and self.general_tc05_ok(page_size):
            per = ops.attn_portion_tc05_tokens(self.H, self.KV)
            qs, cl = ctx.h_q_start, ctx.h_ctx_len
            chosen, items = [], []
            for s in range(ctx.num_seqs):
                row0, n = int(qs[s]), int(qs[s + 1] - qs[s])
                if n < per:
                    continue
                chosen.append(s)
                pos0 = int(cl[s]) - n
                items += [(s, row0 + b, min(per, n - b), pos0 + b) for b in range(0, n, per)]
            if chosen:
                out = {"skip": frozenset(chosen), "all": len(chosen) == ctx.num_seqs,
                       "items": ctx.upload_ints(f"attn_gen_tc05_{self.H}_{self.KV}_{self.hs}_{self.window}",
                                                np.asarray(items, dtype=np.int32)).view(-1, 4)}
        ctx.plans[key] = out
        return out

    def forward_general(self, x, ctx, cache):
        """No rotation; keys (and values of their own size, where the layer has them) into the pages as they are; scores with
        the bias, the slopes and the query temperature; the gate on the heads' results."""
        T = x.shape[0]
        H, KV, hs, vs = self.H, self.KV, self.hs, self.vs
        qkv = ctx.buf("attn_qkv", (T, self.proj_cols), self.dtype)
        linear(x, self.qkv, qkv, ctx.status)
        v_cache = cache.v if self.own_v else None
        if cache.writes:
            ops.kv_store(qkv, ctx.positions, ctx.row_seq, cache.block_table, cache.k, v_cache, cache.page_size,
                         ctx.seq_slots, H, KV, hs, vs if self.own_v else 0, status=ctx.status)
        attn = ctx.buf("attn_out", (T, H * vs), self.dtype)
        gate = qkv[:, self.gate_off:self.gate_off + H * vs] if self.gate_name else None      # applied in the attention's epilogue
        if self.uses_flex():
            big = self._plan_general_tc05(ctx, cache.page_size)
            if not big["all"]:
                flex_plan.attend(flex_plan.plan(ctx, self.device, H, KV, hs, vs, self.own_v, self.window, skip=big["skip"]),
                                 qkv[:, :H * hs], cache.k, v_cache, cache.block_table, attn, cache.page_size, ctx.seq_slots, H, KV,
                                 hs, vs, self.scale, self.window, dist_bias=self.dist_bias, status=ctx.status, slopes=self.slopes,
                                 q_temp=self.q_temp, gate=gate)
            if big["items"] is not None:
                ops.attn_portion_tc05(qkv[:, :H * hs], cache.k, v_cache, cache.block_table, big["items"], attn, cache.page_size,
                                      ctx.seq_slots, H, KV, hs, self.scale, self.window or 0, status=ctx.status,
                                      slopes=self.slopes, q_temp=self.q_temp, gate=gate)
        else:
            ops.attention_general(qkv[:, :H * hs], cache.k, v_cache, cache.block_table, ctx.row_seq, ctx.positions, attn,
                                  cache.page_size, ctx.seq_slots, H, KV, hs, vs, self.scale, self.window or 0,
                                  dist_bias=self.dist_bias, status=ctx.status, slopes=self.slopes, q_temp=self.q_temp, gate=gate)
        out = ctx.buf("delta", (T, self.hidden), self.dtype)
        linear(attn, self.o, out, ctx.status)
        return out

    # ---- kernels ---------------------------------------------------------------------
    def target_blocks(self) -> int:
        """Decode attention blocks that run at once on this part's device."""
        return DECODE_BLOCKS_PER_SM * ops.sm_count(self.device)

    def uses_flex(self) -> bool:
        """The general form on the tensor cores: bfloat16 and sizes in multiples of 8."""
        return (self.general and self.dtype == torch.bfloat16 and USE_TENSOR_CORES
                and ops.attn_flex_ok(self.H, self.KV, self.hs, self.vs, self.own_v))

    def uses_tensor_cores(self) -> bool:
        return not self.general and self.dtype == torch.bfloat16 and USE_TENSOR_CORES and self.hs % 16 == 0

    def prepare(self, ctx, cache):
        """Cut the step's sequences into work items for the tensor-core kernels: runs of few
        tokens (decode rows) for the decode kernel, longer portions in runs of the portion
        kernel's item size. One plan serves every layer with the same head layout and window."""
        if self.general:
            if self.uses_flex() and cache.k is not None:
                big = self._plan_general_tc05(ctx, cache.page_size)
                if not big["all"]:
                    flex_plan.plan(ctx, self.device, self.H, self.KV, self.hs, self.vs, self.own_v, self.window, skip=big["skip"])
            return
        if not self.uses_tensor_cores():
            return
        key = ("attention", self.H, self.KV, self.hs, self.window)
        if key in ctx.plans or cache.k is None:
            return
        G = self.H // self.KV
        tma = USE_TMA and ops.attn_decode_tma_ok(self.H, self.KV, self.hs, cache.page_size)
        dec_rows = ops.attn_decode_tma_rows(self.H, self.KV) if tma else ops.attn_decode_rows(self.H, self.KV, self.hs)
        dec_tokens = dec_rows // G
        tc05 = USE_TC05 and ops.attn_portion_tc05_ok(self.H, self.KV, self.hs, cache.page_size)
        por_tokens = (ops.attn_portion_tc05_tokens(self.H, self.KV) if tc05
                      else ops.attn_portion_tokens(self.H, self.KV, self.hs))
        if por_tokens <= 0:
            raise ops.KernelError(f"attention: {G} query heads per kv head do not fit the tensor-core kernels")
        dec, por = [], []
        S = ctx.num_seqs
        qs, cl = ctx.h_q_start, ctx.h_ctx_len
        for s in range(S):
            row0, n = int(qs[s]), int(qs[s + 1] - qs[s])
            pos0 = int(cl[s]) - n
            if n <= dec_tokens:
                dec.append((s, row0, n, pos0))
            else:
                for b in range(0, n, por_tokens):
                    por.append((s, row0 + b, min(por_tokens, n - b), pos0 + b))
        plan = {"dec": None, "por": None, "nsplit": 1, "scratch": None, "tma": tma, "work": None,
                "dec_rows": max((d[2] for d in dec), default=0) * G,
                "tc05": tc05}
        n_dec = len(dec)
        if ctx.seq_cap is not None:                   # fixed shapes: pad with empty items
            dec += [(0, 0, 0, 0)] * (ctx.seq_cap - n_dec)
        if dec and tma:
            # Shares of about equal length for as many blocks as run at once (two per SM), so that a long
            # sequence beside short ones is cut into more of them; a second wave of blocks would wait.
            tiles = []
            for (_, _, n, pos0) in dec:
                first = max(0, pos0 - self.window + 1) // 64 * 64 if self.window else 0
                tiles.append(-(-(pos0 + n - first) // 64) if n > 0 else 0)
            # Entries: every item whole, the shares that run at once, and room for finer cuts when items outnumber
            # those (entries without work are blocks that start and leave, so not more room than pays)
            budget = max(1, self.target_blocks() // self.KV)
            entries = budget + len(dec) + min(3 * len(dec), 2 * budget)
            work = ops.split_work(tiles, budget, entries, MAX_SPLITS, MIN_TILES_PER_SPLIT)
            if ctx.seq_cap is None:                    # shapes are free: only the entries with work
                work = work[:max(1, int((work[:, 0] >= 0).sum()))]
            both = ctx.upload_ints(f"attn_dec_{self.H}_{self.KV}_{self.hs}_{self.window}",
                                   np.concatenate([np.asarray(dec, dtype=np.int32).reshape(-1), work.reshape(-1)]))
            plan["dec"] = both[:4 * len(dec)].view(-1, 4)
            plan["work"] = both[4 * len(dec):].view(-1, 4)
            plan["scratch"] = ctx.buf("attn_split", (ops.attn_decode_tma_work_floats(entries, self.H, self.KV, self.hs),),
                                      torch.float32)
        elif dec:
            # as many blocks as run at once (two per SM), not more: a second wave would wait
            nsplit = max(1, min(MAX_SPLITS, self.target_blocks() // (len(dec) * self.KV)))
            if ctx.seq_cap is None:
                longest = max(d[3] + d[2] for d in dec)
                nsplit = min(nsplit, max(1, -(-longest // (64 * MIN_TILES_PER_SPLIT))))
            plan["nsplit"] = nsplit
            plan["dec"] = ctx.upload_ints(f"attn_dec_{self.H}_{self.KV}_{self.hs}_{self.window}",
                                          np.asarray(dec, dtype=np.int32)).view(-1, 4)
            if nsplit > 1:
                n = ops.attn_decode_scratch_floats(len(dec), self.H, self.KV, self.hs, nsplit)
                plan["scratch"] = ctx.buf("attn_split", (n,), torch.float32)
        if por:
            plan["por"] = ctx.upload_ints(f"attn_por_{self.H}_{self.KV}_{self.hs}_{self.window}",
                                          np.asarray(por, dtype=np.int32)).view(-1, 4)
        ctx.plans[key] = plan

    def attend(self, q, cache, ctx, out):
        if not self.uses_tensor_cores():
            ops.paged_attention_ref(q, cache.k, cache.v, cache.block_table, ctx.row_seq, ctx.positions,
                                    out, cache.page_size, ctx.seq_slots, self.H, self.KV, self.hs,
                                    self.scale, self.window or 0, status=ctx.status)
            return
        plan = ctx.plans[("attention", self.H, self.KV, self.hs, self.window)]
        args = (cache.page_size, ctx.seq_slots, self.H, self.KV, self.hs, self.scale, self.window or 0)
        if plan["dec"] is not None:
            if plan["tma"]:
                ops.attn_decode_tma(q, cache.k, cache.v, cache.block_table, plan["dec"], out, *args, work=plan["work"],
                                    scratch=plan["scratch"], status=ctx.status, max_rows=plan["dec_rows"])
            else:
                ops.attn_decode(q, cache.k, cache.v, cache.block_table, plan["dec"], out, *args,
                                nsplit=plan["nsplit"], scratch=plan["scratch"], status=ctx.status)
        if plan["por"] is not None:
            portion = ops.attn_portion_tc05 if plan["tc05"] else ops.attn_portion
            portion(q, cache.k, cache.v, cache.block_table, plan["por"], out, *args, status=ctx.status)


def distance_bucket(n: int, rows: int, max_distance: float) -> int:
    """Row of a bias table of ``rows`` rows for distance n: its own row below rows/2, then logarithmic steps that
    reach the last row at ``max_distance``."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(max_distance / half) * (rows - half))))


def spread_by_distance(table: torch.Tensor, max_distance: float) -> torch.Tensor:
    """fp32 [nd, H] with row n = table[bucket(n)] for every distance up to ``max_distance`` rounded up; distances
    beyond that share the last row, which is what the kernels' ``min(distance, nd - 1)`` gives them."""
    rows = table.shape[0]
    if rows < 2 or max_distance <= rows // 2:
        raise ValueError(f"attention: a bias table of {rows} rows needs max_distance above {rows // 2}, found {max_distance}")
    nd = int(math.ceil(max_distance)) + 1
    idx = torch.tensor([distance_bucket(n, rows, max_distance) for n in range(nd)], dtype=torch.long, device=table.device)
    return table.float().index_select(0, idx).contiguous()


register_mixer("attention", Attention)
