"""Work lists of the general tensor-core attention (``attention_flex.cu``), made on the host before a step.

A sequence's rows of the step become work items of at most ``ops.attn_flex_tokens`` tokens. Sequences that bring
few rows (decode rows, short ends of prompts: one item) form one launch whose items have their keys cut into
shares, as many as fill the device; longer portions form another without shares. A plan is kept under a key of
the step's context, so layers with the same head layout make it once.
"""
from __future__ import annotations

import numpy as np
import torch

from ..csrc import ops

MAX_SPLITS = 32
MIN_KEYS_PER_SPLIT = 256
BLOCKS_PER_SM = 2


def plan(ctx, device, H: int, KV: int, dk: int, dv: int, own_v: bool, window, skip=frozenset()) -> dict:
    """``skip``: sequences of the step that get no items (another path serves them)."""
    key = ("flex", H, KV, dk, dv, own_v, window, tuple(sorted(skip)))
    got = ctx.plans.get(key)
    if got is not None:
        return got
    per_item = ops.attn_flex_tokens(H, KV)
    dec, por = [], []
    qs, cl = ctx.h_q_start, ctx.h_ctx_len
    for s in range(ctx.num_seqs):
        if s in skip:
            continue
        row0, n = int(qs[s]), int(qs[s + 1] - qs[s])
        pos0 = int(cl[s]) - n
        if n <= per_item:
            dec.append((s, row0, n, pos0))
        else:
            for b in range(0, n, per_item):
                por.append((s, row0 + b, min(per_item, n - b), pos0 + b))
    fixed = ctx.seq_cap is not None
    if fixed:                                         # fixed shapes: pad with empty items, shares by the shape alone
        dec += [(0, 0, 0, 0)] * (ctx.seq_cap - len(dec))
    out = {"dec": None, "por": None, "nsplit": 1, "scratch": None, "dec_rows": 0}
    tag = f"{H}_{KV}_{dk}_{dv}_{int(own_v)}_{window}" + ("_rest" if skip else "")
    if dec:
        # blocks one item gets without shares: kv heads x parts of the query heads x slices of the value columns
        gb = max(g for g in range(1, min(H // KV, 64) + 1) if (H // KV) % g == 0)
        slices = -(-dv // (128 if dv > 64 else 64))
        # the most rows of any item; in a fixed shape every item is one token
        out["dec_rows"] = gb * (1 if fixed else max(d[2] for d in dec))
        if not own_v and slices > 1 and out["dec_rows"] <= 16:
            slices = -(-slices // 4)                  # a block's four warps take a slice each
        per = KV * ((H // KV) // gb) * slices
        nsplit = max(1, min(MAX_SPLITS, BLOCKS_PER_SM * ops.sm_count(device) // (len(dec) * per)))
        if not fixed:
            longest = max(d[3] + d[2] for d in dec)
            nsplit = min(nsplit, max(1, longest // MIN_KEYS_PER_SPLIT))
        out["nsplit"] = nsplit
        out["dec"] = ctx.upload_ints("flex_dec_" + tag, np.asarray(dec, dtype=np.int32)).view(-1, 4)
        if nsplit > 1:
            out["scratch"] = ctx.buf("flex_split", (ops.attn_flex_scratch_floats(len(dec), H, KV, dv, nsplit),), torch.float32)
    if por:
        por.sort(key=lambda it: -(it[3] + it[2]))     # the items with most keys first: the last blocks to start are short
        out["por"] = ctx.upload_ints("flex_por_" + tag, np.asarray(por, dtype=np.int32)).view(-1, 4)
    ctx.plans[key] = out
    return out


def attend(pl: dict, q, k_cache, v_cache, block_table, out, page_size, seq_slots, H, KV, dk, dv, scale, window,
           dist_bias=None, sink=None, status=None, softcap: float = 0.0, v_share: int = 1, slopes=None, q_temp=None,
           gate=None) -> None:
    args = (page_size, seq_slots, H, KV, dk, dv, scale, window or 0)
    if pl["dec"] is not None:
        ops.attn_flex(q, k_cache, v_cache, block_table, pl["dec"], out, *args, dist_bias=dist_bias, sink=sink,
                      nsplit=pl["nsplit"], scratch=pl["scratch"], status=status, max_rows=pl["dec_rows"], softcap=softcap,
                      v_share=v_share, slopes=slopes, q_temp=q_temp, gate=gate)
    if pl["por"] is not None:
        ops.attn_flex(q, k_cache, v_cache, block_table, pl["por"], out, *args, dist_bias=dist_bias, sink=sink, status=status,
                      softcap=softcap, v_share=v_share, slopes=slopes, q_temp=q_temp, gate=gate)
