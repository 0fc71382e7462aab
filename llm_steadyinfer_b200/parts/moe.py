"""Routed feed-forward (mixture of experts): every row uses ``top`` of ``experts`` small feed-forwards, chosen by a
router, and optionally a shared one that runs for every row.

Per row x:
    z = W_router x (fp32 sums);  s = sigmoid(z)  (``scores``: "sigmoid" or "softmax" over the experts)
    the ``top`` experts with the largest scores are chosen; their weights are s_e * ``scale`` (``renorm``: divided by the
    chosen scores' sum first)
    expert_e(x) = W_down,e act(W_up,e x)              act one of ``ops.MOE_ACTS`` (default relu2: the square of relu), no biases
    out = sum_chosen weight_e * expert_e(x)  +  sigmoid(w_sg . x) * shared(x)      (``shared``: {"intermediate_size": F}
                                                                                   or None; ``shared_gate`` False: no gate)
On the device, with nothing read back: ``moe_route`` (scores, choice, weights, the shared gate), ``moe_plan`` (pairs ordered
by expert), two grouped products over the ordered places (the first reads its rows through the order and applies the
activation in its epilogue; true 32-bit in float32; in bfloat16 on the tensor cores: mma.sync tiles for few places, and
from 128 places on the TMA-fed tcgen05 grouped kernel behind a gather of the rows), ``moe_combine`` (weighted sum in each
row's own order of choices, in fp32, the shared expert included). Within a kernel a row's result does not depend on what
else is in the batch: places only decide where a row lies in a tile, never the order of its sums; which kernel runs
depends on the number of places, as for every product of the package, and changes the rounding of bfloat16 sums only.

Tensor names below the part's prefix: router, e<i>.up, e<i>.down, shared.up, shared.down, shared.sg.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import FeedForward, feed_forward_class, register_feed_forward


class RoutedMLP(FeedForward):
    capturable = True

    def __init__(self, params, dtype, device):
        super().__init__(params, dtype, device)
        p = params
        self.hidden = int(p["hidden_size"])
        self.inter = int(p["intermediate_size"])
        self.E = int(p["experts"])
        self.top = int(p["top"])
        self.scale = float(p.get("scale", 1.0))
        self.scores = p.get("scores", "sigmoid")
        self.renorm = bool(p.get("renorm", False))
        self.activation = p.get("activation", "relu2")
        if not 1 <= self.top <= min(self.E, 32):
            raise ValueError(f"routed_mlp: top {self.top} must be between 1 and min(experts, 32)")
        if self.activation not in ops.MOE_ACTS or self.scores not in ops.MOE_SCORES:
            raise ValueError(f"routed_mlp: activation {self.activation!r} or scores {self.scores!r} is not supported")
        sh = p.get("shared") or None
        self.shared = None
        self.shared_gate = False
        if sh is not None:
            self.shared = feed_forward_class("dense_mlp")(
                {"hidden_size": self.hidden, "intermediate_size": int(sh["intermediate_size"]),
                 "activation": sh.get("activation", self.activation), "up_name": "shared.up", "down_name": "shared.down"}, dtype, device)
            self.shared_gate = bool(p.get("shared_gate", True))
        self.w_route = self.w_up = self.w_down = None

    def weight_shapes(self):
        s = {"router": (self.E, self.hidden)}
        for e in range(self.E):
            s[f"e{e}.up"] = (self.inter, self.hidden)
            s[f"e{e}.down"] = (self.hidden, self.inter)
        if self.shared is not None:
            s.update(self.shared.weight_shapes())
            if self.shared_gate:
                s["shared.sg"] = (1, self.hidden)
        return s

    def load_weights(self, t):
        rows = [t["router"]] + ([t["shared.sg"]] if self.shared_gate else [])
        self.w_route = torch.cat(rows, 0).contiguous()           # the router's rows, then the shared expert's gate row
        self.w_up = torch.stack([t[f"e{e}.up"] for e in range(self.E)]).contiguous()        # [E, F, d]
        self.w_down = torch.stack([t[f"e{e}.down"] for e in range(self.E)]).contiguous()    # [E, d, F]
        if self.shared is not None:
            self.shared.load_weights({n: t[n] for n in self.shared.weight_shapes()})

    def kernel_files(self, page_size):
        return ("moe",) + (("gemm_tc05",) if self.dtype == torch.bfloat16 else ()) + (self.shared.kernel_files(page_size) if self.shared is not None else ())

    def forward(self, x, ctx):
        T = x.shape[0]
        E, top, P = self.E, self.top, x.shape[0] * self.top
        ids = ctx.buf("moe_ids", (T, top), torch.int32)
        wts = ctx.buf("moe_wts", (T, top), torch.float32)
        gates = ctx.buf("moe_gates", (T, 1), torch.float32) if self.shared_gate else None
        ops.moe_route(x, self.w_route, E, top, self.scale, ids, wts, gates, scores=self.scores, renorm=self.renorm)
        scratch = ctx.buf("moe_plan", (ops.moe_plan_ints(P, E),), torch.int32)
        offsets = ctx.buf("moe_offsets", (E + 1,), torch.int32)
        row_of = ctx.buf("moe_row_of", (P,), torch.int32)
        place_of = ctx.buf("moe_place_of", (T, top), torch.int32)
        ops.moe_plan(ids, E, scratch, offsets, row_of, place_of)
        act = ctx.buf("moe_act", (P, self.inter), self.dtype)
        gathered = ctx.buf("moe_x", (P, self.hidden), self.dtype) if ops.moe_gemm_grouped_ok(x, self.w_up, act, P, self.activation) else None
        ops.moe_gemm(x, row_of, self.w_up, act, offsets, act=self.activation, gathered=gathered, status=ctx.status)
        y = ctx.buf("moe_y", (P, self.hidden), torch.float32)
        ops.moe_gemm(act, None, self.w_down, y, offsets, status=ctx.status)
        shared = self.shared.forward(x, ctx) if self.shared is not None else None
        out = ctx.buf("moe_out", (T, self.hidden), self.dtype)
        ops.moe_combine(y, place_of, wts, out, shared=shared, gate=gates[:, 0] if gates is not None else None)
        return out


register_feed_forward("routed_mlp", RoutedMLP)
