"""Routed feed-forward (mixture of experts): every row uses ``top`` of ``experts`` small feed-forwards, chosen by a
router, and optionally a shared one that runs for every row.

Per row x:
    z = W_router x (fp32 sums);  s = sigmoid(z)  (``scores``: "sigmoid" or "softmax" over the experts)
    the ``top`` experts with the largest scores are chosen; their weights are s_e * ``scale`` (``renorm``: divided by the
    chosen scores' sum first)
    expert_e(x) = W_down,e act(W_up,e x)              act one of ``ops.MOE_ACTS`` (default relu2: the square of relu), no biases
    out = sum_chosen weight_e * expert_e(x)  +  sigmoid(w_sg . x) * shared(x)      (``shared``: {"intermediate_size": F}
                                                                                   or None; ``shared_gate`` False: no gate)
Further parameters:
``activation`` "glu_limited"   experts with a gate matrix and limits (``limit``, ``alpha``):
                               g = min(W_gate,e x, limit), u = clamp(W_up,e x, -limit, limit), expert_e(x) = W_down,e (g sigmoid(alpha g) (u + 1));
                               gate and up rows are stacked in turn, and the first grouped product applies the activation to
                               each pair of neighbouring columns in its epilogue.
``choice_bias``                name of a vector [experts + identity]: the ``top`` largest of s + bias are chosen, the weights stay s.
``identity`` I                 the router has I more rows behind the experts'; a choice among them stands for an expert that returns
                               x itself (no tensors, no product: the combining kernel reads the row).
``shared`` with "kind"         the shared expert is the registered feed-forward of that kind, built from ``shared["params"]``.
On the device, with nothing read back: ``moe_route`` (scores, choice, weights, the shared gate), ``moe_plan`` (pairs ordered
by expert), two grouped products over the ordered places (the first reads its rows through the order and applies the
activation in its epilogue; true 32-bit in float32; in bfloat16 on the tensor cores: mma.sync tiles for few places, and
from 128 places on the TMA-fed tcgen05 grouped kernel behind a gather of the rows), ``moe_combine`` (weighted sum in each
row's own order of choices, in fp32, the shared expert included). Within a kernel a row's result does not depend on what
else is in the batch: places only decide where a row lies in a tile, never the order of its sums; which kernel runs
depends on the number of places, as for every product of the package, and changes the rounding of bfloat16 sums only.

Tensor names below the part's prefix: router, e<i>.up, e<i>.down (e<i>.gate), shared.up, shared.down, shared.sg.
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
        self.identity = int(p.get("identity", 0) or 0)
        self.routes = self.E + self.identity              # rows of the router
        self.choice_bias_name = p.get("choice_bias") or None
        self.limit = float(p.get("limit", 0.0) or 0.0)
        self.alpha = float(p.get("alpha", 1.702))
        self.gated = self.activation == "glu_limited"
        if not 1 <= self.top <= min(self.routes, 32) or self.identity < 0:
            raise ValueError(f"routed_mlp: top {self.top} must be between 1 and min(experts + identity, 32)")
        if self.gated and not self.limit > 0:
            raise ValueError("routed_mlp: activation 'glu_limited' needs a positive limit")
        if self.activation not in ops.MOE_ACTS or self.scores not in ops.MOE_SCORES:
            raise ValueError(f"routed_mlp: activation {self.activation!r} or scores {self.scores!r} is not supported")
        sh = p.get("shared") or None
        self.shared = None
        self.shared_gate = False
        if sh is not None and sh.get("kind"):
            self.shared = feed_forward_class(sh["kind"])(dict(sh["params"]), dtype, device)
            self.shared_gate = bool(p.get("shared_gate", False))
        elif sh is not None:
            self.shared = feed_forward_class("dense_mlp")(
                {"hidden_size": self.hidden, "intermediate_size": int(sh["intermediate_size"]),
                 "activation": sh.get("activation", self.activation), "up_name": "shared.up", "down_name": "shared.down"}, dtype, device)
            self.shared_gate = bool(p.get("shared_gate", True))
        self.w_route = self.w_up = self.w_down = self.choice_bias = None

    def weight_shapes(self):
        s = {"router": (self.routes, self.hidden)}
        if self.choice_bias_name:
            s[self.choice_bias_name] = (self.routes,)
        for e in range(self.E):
            if self.gated:
                s[f"e{e}.gate"] = (self.inter, self.hidden)
            s[f"e{e}.up"] = (self.inter, self.hidden)
            s[f"e{e}.down"] = (self.hidden, self.inter)
        if self.shared is not None:
            s.update(self.shared.weight_shapes())
            if self.shared_gate:
                s["shared.sg"] = (1, self.hidden)
        return s

    def keeps_dtype(self, name):
        return name == self.choice_bias_name or (self.shared is not None and self.shared.keeps_dtype(name))

    def norm_like(self, name):
        return False

    def load_weights(self, t):
        rows = [t["router"]] + ([t["shared.sg"]] if self.shared_gate else [])
        self.w_route = torch.cat(rows, 0).contiguous()           # the router's rows, then the shared expert's gate row
        if self.choice_bias_name:
            self.choice_bias = t[self.choice_bias_name].float().contiguous()
        if self.gated:                                            # [E, 2F, d]: row 2i an entry's gate, row 2i + 1 its up
            self.w_up = torch.stack([torch.stack([t[f"e{e}.gate"], t[f"e{e}.up"]], 1).reshape(2 * self.inter, self.hidden)
                                     for e in range(self.E)]).contiguous()
        else:
            self.w_up = torch.stack([t[f"e{e}.up"] for e in range(self.E)]).contiguous()    # [E, F, d]
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
        R = self.routes                                           # experts with weights, then the identity experts
        ops.moe_route(x, self.w_route, R, top, self.scale, ids, wts, gates, scores=self.scores, renorm=self.renorm,
                      choice_bias=self.choice_bias)
        scratch = ctx.buf("moe_plan", (ops.moe_plan_ints(P, R),), torch.int32)
        offsets = ctx.buf("moe_offsets", (R + 1,), torch.int32)
        row_of = ctx.buf("moe_row_of", (P,), torch.int32)
        place_of = ctx.buf("moe_place_of", (T, top), torch.int32)
        ops.moe_plan(ids, R, scratch, offsets, row_of, place_of)
        # the places of the identity experts lie behind offsets[E]: the grouped products never reach them
        act = ctx.buf("moe_act", (P, self.inter), self.dtype)
        gathered = ctx.buf("moe_x", (P, self.hidden), self.dtype) if ops.moe_gemm_grouped_ok(x, self.w_up, act, P, self.activation) else None
        ops.moe_gemm(x, row_of, self.w_up, act, offsets, act=self.activation, gathered=gathered, status=ctx.status,
                     limit=self.limit, alpha=self.alpha)
        y = ctx.buf("moe_y", (P, self.hidden), torch.float32)
        ops.moe_gemm(act, None, self.w_down, y, offsets, status=ctx.status)
        shared = self.shared.forward(x, ctx) if self.shared is not None else None
        out = ctx.buf("moe_out", (T, self.hidden), self.dtype)
        ops.moe_combine(y, place_of, wts, out, shared=shared, gate=gates[:, 0] if gates is not None else None,
                        ids=ids if self.identity else None, real=E, x=x if self.identity else None)
        return out


register_feed_forward("routed_mlp", RoutedMLP)
