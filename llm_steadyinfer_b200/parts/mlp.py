"""Gated feed-forward part: ``down(silu(gate(x)) * up(x))`` without biases, as the reference's
block computes it (src/source/model/llama3.cpp:1149-1180). gate and up are stacked into one
[2F, d] matrix at load so one product feeds the activation: when F is a multiple of 8 the rows
are interleaved in groups of 8 (8 rows of gate, the 8 rows of up that belong to them, ...), so
that the few-row product holds a gate and its up in one block and applies the activation in
its epilogue. So does the product on the tcgen05 tensor cores for 128 rows and more (``gemm_tc05.cu``;
``gemm_rows.cu`` below that, when it is turned on); where none applies (fp32, an intermediate size that is
no multiple of 8, 17 to 127 rows by default), the product runs alone and the activation kernel reads the
same interleaved columns.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import FeedForward, register_feed_forward
from . import linear as linear_mod
from .linear import linear

INTERLEAVE = 8         # rows of gate, then rows of up, in the stacked weight
USE_TC05_GEMM = True   # gate/up product of more than 16 rows through this package's tcgen05 kernels (activation fused)


class GatedMLP(FeedForward):
    capturable = True
    adds_into_residual = True

    def __init__(self, params, dtype, device):
        super().__init__(params, dtype, device)
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        if params.get("activation", "silu") != "silu":
            raise ValueError(f"gated_mlp: activation {params['activation']!r} is not supported")
        self.names = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight"}
        self.names.update(params.get("names") or {})       # checkpoint names of the three matrices
        self.group = INTERLEAVE if self.inter % INTERLEAVE == 0 else self.inter
        self.gate_up = None
        self.down = None

    def weight_shapes(self):
        n = self.names
        return {n["gate"]: (self.inter, self.hidden), n["up"]: (self.inter, self.hidden), n["down"]: (self.hidden, self.inter)}

    def load_weights(self, tensors):
        gate, up = tensors[self.names["gate"]], tensors[self.names["up"]]
        n = self.inter // self.group
        self.gate_up = torch.stack([gate.view(n, self.group, self.hidden), up.view(n, self.group, self.hidden)], 1) \
            .reshape(2 * self.inter, self.hidden).contiguous()
        self.down = tensors[self.names["down"]].contiguous()

    def streams_first(self, rows):
        # few rows in bfloat16 go to the weight-streaming product, which reads every weight once
        return self.gate_up if self.dtype == torch.bfloat16 and rows <= ops.SKINNY_MAX_ROWS else None

    def kernel_files(self, page_size):
        if self.dtype == torch.float32:
            return ("gemm_f32", "swiglu")
        return ("gemm_skinny", "swiglu", "gemm_tc05", "gemm_rows")

    def forward(self, x, ctx, resid=None):
        T = x.shape[0]
        act = ctx.buf("ffn_act", (T, self.inter), self.dtype)
        if (self.group == INTERLEAVE and linear_mod.USE_SKINNY and act.dtype == torch.bfloat16
                and ops.gemm_skinny_ok(x, self.gate_up, act)):
            ops.gemm_skinny_swiglu(x, self.gate_up, act, checked=True)
        elif (self.group == INTERLEAVE and USE_TC05_GEMM and act.dtype == torch.bfloat16 and ops.gemm_tc05_available()
                and ops.gemm_tc05_ok(x, self.gate_up, act)
                and (linear_mod.USE_OWN_GEMM if T >= linear_mod.OWN_GEMM_MIN_ROWS else linear_mod.USE_ROWS)):
            if T >= linear_mod.OWN_GEMM_MIN_ROWS:
                ops.gemm_tc05_swiglu(x, self.gate_up, act, ctx.status)
            else:
                ops.gemm_rows_swiglu(x, self.gate_up, act, ctx.status)
        else:
            gu = ctx.buf("ffn_gate_up", (T, 2 * self.inter), self.dtype)
            linear(x, self.gate_up, gu, ctx.status)
            ops.swiglu(gu, act, self.group)
        if resid is not None and linear_mod.linear_into_residual(act, self.down, resid, ctx.status):
            return None                                   # the down projection added itself into the stream
        out = ctx.buf("delta", (T, self.hidden), self.dtype)
        linear(act, self.down, out, ctx.status)
        return out


register_feed_forward("gated_mlp", GatedMLP)


class DenseMLP(FeedForward):
    """Feed-forward without a gate: ``down(act(up(x)))``; ``activation`` is one of ``ops.ACTIVATIONS`` ("relu2": the
    square of relu). Tensor names are parameters (``up_name``, ``down_name``)."""
    capturable = True

    def __init__(self, params, dtype, device):
        super().__init__(params, dtype, device)
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        self.activation = params.get("activation", "relu2")
        if self.activation not in ops.ACTIVATIONS:
            raise ValueError(f"dense_mlp: activation {self.activation!r} is not one of {sorted(ops.ACTIVATIONS)}")
        self.up_name = params.get("up_name", "up_proj.weight")
        self.down_name = params.get("down_name", "down_proj.weight")
        self.up = None
        self.down = None

    def weight_shapes(self):
        return {self.up_name: (self.inter, self.hidden), self.down_name: (self.hidden, self.inter)}

    def load_weights(self, tensors):
        self.up = tensors[self.up_name].contiguous()
        self.down = tensors[self.down_name].contiguous()

    def streams_first(self, rows):
        return self.up if self.dtype == torch.bfloat16 and rows <= ops.SKINNY_MAX_ROWS else None

    def kernel_files(self, page_size):
        return ("gemm_f32", "activation") if self.dtype == torch.float32 else ("gemm_skinny", "gemm_tc05", "gemm_rows", "activation")

    def forward(self, x, ctx):
        T = x.shape[0]
        act = ctx.buf("ffn_act", (T, self.inter), self.dtype)
        fused = self.activation == "relu2" and act.dtype == torch.bfloat16
        if fused and linear_mod.USE_SKINNY and ops.gemm_skinny_ok(x, self.up, act):
            ops.gemm_skinny_relu2(x, self.up, act, checked=True)              # decode rows: activation in the epilogue
        elif (fused and linear_mod.USE_OWN_GEMM and T >= linear_mod.OWN_GEMM_MIN_ROWS and ops.gemm_tc05_available()
                and ops.gemm_tc05_ok(x, self.up, act)):
            ops.gemm_tc05_relu2(x, self.up, act, ctx.status)                  # prompt portions: likewise, on tcgen05
        else:
            linear(x, self.up, act, ctx.status)
            ops.activation(act, act, self.activation)
        out = ctx.buf("delta", (T, self.hidden), self.dtype)
        linear(act, self.down, out, ctx.status)
        return out


register_feed_forward("dense_mlp", DenseMLP)


class LimitedGatedMLP(FeedForward):
    """Gated feed-forward with limits and biases:
        g = min(W_gate x + b_gate, limit);  u = clamp(W_up x + b_up, -limit, limit)
        y = g * sigmoid(alpha * g) * (u + 1);  out = W_down y + b_down
    ``limit`` and ``alpha`` (default 1.702, which makes g * sigmoid(alpha g) close to gelu) are parameters; so are the
    tensor names (``names``: gate, up, down; each bias is the matrix's name + ``bias_suffix``; ``biases`` False: the
    checkpoint has none and they count as zero). gate and up are
    stacked and interleaved as in ``GatedMLP``, and as there the activation (biases and limits included) runs in the
    epilogue of the first product for decode rows and for prompt portions in bfloat16; elsewhere a kernel of its own
    applies it to the stored product. Either way it is fp32 arithmetic on the product rounded to the compute dtype.
    ``output_bias`` is the down projection's bias; a caller that adds it itself (an arrangement that normalises the
    result anyway) calls ``forward(..., add_bias=False)``."""
    capturable = True

    def __init__(self, params, dtype, device):
        super().__init__(params, dtype, device)
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        self.limit = float(params["limit"])
        self.alpha = float(params.get("alpha", 1.702))
        if not self.limit > 0:
            raise ValueError(f"gated_mlp_limited: limit must be positive, found {self.limit}")
        self.names = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight"}
        self.names.update(params.get("names") or {})
        self.bias_suffix = params.get("bias_suffix", ".bias")
        self.biases = bool(params.get("biases", True))
        self.group = INTERLEAVE if self.inter % INTERLEAVE == 0 else self.inter
        self.gate_up = self.down = self.gate_up_bias = self.output_bias = None

    def weight_shapes(self):
        n, b = self.names, self.bias_suffix
        shapes = {n["gate"]: (self.inter, self.hidden), n["up"]: (self.inter, self.hidden), n["down"]: (self.hidden, self.inter)}
        if self.biases:
            shapes.update({n["gate"] + b: (self.inter,), n["up"] + b: (self.inter,), n["down"] + b: (self.hidden,)})
        return shapes

    def keeps_dtype(self, name):
        return self.biases and name.endswith(self.bias_suffix) and name[:-len(self.bias_suffix)] in self.names.values()

    def norm_like(self, name):
        return False

    def load_weights(self, tensors):
        n, b = self.names, self.bias_suffix
        k = self.inter // self.group
        stack = lambda g, u, *rest: torch.stack([g.view(k, self.group, *rest), u.view(k, self.group, *rest)], 1)
        self.gate_up = stack(tensors[n["gate"]], tensors[n["up"]], self.hidden).reshape(2 * self.inter, self.hidden).contiguous()
        self.down = tensors[n["down"]].contiguous()
        if self.biases:
            self.gate_up_bias = stack(tensors[n["gate"] + b].float(), tensors[n["up"] + b].float()).reshape(2 * self.inter).contiguous()
            self.output_bias = tensors[n["down"] + b].float().contiguous()
        else:                                           # the kernels take a bias vector: zeros
            self.gate_up_bias = torch.zeros(2 * self.inter, dtype=torch.float32, device=self.down.device)
            self.output_bias = None

    def streams_first(self, rows):
        return self.gate_up if self.dtype == torch.bfloat16 and rows <= ops.SKINNY_MAX_ROWS else None

    def kernel_files(self, page_size):
        return ("gemm_f32", "swiglu", "activation") if self.dtype == torch.float32 else \
            ("gemm_skinny", "swiglu", "activation", "gemm_tc05", "gemm_rows")

    def forward(self, x, ctx, add_bias=True):
        T = x.shape[0]
        act = ctx.buf("ffn_act", (T, self.inter), self.dtype)
        fused = self.group == INTERLEAVE and act.dtype == torch.bfloat16
        if fused and linear_mod.USE_SKINNY and ops.gemm_skinny_ok(x, self.gate_up, act):
            # decode rows: biases, limits and the gate in the epilogue of the weight-streaming product
            ops.gemm_skinny_glu_limited(x, self.gate_up, self.gate_up_bias, act, self.limit, self.alpha, checked=True)
        elif (fused and USE_TC05_GEMM and linear_mod.USE_OWN_GEMM and T >= linear_mod.OWN_GEMM_MIN_ROWS
                and ops.gemm_tc05_available() and ops.gemm_tc05_ok(x, self.gate_up, act)):
            ops.gemm_tc05_glu_limited(x, self.gate_up, self.gate_up_bias, act, self.limit, self.alpha, ctx.status)   # prompt portions
        else:
            gu = ctx.buf("ffn_gate_up", (T, 2 * self.inter), self.dtype)
            linear(x, self.gate_up, gu, ctx.status)
            ops.glu_limited(gu, self.gate_up_bias, act, self.group, self.limit, self.alpha)
        out = ctx.buf("delta", (T, self.hidden), self.dtype)
        linear(act, self.down, out, ctx.status)
        if add_bias and self.output_bias is not None:
            ops.add_bias(out, self.output_bias)
        return out


register_feed_forward("gated_mlp_limited", LimitedGatedMLP)
