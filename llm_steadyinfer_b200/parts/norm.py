"""RMSNorm part: ``out = weight * h * rsqrt(mean(h^2) + eps)`` with ``h = resid + delta``
written back to the fp32 residual stream. Formula of the reference's
``row_rmsnorm_f32_dim`` (src/source/op/kernels/cuda/rmsnorm_kernel.cu:8-60), whose eps is a
constant in the kernel; here it is a parameter of the part. With ``scalar`` the checkpoint holds one number
for all coordinates (a tensor without dimensions), which is spread over the width when the weights are loaded.
With ``offset`` c the checkpoint's vector is stored around zero and the norm multiplies by ``c + weight`` (summed in fp32
when the weights are loaded, and kept in fp32).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..csrc import ops
from .base import Norm, NormedDelta, SummedDelta, register_norm


class RMSNorm(Norm):
    capturable = True
    takes_ahead = True

    def __init__(self, params, dtype, device):
        super().__init__(params, dtype, device)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.name = params.get("weight_name", "weight")      # "" where the checkpoint names the vector by the prefix alone
        self.scalar = bool(params.get("scalar", False))     # one number for all coordinates
        self.offset = float(params.get("offset", 0.0))      # added to the stored vector
        self.weight: Optional[torch.Tensor] = None

    def weight_shapes(self):
        return {self.name: () if self.scalar else (self.size,)}

    def keeps_dtype(self, name: str) -> bool:
        return True

    def load_weights(self, tensors):
        w = tensors[self.name]
        if self.offset:
            w = w.float() + self.offset
        self.weight = (w.reshape(1).expand(self.size) if self.scalar else w).contiguous()

    def norm_like(self, name):
        return not self.offset                       # a vector stored around zero is drawn around zero

    def kernel_files(self, page_size):
        return ("norm",)

    def forward(self, resid, delta, out, rows=None, ahead=None):
        if isinstance(delta, NormedDelta):           # the sublayer before has a norm of its own behind it
            ops.add_norm(resid, delta.x, self.weight, self.eps, out, rows=rows, delta_weight=delta.norm.weight,
                         delta_eps=delta.norm.eps, delta_bias=delta.bias)
        elif isinstance(delta, SummedDelta):         # two sublayers side by side: both join the stream here
            ops.add_rmsnorm(resid, delta.a, self.weight, self.eps, out, rows=rows, ahead=ahead, delta2=delta.b)
        else:
            ops.add_rmsnorm(resid, delta, self.weight, self.eps, out, rows=rows, ahead=ahead)

    def add(self, resid, delta: NormedDelta, extra=None, vec=None):
        """``resid += norm(delta) (+ extra) (+ vec)`` with no norm of the stream behind it."""
        ops.add_norm(resid, delta.x, delta_weight=delta.norm.weight, delta_eps=delta.norm.eps, delta_bias=delta.bias,
                     extra=extra, vec=vec)

    def normalize(self, x, out=None):
        ops.rmsnorm_rows(x, self.weight, self.eps, out)


register_norm("rmsnorm", RMSNorm)
