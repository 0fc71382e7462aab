"""A block arranges one mixer, one feed-forward and their norms around the residual stream.

How they are arranged is data as well: an *arrangement* is a function registered under a name,
``fn(block, resid, delta, ctx, cache) -> delta``, and a layer's spec names it. It gets the fp32
residual stream ``resid`` [T, d] and the pending ``delta`` of the block before it (None for the
first block), which it must add into the stream (``Norm.forward`` does the add and the norm in one
kernel), and returns its own pending delta, which the block after it (or the final norm) adds.

The built-in "pre_norm" is the reference's block (src/source/model/llama3.cpp:996-1181):
    h += delta_in;  x = norm1(h);  a = mixer(x);  h += a;  x = norm2(h);  return ffn(x)
(a block whose spec has no feed-forward ends after the mixer and returns ``a``).
"sandwich" has a norm behind each sublayer as well as before it:
    h += delta_in;  a = mixer(norm1(h));  h += norm1b(a);  f = ffn(norm2(h));  return norm2b(f), still to be added
What it hands on is a ``NormedDelta``: the sublayer's raw result with the norm that belongs to it, which the next
norm's launch normalises and adds before its own statistics (no launch of its own).
"parallel_gated" runs both sublayers on the same stream, each behind a norm of its own, and passes each result through
a learned gate (``SublayerGate``: sigmoid of a projection of the sublayer's own input plus a bias, entry by entry):
    h += delta_in;  x1 = norm1(h);  x2 = norm2(h);  h += scale * (gate1(x1) * mixer(x1) + gate2(x2) * ffn(x2))
The add is one kernel in fp32 on the stream itself (``ops.gated_add``), so the block hands no pending delta on.
"parallel" runs both sublayers on the output of one norm and adds both results to the stream:
    h += delta_in;  x = norm1(h);  return (mixer(x), ffn(x)), both still to be added
What it hands on is a ``SummedDelta``: the next norm's launch adds both results in fp32 before its own statistics. While the
feed-forward runs, the scratch key "delta" (where parts put their results) stands for a second buffer, so that the mixer's
result stays alive beside it.
Another arrangement (post-norm, ...) is added with ``register_arrangement`` and needs no change here.
"""
from __future__ import annotations

from typing import Callable, Dict, Optional

import torch

from ..csrc import ops
from .base import FeedForward, Mixer, Norm, NormedDelta, Part, SummedDelta
from .linear import linear

_ARRANGEMENTS: Dict[str, Callable] = {}
_CAPTURABLE: Dict[str, bool] = {}


def register_arrangement(name: str, fn: Callable, capturable: bool = False) -> None:
    """Register ``fn(block, resid, delta, ctx, cache) -> delta`` under a name that layer specs use.
    ``capturable``: the function itself (beside the parts it calls) reads nothing on the host that
    changes from step to step, allocates nothing and never waits for the device, so that a decode
    step through it may be recorded in a CUDA graph (see ``Part.capturable``)."""
    _ARRANGEMENTS[name] = fn
    _CAPTURABLE[name] = bool(capturable)


def arrangement(name: str) -> Callable:
    if name not in _ARRANGEMENTS:
        raise KeyError(f"block arrangement {name!r} is not registered; registered: {sorted(_ARRANGEMENTS)}")
    return _ARRANGEMENTS[name]


class SublayerGate(Part):
    """A learned gate on a sublayer's result: ``sigmoid(W x + b)``, one number per coordinate, from the sublayer's own
    input x. The part owns the matrix and the bias (tensor names: the part's prefix itself and ``.b``) and computes the
    projection; the sigmoid and the product run in the kernel that adds the gated results into the stream."""
    capturable = True

    def __init__(self, params, dtype, device):
        super().__init__(params, dtype, device)
        self.size = int(params["size"])
        self.weight = self.bias = None

    def weight_shapes(self):
        return {"": (self.size, self.size), ".b": (self.size,)}

    def keeps_dtype(self, name):
        return name == ".b"

    def norm_like(self, name):
        return False

    def load_weights(self, tensors):
        self.weight = tensors[""].contiguous()
        self.bias = tensors[".b"].float().contiguous()

    def kernel_files(self, page_size):
        return ("norm",) + (("gemm_f32",) if self.dtype == torch.float32 else ("gemm_skinny", "gemm_rows", "gemm_tc05"))

    def project(self, x, ctx, key: str):
        """``W x`` [T, size] in the compute dtype (the bias and the sigmoid belong to the adding kernel)."""
        z = ctx.buf(key, (x.shape[0], self.size), self.dtype)
        linear(x, self.weight, z, ctx.status)
        return z


class Block:
    def __init__(self, mixer: Mixer, feed_forward: Optional[FeedForward], mixer_norm: Norm,
                 feed_forward_norm: Optional[Norm], arrangement_name: str = "pre_norm",
                 mixer_post_norm: Optional[Norm] = None, feed_forward_post_norm: Optional[Norm] = None,
                 mixer_gate: Optional[SublayerGate] = None, feed_forward_gate: Optional[SublayerGate] = None,
                 residual_scale: float = 1.0):
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.mixer_norm = mixer_norm
        self.feed_forward_norm = feed_forward_norm
        self.mixer_post_norm = mixer_post_norm
        self.feed_forward_post_norm = feed_forward_post_norm
        self.mixer_gate = mixer_gate
        self.feed_forward_gate = feed_forward_gate
        self.residual_scale = float(residual_scale)
        self.arrangement = arrangement_name
        self._run = arrangement(arrangement_name)
        self.capturable = _CAPTURABLE[arrangement_name]

    def forward(self, resid: torch.Tensor, delta: Optional[torch.Tensor], ctx, cache) -> torch.Tensor:
        return self._run(self, resid, delta, ctx, cache)

    @staticmethod
    def norm(norm: Norm, resid, delta, out, ahead=None) -> None:
        """``resid += delta; out = norm(resid)``; ``ahead`` (what the part after the norm streams first)
        is passed on to norms that take it."""
        if ahead is not None and norm.takes_ahead:
            norm.forward(resid, delta, out, ahead=ahead)
        else:
            norm.forward(resid, delta, out)


def pre_norm(block: Block, resid, delta, ctx, cache):
    T, d = resid.shape
    x = ctx.buf("block_x", (T, d), block.mixer.dtype)
    block.norm(block.mixer_norm, resid, delta, x, block.mixer.streams_first(T))
    # a part that can add its result into the stream itself is given the stream and returns None
    if block.mixer.adds_into_residual:
        a = block.mixer.forward(x, ctx, cache, resid=resid)
    else:
        a = block.mixer.forward(x, ctx, cache)
    if block.feed_forward is None:                        # a block of the mixer's sublayer alone
        return a
    block.norm(block.feed_forward_norm, resid, a, x, block.feed_forward.streams_first(T))
    if block.feed_forward.adds_into_residual:
        return block.feed_forward.forward(x, ctx, resid=resid)
    return block.feed_forward.forward(x, ctx)


register_arrangement("pre_norm", pre_norm, capturable=True)


def sandwich(block: Block, resid, delta, ctx, cache):
    if block.mixer_post_norm is None or (block.feed_forward is not None and block.feed_forward_post_norm is None):
        raise ValueError("arrangement 'sandwich' needs a norm behind each sublayer")
    T, d = resid.shape
    x = ctx.buf("block_x", (T, d), block.mixer.dtype)
    block.norm(block.mixer_norm, resid, delta, x)
    a = NormedDelta(block.mixer.forward(x, ctx, cache), block.mixer_post_norm)
    if block.feed_forward is None:
        return a
    block.norm(block.feed_forward_norm, resid, a, x)
    ff = block.feed_forward
    bias = getattr(ff, "output_bias", None)
    if bias is not None:                                  # the last product's bias joins the result inside the adding kernel
        return NormedDelta(ff.forward(x, ctx, add_bias=False), block.feed_forward_post_norm, bias)
    return NormedDelta(ff.forward(x, ctx), block.feed_forward_post_norm)


register_arrangement("sandwich", sandwich, capturable=True)


def parallel(block: Block, resid, delta, ctx, cache):
    T, d = resid.shape
    x = ctx.buf("block_x", (T, d), block.mixer.dtype)
    block.norm(block.mixer_norm, resid, delta, x, block.mixer.streams_first(T))
    a = block.mixer.forward(x, ctx, cache)
    if block.feed_forward is None:
        return a
    ctx.alias["delta"] = "delta_second"                   # the feed-forward's result beside the mixer's
    try:
        f = block.feed_forward.forward(x, ctx)
    finally:
        del ctx.alias["delta"]
    if f.data_ptr() == a.data_ptr():
        raise ValueError("arrangement 'parallel': the mixer and the feed-forward return the same scratch buffer")
    return SummedDelta(a, f)


register_arrangement("parallel", parallel, capturable=True)


def parallel_gated(block: Block, resid, delta, ctx, cache):
    if block.mixer_gate is None or (block.feed_forward is not None and block.feed_forward_gate is None):
        raise ValueError("arrangement 'parallel_gated' needs a gate for each sublayer")
    T, d = resid.shape
    x1 = ctx.buf("block_x", (T, d), block.mixer.dtype)
    block.norm(block.mixer_norm, resid, delta, x1, block.mixer.streams_first(T))
    ff = block.feed_forward
    x2 = None
    if ff is not None:                                     # the same stream through the second norm (nothing left to add)
        x2 = ctx.buf("block_x2", (T, d), block.mixer.dtype)
        block.norm(block.feed_forward_norm, resid, None, x2)
    a = block.mixer.forward(x1, ctx, cache)
    z1 = block.mixer_gate.project(x1, ctx, "block_gate1")
    if ff is None:
        ops.gated_add(resid, z1, block.mixer_gate.bias, a, mult=block.residual_scale)
        return None
    f = ff.forward(x2, ctx)
    if f.data_ptr() == a.data_ptr():
        raise ValueError("arrangement 'parallel_gated': the mixer and the feed-forward return the same scratch buffer; "
                         "the mixer's result must stay alive beside the feed-forward's")
    z2 = block.feed_forward_gate.project(x2, ctx, "block_gate2")
    ops.gated_add(resid, z1, block.mixer_gate.bias, a, z2, block.feed_forward_gate.bias, f, mult=block.residual_scale)
    return None


register_arrangement("parallel_gated", parallel_gated, capturable=True)
