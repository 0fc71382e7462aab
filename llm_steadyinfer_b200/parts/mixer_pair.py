"""Two mixers side by side: both read the same input, and the block gets ``left_scale * left(x) + right_scale * right(x)``.

The two are registered mixer kinds of their own, built from ``params["left"]`` / ``params["right"]`` = ``{"kind": ..,
"params": .., "position": {"kind": .., "params": ..} or None}``; their checkpoint tensors lie below ``left.`` and
``right.`` (``prefixes`` overrides). Between them they may ask for one paged cache and one per-request state, which the
pair passes on as its own needs.

Both kinds must offer the pair their result *before* the output projection: ``forward_heads(x, ctx, cache, out, scale)``
writes the scaled, gated heads into the strided view ``out`` [T, head_width], and ``output_weight`` is the projection
[hidden, head_width]. The pair stacks the two projections along k at load, so that one product over
``[scale_l * heads_l | scale_r * heads_r]`` gives the weighted sum: each scale is applied in fp32 where the heads are
formed, and the two results are added in the product's fp32 sums, never as rounded tensors.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Mixer, mixer_class, position_class, register_mixer
from .linear import linear


class MixerPair(Mixer):
    def __init__(self, params, dtype, device, position=None):
        super().__init__(params, dtype, device, position)
        self.hidden = int(params["hidden_size"])
        self.scales = (float(params.get("left_scale", 1.0)), float(params.get("right_scale", 1.0)))
        self.prefixes = tuple(params.get("prefixes") or ("left.", "right."))
        self.subs = []
        for side in ("left", "right"):
            sp = params[side]
            pos = sp.get("position")
            pos = None if pos is None else position_class(pos["kind"])(pos["params"], dtype, device)
            sub = mixer_class(sp["kind"])(sp["params"], dtype, device, position=pos)
            if not hasattr(sub, "forward_heads") or not hasattr(sub, "head_width"):
                raise ValueError(f"mixer_pair: mixer kind {sp['kind']!r} does not offer its heads before the output projection")
            self.subs.append(sub)
        caches = [s.cache_need() for s in self.subs if s.cache_need() is not None]
        states = [s.state_need() for s in self.subs if s.state_need() is not None]
        if len(caches) > 1 or len(states) > 1:
            raise ValueError("mixer_pair: the two mixers may ask for one paged cache and one state between them")
        self._cache_need = caches[0] if caches else None
        self._state_need = states[0] if states else None
        self.widths = tuple(int(s.head_width) for s in self.subs)
        self.w_o = None

    @property
    def capturable(self):
        return all(s.capturable for s in self.subs)

    def weight_shapes(self):
        return {p + n: shape for p, s in zip(self.prefixes, self.subs) for n, shape in s.weight_shapes().items()}

    def _owner(self, name):
        for p, s in zip(self.prefixes, self.subs):
            if name.startswith(p) and name[len(p):] in s.weight_shapes():
                return s, name[len(p):]
        raise KeyError(name)

    def keeps_dtype(self, name):
        s, n = self._owner(name)
        return s.keeps_dtype(n)

    def norm_like(self, name):
        s, n = self._owner(name)
        return s.norm_like(n)

    def load_weights(self, tensors):
        for p, s in zip(self.prefixes, self.subs):
            s.load_weights({n: tensors[p + n] for n in s.weight_shapes()})
        # one output product for both: [hidden, width_l + width_r], k padded to a multiple of 8 for the kernels' 16-byte rows
        ws = [s.output_weight for s in self.subs]
        k = sum(self.widths)
        self.k_pad = -(-k // 8) * 8
        if self.k_pad > k:
            ws.append(torch.zeros(self.hidden, self.k_pad - k, dtype=ws[0].dtype, device=ws[0].device))
        self.w_o = torch.cat(ws, 1).contiguous()
        for s in self.subs:
            s.output_weight = None                   # the stacked matrix is the one that is used

    def cache_need(self):
        return self._cache_need

    def state_need(self):
        return self._state_need

    def streams_first(self, rows):
        return self.subs[0].streams_first(rows)

    def kernel_files(self, page_size):
        names = set()
        for s in self.subs:
            names.update(s.kernel_files(page_size))
        return tuple(sorted(names))

    def prepare(self, ctx, cache):
        for s in self.subs:
            s.prepare(ctx, cache)

    def forward(self, x, ctx, cache):
        T = x.shape[0]
        heads = ctx.buf("pair_heads", (T, self.k_pad), self.dtype)       # the padding columns stay zero
        at = 0
        for s, w, scale in zip(self.subs, self.widths, self.scales):
            s.forward_heads(x, ctx, cache, heads[:, at:at + w], scale)
            at += w
        out = ctx.buf("pair_delta", (T, self.hidden), self.dtype)     # a buffer of its own: it may live beside a feed-forward's
        linear(heads, self.w_o, out, ctx.status)
        return out


register_mixer("mixer_pair", MixerPair)
