"""The model: embedding, blocks in their run order, final norm and LM head, built from a
``ModelSpec`` with registered parts. It owns no cache and no batch logic: ``forward`` takes
the step's context (token rows, positions, block tables) and the per-layer cache views.

Data flow of the reference's ``forward_batch`` (src/source/model/llama3.cpp:849-1199), except
that the final norm and the LM head run on the wanted rows only (the reference computes
logits for every row of a mixed step and drops the prompt rows, scheduler.cpp:616-621).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..config.base import EmbedderSpec, ModelConfig, ModelSpec
from ..csrc import ops
from ..parts import Block, NormedDelta, SublayerGate, SummedDelta, embedder_class, feed_forward_class, mixer_class, norm_class, position_class
from ..parts.linear import configure_library_gemm, linear
from ..engine import tracing


class Model:
    def __init__(self, config: ModelConfig, dtype: torch.dtype, device):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"compute dtype must be float32 or bfloat16, found {dtype}")
        self.config = config
        self.spec: ModelSpec = config.model_spec()
        self.dtype = dtype
        self.device = torch.device(device)
        configure_library_gemm()
        self.blocks: List[Block] = []
        for ls in self.spec.layers:
            pos = None
            if ls.mixer.position is not None:
                pos = position_class(ls.mixer.position.kind)(ls.mixer.position.params, dtype, self.device)
            mixer = mixer_class(ls.mixer.kind)(ls.mixer.params, dtype, self.device, position=pos)
            ffn = n2 = None
            if ls.feed_forward is not None:
                ffn = feed_forward_class(ls.feed_forward.kind)(ls.feed_forward.params, dtype, self.device)
                if ls.feed_forward_norm is not None:      # None: the feed-forward reads the mixer's norm (an arrangement's choice)
                    n2 = norm_class(ls.feed_forward_norm.kind)(ls.feed_forward_norm.params, dtype, self.device)
            n1 = norm_class(ls.mixer_norm.kind)(ls.mixer_norm.params, dtype, self.device)
            n1b = n2b = None                          # norms behind the sublayers, where the layer has them
            if ls.mixer_post_norm is not None:
                n1b = norm_class(ls.mixer_post_norm.kind)(ls.mixer_post_norm.params, dtype, self.device)
            if ffn is not None and ls.feed_forward_post_norm is not None:
                n2b = norm_class(ls.feed_forward_post_norm.kind)(ls.feed_forward_post_norm.params, dtype, self.device)
            g1 = g2 = None                            # learned gates on the sublayers' results, where the layer has them
            if ls.mixer_gate_name is not None:
                g1 = SublayerGate({"size": self.spec.hidden_size}, dtype, self.device)
            if ffn is not None and ls.feed_forward_gate_name is not None:
                g2 = SublayerGate({"size": self.spec.hidden_size}, dtype, self.device)
            self.blocks.append(Block(mixer, ffn, n1, n2, ls.arrangement, n1b, n2b, g1, g2, ls.residual_scale))
        self.final_norm = norm_class(self.spec.final_norm.kind)(self.spec.final_norm.params, dtype, self.device)
        # the embedder: by default the plain table under the spec's embedding name
        es = self.spec.embedder or EmbedderSpec("table", {})
        self._embed_prefix, _, last = self.spec.embed_name.rpartition(".")
        self._embed_prefix += "." if self._embed_prefix else ""
        eparams = {"vocab_size": self.spec.vocab_size, "hidden_size": self.spec.hidden_size, "name": last}
        eparams.update(es.params)
        self.embedder = embedder_class(es.kind)(eparams, dtype, self.device)
        self.embed: Optional[torch.Tensor] = None
        self.lm_head: Optional[torch.Tensor] = None
        self._layer_hook = None
        # what the stream gains between layers: place of the run order -> spec; the vectors come with the weights
        self.stream_adds = {a.place: a for a in self.spec.stream_adds}
        self.stream_vectors: Dict[str, torch.Tensor] = {}
        self._keeps_embedding = any(a.embedding for a in self.spec.stream_adds)
        for a in self.spec.stream_adds:
            if not 0 <= a.place < len(self.spec.order):
                raise ValueError(f"a stream addition names place {a.place} of a run order of {len(self.spec.order)}")
        for i in self.spec.order:
            if not 0 <= i < len(self.blocks):
                raise ValueError(f"run order names layer {i}, but the model has {len(self.blocks)} layers")

    # ---- weights -------------------------------------------------------------------
    def _named_parts(self):
        for ls, b in zip(self.spec.layers, self.blocks):
            p = ls.weight_prefix
            yield p + ls.mixer_prefix, b.mixer
            yield p + ls.mixer_norm_name, b.mixer_norm
            if b.mixer_post_norm is not None:
                yield p + ls.mixer_post_norm_name, b.mixer_post_norm
            if b.mixer_gate is not None:
                yield p + ls.mixer_gate_name, b.mixer_gate
            if b.feed_forward_gate is not None:
                yield p + ls.feed_forward_gate_name, b.feed_forward_gate
            if b.feed_forward is not None:
                yield p + ls.feed_forward_prefix, b.feed_forward
                if b.feed_forward_norm is not None:
                    yield p + ls.feed_forward_norm_name, b.feed_forward_norm
                if b.feed_forward_post_norm is not None:
                    yield p + ls.feed_forward_post_norm_name, b.feed_forward_post_norm
        yield self.spec.final_norm_name, self.final_norm
        yield self._embed_prefix, self.embedder

    def weight_shapes(self) -> Dict[str, Tuple[int, ...]]:
        """Every checkpoint tensor the model wants: full name -> shape."""
        shapes = {}
        if not self.spec.tie_word_embeddings:
            shapes[self.spec.lm_head_name] = (self.spec.vocab_size, self.spec.hidden_size)
        for prefix, part in self._named_parts():
            for n, s in part.weight_shapes().items():
                shapes[prefix + n] = tuple(s)
        for n, s in (self.spec.stream_vector_shapes or {}).items():
            shapes[n] = tuple(s)
        return shapes

    def optional_weights(self) -> List[str]:
        """Tensors that may be in a checkpoint without being used (a stored head of a tied model)."""
        return [self.spec.lm_head_name] if self.spec.tie_word_embeddings else []

    def keeps_dtype(self, name: str) -> bool:
        if name in (self.spec.stream_vector_shapes or {}):
            return True
        for prefix, part in self._named_parts():
            if name.startswith(prefix) and name[len(prefix):] in part.weight_shapes():
                return part.keeps_dtype(name[len(prefix):])
        return False

    def norm_like(self, name: str) -> bool:
        """True for tensors that random weights draw around one (norm weights), as far as the owning part says
        (``Part.norm_like``; by default the vectors that keep their dtype)."""
        for prefix, part in self._named_parts():
            if name.startswith(prefix) and name[len(prefix):] in part.weight_shapes():
                return part.norm_like(name[len(prefix):])
        return False

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        """``tensors`` holds every name of ``weight_shapes`` on the device, matrices in the
        compute dtype."""
        for prefix, part in self._named_parts():
            part.load_weights({n: tensors[prefix + n] for n in part.weight_shapes()})
        self.stream_vectors = {n: tensors[n].float().contiguous() for n in (self.spec.stream_vector_shapes or {})}
        self.embed = self.embedder.table
        self.lm_head = self.embed if self.spec.tie_word_embeddings else tensors[self.spec.lm_head_name].contiguous()

    def kernel_files(self, page_size: int) -> List[str]:
        """CUDA sources of the model's own kernels and of its parts (see ``Part.kernel_files``)."""
        names = {"sampling"} | ({"gemm_f32"} if self.dtype == torch.float32 else {"gemm_skinny", "gemm_rows", "gemm_tc05"})
        if self.spec.logit_softcap > 0:
            names.add("activation")
        for _, part in self._named_parts():
            names.update(part.kernel_files(page_size))
        return sorted(names)

    def capturable(self) -> bool:
        """True if every part's ``forward`` may be captured into a CUDA graph (see ``Part.capturable``)."""
        return all(part.capturable for _, part in self._named_parts()) and all(b.capturable for b in self.blocks)

    def hook_layers(self, fn) -> None:
        """``fn(run, resid)`` is called after every layer run with the fp32 residual stream as it then stands, the
        run's own pending delta added (tests compare layer by layer through this); None takes the hook off."""
        self._layer_hook = fn

    # ---- cache and state --------------------------------------------------------------
    def cache_places(self):
        """What the cache layout is made of: (cache needs, state needs) per place. The places are the run order's,
        then one for the embedder (it keeps no pages, but may keep state per request)."""
        mixers = [self.blocks[i].mixer for i in self.spec.order]
        return ([m.cache_need() for m in mixers] + [None],
                [m.state_need() for m in mixers] + [self.embedder.state_need()])

    # ---- forward -------------------------------------------------------------------
    def prepare(self, ctx, caches) -> None:
        """Host-side planning of the parts for this step (work lists, uploads); runs before
        ``forward`` and also before a captured step is replayed."""
        for o, i in enumerate(self.spec.order):
            self.blocks[i].mixer.prepare(ctx, caches[o])

    def forward(self, ctx, caches) -> Optional[torch.Tensor]:
        """Run the step's rows through all layers; returns fp32 logits [R, vocab] for
        ``ctx.logit_rows`` or None when no row is wanted. ``caches[o]`` is the view of the o-th
        place in the run order (a layer that runs twice has a cache per run)."""
        T, d = ctx.num_tokens, self.spec.hidden_size
        resid = ctx.buf("resid", (T, d), torch.float32)
        self.embedder.forward(ctx, resid, caches[len(self.spec.order)].state)
        embed_out = None
        if self._keeps_embedding:
            embed_out = ctx.buf("embed_out", (T, d), torch.float32)
            embed_out.copy_(resid)
        delta = None
        for o, i in enumerate(self.spec.order):
            add = self.stream_adds.get(o)
            if add is not None:                       # the pending delta goes in with what the stream gains here
                vec = self.stream_vectors[add.vector_name][add.row] if add.vector_name is not None else None
                self._stream_add(resid, delta, embed_out if add.embedding else None, vec)
                delta = None
            if tracing.ENABLED:
                with tracing.span(f"layer {i}"):
                    delta = self.blocks[i].forward(resid, delta, ctx, caches[o])
            else:
                delta = self.blocks[i].forward(resid, delta, ctx, caches[o])
            if self._layer_hook is not None:
                self._layer_hook(o, resid if delta is None else resid + (
                    delta.value() if isinstance(delta, (NormedDelta, SummedDelta)) else delta.float()))
        R = ctx.num_logit_rows
        if R == 0:
            return None
        x = ctx.buf("final_x", (R, d), self.dtype)
        self.final_norm.forward(resid, delta, x, rows=ctx.logit_rows)
        logits = ctx.buf("logits", (R, self.spec.vocab_size), torch.float32)
        linear(x, self.lm_head, logits, ctx.status)
        if self.spec.logit_softcap > 0:
            ops.softcap(logits, self.spec.logit_softcap)
        return logits

    @staticmethod
    def _stream_add(resid, delta, extra, vec) -> None:
        """``resid += delta (+ extra) (+ vec)`` in one launch; ``delta`` may be None, a tensor or a ``NormedDelta``."""
        if isinstance(delta, SummedDelta):
            ops.add_norm(resid, delta.a)
            ops.add_norm(resid, delta.b, extra=extra, vec=vec)
        elif isinstance(delta, NormedDelta):
            ops.add_norm(resid, delta.x, delta_weight=delta.norm.weight, delta_eps=delta.norm.eps, delta_bias=delta.bias,
                         extra=extra, vec=vec)
        elif delta is not None or extra is not None or vec is not None:
            ops.add_norm(resid, delta, extra=extra, vec=vec)
