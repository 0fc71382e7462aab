"""Vibunex: a decoder whose config.json lists its layers one by one. Every layer runs two sublayers on the same stream,
each behind a norm with a single learned number as weight and each passed through a learned gate before the two join the
stream together. The first sublayer is a pair of mixers side by side, attention whose softmax weights are mixed over the
heads (norm over the whole query and key projections, partial rotation with YaRN scaling, a sink, an output gate) and
time mixing with a decaying matrix state; the second is a routed feed-forward with a shared expert.

config.json:
    architecture    "Vibunex"
    vocab, width    sizes of the embedding and of the residual stream
    norm.eps        of every RMS norm
    residual_mult   what a layer adds to the stream is multiplied by it
    layers[i]       {type: "parallel", mixer{left{...}, right{...}, left_scale, right_scale}, mlp{...} | null}
      mixer.left    {heads, kv_heads, dim, vdim, scale, rot{base, dims, scaling{factor, original, fast, slow} | null} | null}
      mixer.right   {heads, dim} (and ``rank``, the decay's low rank, where no checkpoint is there to say it)
      mlp           {kind: "moe", expert{ff}, router{experts, top, scale}, shared{ff} | null}
Tensors: embed, l<i>.norm1, l<i>.norm2, l<i>.rg1[.b], l<i>.rg2[.b], l<i>.mix.left.*, l<i>.mix.right.*, l<i>.mlp.*,
final.norm, head.

Everything is expressed with registered parts: the model below is a ``ModelSpec`` and nothing else.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from ..config.base import (ConfigError, FeedForwardSpec, LayerSpec, MixerSpec, ModelConfig, ModelSpec, NormSpec, read_key,
                           register_architecture)


def _sub(d: Dict[str, Any], key: str, where: str, optional: bool = False) -> Optional[Dict[str, Any]]:
    v = d.get(key)
    if v is None and optional:
        return None
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: {where}{key!r} must be an object")
    return v


def _keyed(fn, where: str):
    try:
        return fn()
    except ConfigError as e:
        raise ConfigError(str(e).replace("key ", f"key {where}", 1)) from None


@dataclass(frozen=True)
class VibunexConfig(ModelConfig):
    vocab: int
    width: int
    eps: float
    residual_mult: float
    layers: Tuple[Dict[str, Any], ...]              # as in config.json, checked

    architecture = "Vibunex"

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "VibunexConfig":
        vocab = read_key(d, "vocab", int, positive=True)
        width = read_key(d, "width", int, positive=True)
        eps = _keyed(lambda: read_key(_sub(d, "norm", ""), "eps", float, positive=True), "norm.")
        mult = read_key(d, "residual_mult", float, 1.0)
        raw = d.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: key 'layers' must be a non-empty list")
        layers: List[Dict[str, Any]] = []
        for i, ent in enumerate(raw):
            where = f"layers[{i}]."
            if not isinstance(ent, dict):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            kind = read_key(ent, "type", str)
            if kind != "parallel":
                raise ConfigError(f"config.json: {where}type {kind!r} is not supported (supported: 'parallel')")
            mx = _sub(ent, "mixer", where)
            for side in ("left_scale", "right_scale"):
                _keyed(lambda: read_key(mx, side, float, 1.0), where + "mixer.")
            left = _sub(mx, "left", where + "mixer.")
            for key, typ in (("heads", int), ("kv_heads", int), ("dim", int), ("vdim", int), ("scale", float)):
                _keyed(lambda: read_key(left, key, typ, positive=True), where + "mixer.left.")
            if left["heads"] % left["kv_heads"]:
                raise ConfigError(f"config.json: {where}mixer.left.heads is not a multiple of kv_heads")
            rot = _sub(left, "rot", where + "mixer.left.", optional=True)
            if rot is not None:
                _keyed(lambda: read_key(rot, "base", float, positive=True), where + "mixer.left.rot.")
                dims = _keyed(lambda: read_key(rot, "dims", int), where + "mixer.left.rot.")
                if dims < 0 or dims % 2 or dims > left["dim"]:
                    raise ConfigError(f"config.json: {where}mixer.left.rot.dims must be even and at most dim")
                sc = _sub(rot, "scaling", where + "mixer.left.rot.", optional=True)
                if sc is not None:
                    for key in ("factor", "original", "fast", "slow"):
                        _keyed(lambda: read_key(sc, key, float, positive=True), where + "mixer.left.rot.scaling.")
            right = _sub(mx, "right", where + "mixer.")
            for key in ("heads", "dim"):
                _keyed(lambda: read_key(right, key, int, positive=True), where + "mixer.right.")
            _keyed(lambda: read_key(right, "rank", int, 1, positive=True), where + "mixer.right.")
            mlp = ent.get("mlp")
            if mlp is not None:
                mlp = _sub(ent, "mlp", where)
                if _keyed(lambda: read_key(mlp, "kind", str), where + "mlp.") != "moe":
                    raise ConfigError(f"config.json: {where}mlp.kind {mlp['kind']!r} is not supported (supported: 'moe')")
                _keyed(lambda: read_key(_sub(mlp, "expert", where + "mlp."), "ff", int, positive=True), where + "mlp.expert.")
                router = _sub(mlp, "router", where + "mlp.")
                experts = _keyed(lambda: read_key(router, "experts", int, positive=True), where + "mlp.router.")
                top = _keyed(lambda: read_key(router, "top", int, positive=True), where + "mlp.router.")
                _keyed(lambda: read_key(router, "scale", float, 1.0), where + "mlp.router.")
                if top > experts:
                    raise ConfigError(f"config.json: {where}mlp.router.top exceeds experts")
                shared = _sub(mlp, "shared", where + "mlp.", optional=True)
                if shared is not None:
                    _keyed(lambda: read_key(shared, "ff", int, positive=True), where + "mlp.shared.")
            layers.append(copy.deepcopy(ent))
        return cls(vocab=vocab, width=width, eps=eps, residual_mult=mult, layers=tuple(layers))

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
                "residual_mult": self.residual_mult, "layers": copy.deepcopy(list(self.layers))}

    def eos_token_ids(self) -> List[int]:
        return []

    # ---- the model as data ---------------------------------------------------------------------
    def _mixer(self, mx: Dict[str, Any]) -> MixerSpec:
        left, right = mx["left"], mx["right"]
        rot = left.get("rot")
        position = None
        if rot is not None and rot["dims"] > 0:
            sc = rot.get("scaling")
            scaling = None if sc is None else {"rope_type": "yarn", "factor": float(sc["factor"]), "original": float(sc["original"]),
                                               "fast": float(sc["fast"]), "slow": float(sc["slow"])}
            position = {"kind": "rotary", "params": {"head_dim": left["dim"], "rot_dim": rot["dims"], "theta": float(rot["base"]),
                                                     "scaling": scaling}}
        return MixerSpec("mixer_pair", {
            "hidden_size": self.width, "left_scale": float(mx.get("left_scale", 1.0)), "right_scale": float(mx.get("right_scale", 1.0)),
            "left": {"kind": "talking_attention", "position": position, "params": {
                "hidden_size": self.width, "num_heads": left["heads"], "num_kv_heads": left["kv_heads"], "head_dim": left["dim"],
                "value_dim": left["vdim"], "scale": float(left["scale"]), "eps": self.eps}},
            "right": {"kind": "time_mix", "position": None, "params": {
                "hidden_size": self.width, "num_heads": right["heads"], "head_dim": right["dim"], "eps": self.eps,
                "decay_rank": right.get("rank")}}})

    def model_spec(self) -> ModelSpec:
        norm = NormSpec("rmsnorm", {"size": self.width, "eps": self.eps, "weight_name": "", "scalar": True})
        specs: List[LayerSpec] = []
        for i, ent in enumerate(self.layers):
            mlp = ent.get("mlp")
            ffn = None
            if mlp is not None:
                shared = mlp.get("shared")
                ffn = FeedForwardSpec("routed_mlp", {
                    "hidden_size": self.width, "intermediate_size": mlp["expert"]["ff"], "experts": mlp["router"]["experts"],
                    "top": mlp["router"]["top"], "scale": float(mlp["router"].get("scale", 1.0)), "scores": "sigmoid",
                    "renorm": False, "activation": "relu2",
                    "shared": None if shared is None else {"intermediate_size": shared["ff"]}, "shared_gate": True})
            specs.append(LayerSpec(
                mixer=self._mixer(ent["mixer"]), feed_forward=ffn, mixer_norm=norm,
                feed_forward_norm=None if ffn is None else norm, weight_prefix=f"l{i}.", arrangement="parallel_gated",
                mixer_prefix="mix.", feed_forward_prefix="mlp.", mixer_norm_name="norm1", feed_forward_norm_name="norm2",
                mixer_gate_name="rg1", feed_forward_gate_name=None if ffn is None else "rg2",
                residual_scale=self.residual_mult))
        return ModelSpec(hidden_size=self.width, vocab_size=self.vocab, layers=specs, order=list(range(len(specs))),
                         final_norm=norm, tie_word_embeddings=False, embed_name="embed", final_norm_name="final.norm",
                         lm_head_name="head", max_position=0)


register_architecture(VibunexConfig.architecture, VibunexConfig)
