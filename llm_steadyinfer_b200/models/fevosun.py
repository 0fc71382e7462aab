"""Fevosun: a decoder whose config.json lists its layers one by one. Every layer has one norm (its weight stored around
zero) whose output feeds a mixer and a feed-forward side by side; both results join the stream together. Three mixers:
grouped-query attention whose values are its keys (no rotation; a query temperature by position, a penalty in proportion
to the distance with a slope per head, a window, an output gate), and latent attention in two forms (queries straight
from the input, rotate-half pairs and YaRN scaling; queries through a latent, interleaved pairs), both with a window. The
feed-forward is dense (silu gate) or routed: softmax scores over all router rows, a correction added for the choice only,
experts with limited gate and up sums, identity experts that return their input, a shared expert.

config.json:
    architecture     "Fevosun"
    vocab, width     sizes of the embedding and of the residual stream
    norm.eps         of every RMS norm
    embedding.scale  what the embedding is multiplied by
    layers[i]        {type, mixer{...}, mlp{...} | null}
      type "attention":           mixer {heads, kv_heads, dim, vdim, scale, mask{size}, q_temp{coef, every}}
      type "latent_attention":    mixer {heads, dim, rot_dim, vdim, kv_rank, scale, mask{size},
                                         rot{base, dims, scaling{factor, original, fast, slow}}}
      type "latent_attention_2":  mixer {heads, dim, rot_dim, vdim, kv_rank, [q_rank,] scale, mask{size}, rot{base, dims}}
      mlp {kind: "dense", ff}  or  {kind: "moe", expert{ff, limit}, router{experts, identity, top}, shared{ff, limit} | null}
Tensors: embed, l<i>.norm1, l<i>.mix.*, l<i>.mlp.*, final.norm, head.

Everything is expressed with registered parts: the model below is a ``ModelSpec`` and nothing else.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from ..config.base import (ConfigError, EmbedderSpec, FeedForwardSpec, LayerSpec, MixerSpec, ModelConfig, ModelSpec, NormSpec,
                           read_key, register_architecture)

# constants of the design
SLOPE_BASE, SLOPE_EXPONENT = 2.0, -8.0        # slope of head h: 2^(-8 (h + 1) / heads)
EXPERT_ALPHA = 1.702                          # g * sigmoid(alpha g)

MIXER_KEYS = {
    "attention": (("heads", int), ("kv_heads", int), ("dim", int), ("vdim", int), ("scale", float)),
    "latent_attention": (("heads", int), ("dim", int), ("rot_dim", int), ("vdim", int), ("kv_rank", int), ("scale", float)),
    "latent_attention_2": (("heads", int), ("dim", int), ("rot_dim", int), ("vdim", int), ("kv_rank", int), ("scale", float)),
}


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
class FevosunConfig(ModelConfig):
    vocab: int
    width: int
    eps: float
    embed_scale: float
    layers: Tuple[Dict[str, Any], ...]              # as in config.json, checked

    architecture = "Fevosun"

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "FevosunConfig":
        vocab = read_key(d, "vocab", int, positive=True)
        width = read_key(d, "width", int, positive=True)
        eps = _keyed(lambda: read_key(_sub(d, "norm", ""), "eps", float, positive=True), "norm.")
        emb = _sub(d, "embedding", "", optional=True)
        embed_scale = 1.0 if emb is None else _keyed(lambda: read_key(emb, "scale", float, 1.0), "embedding.")
        raw = d.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: key 'layers' must be a non-empty list")
        layers: List[Dict[str, Any]] = []
        for i, ent in enumerate(raw):
            where = f"layers[{i}]."
            if not isinstance(ent, dict):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            kind = read_key(ent, "type", str)
            if kind not in MIXER_KEYS:
                raise ConfigError(f"config.json: {where}type {kind!r} is not one of {sorted(MIXER_KEYS)}")
            mx = _sub(ent, "mixer", where)
            for key, typ in MIXER_KEYS[kind]:
                _keyed(lambda: read_key(mx, key, typ, positive=True), where + "mixer.")
            mask = _sub(mx, "mask", where + "mixer.", optional=True)
            if mask is not None:
                _keyed(lambda: read_key(mask, "size", int, positive=True), where + "mixer.mask.")
            if kind == "attention":
                if mx["heads"] % mx["kv_heads"]:
                    raise ConfigError(f"config.json: {where}mixer.heads is not a multiple of kv_heads")
                if mx["vdim"] > mx["dim"]:
                    raise ConfigError(f"config.json: {where}mixer.vdim exceeds dim, but the values are the keys")
                qt = _sub(mx, "q_temp", where + "mixer.", optional=True)
                if qt is not None:
                    _keyed(lambda: read_key(qt, "coef", float), where + "mixer.q_temp.")
                    if isinstance(qt.get("every"), float) and qt["every"].is_integer():
                        qt["every"] = int(qt["every"])              # a whole number written with a point
                    _keyed(lambda: read_key(qt, "every", int, positive=True), where + "mixer.q_temp.")
            else:
                rot = _sub(mx, "rot", where + "mixer.")
                _keyed(lambda: read_key(rot, "base", float, positive=True), where + "mixer.rot.")
                dims = _keyed(lambda: read_key(rot, "dims", int), where + "mixer.rot.")
                if dims < 0 or dims % 2 or dims > mx["rot_dim"]:
                    raise ConfigError(f"config.json: {where}mixer.rot.dims must be even and at most rot_dim")
                sc = _sub(rot, "scaling", where + "mixer.rot.", optional=True)
                if sc is not None:
                    for key in ("factor", "original", "fast", "slow"):
                        _keyed(lambda: read_key(sc, key, float, positive=True), where + "mixer.rot.scaling.")
                if kind == "latent_attention_2" and mx.get("q_rank") is not None:
                    _keyed(lambda: read_key(mx, "q_rank", int, positive=True), where + "mixer.")
            mlp = ent.get("mlp")
            if mlp is not None:
                mlp = _sub(ent, "mlp", where)
                mk = _keyed(lambda: read_key(mlp, "kind", str), where + "mlp.")
                if mk == "dense":
                    _keyed(lambda: read_key(mlp, "ff", int, positive=True), where + "mlp.")
                elif mk == "moe":
                    ex = _sub(mlp, "expert", where + "mlp.")
                    _keyed(lambda: read_key(ex, "ff", int, positive=True), where + "mlp.expert.")
                    _keyed(lambda: read_key(ex, "limit", float, positive=True), where + "mlp.expert.")
                    router = _sub(mlp, "router", where + "mlp.")
                    experts = _keyed(lambda: read_key(router, "experts", int, positive=True), where + "mlp.router.")
                    top = _keyed(lambda: read_key(router, "top", int, positive=True), where + "mlp.router.")
                    ident = _keyed(lambda: read_key(router, "identity", int, 0), where + "mlp.router.")
                    if ident < 0 or top > experts + ident:
                        raise ConfigError(f"config.json: {where}mlp.router: identity must not be negative and top at most experts + identity")
                    shared = _sub(mlp, "shared", where + "mlp.", optional=True)
                    if shared is not None:
                        _keyed(lambda: read_key(shared, "ff", int, positive=True), where + "mlp.shared.")
                        _keyed(lambda: read_key(shared, "limit", float, positive=True), where + "mlp.shared.")
                else:
                    raise ConfigError(f"config.json: {where}mlp.kind {mk!r} is not supported (supported: 'dense', 'moe')")
            layers.append(copy.deepcopy(ent))
        return cls(vocab=vocab, width=width, eps=eps, embed_scale=embed_scale, layers=tuple(layers))

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
                "embedding": {"scale": self.embed_scale}, "layers": copy.deepcopy(list(self.layers))}

    def eos_token_ids(self) -> List[int]:
        return []

    # ---- the model as data ---------------------------------------------------------------------
    def _mixer(self, kind: str, mx: Dict[str, Any]) -> MixerSpec:
        window = (mx.get("mask") or {}).get("size")
        if kind == "attention":
            qt = mx.get("q_temp")
            return MixerSpec("attention", {
                "hidden_size": self.width, "num_heads": mx["heads"], "num_kv_heads": mx["kv_heads"], "head_dim": mx["dim"],
                "value_dim": mx["vdim"], "scale": float(mx["scale"]), "window": window, "values_are_keys": True,
                "distance_slopes": {"base": SLOPE_BASE, "exponent": SLOPE_EXPONENT},
                "query_temperature": None if qt is None else {"coef": float(qt["coef"]), "every": int(qt["every"])},
                "output_gate": "g", "names": {"q": "q", "k": "k", "o": "o"}})
        rot = mx["rot"]
        sc = rot.get("scaling")
        scaling = None if sc is None else {"rope_type": "yarn", "factor": float(sc["factor"]), "original": float(sc["original"]),
                                           "fast": float(sc["fast"]), "slow": float(sc["slow"])}
        second = kind == "latent_attention_2"
        return MixerSpec("latent_attention", {
            "hidden_size": self.width, "num_heads": mx["heads"], "head_dim": mx["dim"], "rot_dim": mx["rot_dim"],
            "value_dim": mx["vdim"], "kv_rank": mx["kv_rank"], "scale": float(mx["scale"]), "eps": self.eps, "sink": False,
            "window": window, "rot_base": float(rot["base"]), "rot_dims": rot["dims"], "rot_scaling": scaling,
            "rot_interleaved": second,
            # the second form's queries go through a latent whose size the stored tensors give where the configuration does not
            "q_rank": (mx.get("q_rank") or "checkpoint") if second else None})

    def _feed_forward(self, mlp: Optional[Dict[str, Any]]) -> Optional[FeedForwardSpec]:
        if mlp is None:
            return None
        if mlp["kind"] == "dense":
            return FeedForwardSpec("gated_mlp", {"hidden_size": self.width, "intermediate_size": mlp["ff"],
                                                 "names": {"gate": "gate", "up": "up", "down": "down"}})
        shared = mlp.get("shared")
        router = mlp["router"]
        return FeedForwardSpec("routed_mlp", {
            "hidden_size": self.width, "intermediate_size": mlp["expert"]["ff"], "experts": router["experts"],
            "identity": int(router.get("identity") or 0), "top": router["top"], "scale": 1.0, "scores": "softmax", "renorm": False,
            "choice_bias": "correction", "activation": "glu_limited", "limit": float(mlp["expert"]["limit"]), "alpha": EXPERT_ALPHA,
            "shared": None if shared is None else {"kind": "gated_mlp_limited", "params": {
                "hidden_size": self.width, "intermediate_size": shared["ff"], "limit": float(shared["limit"]), "alpha": EXPERT_ALPHA,
                "biases": False, "names": {"gate": "shared.gate", "up": "shared.up", "down": "shared.down"}}},
            "shared_gate": False})

    def model_spec(self) -> ModelSpec:
        norm = NormSpec("rmsnorm", {"size": self.width, "eps": self.eps, "weight_name": "", "offset": 1.0})
        specs: List[LayerSpec] = []
        for i, ent in enumerate(self.layers):
            ffn = self._feed_forward(ent.get("mlp"))
            specs.append(LayerSpec(
                mixer=self._mixer(ent["type"], ent["mixer"]), feed_forward=ffn, mixer_norm=norm,
                feed_forward_norm=None, weight_prefix=f"l{i}.", arrangement="parallel", mixer_prefix="mix.",
                feed_forward_prefix="mlp.", mixer_norm_name="norm1"))
        return ModelSpec(hidden_size=self.width, vocab_size=self.vocab, layers=specs, order=list(range(len(specs))),
                         final_norm=norm, tie_word_embeddings=False, embed_name="embed", final_norm_name="final.norm",
                         lm_head_name="head", max_position=0, embedder=EmbedderSpec("table", {"scale": self.embed_scale}))


register_architecture(FevosunConfig.architecture, FevosunConfig)
