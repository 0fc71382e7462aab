"""Small Vibunex configurations for the tests and a writer of model folders whose weights make every mechanism count:
query and key norm weights large enough for peaked attention, sinks of the size of a typical largest score, a head-mixing
matrix with negative entries away from the identity, decays that keep the matrix state for hundreds of tokens, a bonus
of order one, routers whose scores lie well apart, gates on both sides of one half. The sizes differ from layer to layer
and avoid coincidences (key size != value size, kv_heads != 1 and != heads, rotated part smaller than the key, a layer
without scaling of the rotation and one without rotation, top == 1 and top == experts, a layer without feed-forward and
one without shared expert, a decay rank that is no multiple of 8, scales that are not one).
"""
import json
import math
import os

import numpy as np
import torch


def _left(heads, kv, dim, vdim, rot_dims, base=10000.0, scale=None, scaling="yarn"):
    rot = None
    if rot_dims is not None:
        rot = {"base": base, "dims": rot_dims}
        if scaling == "yarn":
            rot["scaling"] = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}
        elif scaling is not None:
            rot["scaling"] = scaling
    d = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5}
    if rot is not None:
        d["rot"] = rot
    return d


def _moe(ff, experts, top, scale=1.0, shared=None):
    d = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale}}
    if shared is not None:
        d["shared"] = {"ff": shared}
    return d


def _layer(left, right, mlp=None, left_scale=1.0, right_scale=1.0, rank=8):
    """``rank`` (the decay's low rank) is not part of config.json: the checkpoint's shapes give it. It rides along here
    for the weight writer and is taken out before the file is written."""
    return {"type": "parallel", "mixer": {"left": left, "right": {"heads": right[0], "dim": right[1]}, "left_scale": left_scale,
                                          "right_scale": right_scale}, "mlp": mlp, "_rank": rank}


def _model(vocab, width, eps, layers, mult=1.0):
    return {"architecture": "Vibunex", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult,
            "layers": layers}


def clean(cfg):
    """The configuration as config.json holds it (without the writer's own keys)."""
    out = json.loads(json.dumps(cfg))
    for layer in out["layers"]:
        layer.pop("_rank", None)
    return out


# one mechanism each between embedding and head: the other mixer's scale is zero, no feed-forward
ONLY_LEFT = _model(200, 64, 1e-5, [_layer(_left(6, 2, 16, 24, 8), (2, 8), left_scale=1.3, right_scale=0.0, rank=4)])
ONLY_RIGHT = _model(200, 64, 1e-5, [_layer(_left(2, 1, 8, 8, None), (4, 12), left_scale=0.0, right_scale=0.8, rank=5)], mult=1.5)
ONLY_MLP = _model(200, 64, 1e-6, [_layer(_left(2, 1, 8, 8, 8, scaling=None), (2, 8), _moe(40, 7, 3, 1.7, shared=24),
                                         left_scale=0.05, right_scale=0.05)], mult=2.0)

# all of it, every layer different
MIXED_A = _model(331, 96, 1e-5, [
    _layer(_left(4, 2, 24, 16, 12, base=50000.0), (3, 16), _moe(48, 6, 2, 2.5, shared=72), 1.15, 0.45, rank=6),
    _layer(_left(3, 3, 16, 32, 16, scale=0.3, scaling=None), (4, 24), None, 0.7, 1.1, rank=16),
    _layer(_left(6, 1, 8, 16, 4, scaling={"factor": 8.0, "original": 32, "fast": 4.0, "slow": 2.0}), (2, 40),
           _moe(32, 5, 5, 0.6), 1.0, 1.0, rank=3),
    _layer(_left(2, 2, 32, 8, None), (6, 8), _moe(64, 9, 1, 1.0, shared=16), 0.9, 1.4, rank=8),
], mult=0.65)
# sizes in multiples of 16 (what tensor-core kernels take), more heads, wider
MIXED_B = _model(500, 256, 2e-6, [
    _layer(_left(8, 2, 64, 32, 32, base=250.0), (4, 64), _moe(128, 8, 2, 1.0, shared=128), 1.0, 0.6, rank=32),
    _layer(_left(4, 4, 32, 64, 32), (8, 32), _moe(64, 16, 4, 2.0, shared=192), 1.1, 0.9, rank=16),
    _layer(_left(8, 1, 48, 80, 16, scale=0.2), (2, 128), None, 0.8, 1.0, rank=24),
    _layer(_left(16, 4, 16, 16, 16, scaling=None), (16, 16), _moe(256, 4, 3, 1.5), 1.3, 0.4, rank=8),
], mult=0.9)
# sizes that are multiples of nothing useful
ODD = _model(97, 70, 3e-5, [
    _layer(_left(3, 1, 10, 14, 6, base=77.0), (5, 6), _moe(18, 3, 2, 1.1, shared=10), 1.0, 1.0, rank=1),
    _layer(_left(5, 5, 20, 12, 20), (2, 7), None, 0.6, 1.7, rank=7),
    _layer(_left(6, 3, 6, 22, 2), (7, 10), _moe(26, 11, 4, 3.0, shared=50), 1.5, 0.3, rank=9),
], mult=1.2)
CONFIGS = {"odd": ODD, "left": ONLY_LEFT, "right": ONLY_RIGHT, "mlp": ONLY_MLP, "mixed_a": MIXED_A, "mixed_b": MIXED_B}
PAGE_SIZE = {"odd": 4, "left": 8, "right": 16, "mlp": 4, "mixed_a": 8, "mixed_b": 16}


def _tensors(cfg, seed):
    """{name: float32 array}, from a numpy generator; rounded to bfloat16 when written."""
    rng = np.random.default_rng(seed)
    W = cfg["width"]
    out = {}

    def lin(name, n_out, n_in, gain=1.0):
        out[name] = (rng.standard_normal((n_out, n_in)) * gain / math.sqrt(n_in)).astype(np.float32)

    def vec(name, n, mean=0.0, std=1.0):
        out[name] = (mean + std * rng.standard_normal(n)).astype(np.float32)

    def one(name, mean, std):
        out[name] = np.asarray(mean + std * rng.standard_normal(), dtype=np.float32)

    out["embed"] = rng.standard_normal((cfg["vocab"], W)).astype(np.float32)
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        one(p + "norm1", 1.0, 0.15)
        lin(p + "rg1", W, W, 2.0)
        vec(p + "rg1.b", W, 0.5, 1.0)
        a, b = layer["mixer"]["left"], layer["mixer"]["right"]
        H, G, dk, dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
        q = p + "mix.left."
        lin(q + "q", H * dk, W); lin(q + "k", G * dk, W); lin(q + "v", G * dv, W)
        # normed queries and keys have entries of order (norm weight): scores of standard deviation about 2.5
        g = (2.5 / (a["scale"] * math.sqrt(dk))) ** 0.5
        vec(q + "q.norm", H * dk, g, 0.2 * g); vec(q + "k.norm", G * dk, g, 0.2 * g)
        out[q + "talk"] = (np.eye(H) * 0.8 + 0.35 * rng.standard_normal((H, H))).astype(np.float32)
        vec(q + "sink", H, 2.0, 1.5)
        lin(q + "g", H * dv, W, 2.0)
        lin(q + "o", W, H * dv)
        r = p + "mix.right."
        Hr, n, L = b["heads"], b["dim"], layer["_rank"]
        C = Hr * n
        for s in "rkvgw":
            out[r + "mu." + s] = rng.uniform(0.0, 1.0, W).astype(np.float32)
        lin(r + "r", C, W); lin(r + "k", C, W); lin(r + "v", C, W); lin(r + "g", C, W, 2.0)
        lin(r + "w1", L, W, 1.5); lin(r + "w2", C, L, 1.0)
        out[r + "w0"] = rng.uniform(-6.0, -1.0, C).astype(np.float32)          # decays of 0.69 to 0.9975 a token
        out[r + "u"] = (0.7 * rng.standard_normal((Hr, n))).astype(np.float32)
        vec(r + "norm", C, 1.0, 0.2)
        lin(r + "o", W, C)
        mlp = layer.get("mlp")
        if mlp is not None:
            one(p + "norm2", 1.0, 0.15)
            lin(p + "rg2", W, W, 2.0)
            vec(p + "rg2.b", W, -0.3, 1.0)
            m = p + "mlp."
            F, E = mlp["expert"]["ff"], mlp["router"]["experts"]
            lin(m + "router", E, W, 3.0)
            for e in range(E):
                lin(m + f"e{e}.up", F, W, 1.4); lin(m + f"e{e}.down", W, F)
            if mlp.get("shared"):
                lin(m + "shared.up", mlp["shared"]["ff"], W, 1.4); lin(m + "shared.down", W, mlp["shared"]["ff"])
                lin(m + "shared.sg", 1, W, 2.0)
    one("final.norm", 1.0, 0.1)
    lin("head", cfg["vocab"], W, 3.0)
    return out


def write_folder(folder, cfg, seed, change=None):
    """A model folder with the weights above in bfloat16. ``change(tensors)`` may edit the float32 arrays first (a test
    that builds a key which stands out, say)."""
    from llm_steadyinfer_b200.weights import write_safetensors
    os.makedirs(folder, exist_ok=True)
    arrays = _tensors(cfg, seed)
    if change is not None:
        change(arrays)
    tensors = {n: torch.tensor(a).to(torch.bfloat16) for n, a in arrays.items()}
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors, metadata={"format": "pt"})
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
        json.dump(clean(cfg), f, indent=1)
    return folder
