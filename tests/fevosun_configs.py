"""Small Fevosun configurations for the tests and a writer of model folders whose weights make every mechanism count:
query and key matrices large enough for peaked attention, windows of a few dozen tokens so that every prompt crosses
their edges, query temperatures that change every few tokens, routers whose scores lie apart with corrections large
enough to change the choice, limits that cut a good part of the gate and up sums, gates on both sides of one half, norm
vectors around zero. The sizes differ from layer to layer and avoid coincidences (value size != key size in the latent
layers, kv_heads != 1 and != heads, top == 1 and top == experts + identity, a layer without identity experts, without
shared expert, without feed-forward, without window, a window of one, sizes that are multiples of nothing).
"""
import json
import math
import os

import numpy as np
import torch


def attn(heads, kv, dim, window=None, coef=0.6, every=16, scale=None, vdim=None):
    d = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim if vdim is None else vdim,
         "scale": scale if scale is not None else dim ** -0.5}
    if window is not None:
        d["mask"] = {"size": window}
    if every is not None:
        d["q_temp"] = {"coef": coef, "every": every}
    return "attention", d


def latent(heads, dim, rot_dim, vdim, kv_rank, window=None, base=10000.0, scaling=None, scale=None, q_rank=None, with_rank=True):
    """``q_rank`` given: the form whose queries go through a latent (interleaved pairs); ``with_rank`` False leaves its
    size out of config.json (the stored tensors say it). The writer finds it under "_q_rank"."""
    rot = {"base": base, "dims": rot_dim}
    if scaling is not None:
        rot["scaling"] = scaling
    d = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "rot": rot,
         "scale": scale if scale is not None else (dim + rot_dim) ** -0.5}
    if window is not None:
        d["mask"] = {"size": window}
    if q_rank is not None:
        d["_q_rank"] = q_rank
        if with_rank:
            d["q_rank"] = q_rank
    return ("latent_attention_2" if q_rank is not None else "latent_attention"), d


YARN = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, experts, identity, top, limit=1.0, shared=None, shared_limit=1.5):
    d = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "identity": identity, "top": top}}
    if shared is not None:
        d["shared"] = {"ff": shared, "limit": shared_limit}
    return d


def layer(mixer, mlp=None):
    return {"type": mixer[0], "mixer": mixer[1], "mlp": mlp}


def model(vocab, width, eps, layers, embed_scale=1.0):
    return {"architecture": "Fevosun", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": embed_scale},
            "layers": layers}


def clean(cfg):
    """The configuration as config.json holds it (without the writer's own keys)."""
    out = json.loads(json.dumps(cfg))
    for ly in out["layers"]:
        ly["mixer"].pop("_q_rank", None)
    return out


# one mechanism each between embedding and head
ONLY_ATTN = model(200, 64, 1e-5, [layer(attn(6, 2, 16, window=23, coef=0.7, every=9))], embed_scale=1.5)
ONLY_LAT1 = model(200, 64, 1e-5, [layer(latent(4, 16, 8, 24, 40, window=29, scaling=YARN))], embed_scale=0.8)
ONLY_LAT2 = model(200, 64, 1e-6, [layer(latent(3, 8, 16, 8, 24, window=17, base=500.0, q_rank=20, with_rank=False))])
# the mixer's output projection is zeroed by the tests that use these two: the feed-forward alone answers
ONLY_DENSE = model(200, 64, 1e-5, [layer(attn(2, 1, 8, window=5), dense(72))])
ONLY_MOE = model(200, 64, 1e-5, [layer(attn(2, 1, 8, window=5), moe(40, 5, 3, 3, limit=0.8, shared=24, shared_limit=1.2))], embed_scale=2.0)

# all of it, every layer different
MIXED_A = model(331, 96, 1e-5, [
    layer(attn(4, 2, 24, window=19, coef=0.4, every=7), moe(48, 6, 2, 2, limit=1.0, shared=72)),
    layer(latent(4, 16, 8, 24, 40, window=50, base=30000.0, scaling=YARN), dense(136)),
    layer(latent(3, 24, 16, 8, 32, window=13, q_rank=24), moe(32, 5, 0, 5, limit=0.6)),
    layer(attn(6, 6, 8, window=1, coef=1.0, every=3), None),
    layer(attn(3, 1, 16, window=None, every=None, scale=0.3), moe(64, 7, 1, 1, limit=2.0, shared=16, shared_limit=0.5)),
], embed_scale=2.5)
# sizes in multiples of 16 (what the tensor-core kernels take), more heads, wider
MIXED_B = model(500, 256, 2e-6, [
    layer(latent(8, 32, 16, 40, 80, window=72, base=250.0, scaling={"factor": 8.0, "original": 32, "fast": 4.0, "slow": 2.0}),
          moe(128, 8, 3, 2, limit=1.3, shared=128, shared_limit=1.8)),
    layer(attn(4, 2, 64, window=33, coef=0.45, every=32), dense(384)),
    layer(latent(4, 64, 32, 32, 96, window=40, q_rank=48, with_rank=False), moe(64, 16, 2, 4, limit=1.0, shared=192)),
    layer(attn(16, 4, 16, window=130, coef=0.25, every=50), moe(256, 4, 4, 8, limit=1.2)),
], embed_scale=3.5)
# sizes that are multiples of nothing useful
ODD = model(97, 70, 3e-5, [
    layer(attn(3, 1, 10, window=11, coef=0.9, every=5), moe(18, 3, 2, 2, limit=0.9, shared=10)),
    layer(latent(5, 6, 4, 14, 18, window=27, base=77.0, scaling={"factor": 2.0, "original": 16, "fast": 6.0, "slow": 1.5}), None),
    layer(latent(2, 10, 6, 22, 14, window=6, q_rank=9), dense(50)),
    layer(attn(6, 3, 6, window=64, coef=0.3, every=20), moe(26, 11, 3, 4, limit=1.4, shared=50, shared_limit=0.7)),
], embed_scale=0.7)
CONFIGS = {"odd": ODD, "attn": ONLY_ATTN, "lat1": ONLY_LAT1, "lat2": ONLY_LAT2, "dense": ONLY_DENSE, "moe": ONLY_MOE,
           "mixed_a": MIXED_A, "mixed_b": MIXED_B}
PAGE_SIZE = {"odd": 4, "attn": 8, "lat1": 16, "lat2": 4, "dense": 8, "moe": 8, "mixed_a": 8, "mixed_b": 16}


def random_config(rng, aligned):
    """A configuration drawn at random (``rng``: random.Random): two to six layers of any kind in any order, windows from
    1 to 300, heads, sizes, experts and constants over wide ranges; ``aligned``: sizes in multiples of 8 and key sizes that
    the tensor-core kernels take, else any."""
    m8 = (lambda lo, hi: 8 * rng.randint(max(1, lo // 8), hi // 8)) if aligned else (lambda lo, hi: rng.randint(lo, hi))
    layers = []
    for _ in range(rng.randint(2, 6)):
        kind = rng.choice(["attention", "latent", "latent2"])
        window = rng.choice([1, 2, 5, 16, 17, 31, 48, 64, 100, 300])
        if kind == "attention":
            kv = rng.choice([1, 2, 3, 4])
            mx = attn(kv * rng.choice([1, 2, 3, 4]), kv, (rng.choice([16, 64, 64, 128, 24]) if aligned else rng.randint(4, 72)), window=window,
                      coef=rng.choice([0.0, 0.3, 1.0]), every=rng.choice([1, 4, 13, 64, 1000]), scale=rng.uniform(0.05, 0.4))
        else:
            dr = 8 * rng.randint(1, 4) if aligned else 2 * rng.randint(1, 12)
            sc = rng.choice([None, {"factor": rng.choice([2.0, 8.0, 32.0]), "original": rng.choice([16, 64, 512]),
                                    "fast": rng.choice([4.0, 32.0]), "slow": rng.choice([1.0, 2.0])}])
            mx = latent(rng.randint(1, 8), m8(4, 64), dr, m8(4, 64), m8(8, 96), window=window, base=rng.choice([100.0, 10000.0, 1e6]),
                        scaling=sc, scale=rng.uniform(0.05, 0.3), q_rank=(m8(8, 64) if kind == "latent2" else None),
                        with_rank=rng.random() < 0.5)
        r = rng.random()
        if r < 0.15:
            mlp = None
        elif r < 0.4:
            mlp = dense(m8(8, 200))
        else:
            E = rng.randint(1, 20)
            I = rng.choice([0, 0, 1, 3, 6])
            mlp = moe(m8(8, 96), E, I, rng.randint(1, min(E + I, 6)), limit=rng.uniform(0.4, 3.0), shared=rng.choice([None, m8(8, 120)]),
                      shared_limit=rng.uniform(0.4, 3.0))
        layers.append(layer(mx, mlp))
    return model(rng.randint(30, 600), m8(24, 160), rng.choice([1e-6, 1e-5]), layers, embed_scale=rng.uniform(0.5, 4.0))


def silence_mixer(t):
    """For the configurations that test a feed-forward alone: the mixer's output projection becomes zero."""
    t["l0.mix.o"][:] = 0.0


def _tensors(cfg, seed):
    """{name: float32 array}, from a numpy generator; rounded to bfloat16 when written."""
    rng = np.random.default_rng(seed)
    W = cfg["width"]
    out = {}

    def lin(name, n_out, n_in, gain=1.0):
        out[name] = (rng.standard_normal((n_out, n_in)) * gain / math.sqrt(n_in)).astype(np.float32)

    def vec(name, n, mean=0.0, std=1.0):
        out[name] = (mean + std * rng.standard_normal(n)).astype(np.float32)

    out["embed"] = rng.standard_normal((cfg["vocab"], W)).astype(np.float32)
    for i, ly in enumerate(cfg["layers"]):
        p = f"l{i}."
        vec(p + "norm1", W, 0.0, 0.15)
        m = ly["mixer"]
        q = p + "mix."
        if ly["type"] == "attention":
            H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            # entries of q and k of order g each: scores of standard deviation about 3
            g = (3.0 / (m["scale"] * math.sqrt(dk))) ** 0.5
            lin(q + "q", H * dk, W, g); lin(q + "k", G * dk, W, g)
            lin(q + "g", H * dv, W, 2.0)
            lin(q + "o", W, H * dv, 1.0 / g)
        else:
            H, dq, dr, dv, rk = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            g = (3.0 / (m["scale"] * math.sqrt(dq + dr))) ** 0.5
            if ly["type"] == "latent_attention_2":
                r = m["_q_rank"]
                lin(q + "dq", r, W); vec(q + "dq.norm", r, 1.0, 0.2); lin(q + "uq", H * (dq + dr), r, g)
            else:
                lin(q + "q", H * (dq + dr), W, g)
            lin(q + "dkv", rk + dr, W, g)                    # the shared key part comes straight out of this product
            vec(q + "dkv.norm", rk, 1.0, 0.2)
            lin(q + "uk", H * dq, rk, g); lin(q + "uv", H * dv, rk); lin(q + "o", W, H * dv)
        mlp = ly.get("mlp")
        if mlp is None:
            continue
        f = p + "mlp."
        if mlp["kind"] == "dense":
            lin(f + "gate", mlp["ff"], W, 1.5); lin(f + "up", mlp["ff"], W, 1.5); lin(f + "down", W, mlp["ff"])
            continue
        F, E, I = mlp["expert"]["ff"], mlp["router"]["experts"], mlp["router"].get("identity", 0)
        lin(f + "router", E + I, W, 2.5)
        vec(f + "correction", E + I, 0.0, 0.15)
        for e in range(E):
            lin(f + f"e{e}.gate", F, W, 1.4); lin(f + f"e{e}.up", F, W, 1.4); lin(f + f"e{e}.down", W, F)
        if mlp.get("shared"):
            S = mlp["shared"]["ff"]
            lin(f + "shared.gate", S, W, 1.4); lin(f + "shared.up", S, W, 1.4); lin(f + "shared.down", W, S)
    vec("final.norm", W, 0.0, 0.1)
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
