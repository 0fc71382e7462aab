"""Fevosun without a GPU: configuration (keys, errors, round trip), the model as a specification (attention whose values
are its keys, latent attention in two forms, parallel sublayers on one norm, a routed feed-forward with identity experts),
checkpoint names and shapes, cache places, what the parts make of their weights, and the plain implementation's own
consistency (closed forms of its mechanisms)."""
import math

import pytest
import torch

import fevosun_configs as fc
import plain_fevosun as pf
from llm_steadyinfer_b200.config import ConfigError, config_from_dict, load_config
from llm_steadyinfer_b200.models import Model
from llm_steadyinfer_b200.weights.loader import load_weights_into

F64 = torch.float64


def test_configuration_round_trip_and_spec():
    cfg = config_from_dict(fc.clean(fc.MIXED_A))
    assert config_from_dict(cfg.to_dict()) == cfg
    spec = cfg.model_spec()
    assert spec.order == [0, 1, 2, 3, 4] and spec.vocab_size == 331 and spec.hidden_size == 96
    assert spec.embedder.kind == "table" and spec.embedder.params["scale"] == 2.5
    assert all(l.arrangement == "parallel" and l.feed_forward_norm is None and l.mixer_norm.params["offset"] == 1.0 for l in spec.layers)
    assert spec.final_norm.params["offset"] == 1.0
    a = spec.layers[0].mixer
    assert a.kind == "attention" and a.position is None and a.params["values_are_keys"] and a.params["window"] == 19
    assert a.params["distance_slopes"] == {"base": 2.0, "exponent": -8.0} and a.params["output_gate"] == "g"
    assert a.params["query_temperature"] == {"coef": 0.4, "every": 7}
    assert spec.layers[4].mixer.params["window"] is None and spec.layers[4].mixer.params["query_temperature"] is None
    l1 = spec.layers[1].mixer
    assert l1.kind == "latent_attention" and l1.params["q_rank"] is None and not l1.params["rot_interleaved"] and not l1.params["sink"]
    assert l1.params["rot_scaling"] == {"rope_type": "yarn", "factor": 4.0, "original": 64.0, "fast": 8.0, "slow": 1.0}
    assert (l1.params["head_dim"], l1.params["rot_dim"], l1.params["value_dim"], l1.params["kv_rank"], l1.params["window"]) == (16, 8, 24, 40, 50)
    l2 = spec.layers[2].mixer
    assert l2.kind == "latent_attention" and l2.params["q_rank"] == 24 and l2.params["rot_interleaved"] and l2.params["rot_scaling"] is None
    ff = spec.layers[0].feed_forward
    assert ff.kind == "routed_mlp" and (ff.params["experts"], ff.params["identity"], ff.params["top"]) == (6, 2, 2)
    assert ff.params["scores"] == "softmax" and not ff.params["renorm"] and ff.params["choice_bias"] == "correction"
    assert ff.params["activation"] == "glu_limited" and ff.params["limit"] == 1.0 and ff.params["alpha"] == 1.702
    assert ff.params["shared"]["kind"] == "gated_mlp_limited" and ff.params["shared"]["params"]["limit"] == 1.5
    assert not ff.params["shared"]["params"]["biases"] and not ff.params["shared_gate"]
    assert spec.layers[1].feed_forward.kind == "gated_mlp" and spec.layers[3].feed_forward is None
    assert spec.layers[2].feed_forward.params["shared"] is None and spec.layers[2].feed_forward.params["identity"] == 0
    # the query latent's size may be left to the checkpoint
    assert config_from_dict(fc.clean(fc.ONLY_LAT2)).model_spec().layers[0].mixer.params["q_rank"] == "checkpoint"


@pytest.mark.parametrize("edit,word", [
    (lambda d: d.pop("vocab"), "vocab"),
    (lambda d: d["norm"].pop("eps"), "eps"),
    (lambda d: d.update(layers=[]), "layers"),
    (lambda d: d["layers"][0].update(type="mamba"), "type"),
    (lambda d: d["layers"][0].pop("mixer"), "mixer"),
    (lambda d: d["layers"][0]["mixer"].pop("dim"), "dim"),
    (lambda d: d["layers"][0]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda d: d["layers"][0]["mixer"].update(vdim=25), "vdim"),
    (lambda d: d["layers"][0]["mixer"]["mask"].update(size=0), "size"),
    (lambda d: d["layers"][0]["mixer"]["q_temp"].update(every=0), "every"),
    (lambda d: d["layers"][1]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda d: d["layers"][1]["mixer"]["rot"]["scaling"].pop("fast"), "fast"),
    (lambda d: d["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda d: d["layers"][1]["mlp"].update(kind="sparse"), "kind"),
    (lambda d: d["layers"][0]["mlp"]["router"].update(top=9), "top"),
    (lambda d: d["layers"][0]["mlp"]["expert"].pop("limit"), "limit"),
    (lambda d: d["layers"][0]["mlp"]["shared"].update(ff=0), "ff"),
])
def test_configuration_errors_name_the_key(edit, word):
    d = fc.clean(fc.MIXED_A)
    edit(d)
    with pytest.raises(ConfigError) as e:
        config_from_dict(d)
    assert word in str(e.value)


def test_checkpoint_names_shapes_and_cache_places(tmp_path):
    folder = fc.write_folder(str(tmp_path / "m"), fc.MIXED_A, 3)
    model = Model(load_config(folder), torch.float32, "cpu")
    shapes = model.weight_shapes()
    assert shapes["embed"] == (331, 96) and shapes["head"] == (331, 96) and shapes["l0.norm1"] == (96,) and shapes["final.norm"] == (96,)
    assert shapes["l0.mix.q"] == (4 * 24, 96) and shapes["l0.mix.k"] == (2 * 24, 96) and shapes["l0.mix.g"] == (4 * 24, 96)
    assert shapes["l0.mix.o"] == (96, 4 * 24) and "l0.mix.v" not in shapes and "l0.norm2" not in shapes
    assert shapes["l1.mix.q"] == (4 * 24, 96) and shapes["l1.mix.dkv"] == (48, 96) and shapes["l1.mix.dkv.norm"] == (40,)
    assert shapes["l1.mix.uk"] == (64, 40) and shapes["l1.mix.uv"] == (96, 40) and shapes["l1.mix.o"] == (96, 96) and "l1.mix.dq" not in shapes
    assert shapes["l2.mix.dq"] == (24, 96) and shapes["l2.mix.dq.norm"] == (24,) and shapes["l2.mix.uq"] == (3 * 40, 24) and "l2.mix.q" not in shapes
    assert shapes["l1.mlp.gate"] == (136, 96) and shapes["l1.mlp.down"] == (96, 136)
    assert shapes["l0.mlp.router"] == (8, 96) and shapes["l0.mlp.correction"] == (8,) and shapes["l0.mlp.e5.gate"] == (48, 96)
    assert "l0.mlp.e6.up" not in shapes and shapes["l0.mlp.shared.gate"] == (72, 96) and "l2.mlp.shared.up" not in shapes
    assert set(shapes) == set(fc._tensors(fc.MIXED_A, 0))
    load_weights_into(model, folder)
    needs, states = model.cache_places()
    assert len(needs) == 6 and needs[-1] is None and all(s is None for s in states)
    # keys alone (they serve as values); a latent and the shared key part as one key that is its own value
    assert (needs[0].num_kv_heads, needs[0].head_dim, needs[0].v_dim, needs[0].window) == (2, 24, 0, 19)
    assert (needs[1].num_kv_heads, needs[1].head_dim, needs[1].v_dim, needs[1].window) == (1, 48, 0, 50)
    assert needs[3].window == 1 and needs[4].window is None
    assert model.capturable()


def test_what_the_parts_make_of_their_weights(tmp_path):
    folder = fc.write_folder(str(tmp_path / "m"), fc.ONLY_LAT2, 4)
    model = Model(load_config(folder), torch.float32, "cpu")
    assert model.weight_shapes()["l0.mix.dq"] == (-1, 64)          # the checkpoint says how large the query latent is
    load_weights_into(model, folder)
    _, w = pf.read_model_folder(folder)
    mixer = model.blocks[0].mixer
    assert mixer.q_rank == 20 and mixer.down.shape == (20 + 24 + 16, 64) and mixer.interleaved and mixer.rot_scale == 1.0
    # the norm multiplies by one plus the stored vector, in fp32
    assert torch.equal(model.blocks[0].mixer_norm.weight, (1.0 + w["l0.norm1"]).float())
    folder = fc.write_folder(str(tmp_path / "a"), fc.MIXED_A, 5)
    model = Model(load_config(folder), torch.float32, "cpu")
    load_weights_into(model, folder)
    _, w = pf.read_model_folder(folder)
    att = model.blocks[0].mixer
    assert torch.allclose(att.slopes.double(), pf.distance_slopes(4), rtol=1e-7) and att.q_temp == (0.4, 7)
    assert att.qkv.shape[0] == att.proj_cols == 4 * 24 + 2 * 24 + 4 * 24 and att.gate_off == 144
    lat = model.blocks[1].mixer
    f, mag = pf.rotary_frequencies(8, 30000.0, fc.YARN)
    assert torch.allclose(lat.inv_freq.double(), f, rtol=1e-6) and abs(lat.rot_scale - mag) < 1e-12 and lat.q_rank is None
    ff = model.blocks[0].feed_forward
    assert ff.routes == 8 and ff.w_up.shape == (6, 96, 96)
    assert torch.equal(ff.w_up[2, 0::2].double(), w["l0.mlp.e2.gate"]) and torch.equal(ff.w_up[2, 1::2].double(), w["l0.mlp.e2.up"])
    assert torch.equal(ff.choice_bias.double(), w["l0.mlp.correction"]) and ff.shared.output_bias is None


def test_plain_rotation():
    f, mag = pf.rotary_frequencies(8, 100.0, None)
    assert mag == 1.0 and torch.allclose(f, torch.tensor([1.0, 100 ** -0.25, 100 ** -0.5, 100 ** -0.75], dtype=F64))
    sc = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}
    f2, mag2 = pf.rotary_frequencies(8, 100.0, sc)
    edge = lambda t: 8 * math.log(64 / (2 * math.pi * t)) / (2 * math.log(100.0))
    lo, hi = max(math.floor(edge(8.0)), 0), min(math.ceil(edge(1.0)), 7)
    assert (lo, hi) == (0, 3) and abs(mag2 - (0.1 * math.log(4.0) + 1)) < 1e-15
    for i in range(4):
        r = min(max((i - lo) / (hi - lo), 0.0), 1.0)
        assert abs(f2[i].item() - (f[i].item() / 4 * r + f[i].item() * (1 - r))) < 1e-15
    # a rotation keeps a pair's length (times the magnitude) and composes; the two pairings move different entries
    x = torch.randn(1, 2, 12, dtype=F64)
    for inter, (i, j) in ((False, (0, 4)), (True, (0, 1))):
        a = pf.rotate(x, torch.tensor([5]), f, 1.0, inter)
        b = pf.rotate(pf.rotate(x, torch.tensor([2]), f, 1.0, inter), torch.tensor([3]), f, 1.0, inter)
        assert torch.allclose(a, b) and torch.equal(a[..., 8:], x[..., 8:])
        assert torch.allclose(a[..., i] ** 2 + a[..., j] ** 2, x[..., i] ** 2 + x[..., j] ** 2)
        assert torch.allclose(pf.rotate(x, torch.tensor([5]), f, 1.5, inter), torch.cat([1.5 * a[..., :8], x[..., 8:]], -1))


def test_plain_attention_closed_forms():
    # the window's mask: row i sees i - window + 1 .. i
    m = pf.window_mask(6, 3)
    assert m.sum(1).tolist() == [1, 2, 3, 3, 3, 3] and m[5].tolist() == [False, False, False, True, True, True]
    assert pf.window_mask(4, None).sum().item() == 10
    # equal raw scores: the weights fall off by exp(-slope) a step back, within the window
    W, H, dk = 4, 2, 3
    w = {"m.q": torch.zeros(H * dk, W, dtype=F64), "m.k": torch.randn(dk, W, dtype=F64), "m.g": torch.zeros(H * dk, W, dtype=F64),
         "m.o": torch.eye(H * dk, dtype=F64)[:W].contiguous()}
    h = torch.randn(5, W, dtype=F64)
    mix = {"heads": H, "kv_heads": 1, "dim": dk, "vdim": dk, "scale": 0.5, "mask": {"size": 3}, "q_temp": {"coef": 0.3, "every": 2}}
    out = pf.attention(h, w, "m.", mix)
    k = h @ w["m.k"].T
    slopes = pf.distance_slopes(H)
    assert torch.allclose(slopes, torch.tensor([2.0 ** -4, 2.0 ** -8], dtype=F64))
    for i in range(5):
        js = list(range(max(0, i - 2), i + 1))
        for hd in range(1):                               # the output keeps the first W of H * dk entries: head 0 and a part of head 1
            e = torch.tensor([math.exp(-slopes[hd].item() * (i - j)) for j in js], dtype=F64)
            want = (e / e.sum()) @ k[js] * 0.5            # gate sums of zero: a half
            assert torch.allclose(out[i, :dk], want)
    # the temperature: one until position every - 1, then 1 + coef ln(2), ...
    t = pf.query_temperature(torch.arange(6), 0.3, 2.0)
    assert torch.allclose(t, torch.tensor([1.0, 1 + 0.3 * math.log(2), 1 + 0.3 * math.log(2), 1 + 0.3 * math.log(3), 1 + 0.3 * math.log(3),
                                          1 + 0.3 * math.log(4)], dtype=F64))


def test_plain_latent_attention_equals_its_absorbed_form():
    """Scores against the latent itself with W_uk moved to the query side, values expanded behind the weighted sum: the same
    function as with keys and values expanded per head (what an engine that caches only the latent computes)."""
    torch.manual_seed(2)
    W, H, dq, dr, dv, rk, T = 12, 2, 4, 2, 3, 5, 7
    w = {"m.q": torch.randn(H * (dq + dr), W, dtype=F64), "m.dkv": torch.randn(rk + dr, W, dtype=F64), "m.dkv.norm": torch.rand(rk, dtype=F64) + 0.5,
         "m.uk": torch.randn(H * dq, rk, dtype=F64), "m.uv": torch.randn(H * dv, rk, dtype=F64), "m.o": torch.randn(W, H * dv, dtype=F64)}
    mix = {"heads": H, "dim": dq, "rot_dim": dr, "vdim": dv, "kv_rank": rk, "scale": 0.4, "mask": {"size": 4}, "rot": {"base": 50.0, "dims": dr}}
    h = torch.randn(T, W, dtype=F64)
    got = pf.latent_attention(h, w, "m.", mix, 1e-6, query_latent=False, interleaved=False)
    pos = torch.arange(T)
    q = (h @ w["m.q"].T).view(T, H, dq + dr)
    lat = h @ w["m.dkv"].T
    c = pf.plain_norm(lat[:, :rk], w["m.dkv.norm"], 1e-6)
    f, mag = pf.rotary_frequencies(dr, 50.0, None)
    kr = pf.rotate(lat[:, rk:].view(T, 1, dr), pos, f, mag, False)[:, 0]
    qr = pf.rotate(q[:, :, dq:], pos, f, mag, False)
    uk, uv = w["m.uk"].view(H, dq, rk), w["m.uv"].view(H, dv, rk)
    q_lat = torch.einsum("ihd,hdr->ihr", q[:, :, :dq], uk)
    s = (torch.einsum("ihr,jr->hij", q_lat, c) + torch.einsum("ihd,jd->hij", qr, kr)) * 0.4
    o_lat = pf.softmax_attend(s, pf.window_mask(T, 4), c.unsqueeze(0).expand(H, T, rk))           # [T, H, rk]
    o = torch.einsum("ihr,hvr->ihv", o_lat, uv).reshape(T, H * dv)
    assert torch.allclose(got, o @ w["m.o"].T)


def test_plain_router_choice_identity_and_limits():
    torch.manual_seed(1)
    W, E, I, F = 8, 3, 2, 6
    w = {"m.router": torch.randn(E + I, W, dtype=F64), "m.correction": torch.tensor([0.0, 0.0, 5.0, 0.0, -5.0], dtype=F64)}
    for e in range(E):
        w[f"m.e{e}.gate"], w[f"m.e{e}.up"], w[f"m.e{e}.down"] = torch.randn(F, W, dtype=F64) * 2, torch.randn(F, W, dtype=F64) * 2, torch.randn(W, F, dtype=F64)
    h = torch.randn(4, W, dtype=F64)
    mlp = {"router": {"experts": E, "identity": I, "top": 2}, "expert": {"ff": F, "limit": 0.5}}
    ids, wts, margin = pf.route(h, w, "m.", 2)
    s = torch.softmax(h @ w["m.router"].T, -1)
    assert (ids[:, 0] == 2).all() and (ids != 4).all()                  # the correction decides the choice ...
    assert torch.allclose(wts, torch.gather(s, 1, ids)) and (margin > 0).all()        # ... and stays out of the weights
    got = pf.routed_ff(h, w, "m.", mlp)
    for t in range(4):
        want = torch.zeros(W, dtype=F64)
        for c in range(2):
            e = int(ids[t, c])
            if e >= E:
                y = h[t]                                                # an identity expert returns its input
            else:
                g = torch.clamp(w[f"m.e{e}.gate"] @ h[t], max=0.5)
                u = torch.clamp(w[f"m.e{e}.up"] @ h[t], -0.5, 0.5)
                assert (w[f"m.e{e}.gate"] @ h[t] > 0.5).any()           # the limit cuts
                y = w[f"m.e{e}.down"] @ (g / (1 + torch.exp(-1.702 * g)) * (u + 1))
            want += s[t, e] * y
        assert torch.allclose(got[t], want)
    # a tie in the choice goes to the lower index
    w2 = {"m.router": torch.zeros(4, W, dtype=F64), "m.correction": torch.zeros(4, dtype=F64)}
    assert pf.route(h, w2, "m.", 2)[0].tolist() == [[0, 1]] * 4


def test_plain_layer_is_parallel_and_norm_has_an_offset():
    cfg = fc.clean(fc.model(20, 8, 1e-5, [fc.layer(fc.attn(2, 1, 4, window=3), fc.dense(6))], embed_scale=3.0))
    w = {n: torch.tensor(a, dtype=F64) for n, a in fc._tensors(cfg, 1).items()}
    toks = [3, 7, 7, 1]
    layers = []
    logits = pf.forward(cfg, w, toks, layers_out=layers)
    x = w["embed"][toks] * 3.0
    h = x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-5) * (1.0 + w["l0.norm1"])
    want = x + pf.attention(h, w, "l0.mix.", cfg["layers"][0]["mixer"]) + pf.dense_ff(h, w, "l0.mlp.")       # both read h
    assert torch.allclose(layers[0], want)
    assert torch.allclose(logits, pf.offset_norm(want, w["final.norm"], 1e-5) @ w["head"].T)
