"""Vibunex without a GPU: configuration (keys, errors, round trip), the model as a specification (a pair of mixers, a
routed feed-forward, gated parallel sublayers, a norm with one number), checkpoint names and shapes, cache and state
places, and the plain implementation's own consistency (closed forms of its mechanisms)."""
import copy
import math

import pytest
import torch

import plain_vibunex as pv
import vibunex_configs as vc
from llm_steadyinfer_b200.config import ConfigError, config_from_dict, load_config
from llm_steadyinfer_b200.models import Model
from llm_steadyinfer_b200.weights.loader import load_weights_into

F64 = torch.float64


def test_configuration_round_trip_and_spec():
    cfg = config_from_dict(vc.clean(vc.MIXED_A))
    assert config_from_dict(cfg.to_dict()) == cfg
    spec = cfg.model_spec()
    assert spec.order == [0, 1, 2, 3] and len(spec.layers) == 4 and spec.vocab_size == 331 and spec.hidden_size == 96
    assert all(l.arrangement == "parallel_gated" and l.mixer.kind == "mixer_pair" and l.residual_scale == 0.65 for l in spec.layers)
    assert all(l.mixer_norm.params["scalar"] and l.mixer_gate_name == "rg1" for l in spec.layers) and spec.final_norm.params["scalar"]
    assert spec.layers[1].feed_forward is None and spec.layers[1].feed_forward_norm is None and spec.layers[1].feed_forward_gate_name is None
    ff = spec.layers[0].feed_forward
    assert ff.kind == "routed_mlp" and ff.params["experts"] == 6 and ff.params["top"] == 2 and ff.params["scale"] == 2.5
    assert ff.params["shared"] == {"intermediate_size": 72} and ff.params["activation"] == "relu2" and not ff.params["renorm"]
    assert spec.layers[2].feed_forward.params["shared"] is None and spec.layers[2].feed_forward.params["top"] == 5
    mx = spec.layers[0].mixer.params
    assert (mx["left_scale"], mx["right_scale"]) == (1.15, 0.45)
    left, right = mx["left"], mx["right"]
    assert left["kind"] == "talking_attention" and right["kind"] == "time_mix" and right["position"] is None
    assert (left["params"]["num_heads"], left["params"]["num_kv_heads"], left["params"]["head_dim"], left["params"]["value_dim"]) == (4, 2, 24, 16)
    pos = left["position"]
    assert pos["kind"] == "rotary" and pos["params"]["rot_dim"] == 12 and pos["params"]["theta"] == 50000.0
    assert pos["params"]["scaling"] == {"rope_type": "yarn", "factor": 4.0, "original": 64.0, "fast": 8.0, "slow": 1.0}
    assert spec.layers[1].mixer.params["left"]["position"]["params"]["scaling"] is None           # rotation without scaling
    assert spec.layers[3].mixer.params["left"]["position"] is None                                  # no rotation at all
    assert (right["params"]["num_heads"], right["params"]["head_dim"]) == (3, 16)


@pytest.mark.parametrize("edit,word", [
    (lambda d: d.pop("vocab"), "vocab"),
    (lambda d: d["norm"].pop("eps"), "eps"),
    (lambda d: d.update(layers=[]), "layers"),
    (lambda d: d["layers"][0].update(type="serial"), "type"),
    (lambda d: d["layers"][0]["mixer"].pop("left"), "left"),
    (lambda d: d["layers"][0]["mixer"]["left"].pop("vdim"), "vdim"),
    (lambda d: d["layers"][0]["mixer"]["left"].update(kv_heads=3), "kv_heads"),
    (lambda d: d["layers"][0]["mixer"]["left"]["rot"].update(dims=13), "rot.dims"),
    (lambda d: d["layers"][0]["mixer"]["left"]["rot"]["scaling"].pop("fast"), "fast"),
    (lambda d: d["layers"][1]["mixer"]["right"].pop("dim"), "dim"),
    (lambda d: d["layers"][0]["mlp"].update(kind="dense"), "kind"),
    (lambda d: d["layers"][0]["mlp"]["router"].update(top=7), "top"),
    (lambda d: d["layers"][0]["mlp"]["expert"].pop("ff"), "ff"),
    (lambda d: d["layers"][0]["mlp"]["shared"].update(ff=0), "ff"),
])
def test_configuration_errors_name_the_key(edit, word):
    d = vc.clean(vc.MIXED_A)
    edit(d)
    with pytest.raises(ConfigError) as e:
        config_from_dict(d)
    assert word in str(e.value)


def test_checkpoint_names_shapes_cache_and_state(tmp_path):
    folder = vc.write_folder(str(tmp_path / "m"), vc.MIXED_A, 3)
    model = Model(load_config(folder), torch.float32, "cpu")
    shapes = model.weight_shapes()
    assert shapes["l0.norm1"] == () and shapes["final.norm"] == () and shapes["l0.rg1"] == (96, 96) and shapes["l0.rg2.b"] == (96,)
    assert shapes["l0.mix.left.q"] == (4 * 24, 96) and shapes["l0.mix.left.k"] == (2 * 24, 96) and shapes["l0.mix.left.v"] == (2 * 16, 96)
    assert shapes["l0.mix.left.q.norm"] == (96,) and shapes["l0.mix.left.k.norm"] == (48,) and shapes["l0.mix.left.talk"] == (4, 4)
    assert shapes["l0.mix.left.sink"] == (4,) and shapes["l0.mix.left.g"] == (64, 96) and shapes["l0.mix.left.o"] == (96, 64)
    assert shapes["l0.mix.right.mu.w"] == (96,) and shapes["l0.mix.right.r"] == (48, 96) and shapes["l0.mix.right.u"] == (3, 16)
    assert shapes["l0.mix.right.w0"] == (48,) and shapes["l0.mix.right.norm"] == (48,) and shapes["l0.mix.right.o"] == (96, 48)
    assert shapes["l0.mlp.router"] == (6, 96) and shapes["l0.mlp.e5.up"] == (48, 96) and shapes["l0.mlp.e0.down"] == (96, 48)
    assert shapes["l0.mlp.shared.up"] == (72, 96) and shapes["l0.mlp.shared.sg"] == (1, 96)
    assert "l1.norm2" not in shapes and "l1.rg2" not in shapes and "l2.mlp.shared.up" not in shapes and "l2.mlp.shared.sg" not in shapes
    assert set(shapes) == set(vc._tensors(vc.MIXED_A, 0))
    load_weights_into(model, folder)                      # the decay's rank comes from the checkpoint: 6, 16, 3, 8
    assert [b.mixer.subs[1].L for b in model.blocks] == [6, 16, 3, 8]
    needs, states = model.cache_places()
    assert len(needs) == 5 and needs[-1] is None and states[-1] is None
    # keys of G heads; a token's values, all key/value heads side by side, as one value head
    assert (needs[0].num_kv_heads, needs[0].head_dim, needs[0].v_dim, needs[0].v_heads, needs[0].window) == (2, 24, 32, 1, None)
    assert (needs[2].num_kv_heads, needs[2].head_dim, needs[2].v_dim, needs[2].v_heads) == (1, 8, 16, 1)
    from llm_steadyinfer_b200.csrc import ops
    assert ops.decay_state_floats(16) >= 16 * 16 and ops.decay_state_floats(40) >= 40 * 40
    # per slot: the heads' matrices in the scan's layout, then the last row of the mixer's input
    assert states[0].shape == (3 * ops.decay_state_floats(16) + 96,) and states[2].shape == (2 * ops.decay_state_floats(40) + 96,)


def test_plain_rotation_frequencies():
    f, mag = pv.yarn_frequencies(8, 100.0, None)
    assert mag == 1.0 and torch.allclose(f, torch.tensor([1.0, 100 ** -0.25, 100 ** -0.5, 100 ** -0.75], dtype=F64))
    # with scaling: below ``lo`` the frequency stays, from ``hi`` on it is divided by the factor, a ramp between
    sc = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}
    f2, mag2 = pv.yarn_frequencies(8, 100.0, sc)
    edge = lambda t: 8 * math.log(64 / (2 * math.pi * t)) / (2 * math.log(100.0))
    lo, hi = max(math.floor(edge(8.0)), 0), min(math.ceil(edge(1.0)), 7)
    assert (lo, hi) == (0, 3) and abs(mag2 - (0.1 * math.log(4.0) + 1)) < 1e-15
    for i in range(4):
        r = min(max((i - lo) / (hi - lo), 0.0), 1.0)
        assert abs(f2[i].item() - (f[i].item() / 4 * r + f[i].item() * (1 - r))) < 1e-15
    # a rotation keeps a pair's length (times the magnitude) and composes: position 5 is position 2 then 3
    x = torch.randn(1, 2, 12, dtype=F64)
    a = pv.rotate_halves(x, torch.tensor([5]), f, 1.0)
    b = pv.rotate_halves(pv.rotate_halves(x, torch.tensor([2]), f, 1.0), torch.tensor([3]), f, 1.0)
    assert torch.allclose(a, b) and torch.equal(a[..., 8:], x[..., 8:])
    assert torch.allclose(a[..., 0] ** 2 + a[..., 4] ** 2, x[..., 0] ** 2 + x[..., 4] ** 2)


def test_plain_sink_softmax_and_recurrence_closed_forms():
    # equal scores: each of the i + 1 keys gets 1 / (i + 1 + exp(sink)) -- one more term in the denominator, exp(sink) as it stands
    q, k = torch.zeros(4, 3, dtype=F64), torch.randn(4, 3, dtype=F64)
    w = pv.sink_softmax_weights(q, k, 0.7, torch.tensor(math.log(2.0), dtype=F64))
    for i in range(4):
        assert torch.allclose(w[i, :i + 1], torch.full((i + 1,), 1.0 / (i + 3), dtype=F64)) and w[i, i + 1:].abs().sum() == 0
    # constant decay w, constant k, v, r: S_t = (1 + w + .. + w^(t-1)) k v^T, o_t = (r.k)(that) v + (r . (u k)) v
    n, T, wd = 3, 6, 0.5
    k, v, r, u = torch.tensor([1.0, 2.0, -1.0], dtype=F64), torch.tensor([0.5, -2.0], dtype=F64), torch.tensor([0.3, 0.1, 0.2], dtype=F64), torch.tensor([2.0, 0.0, 1.0], dtype=F64)
    o = pv.decay_recurrence(r.expand(T, n), k.expand(T, n), v.expand(T, 2), torch.full((T, n), wd, dtype=F64), u)
    for t in range(T):
        geo = sum(wd ** j for j in range(t))
        assert torch.allclose(o[t], ((r @ k) * geo + (r * u) @ k) * v)


def test_plain_router_choice_and_weights():
    torch.manual_seed(1)
    W, E, F = 8, 5, 6
    w = {"m.router": torch.randn(E, W, dtype=F64)}
    for e in range(E):
        w[f"m.e{e}.up"], w[f"m.e{e}.down"] = torch.randn(F, W, dtype=F64), torch.randn(W, F, dtype=F64)
    h = torch.randn(3, W, dtype=F64)
    mlp = {"router": {"experts": E, "top": 2, "scale": 1.5}, "expert": {"ff": F}}
    got = pv.routed_feed_forward(h, w, "m.", mlp)
    s = 1 / (1 + torch.exp(-(h @ w["m.router"].t())))
    for t in range(3):
        order = sorted(range(E), key=lambda e: -s[t, e].item())[:2]
        want = sum(1.5 * s[t, e] * (torch.relu(w[f"m.e{e}.up"] @ h[t]) ** 2) @ w[f"m.e{e}.down"].t() for e in order)
        assert torch.allclose(got[t], want)            # weights are the scores themselves, not renormalised
