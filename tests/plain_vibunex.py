"""Plain implementation of the Vibunex decoder for the tests: whole sequences, float64, no cache, no batching,
one function per mechanism. It shares no code with the package: it reads config.json and the safetensors file
itself and computes every layer from the equations in each function's docstring.
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np
import torch

F64 = torch.float64


# ---- model folder ---------------------------------------------------------------------------

def read_model_folder(folder: str):
    """(config dictionary, {tensor name: float64 or int64 tensor})."""
    with open(os.path.join(folder, "config.json"), "r", encoding="utf-8") as f:
        cfg = json.load(f)
    with open(os.path.join(folder, "model.safetensors"), "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        head = json.loads(f.read(n))
        data = f.read()
    w = {}
    for name, ent in head.items():
        if name == "__metadata__":
            continue
        a, b = ent["data_offsets"]
        raw = np.frombuffer(data[a:b], dtype=np.uint8)
        dt = ent["dtype"]
        if dt == "BF16":
            u = raw.view("<u2").astype(np.uint32) << 16
            t = torch.from_numpy(u.view(np.float32).astype(np.float64))
        elif dt == "F32":
            t = torch.from_numpy(raw.view("<f4").astype(np.float64))
        elif dt == "I32":
            t = torch.from_numpy(raw.view("<i4").astype(np.int64))
        else:
            raise ValueError(f"dtype {dt} of {name}")
        w[name] = t.reshape(ent["shape"])
    return cfg, w


# ---- mechanisms -----------------------------------------------------------------------------

def sigmoid(z):
    return 1.0 / (1.0 + torch.exp(-z))


def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last dimension."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def yarn_frequencies(dims, base, scaling):
    """(f [dims/2], magnitude). f_i = base^(-2i/dims); with scaling {factor, original, fast, slow}:
    edge(t) = dims ln(original / (2 pi t)) / (2 ln base), lo = max(floor(edge(fast)), 0), hi = min(ceil(edge(slow)), dims-1),
    r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), f_i <- f_i / factor * r_i + f_i (1 - r_i), magnitude 0.1 ln(factor) + 1."""
    i = torch.arange(dims // 2, dtype=F64)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])
    edge = lambda t: dims * math.log(orig / (2.0 * math.pi * t)) / (2.0 * math.log(base))
    lo = max(math.floor(edge(float(scaling["fast"]))), 0)
    hi = min(math.ceil(edge(float(scaling["slow"]))), dims - 1)
    r = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * r + f * (1.0 - r), 0.1 * math.log(factor) + 1.0


def rotate_halves(x, positions, freqs, magnitude):
    """x [T, heads, size]: entry i < dims/2 is paired with entry i + dims/2 (dims = 2 len(freqs)); the pair (u, v) at
    position p becomes (u c - v s, v c + u s) with c = magnitude cos(p f_i), s = magnitude sin(p f_i); entries from
    dims on pass unchanged."""
    half = freqs.numel()
    if half == 0:
        return x
    a = positions.to(F64)[:, None] * freqs[None, :]
    c, s = (torch.cos(a) * magnitude)[:, None, :], (torch.sin(a) * magnitude)[:, None, :]
    u, v = x[..., :half], x[..., half:2 * half]
    out = x.clone()
    out[..., :half] = u * c - v * s
    out[..., half:2 * half] = v * c + u * s
    return out


def sink_softmax_weights(q, k, scale, sink):
    """Causal attention weights of one head, [T, T]: w_ij = exp(s_ij) / (sum_{j' <= i} exp(s_ij') + exp(sink)),
    s_ij = scale q_i . k_j for j <= i, 0 for j > i. The rows do not sum to one: the sink takes its share."""
    T = q.shape[0]
    s = (q @ k.t()) * scale
    mask = torch.ones(T, T, dtype=torch.bool).tril()
    s = s.masked_fill(~mask, -math.inf)
    m = torch.maximum(s.max(-1, keepdim=True).values, torch.as_tensor(sink, dtype=F64))
    e = torch.exp(s - m)
    return e / (e.sum(-1, keepdim=True) + torch.exp(sink - m))


def talking_attention(h, w, p, mx, eps):
    """The left mixer. q = W_q h, k = W_k h, v = W_v h; q and k normalised over their whole width (weights q.norm,
    k.norm), split into H and G heads, rotated; per head sink-softmax weights; the weights of the heads are mixed,
    w'_h = sum_g talk[h, g] w_g, and head h applies w'_h to the values of key/value head h // (H / G); the
    concatenated heads are multiplied by sigmoid(W_g h) and go through W_o."""
    H, G, dk, dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    T = h.shape[0]
    pos = torch.arange(T)
    q = rms(h @ w[p + "q"].t(), eps) * w[p + "q.norm"]
    k = rms(h @ w[p + "k"].t(), eps) * w[p + "k.norm"]
    v = (h @ w[p + "v"].t()).view(T, G, dv)
    rot = mx.get("rot")
    q, k = q.view(T, H, dk), k.view(T, G, dk)
    if rot and rot["dims"] > 0:
        f, mag = yarn_frequencies(rot["dims"], float(rot["base"]), rot.get("scaling"))
        q, k = rotate_halves(q, pos, f, mag), rotate_halves(k, pos, f, mag)
    ratio = H // G
    weights = torch.stack([sink_softmax_weights(q[:, g], k[:, g // ratio], float(mx["scale"]), w[p + "sink"][g])
                           for g in range(H)])                       # [H, T, T]
    mixed = torch.einsum("hg,gij->hij", w[p + "talk"], weights)
    heads = [mixed[hh] @ v[:, hh // ratio] for hh in range(H)]
    o = torch.cat(heads, -1) * sigmoid(h @ w[p + "g"].t())
    return o @ w[p + "o"].t()


def decay_recurrence(r, k, v, wdec, u):
    """One head of the right mixer's recurrence. r, k, wdec [T, n], v [T, m], u [n]; S is n x m, zero at the start:
        o_t = (S + diag(u) k_t v_t^T)^T r_t;   S <- diag(wdec_t) S + k_t v_t^T."""
    T, n = k.shape
    S = torch.zeros(n, v.shape[1], dtype=F64)
    out = []
    for t in range(T):
        kv = k[t][:, None] * v[t][None, :]
        out.append((S + u[:, None] * kv).t() @ r[t])
        S = wdec[t][:, None] * S + kv
    return torch.stack(out)


def time_mix(h, w, p, mx, eps):
    """The right mixer. With h' the previous token's h (zeros for the first), each of r, k, v, g, w reads
    h + (h' - h) mu_s. r, k, v = W_s mix_s [heads, dim]; gate = silu(W_g mix_g); decay = exp(-exp(W_w2 tanh(W_w1 mix_w)
    + w0)); the recurrence per head; each head's result divided by its root mean square, times ``norm``, times the
    gate, through W_o."""
    H, n = mx["heads"], mx["dim"]
    T = h.shape[0]
    prev = torch.cat([torch.zeros(1, h.shape[1], dtype=F64), h[:-1]], 0)
    mix = lambda s: h + (prev - h) * w[p + "mu." + s]
    r = (mix("r") @ w[p + "r"].t()).view(T, H, n)
    k = (mix("k") @ w[p + "k"].t()).view(T, H, n)
    v = (mix("v") @ w[p + "v"].t()).view(T, H, n)
    gz = mix("g") @ w[p + "g"].t()
    gate = gz * sigmoid(gz)
    dec = torch.exp(-torch.exp(torch.tanh(mix("w") @ w[p + "w1"].t()) @ w[p + "w2"].t() + w[p + "w0"])).view(T, H, n)
    o = torch.stack([decay_recurrence(r[:, i], k[:, i], v[:, i], dec[:, i], w[p + "u"][i]) for i in range(H)], 1)
    o = rms(o, eps).reshape(T, H * n) * w[p + "norm"] * gate
    return o @ w[p + "o"].t()


def expert(h, up, down):
    """W_down relu(W_up h)^2."""
    a = torch.relu(h @ up.t())
    return (a * a) @ down.t()


def routed_feed_forward(h, w, p, mlp):
    """s = sigmoid(W_router h); the ``top`` experts with the largest scores each add s_e * scale * expert_e(h); the
    shared expert adds sigmoid(W_sg h) * expert_shared(h)."""
    E, top, scale = mlp["router"]["experts"], mlp["router"]["top"], float(mlp["router"]["scale"])
    s = sigmoid(h @ w[p + "router"].t())
    out = torch.zeros_like(h)
    chosen = torch.topk(s, top, dim=-1).indices
    for e in range(E):
        rows = (chosen == e).any(-1).nonzero().flatten()
        if rows.numel():
            out[rows] += expert(h[rows], w[f"{p}e{e}.up"], w[f"{p}e{e}.down"]) * (s[rows, e] * scale)[:, None]
    if mlp.get("shared"):
        out = out + expert(h, w[p + "shared.up"], w[p + "shared.down"]) * sigmoid(h @ w[p + "shared.sg"].t())
    return out


def routing_margin(h, w, p, mlp):
    """Per row, the gap between the smallest chosen score and the largest one left out (inf when all are chosen): a
    row whose gap is tiny may choose otherwise when h is rounded, which is no fault."""
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    if top >= E:
        return torch.full((h.shape[0],), math.inf, dtype=F64)
    s = sigmoid(h @ w[p + "router"].t()).sort(-1, descending=True).values
    return s[:, top - 1] - s[:, top]


# ---- the model ------------------------------------------------------------------------------

def forward(cfg, w, tokens, return_layers=False, margins=None):
    """Logits [T, vocab] of one whole sequence (and the residual stream after every layer; ``margins``, a list, gains
    every routed layer's ``routing_margin``).
    A layer: x <- x + m (sigmoid(W_rg1 h1 + b1) * mixer(h1) + sigmoid(W_rg2 h2 + b2) * ff(h2)), h1 = norm1(x),
    h2 = norm2(x), norm(x) = x / sqrt(mean(x^2) + eps) * g with one number g."""
    eps = cfg["norm"]["eps"]
    m = float(cfg["residual_mult"])
    x = w["embed"][torch.tensor(list(tokens))]
    layers = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        if layer["type"] != "parallel":
            raise ValueError(layer["type"])
        mx = layer["mixer"]
        h1 = rms(x, eps) * w[p + "norm1"]
        left = talking_attention(h1, w, p + "mix.left.", mx["left"], eps)
        right = time_mix(h1, w, p + "mix.right.", mx["right"], eps)
        mixed = float(mx["left_scale"]) * left + float(mx["right_scale"]) * right
        delta = mixed * sigmoid(h1 @ w[p + "rg1"].t() + w[p + "rg1.b"])
        if layer.get("mlp") is not None:
            h2 = rms(x, eps) * w[p + "norm2"]
            ff = routed_feed_forward(h2, w, p + "mlp.", layer["mlp"])
            if margins is not None:
                margins.append(routing_margin(h2, w, p + "mlp.", layer["mlp"]))
            delta = delta + ff * sigmoid(h2 @ w[p + "rg2"].t() + w[p + "rg2.b"])
        x = x + m * delta
        layers.append(x.clone())
    logits = (rms(x, eps) * w["final.norm"]) @ w["head"].t()
    if return_layers:
        return logits, torch.stack(layers)
    return logits


def greedy(cfg, w, prompt, n):
    """n greedy tokens after the prompt (each from a forward pass over the whole sequence so far)."""
    toks = list(prompt)
    out = []
    for _ in range(n):
        nxt = int(forward(cfg, w, toks)[-1].argmax())
        out.append(nxt)
        toks.append(nxt)
    return out
