"""Plain implementation of the Fevosun decoder for the tests: whole sequences, float64, no cache, no batching,
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


def offset_norm(x, w, eps):
    """The norm on the residual stream: rms(x) * (1 + w), the stored vector lying around zero."""
    return rms(x, eps) * (1.0 + w)


def plain_norm(x, w, eps):
    """The norm of a latent: rms(x) * w."""
    return rms(x, eps) * w


def rotary_frequencies(dims, base, scaling):
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


def rotate(x, positions, freqs, magnitude, interleaved):
    """x [T, heads, size], dims = 2 len(freqs) <= size. Pair i is (entry i, entry i + dims/2), or (entry 2i, entry 2i+1)
    when ``interleaved``; the pair (u, v) at position p becomes (u c - v s, v c + u s) with c = magnitude cos(p f_i),
    s = magnitude sin(p f_i); entries from dims on pass unchanged."""
    half = freqs.numel()
    if half == 0:
        return x
    ang = positions.to(F64).view(-1, 1, 1) * freqs.view(1, 1, -1)
    c, s = magnitude * torch.cos(ang), magnitude * torch.sin(ang)
    out = x.clone()
    if interleaved:
        u, v = x[..., 0:2 * half:2], x[..., 1:2 * half:2]
        out[..., 0:2 * half:2] = u * c - v * s
        out[..., 1:2 * half:2] = v * c + u * s
    else:
        u, v = x[..., :half], x[..., half:2 * half]
        out[..., :half] = u * c - v * s
        out[..., half:2 * half] = v * c + u * s
    return out


def window_mask(T, window):
    """[T, T] True where query i sees key j: j <= i, and i - j < window when there is a window."""
    i = torch.arange(T).view(-1, 1)
    j = torch.arange(T).view(1, -1)
    m = j <= i
    if window:
        m = m & (i - j < window)
    return m


def softmax_attend(scores, mask, values):
    """scores [H, T, T], mask [T, T], values [H, T, dv]: softmax over the visible keys, then the weighted sum."""
    s = scores.masked_fill(~mask.unsqueeze(0), -math.inf)
    p = torch.softmax(s, dim=-1)
    return torch.einsum("hij,hjd->ihd", p, values)


def query_temperature(positions, coef, every):
    """1 + coef * ln(floor((p + 1) / every) + 1) per position p."""
    return 1.0 + coef * torch.log(torch.floor((positions.to(F64) + 1.0) / every) + 1.0)


def distance_slopes(H):
    """slope_h = 2^(-8 (h + 1) / H), h = 0 .. H-1."""
    return torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], dtype=F64)


def attention(h, w, pre, m):
    """Grouped-query attention whose values are its keys, with a query temperature, a linear penalty by distance,
    a window and an output gate:
        q_i = temp(i) W_q h_i [H, dk];  k_j = W_k h_j [G, dk];  v_j = k_j
        s_h(i, j) = scale q_h(i) . k_g(j) - slope_h (i - j),  g = h // (H / G);  softmax over the window
        out = W_o (concat_h o_h * sigmoid(W_g h_i))"""
    T = h.shape[0]
    H, G, dk = m["heads"], m["kv_heads"], m["dim"]
    pos = torch.arange(T)
    q = (h @ w[pre + "q"].T).view(T, H, dk)
    k = (h @ w[pre + "k"].T).view(T, G, dk)
    qt = m.get("q_temp")
    if qt:
        q = q * query_temperature(pos, float(qt["coef"]), float(qt["every"])).view(T, 1, 1)
    kh = k.repeat_interleave(H // G, dim=1)                       # [T, H, dk]
    s = torch.einsum("ihd,jhd->hij", q, kh) * float(m["scale"])
    dist = (pos.view(-1, 1) - pos.view(1, -1)).to(F64)
    s = s - distance_slopes(H).view(H, 1, 1) * dist.unsqueeze(0)
    mask = window_mask(T, (m.get("mask") or {}).get("size"))
    o = softmax_attend(s, mask, kh.permute(1, 0, 2)).reshape(T, H * dk)
    o = o * sigmoid(h @ w[pre + "g"].T)
    return o @ w[pre + "o"].T


def latent_attention(h, w, pre, m, eps, query_latent, interleaved):
    """Attention through a key/value latent:
        q = W_q h, or with ``query_latent`` q = W_uq norm(W_dq h);  per head [dq plain | dr rotated]
        [l | r] = W_dkv h;  c = norm(l);  shared rotated key part rot(r)
        k_h(j) = [W_uk,h c_j | rot(r_j)];  v_h(j) = W_uv,h c_j
        s_h(i, j) = scale (q_plain . k_plain + rot(q_rot) . rot(r_j));  softmax over the window;  out = W_o concat_h o_h"""
    T = h.shape[0]
    H, dq, dr, dv, rk = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    if query_latent:
        cq = plain_norm(h @ w[pre + "dq"].T, w[pre + "dq.norm"], eps)
        q = cq @ w[pre + "uq"].T
    else:
        q = h @ w[pre + "q"].T
    q = q.view(T, H, dq + dr)
    lat = h @ w[pre + "dkv"].T
    c = plain_norm(lat[:, :rk], w[pre + "dkv.norm"], eps)
    rot = m["rot"]
    f, mag = rotary_frequencies(int(rot["dims"]), float(rot["base"]), rot.get("scaling"))
    kr = rotate(lat[:, rk:].view(T, 1, dr), pos, f, mag, interleaved)         # [T, 1, dr]
    qr = rotate(q[:, :, dq:], pos, f, mag, interleaved)
    kp = (c @ w[pre + "uk"].T).view(T, H, dq)
    v = (c @ w[pre + "uv"].T).view(T, H, dv)
    s = (torch.einsum("ihd,jhd->hij", q[:, :, :dq], kp) + torch.einsum("ihd,jd->hij", qr, kr[:, 0])) * float(m["scale"])
    mask = window_mask(T, (m.get("mask") or {}).get("size"))
    o = softmax_attend(s, mask, v.permute(1, 0, 2)).reshape(T, H * dv)
    return o @ w[pre + "o"].T


def dense_ff(h, w, pre):
    """W_down (silu(W_gate h) * (W_up h))."""
    g = h @ w[pre + "gate"].T
    return (g * sigmoid(g) * (h @ w[pre + "up"].T)) @ w[pre + "down"].T


def limited_expert(h, w, pre, limit):
    """g = min(W_gate h, limit); u = clamp(W_up h, -limit, limit); W_down (g sigmoid(1.702 g) (u + 1))."""
    g = torch.clamp(h @ w[pre + "gate"].T, max=limit)
    u = torch.clamp(h @ w[pre + "up"].T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ w[pre + "down"].T


def route(h, w, pre, top):
    """s = softmax(W_router h) over all router rows; the ``top`` largest of s + correction are chosen (the lower index on a
    tie); the weights are their s. Returns (ids [T, top], weights [T, top], margin [T]: by how much the last chosen row's
    choice score lies above the first one left out, infinite where none is left out)."""
    s = torch.softmax(h @ w[pre + "router"].T, dim=-1)
    choice = s + w[pre + "correction"]
    order = torch.sort(choice, dim=-1, descending=True, stable=True)
    ids = order.indices[:, :top]
    if top < choice.shape[1]:
        margin = order.values[:, top - 1] - order.values[:, top]
    else:
        margin = torch.full((h.shape[0],), math.inf, dtype=F64)
    return ids, torch.gather(s, 1, ids), margin


def routed_ff(h, w, pre, mlp, margins=None):
    """sum over the chosen e of weight_e * expert_e(h), where the last ``identity`` router rows stand for experts that
    return h itself; plus the shared expert for every row."""
    r = mlp["router"]
    E, top = int(r["experts"]), int(r["top"])
    ids, wts, margin = route(h, w, pre, top)
    if margins is not None:
        margins.append(margin)
    limit = float(mlp["expert"]["limit"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for c in range(top):
            e = int(ids[t, c])
            y = limited_expert(h[t:t + 1], w, f"{pre}e{e}.", limit)[0] if e < E else h[t]
            out[t] += wts[t, c] * y
    sh = mlp.get("shared")
    if sh:
        out = out + limited_expert(h, w, pre + "shared.", float(sh["limit"]))
    return out


# ---- the model --------------------------------------------------------------------------------

def mixer(kind, h, w, pre, m, eps):
    if kind == "attention":
        return attention(h, w, pre, m)
    if kind == "latent_attention":
        return latent_attention(h, w, pre, m, eps, query_latent=False, interleaved=False)
    if kind == "latent_attention_2":
        return latent_attention(h, w, pre, m, eps, query_latent=True, interleaved=True)
    raise ValueError(kind)


def forward(cfg, w, tokens, layers_out=None, margins=None):
    """Logits [T, vocab] of a whole sequence. Every layer: h = norm1(x); x <- x + mixer(h) + ff(h).
    ``layers_out``: a list that receives the stream after every layer; ``margins``: a list that receives every routed
    layer's margins [T] (see ``route``)."""
    eps = float(cfg["norm"]["eps"])
    x = w["embed"][torch.tensor(list(tokens), dtype=torch.long)] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = offset_norm(x, w[p + "norm1"], eps)
        d = mixer(layer["type"], h, w, p + "mix.", layer["mixer"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            d = d + (dense_ff(h, w, p + "mlp.") if mlp["kind"] == "dense" else routed_ff(h, w, p + "mlp.", mlp, margins))
        x = x + d
        if layers_out is not None:
            layers_out.append(x.clone())
    return offset_norm(x, w["final.norm"], eps) @ w["head"].T


def greedy(cfg, w, prompt, new):
    """``new`` tokens, each the largest logit after the sequence so far (the whole sequence computed again every time)."""
    toks = list(prompt)
    for _ in range(new):
        toks.append(int(forward(cfg, w, toks)[-1].argmax()))
    return toks[len(prompt):]
