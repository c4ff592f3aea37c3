"""Plain, slow float64 statement of the Timerax design, one function per mechanism (numpy only).

It is test infrastructure: it shares no code with the product path and is written for reading, not speed.
Notation: T tokens of ONE sequence, positions 0..T-1; matrices are stored [out, in] and applied as x @ W.T.
A model is (cfg, w): cfg the parsed config.json, w a dict name -> float64 array.
"""
from __future__ import annotations

import json
import math
import struct

import numpy as np


# ---- files -----------------------------------------------------------------------------------------------
def bf16_round(a):
    """Round float32 values to the nearest-even bfloat16, returned as float32."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    u = a.view(np.uint32).astype(np.uint64)
    u = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return u.astype(np.uint32).view(np.float32).reshape(a.shape)


def read_safetensors(path):
    with open(path, "rb") as f:
        n = struct.unpack("<Q", f.read(8))[0]
        head = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, d in head.items():
        if name == "__metadata__":
            continue
        lo, hi = d["data_offsets"]
        raw = data[lo:hi]
        if d["dtype"] == "BF16":
            a = (np.frombuffer(raw, np.uint16).astype(np.uint32) << 16).view(np.float32)
        elif d["dtype"] == "F32":
            a = np.frombuffer(raw, np.float32)
        elif d["dtype"] == "I32":
            a = np.frombuffer(raw, np.int32)
        else:
            raise ValueError(d["dtype"])
        out[name] = a.reshape(d["shape"]).astype(np.float64)
    return out


def write_safetensors(path, tensors):
    """tensors: name -> float array (stored as bfloat16; values must already be bf16-representable or get rounded)."""
    head, blobs, off = {}, [], 0
    for name, a in tensors.items():
        r = bf16_round(np.asarray(a, np.float32))
        b = (r.view(np.uint32) >> 16).astype(np.uint16).tobytes()
        head[name] = {"dtype": "BF16", "shape": list(np.shape(a)), "data_offsets": [off, off + len(b)]}
        blobs.append(b)
        off += len(b)
    hj = json.dumps(head).encode()
    hj += b" " * (-len(hj) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


def load_model(folder):
    with open(folder + "/config.json") as f:
        cfg = json.load(f)
    return cfg, read_safetensors(folder + "/model.safetensors")


# ---- small pieces ----------------------------------------------------------------------------------------
def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def logsigmoid(z):
    return -np.logaddexp(0.0, -z)


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def layer_norm_weight(x, w, eps):
    """The layers' norm: the weight is stored around zero."""
    return unit_rms(x, eps) * (1.0 + w)


# ---- rotary positions with YaRN ----------------------------------------------------------------------------
def rotary_tables(rot, positions):
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    f = np.array([base ** (-2.0 * i / dims) for i in range(half)])
    mag = 1.0
    sc = rot.get("scaling")
    if sc:
        factor, orig = float(sc["factor"]), float(sc["original"])

        def where(t):
            return dims * math.log(orig / (2.0 * math.pi * t)) / (2.0 * math.log(base))
        lo = max(math.floor(where(float(sc["fast"]))), 0)
        hi = min(math.ceil(where(float(sc["slow"]))), dims - 1)
        ramp = np.clip((np.arange(half) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        f = f / factor * ramp + f * (1.0 - ramp)
        mag = 0.1 * math.log(factor) + 1.0
    ang = np.asarray(positions, np.float64)[:, None] * f[None, :]
    return np.cos(ang) * mag, np.sin(ang) * mag


def rotate_interleaved(x, cos, sin):
    """x [T, H, D]; the first 2*cos.shape[1] dimensions of every head are rotated as pairs (2i, 2i+1)."""
    out = x.copy()
    n = 2 * cos.shape[1]
    a, b = x[..., 0:n:2], x[..., 1:n:2]
    c, s = cos[:, None, :], sin[:, None, :]
    out[..., 0:n:2] = a * c - b * s
    out[..., 1:n:2] = b * c + a * s
    return out


# ---- the attention side -----------------------------------------------------------------------------------
def chunked_attention(q, k, v, scale, size):
    """q [T, H, D], k [T, G, D], v [T, G, E]; token i sees j <= i of its own block of `size` positions."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]))
    for i in range(T):
        lo = (i // size) * size
        for h in range(H):
            g = h // (H // G)
            s = (k[lo:i + 1, g] @ q[i, h]) * scale
            p = np.exp(s - s.max())
            p /= p.sum()
            out[i, h] = p @ v[lo:i + 1, g]
    return out


def attention_side(h, w, pre, m, eps):
    T = h.shape[0]
    H, G, D, E = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[pre + "q"].T).reshape(T, H, D)
    k = (h @ w[pre + "k"].T).reshape(T, G, D)
    v = (h @ w[pre + "v"].T).reshape(T, G, E)
    if m.get("rot"):
        cos, sin = rotary_tables(m["rot"], np.arange(T))
        q, k = rotate_interleaved(q, cos, sin), rotate_interleaved(k, cos, sin)
    q, k = unit_rms(q, eps), unit_rms(k, eps)
    o = chunked_attention(q, k, v, float(m["scale"]), int(m["mask"]["size"]) if m.get("mask") else max(T, 1))
    return o.reshape(T, H * E) @ w[pre + "o"].T


# ---- the matrix-memory side ---------------------------------------------------------------------------------
def matrix_memory(q, k, v, ig, fg, state=None):
    """One head.  q, k [T, D], v [T, E], ig / fg [T] log gates.  state = (S [D, E], n [D], m) or None for zeros."""
    T, D = q.shape
    E = v.shape[1]
    S, n, m = (np.zeros((D, E)), np.zeros(D), 0.0) if state is None else state
    out = np.zeros((T, E))
    for t in range(T):
        m_new = max(fg[t] + m, ig[t])
        a, b = math.exp(fg[t] + m - m_new), math.exp(ig[t] - m_new)
        S = a * S + b * np.outer(k[t], v[t])
        n = a * n + b * k[t]
        m = m_new
        out[t] = (S.T @ q[t]) / (max(abs(n @ q[t]), math.exp(-m)) + 1e-6)
    return out, (S, n, m)


def memory_side(h, w, pre, m, eps):
    T = h.shape[0]
    H, D, E, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    q = (h @ w[pre + "q"].T).reshape(T, H, D) * D ** -0.5
    k = (h @ w[pre + "k"].T).reshape(T, H, D)
    v = (h @ w[pre + "v"].T).reshape(T, H, E)
    ig = cap * np.tanh((h @ w[pre + "i"].T + w[pre + "i.b"]) / cap)
    fg = logsigmoid(cap * np.tanh((h @ w[pre + "f"].T + w[pre + "f.b"]) / cap))
    o = np.zeros((T, H, E))
    for a in range(H):
        o[:, a], _ = matrix_memory(q[:, a], k[:, a], v[:, a], ig[:, a], fg[:, a])
    o = unit_rms(o, eps).reshape(T, H * E) * w[pre + "norm"] * sigmoid(h @ w[pre + "g"].T)
    return o @ w[pre + "o"].T


def parallel_mixer(h, w, pre, m, eps):
    left = attention_side(h, w, pre + "left.", m["left"], eps)
    right = memory_side(h, w, pre + "right.", m["right"], eps)
    return 0.5 * (unit_rms(left, eps) * w[pre + "left.out"] + unit_rms(right, eps) * w[pre + "right.out"])


# ---- the gated delta rule ---------------------------------------------------------------------------------
def causal_conv(x, taps):
    """x [T, C], taps [C, K]; the last column multiplies the current token, zeros before the start."""
    T, C = x.shape
    K = taps.shape[1]
    pad = np.concatenate([np.zeros((K - 1, C)), x], 0)
    out = np.zeros((T, C))
    for j in range(K):
        out += pad[j:j + T] * taps[:, j][None, :]
    return out


def delta_rule(q, k, v, beta, g, state=None):
    """One head.  q, k [T, D] (unit vectors, q scaled), v [T, E], beta [T], g [T, D] decays of the key channels."""
    T, D = q.shape
    E = v.shape[1]
    S = np.zeros((D, E)) if state is None else state
    out = np.zeros((T, E))
    for t in range(T):
        S = g[t][:, None] * S
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + np.outer(k[t], u)
        out[t] = S.T @ q[t]
    return out, S


def delta_mixer(h, w, pre, m, eps):
    T = h.shape[0]
    H, G, D, E = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ w[pre + "q"].T, w[pre + "q.conv"])).reshape(T, G, D)
    k = silu(causal_conv(h @ w[pre + "k"].T, w[pre + "k.conv"])).reshape(T, G, D)
    v = silu(causal_conv(h @ w[pre + "v"].T, w[pre + "v.conv"])).reshape(T, H, E)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * D ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    beta = sigmoid(h @ w[pre + "b"].T)
    dt = softplus((h @ w[pre + "a1"].T) @ w[pre + "a2"].T + w[pre + "dt_bias"]).reshape(T, H, D)
    g = np.exp(-np.exp(w[pre + "A_log"])[None, :, None] * dt)
    o = np.zeros((T, H, E))
    for a in range(H):
        b = a // (H // G)
        o[:, a], _ = delta_rule(q[:, b], k[:, b], v[:, a], beta[:, a], g[:, a])
    gate = sigmoid((h @ w[pre + "g1"].T) @ w[pre + "g2"].T).reshape(T, H, E)
    o = unit_rms(o, eps) * w[pre + "norm"][None, None, :] * gate
    return o.reshape(T, H * E) @ w[pre + "o"].T


# ---- feed-forward -----------------------------------------------------------------------------------------
def expert(h, w, pre, limit):
    g = np.minimum(h @ w[pre + "gate"].T, limit)
    u = np.clip(h @ w[pre + "up"].T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ w[pre + "down"].T


def route(z, top):
    """z [T, experts] -> (indices [T, top], weights [T, top]): largest logits, softmax over the chosen ones."""
    idx = np.argsort(-z, axis=1, kind="stable")[:, :top]
    zz = np.take_along_axis(z, idx, 1)
    p = np.exp(zz - zz.max(1, keepdims=True))
    return idx, p / p.sum(1, keepdims=True)


def moe(h, w, pre, m):
    T = h.shape[0]
    idx, wt = route(h @ w[pre + "router"].T, int(m["router"]["top"]))
    out = np.zeros((T, w[pre + "e0.down"].shape[0]))
    for t in range(T):
        for j in range(idx.shape[1]):
            out[t] += wt[t, j] * expert(h[t:t + 1], w, pre + "e%d." % idx[t, j], float(m["expert"]["limit"]))[0]
    if m.get("shared"):
        out += expert(h, w, pre + "shared.", float(m["shared"]["limit"]))
    return out


# ---- the model --------------------------------------------------------------------------------------------
def forward(cfg, w, tokens, layers_out=None):
    """Logits [T, vocab] of one whole sequence; layers_out (a list) receives the residual stream after every layer."""
    eps = float(cfg["norm"]["eps"])
    x = w["embed"][np.asarray(tokens)]
    for i, L in enumerate(cfg["layers"]):
        pre = "l%d." % i
        h = layer_norm_weight(x, w[pre + "norm1"], eps)
        if L["type"] == "parallel":
            y = parallel_mixer(h, w, pre + "mix.", L["mixer"], eps)
        elif L["type"] == "channel_delta":
            y = delta_mixer(h, w, pre + "mix.", L["mixer"], eps)
        else:
            raise ValueError(L["type"])
        if L.get("mlp"):
            y = y + moe(h, w, pre + "mlp.", L["mlp"])
        x = x + y
        if layers_out is not None:
            layers_out.append(x.copy())
    z = layer_norm_weight(x, w["final.norm"], eps) @ w["head"].T
    cap = cfg.get("logit_softcap")
    return cap * np.tanh(z / cap) if cap else z
