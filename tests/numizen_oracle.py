"""Plain float64 statement of the Numizen design (numpy; one function per mechanism; shares no code with the product).

A model is (cfg, W): cfg the parsed config.json, W a dict name -> float64 array.  `forward` runs whole sequences from
position 0; `Stepper` runs one token at a time through explicit caches and recurrent states, which is the second,
independent statement that prefill is compared with.

Layer:            x <- x + ls1 * mixer(dyt1(x)) + ls2 * ff(dyt2(x))          (both read the same x)
Dynamic tanh:     dyt(x) = tanh(a x) * w + b                                  (scalar a; no statistics)
Loop:             layers [start, stop) run `times` times with the same weights, every pass with a cache / state of its own
"""
import math

import numpy as np


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def softplus(z):
    return np.logaddexp(0.0, z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rms_unit(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def dyt(x, W, name):
    return np.tanh(W[name + ".alpha"] * x) * W[name] + W[name + ".b"]


def layer_runs(cfg):
    """The order in which layers run: indices into cfg['layers'], looped segment repeated."""
    n = len(cfg["layers"])
    lp = cfg.get("loop")
    if not lp:
        return list(range(n))
    a, b, t = lp["start"], lp["stop"], lp["times"]
    return list(range(a)) + list(range(a, b)) * t + list(range(b, n))


# ---- rotary: interleaved pairs (2i, 2i+1) on the first `dims` entries ---------------------------------------------
def rotate(x, pos, dims, base):
    """x [..., T, n], pos [T]"""
    out = x.copy()
    half = dims // 2
    f = base ** (-2.0 * np.arange(half) / dims)
    ang = np.asarray(pos, dtype=np.float64)[:, None] * f[None, :]
    c, s = np.cos(ang), np.sin(ang)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


# ---- latent attention ---------------------------------------------------------------------------------------------
def latent_project(h, pos, m, W, p, eps):
    """h [T, width] -> q [H, T, dim + rot_dim] (rotated part last, rotated), c [T, kv_rank], kr [T, rot_dim] (rotated),
    gate [T, H * vdim]"""
    H, D, R, K = m["heads"], m["dim"], m["rot_dim"], m["kv_rank"]
    cq = rms_unit(h @ W[p + "dq"].T, eps) * W[p + "dq.norm"]
    q = (cq @ W[p + "uq"].T).reshape(len(h), H, D + R).transpose(1, 0, 2)
    kv = h @ W[p + "dkv"].T
    c = rms_unit(kv[:, :K], eps) * W[p + "dkv.norm"]
    kr = kv[:, K:]
    if m.get("rot"):                                           # no rotary setting: nothing is rotated
        dims, base = m["rot"]["dims"], m["rot"]["base"]
        q = np.concatenate([q[..., :D], rotate(q[..., D:], pos, dims, base)], axis=-1)
        kr = rotate(kr, pos, dims, base)
    return q, c, kr, h @ W[p + "g"].T


def latent_attend(q, qpos, c, kr, m, W, p):
    """queries q [H, Tq, D + R] at positions qpos against cached latents c [Tk, K], kr [Tk, R] of positions 0..Tk-1"""
    H, D, E = m["heads"], m["dim"], m["vdim"]
    Tk = len(c)
    k = (c @ W[p + "uk"].T).reshape(Tk, H, D).transpose(1, 0, 2)
    v = (c @ W[p + "uv"].T).reshape(Tk, H, E).transpose(1, 0, 2)
    s = (q[..., :D] @ k.transpose(0, 2, 1) + q[..., D:] @ kr.T[None]) * m["scale"]
    vis = np.arange(Tk)[None, :] <= np.asarray(qpos)[:, None]
    s = np.where(vis[None], s, -np.inf)
    s = s - s.max(axis=-1, keepdims=True)
    w = np.exp(s)
    w /= w.sum(axis=-1, keepdims=True)
    return (w @ v).transpose(1, 0, 2).reshape(len(qpos), H * E)


def latent_mixer(h, m, W, p, eps, cache=None, pos0=0):
    pos = np.arange(pos0, pos0 + len(h))
    q, c, kr, g = latent_project(h, pos, m, W, p, eps)
    if cache is not None:
        cache["c"] = c = np.concatenate([cache["c"], c]) if "c" in cache else c
        cache["kr"] = kr = np.concatenate([cache["kr"], kr]) if "kr" in cache else kr
    o = latent_attend(q, pos, c, kr, m, W, p)
    return (o * sigmoid(g)) @ W[p + "o"].T


# ---- gated linear attention -------------------------------------------------------------------------------------------
def gla_mixer(h, m, W, p, eps, state=None):
    """state: dict with 'S' [H, D, E] carried between calls (None: starts at zero, not kept)"""
    H, D, E, tau = m["heads"], m["dim"], m["vdim"], m["tau"]
    T = len(h)
    q = (h @ W[p + "q"].T).reshape(T, H, D) * D ** -0.5
    k = (h @ W[p + "k"].T).reshape(T, H, D)
    v = (h @ W[p + "v"].T).reshape(T, H, E)
    z = (h @ W[p + "a1"].T) @ W[p + "a2"].T + W[p + "a2.b"]
    decay = np.exp(-softplus(-z) / tau).reshape(T, H, D)          # sigmoid(z) ** (1 / tau)
    S = np.zeros((H, D, E)) if state is None or "S" not in state else state["S"]
    o = np.zeros((T, H, E))
    for t in range(T):
        S = decay[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = np.einsum("hde,hd->he", S, q[t])
    if state is not None:
        state["S"] = S
    o = rms_unit(o, eps) * W[p + "norm"]
    g = h @ W[p + "g"].T
    return (o.reshape(T, H * E) * (g * sigmoid(g))) @ W[p + "o"].T


# ---- feed-forward ---------------------------------------------------------------------------------------------------
def dense_ff(h, W, p):
    return (gelu_tanh(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def relu2_expert(h, W, p):
    return np.maximum(h @ W[p + "up"].T, 0.0) ** 2 @ W[p + "down"].T


def route(h, f, W, p):
    """-> chosen experts [T, top] and their weights"""
    r = f["router"]
    n, top = r["experts"], r["top"]
    z = h @ W[p + "router"].T
    z = z - z.max(axis=-1, keepdims=True)
    s = np.exp(z)
    s /= s.sum(axis=-1, keepdims=True)
    choice = s + W[p + "correction"]
    g = r.get("groups")
    if g:
        per = n // g["count"]
        best = choice.reshape(len(h), g["count"], per).max(axis=-1)
        order = np.argsort(-best, axis=-1, kind="stable")[:, : g["keep"]]
        allowed = np.zeros((len(h), g["count"]), dtype=bool)
        np.put_along_axis(allowed, order, True, axis=-1)
        choice = np.where(np.repeat(allowed, per, axis=-1), choice, -np.inf)
    picked = np.argsort(-choice, axis=-1, kind="stable")[:, :top]
    w = np.take_along_axis(s, picked, axis=-1)
    return picked, w / (w.sum(axis=-1, keepdims=True) + 1e-20)


def moe_ff(h, f, W, p):
    picked, w = route(h, f, W, p)
    out = np.zeros((len(h), W[p + "e0.down"].shape[0]))
    for t in range(len(h)):
        for j, e in enumerate(picked[t]):
            out[t] += w[t, j] * relu2_expert(h[t : t + 1], W, "%se%d." % (p, e))[0]
    if f.get("shared"):
        out += relu2_expert(h, W, p + "shared.") * sigmoid(h @ W[p + "shared.sg"].T)
    return out


def feed_forward(h, f, W, p):
    if f is None:
        return 0.0
    return dense_ff(h, W, p) if f["kind"] == "dense" else moe_ff(h, f, W, p)


# ---- the model --------------------------------------------------------------------------------------------------------
def embed(cfg, W, tokens, pos0=0):
    tokens = np.asarray(tokens)
    return W["embed"][tokens] + W["pos"][pos0 : pos0 + len(tokens)]


def run_layer(x, L, W, i, eps, carry=None, pos0=0):
    pre = "l%d." % i
    h1, h2 = dyt(x, W, pre + "norm1"), dyt(x, W, pre + "norm2")
    if L["type"] == "latent_attention":
        y = latent_mixer(h1, L["mixer"], W, pre + "mix.", eps, carry, pos0)
    elif L["type"] == "gla":
        y = gla_mixer(h1, L["mixer"], W, pre + "mix.", eps, carry)
    else:
        raise ValueError(L["type"])
    out = x + W[pre + "ls1"] * y
    if L.get("mlp") is not None:
        out = out + W[pre + "ls2"] * feed_forward(h2, L["mlp"], W, pre + "mlp.")
    return out


def forward(cfg, W, tokens, taps=None):
    """logits [T, vocab] of a whole sequence; taps (a list) receives the residual stream after every layer run"""
    eps = cfg["norm"]["eps"]
    x = embed(cfg, W, tokens)
    for i in layer_runs(cfg):
        x = run_layer(x, cfg["layers"][i], W, i, eps)
        if taps is not None:
            taps.append(x.copy())
    return dyt(x, W, "final.norm") @ W["head"].T


class Stepper:
    """Token-by-token decoding through explicit caches and states, one per layer RUN."""

    def __init__(self, cfg, W):
        self.cfg, self.W, self.t = cfg, W, 0
        self.carry = [dict() for _ in layer_runs(cfg)]

    def feed(self, tokens):
        cfg, W = self.cfg, self.W
        x = embed(cfg, W, tokens, self.t)
        for n, i in enumerate(layer_runs(cfg)):
            x = run_layer(x, cfg["layers"][i], W, i, cfg["norm"]["eps"], self.carry[n], self.t)
        self.t += len(tokens)
        return dyt(x, W, "final.norm") @ W["head"].T


# ---- random models ----------------------------------------------------------------------------------------------------
def bf16_round(a):
    a = np.asarray(a, dtype=np.float32)
    u = a.view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) >> 16 << 16
    return u.astype(np.uint32).view(np.float32).reshape(a.shape)


def tensor_shapes(cfg, gla_rank=8):
    """name -> shape of every tensor the design needs (the rank of the decay projection is a property of the tensors)"""
    Wd, out = cfg["width"], {}
    out["embed"] = (cfg["vocab"], Wd)
    out["pos"] = (cfg["max_positions"], Wd)
    out["head"] = (cfg["vocab"], Wd)

    def norm(n):
        out[n], out[n + ".b"], out[n + ".alpha"] = (Wd,), (Wd,), ()

    norm("final.norm")
    for i, L in enumerate(cfg["layers"]):
        p, m = "l%d." % i, L["mixer"]
        norm(p + "norm1")
        norm(p + "norm2")
        out[p + "ls1"] = out[p + "ls2"] = (Wd,)
        q = p + "mix."
        if L["type"] == "latent_attention":
            H, D, R, E = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
            out[q + "dq"], out[q + "dq.norm"] = (m["q_rank"], Wd), (m["q_rank"],)
            out[q + "uq"] = (H * (D + R), m["q_rank"])
            out[q + "dkv"], out[q + "dkv.norm"] = (m["kv_rank"] + R, Wd), (m["kv_rank"],)
            out[q + "uk"], out[q + "uv"] = (H * D, m["kv_rank"]), (H * E, m["kv_rank"])
            out[q + "g"], out[q + "o"] = (H * E, Wd), (Wd, H * E)
        else:
            H, D, E = m["heads"], m["dim"], m["vdim"]
            rank = gla_rank
            out[q + "q"] = out[q + "k"] = (H * D, Wd)
            out[q + "v"] = out[q + "g"] = (H * E, Wd)
            out[q + "o"], out[q + "norm"] = (Wd, H * E), (E,)
            out[q + "a1"], out[q + "a2"], out[q + "a2.b"] = (rank, Wd), (H * D, rank), (H * D,)
        f = L.get("mlp")
        if f is None:
            continue
        q = p + "mlp."
        if f["kind"] == "dense":
            out[q + "gate"] = out[q + "up"] = (f["ff"], Wd)
            out[q + "down"] = (Wd, f["ff"])
        else:
            for e in range(f["router"]["experts"]):
                out["%se%d.up" % (q, e)], out["%se%d.down" % (q, e)] = (f["expert"]["ff"], Wd), (Wd, f["expert"]["ff"])
            out[q + "router"], out[q + "correction"] = (f["router"]["experts"], Wd), (f["router"]["experts"],)
            if f.get("shared"):
                out[q + "shared.up"], out[q + "shared.down"] = (f["shared"]["ff"], Wd), (Wd, f["shared"]["ff"])
                out[q + "shared.sg"] = (1, Wd)
    return out


def random_weights(cfg, seed=0, gain=1.0, gla_rank=8):
    """bf16-representable float64 weights, scaled so that activations stay of order one"""
    rng = np.random.default_rng(seed)
    W = {}
    for name, shape in tensor_shapes(cfg, gla_rank).items():
        last = name.rsplit(".", 1)[-1]
        if last == "alpha":
            a = np.array(rng.uniform(0.5, 1.0))
        elif last == "b" and "norm" in name:
            a = 0.1 * rng.standard_normal(shape)
        elif last in ("norm", "norm1", "norm2", "ls1", "ls2"):
            a = 1.0 + 0.2 * rng.standard_normal(shape)
        elif last == "correction":
            a = 0.05 * rng.standard_normal(shape)
        elif name.endswith("a2.b"):
            a = 2.0 + rng.standard_normal(shape)
        elif len(shape) == 2 and name not in ("embed", "pos"):
            a = gain * rng.standard_normal(shape) / math.sqrt(shape[1])
        else:
            a = rng.standard_normal(shape) * (0.3 if name == "pos" else 1.0)
        W[name] = bf16_round(a).astype(np.float64)
    return W
