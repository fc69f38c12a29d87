"""Plain, slow restatement of the Megolorn design in float64 numpy, one function per mechanism.

It shares no code with the product path (krasis_b200/): tests compare the framework against these functions.
Weights are a dict name -> numpy array, the configuration is the dict that config.json holds.  A sequence is always
evaluated whole; there is no cache here.

Notation: W is [out, in] and applied as W @ h; positions count from 0.  T tokens, H query heads, G key/value heads,
d = per-map query/key size, dv = value size.
"""
import numpy as np


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def layer_norm_nobias(x, w, eps):
    mu = x.mean(-1, keepdims=True)
    var = ((x - mu) ** 2).mean(-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * w


def rms_unit(x, eps):
    return x / np.sqrt((x ** 2).mean(-1, keepdims=True) + eps)


def rotary_frequencies(dims, base, factor=1.0):
    i = np.arange(dims // 2, dtype=np.float64)
    return base ** (-2.0 * i / dims) / factor


def rotate_pairs(x, pos, freq):
    """x [T, ..., n]; the pairs (2i, 2i+1), i < len(freq), of the last axis turn by pos[t] * freq[i]; the rest is kept."""
    out = x.copy()
    n = 2 * len(freq)
    if n == 0:
        return out
    shape = (len(pos),) + (1,) * (x.ndim - 2) + (len(freq),)
    ang = (np.asarray(pos, dtype=np.float64)[:, None] * freq[None, :]).reshape(shape)
    u, v = x[..., 0:n:2], x[..., 1:n:2]
    out[..., 0:n:2] = u * np.cos(ang) - v * np.sin(ang)
    out[..., 1:n:2] = v * np.cos(ang) + u * np.sin(ang)
    return out


def visible(T, chunk=None, window=None):
    """[T, T] boolean: may query i read key j.  Causal; chunk: same block of `chunk` positions; window: i - j < window."""
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    m = j <= i
    if chunk:
        m &= (i // chunk) == (j // chunk)
    if window:
        m &= (i - j) < window
    return m


def softmax_rows(s, mask):
    s = np.where(mask, s, -np.inf)
    s = s - s.max(-1, keepdims=True)
    e = np.exp(s)
    return e / e.sum(-1, keepdims=True)


def attention_keys_values(h, w, m, eps):
    """Keys after norm and rotation [T, G, 2, d] and values [T, G, dv] of a layer that projects its own."""
    T = h.shape[0]
    G, d, dv = m["kv_heads"], m["dim"], m["vdim"]
    k = (h @ w["k"].T + w["k.b"]).reshape(T, G, 2, d)
    v = (h @ w["v"].T + w["v.b"]).reshape(T, G, dv)
    k = rms_unit(k, eps) * w["k.norm"]
    rot = m.get("rot") or {}
    if rot.get("dims", 0):
        f = rotary_frequencies(rot["dims"], rot["base"], (rot.get("scaling") or {}).get("factor", 1.0))
        k = rotate_pairs(k, np.arange(T), f)
    return k, v


def differential_lambda(w, diff):
    return np.exp(np.sum(w["lq1"] * w["lk1"])) - np.exp(np.sum(w["lq2"] * w["lk2"])) + diff


def differential_attention(h, w, m, eps, kv=None):
    """h [T, W] -> (mixer output [T, W], (k, v) as a later layer may reuse them)."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w["q"].T + w["q.b"]).reshape(T, H, 2, d)
    q = rms_unit(q, eps) * w["q.norm"]
    rot = m.get("rot") or {}
    if rot.get("dims", 0):
        f = rotary_frequencies(rot["dims"], rot["base"], (rot.get("scaling") or {}).get("factor", 1.0))
        q = rotate_pairs(q, np.arange(T), f)
    k, v = kv if kv is not None else attention_keys_values(h, w, m, eps)
    mask = visible(T, chunk=(m.get("mask") or {}).get("size"))
    lam = differential_lambda(w, m["diff"])
    gate = sigmoid(h @ w["g"].T)                                   # [T, H]
    out = np.zeros((T, H, dv))
    for hh in range(H):
        g = hh // (H // G)
        a = []
        for mp in range(2):
            s = (q[:, hh, mp] @ k[:, g, mp].T) * m["scale"]
            a.append(softmax_rows(s, mask) @ v[:, g])
        o = a[0] - lam * a[1]
        o = rms_unit(o, eps) * (1.0 - m["diff"])
        out[:, hh] = o * gate[:, hh:hh + 1]
    return out.reshape(T, H * dv) @ w["o"].T, (k, v)


def clamped_glu(h, w, limit):
    g = np.minimum(h @ w["gate"].T, limit)
    u = np.clip(h @ w["up"].T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ w["down"].T


def silu_glu(h, gate, up, down):
    return (silu(h @ gate.T) * (h @ up.T)) @ down.T


def route(h, router_w, correction, top, groups, keep):
    """-> (chosen [T, top] indices into experts + identity experts, weights [T, top])."""
    z = h @ router_w.T
    z = z - z.max(-1, keepdims=True)
    s = np.exp(z) / np.exp(z).sum(-1, keepdims=True)
    c = s + correction
    T, E = c.shape
    if groups and groups > 1:
        gs = c.reshape(T, groups, E // groups).max(-1)
        best = np.argsort(-gs, axis=-1, kind="stable")[:, :keep]
        ok = np.zeros((T, groups), dtype=bool)
        np.put_along_axis(ok, best, True, axis=-1)
        c = np.where(np.repeat(ok, E // groups, axis=1), c, -np.inf)
    chosen = np.argsort(-c, axis=-1, kind="stable")[:, :top]
    return chosen, np.take_along_axis(s, chosen, axis=-1)


def mixture(h, w, mlp):
    r = mlp["router"]
    E, ident = r["experts"], r.get("identity", 0)
    grp = r.get("groups") or {}
    chosen, weight = route(h, w["router"], w["correction"], r["top"], grp.get("count", 1), grp.get("keep", 1))
    y = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, p in zip(chosen[t], weight[t]):
            if e >= E:
                assert e < E + ident
                y[t] += p * h[t]
            else:
                y[t] += p * silu_glu(h[t:t + 1], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"])[0]
    if mlp.get("shared"):
        y += silu_glu(h, w["shared.gate"], w["shared.up"], w["shared.down"])
    return y


def sub(weights, prefix):
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def forward(cfg, weights, tokens, collect=None):
    """tokens [T] -> logits [T, vocab]; `collect`, a list, receives the residual stream after every layer."""
    eps = cfg["norm"]["eps"]
    x = weights["embed"][np.asarray(tokens)] * cfg["embedding"]["scale"]
    kv = {}
    for i, L in enumerate(cfg["layers"]):
        assert L["type"] == "attention"
        h = layer_norm_nobias(x, weights[f"l{i}.norm1"], eps)
        m = L["mixer"]
        src = m.get("kv_from")
        y, kv[i] = differential_attention(h, sub(weights, f"l{i}.mix."), m, eps, kv[src] if src is not None else None)
        if L.get("mlp"):
            mw = sub(weights, f"l{i}.mlp.")
            if L["mlp"]["kind"] == "dense":
                y = y + clamped_glu(h, mw, L["mlp"]["limit"])
            else:
                y = y + mixture(h, mw, L["mlp"])
        x = x + y
        if collect is not None:
            collect.append(x.copy())
    return layer_norm_nobias(x, weights["final.norm"], eps) @ weights["head"].T
