"""Plain, slow restatement of the Vofelix design in float64 numpy, one function per mechanism.

It shares no code with the product path (krasis_b200/): tests compare the framework against these functions.
Weights are a dict name -> numpy array, the configuration is the dict that config.json holds.  A sequence is always
evaluated whole, token by token where the design is recurrent; there is no cache here.

Notation: W is [out, in] and applied as W @ h; positions count from 0.
"""
import math

import numpy as np


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z / (1.0 + np.exp(-z))


def softplus(z):
    return np.logaddexp(0.0, z)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def layer_norm(x, w, b, eps):
    mu = x.mean(-1, keepdims=True)
    var = ((x - mu) ** 2).mean(-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * w + b


def rms_norm(x, w, eps):
    return x / np.sqrt((x ** 2).mean(-1, keepdims=True) + eps) * w


def yarn_frequencies(dims, base, scaling):
    """Per-pair angular frequencies and the common amplitude of the rotation table."""
    i = np.arange(dims // 2, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])

    def dim_of(turns):
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(dim_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(dim_of(float(scaling["slow"]))), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_interleaved(x, pos, freq, amp):
    """x [..., T, n] with n >= 2 * len(freq); pairs (2i, 2i+1) of the first 2*len(freq) dims turn by pos * freq[i]."""
    out = x.copy()
    n = 2 * len(freq)
    a = pos[:, None] * freq[None, :]
    c, s = np.cos(a) * amp, np.sin(a) * amp
    u, v = x[..., 0:n:2], x[..., 1:n:2]
    out[..., 0:n:2] = u * c - v * s
    out[..., 1:n:2] = v * c + u * s
    return out


def latent_attention(h, w, p, m, eps):
    """Sliding-window attention over a shared latent with a per-head sink.  h [T, width]; w: mixer tensors by short name."""
    T = h.shape[0]
    H, dn, dr, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = np.arange(T, dtype=np.float64)
    rot = m.get("rot") or {}
    freq, amp = yarn_frequencies(rot.get("dims", 0), rot.get("base", 10000.0), rot.get("scaling")) if rot.get("dims", 0) else (np.zeros(0), 1.0)
    q = (h @ w["q"].T).reshape(T, H, dn + dr)
    dkv = h @ w["dkv"].T
    c = rms_norm(dkv[:, :r], w["dkv.norm"], eps)
    k_rot = rotate_interleaved(dkv[:, r:], pos, freq, amp)                      # one rotated key part for all heads
    q_rot = rotate_interleaved(q[:, :, dn:].transpose(1, 0, 2), pos, freq, amp)  # [H, T, dr]
    k_nope = (c @ w["uk"].T).reshape(T, H, dn)
    v = (c @ w["uv"].T).reshape(T, H, dv)
    out = np.zeros((T, H, dv))
    win = (m.get("mask") or {}).get("size") or T + 1          # no mask: every earlier position is seen
    for hd in range(H):
        s = (q[:, hd, :dn] @ k_nope[:, hd].T + q_rot[hd] @ k_rot.T) * m["scale"]
        i, j = np.arange(T)[:, None], np.arange(T)[None, :]
        s = np.where((i - j >= 0) & (i - j < win), s, -np.inf)
        sink = float(w["sink"][hd])
        mx = np.maximum(s.max(-1, keepdims=True), sink)
        e = np.exp(s - mx)
        den = e.sum(-1, keepdims=True) + np.exp(sink - mx)
        out[:, hd] = (e / den) @ v[:, hd]
    return out.reshape(T, H * dv) @ w["o"].T


def causal_conv(x, taps):
    """x [T, C], taps [C, K]; the last column multiplies the current token, zeros before the start."""
    T, C = x.shape
    K = taps.shape[1]
    xp = np.concatenate([np.zeros((K - 1, C)), x], 0)
    y = np.zeros((T, C))
    for j in range(K):
        y += xp[j:j + T] * taps[:, j][None, :]
    return y


def delta_mixer(h, w, m, eps):
    """Gated delta rule, token by token.  h [T, width]."""
    T = h.shape[0]
    H, Hk, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ w["q"].T, w["q.conv"])).reshape(T, Hk, dk)
    k = silu(causal_conv(h @ w["k"].T, w["k.conv"])).reshape(T, Hk, dk)
    v = silu(causal_conv(h @ w["v"].T, w["v.conv"])).reshape(T, H, dv)
    q = q / np.sqrt((q ** 2).sum(-1, keepdims=True) + 1e-6) * dk ** -0.5
    k = k / np.sqrt((k ** 2).sum(-1, keepdims=True) + 1e-6)
    beta = sigmoid(h @ w["b"].T)                                                # [T, H]
    decay = np.exp(-np.exp(w["A_log"])[None, :] * softplus(h @ w["a"].T + w["dt_bias"][None, :]))
    gate = silu(h @ w["g"].T).reshape(T, H, dv)
    rep = H // Hk
    S = np.zeros((H, dk, dv))
    o = np.zeros((T, H, dv))
    for t in range(T):
        for hd in range(H):
            kk, qq = k[t, hd // rep], q[t, hd // rep]
            S[hd] *= decay[t, hd]
            u = beta[t, hd] * (v[t, hd] - S[hd].T @ kk)
            S[hd] += np.outer(kk, u)
            o[t, hd] = S[hd].T @ qq
    o = o / np.sqrt((o ** 2).mean(-1, keepdims=True) + eps) * w["norm"][None, None, :] * gate
    return o.reshape(T, H * dv) @ w["o"].T


def feed_forward(h, w):
    return (gelu_tanh(h @ w["gate"].T) * (h @ w["up"].T)) @ w["down"].T


def token_side(x, tokens, layer, w, side_embed, dim, eps):
    e = side_embed[tokens][:, layer * dim:(layer + 1) * dim]
    y = (gelu_tanh(x @ w["gate"].T) * e) @ w["proj"].T
    return y / np.sqrt((y ** 2).mean(-1, keepdims=True) + eps) * w["norm"]


def sub(weights, prefix):
    n = len(prefix)
    return {k[n:]: v for k, v in weights.items() if k.startswith(prefix)}


def layer_schedule(cfg):
    """Layer indices in the order they run; a looped span appears `times` times.  Returns [(layer, starts_later_pass)]."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop or loop["times"] <= 1 or loop["stop"] <= loop["start"]:
        return [(i, False) for i in range(n)]
    out = [(i, False) for i in range(loop["start"])]
    for t in range(loop["times"]):
        for i in range(loop["start"], loop["stop"]):
            out.append((i, t > 0 and i == loop["start"]))
    out += [(i, False) for i in range(loop["stop"], n)]
    return out


def forward(cfg, weights, tokens, return_layers=False):
    """Logits [T, vocab] of one whole sequence (and the residual stream after every layer run)."""
    W = {k: np.asarray(v, dtype=np.float64) for k, v in weights.items()}
    tokens = np.asarray(tokens, dtype=np.int64)
    eps = cfg["norm"]["eps"]
    x0 = W["embed"][tokens] * cfg["embedding"]["scale"]
    x = x0.copy()
    trace = []
    for i, again in layer_schedule(cfg):
        L = cfg["layers"][i]
        p = f"l{i}."
        if again:
            x = x + x0
        h = layer_norm(x, W[p + "norm1"], W[p + "norm1.b"], eps)
        mw = sub(W, p + "mix.")
        if L["type"] == "latent_attention":
            y = latent_attention(h, mw, None, L["mixer"], eps)
        elif L["type"] == "delta":
            y = delta_mixer(h, mw, L["mixer"], eps)
        else:
            raise ValueError(L["type"])
        x = x + layer_norm(y, W[p + "norm1b"], W[p + "norm1b.b"], eps)
        if L.get("mlp"):
            h = layer_norm(x, W[p + "norm2"], W[p + "norm2.b"], eps)
            x = x + layer_norm(feed_forward(h, sub(W, p + "mlp.")), W[p + "norm2b"], W[p + "norm2b.b"], eps)
        if cfg.get("token_side"):
            x = x + token_side(x, tokens, i, sub(W, p + "side."), W["side.embed"], cfg["token_side"]["dim"], eps)
        trace.append(x.copy())
    logits = layer_norm(x, W["final.norm"], W["final.norm.b"], eps) @ W["head"].T
    return (logits, np.stack(trace)) if return_layers else logits
