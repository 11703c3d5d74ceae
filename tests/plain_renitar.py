"""The Renitar design restated in numpy (float64), slowly and plainly: one function per mechanism, no cache, no batch,
nothing shared with the library.  A model is a configuration (the dict of config.json) and a dict name -> array.

    tokens -> embedding rows -> layers -> final norm -> head

A layer reads the stream once through ONE norm and adds both branches, times a constant m:
x <- x + m (mixer(n(x)) + ff(n(x))).  The norm's weight is stored around zero: n(x) = x / rms(x) * (1 + w).
A layer's mixer is either a linear recurrence with a decay per key channel (``gla``) or two mixers side by side whose
normed outputs are averaged (``parallel``): softmax attention within blocks of positions, and a linear recurrence with
one constant decay per head.  The feed-forward is a mixture of experts, some of which only hand their input on.
"""
import math

import numpy as np


# -- small pieces -----------------------------------------------------------------------------------------------------

def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last axis."""
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * w


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


_erf = np.vectorize(math.erf, otypes=[np.float64])


def gelu(z):
    """The exact form: z * Phi(z)."""
    return 0.5 * z * (1.0 + _erf(z / math.sqrt(2.0)))


def softmax(z):
    e = np.exp(z - z.max())
    return e / e.sum()


# -- pieces of the mixers ---------------------------------------------------------------------------------------------

def rotate_half(x, pos, base, dims):
    """x [heads, head size] at position ``pos``: entry i < dims/2 turns together with entry i + dims/2 by the angle
    pos * base^(-2i/dims); entries from ``dims`` on pass."""
    y = x.copy()
    half = dims // 2
    a = pos * np.array([base ** (-2.0 * i / dims) for i in range(half)])
    c, s = np.cos(a), np.sin(a)
    u, v = x[..., :half], x[..., half:dims]
    y[..., :half] = u * c - v * s
    y[..., half:dims] = v * c + u * s
    return y


def short_conv(u, w):
    """u [tokens, channels], w [channels, taps]: y[t] = sum_j w[:, j] * u[t - (taps-1) + j], zeros before token 0."""
    T, taps = u.shape[0], w.shape[1]
    y = np.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            s = t - (taps - 1) + j
            if s >= 0:
                y[t] += w[:, j] * u[s]
    return y


def sees(i, j, size):
    """Does the query at position i see the key at position j?  Causal, and with ``size`` only within its own block of
    ``size`` positions (blocks counted from position 0)."""
    return j <= i and (not size or i // size == j // size)


def linear_recurrence(q, k, v, decay):
    """One head.  q, k [tokens, dk], v [tokens, dv]; decay [tokens, dk] (a factor per key channel and token) or a
    number.  S_t = diag(decay_t) S_{t-1} + k_t v_t^T from S = 0;  o_t = S_t^T q_t."""
    T, dk = k.shape
    S = np.zeros((dk, v.shape[1]))
    o = np.zeros((T, v.shape[1]))
    for t in range(T):
        d = decay[t][:, None] if np.ndim(decay) else decay
        S = d * S + np.outer(k[t], v[t])
        o[t] = S.T @ q[t]
    return o


# -- mixers -----------------------------------------------------------------------------------------------------------

def gla_mixer(m, w, p, h, eps):
    """h [tokens, width].  Queries times dk^-1/2; the decay of key channel c is logistic(z_c)^(1/tau) with z from a
    low-rank path with a bias; every head's read-out is normed over its values (one weight for all heads), the heads
    are gated by silu(W_g h) and projected."""
    H, dk, dv, tau = int(m["heads"]), int(m["dim"]), int(m["vdim"]), float(m["tau"])
    T = h.shape[0]
    q = (h @ w[p + "q"].T).reshape(T, H, dk) * dk ** -0.5
    k = (h @ w[p + "k"].T).reshape(T, H, dk)
    v = (h @ w[p + "v"].T).reshape(T, H, dv)
    z = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "a2.b"]
    alpha = (sigmoid(z) ** (1.0 / tau)).reshape(T, H, dk)
    o = np.stack([linear_recurrence(q[:, a], k[:, a], v[:, a], alpha[:, a]) for a in range(H)], axis=1)     # [T, H, dv]
    o = rms_norm(o, w[p + "norm"], eps).reshape(T, H * dv)
    return (o * silu(h @ w[p + "g"].T)) @ w[p + "o"].T


def block_attention(m, w, p, h, eps):
    """Softmax attention of grouped queries: projections with biases, a short convolution over time on every channel of
    q, k and v, a norm over the whole q row and the whole k row, a rotation of the first entries of every q and k head,
    scores capped by a tanh, keys of the query's own block of positions only, a logistic gate per output entry."""
    H, G, dk, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    T = h.shape[0]
    q = h @ w[p + "q"].T + w[p + "q.b"]
    k = h @ w[p + "k"].T + w[p + "k.b"]
    v = h @ w[p + "v"].T + w[p + "v.b"]
    if m.get("conv"):
        q, k, v = short_conv(q, w[p + "q.conv"]), short_conv(k, w[p + "k.conv"]), short_conv(v, w[p + "v.conv"])
    q = rms_norm(q, w[p + "q.norm"], eps).reshape(T, H, dk)
    k = rms_norm(k, w[p + "k.norm"], eps).reshape(T, G, dk)
    v = v.reshape(T, G, dv)
    rot = m.get("rot")
    if rot and rot.get("dims"):
        q = np.stack([rotate_half(q[t], t, float(rot["base"]), int(rot["dims"])) for t in range(T)])
        k = np.stack([rotate_half(k[t], t, float(rot["base"]), int(rot["dims"])) for t in range(T)])
    size = int((m.get("mask") or {}).get("size") or 0)
    cap = float(m.get("softcap") or 0.0)
    o = np.zeros((T, H, dv))
    for i in range(T):
        js = [j for j in range(i + 1) if sees(i, j, size)]
        for a in range(H):
            g = a // (H // G)
            s = np.array([q[i, a] @ k[j, g] for j in js]) * float(m["scale"])
            if cap:
                s = cap * np.tanh(s / cap)
            pr = softmax(s)
            o[i, a] = sum(pr[n] * v[j, g] for n, j in enumerate(js))
    o = o.reshape(T, H * dv) * sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T + w[p + "o.b"]


def constant_decay_mixer(m, w, p, h, eps):
    """A linear recurrence whose head a forgets by the constant factor decay[a] a token: q, k, v through silu, no scale;
    the heads' read-outs are normed TOGETHER (one row of heads * dv entries), gated by logistic(W_g h) and projected."""
    H, dk, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    T = h.shape[0]
    q = silu(h @ w[p + "q"].T).reshape(T, H, dk)
    k = silu(h @ w[p + "k"].T).reshape(T, H, dk)
    v = silu(h @ w[p + "v"].T).reshape(T, H, dv)
    o = np.stack([linear_recurrence(q[:, a], k[:, a], v[:, a], float(m["decay"][a])) for a in range(H)], axis=1)
    o = rms_norm(o.reshape(T, H * dv), w[p + "norm"], eps)
    return (o * sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


def side_by_side_mixer(m, w, p, h, eps):
    """Two mixers read the same h; each output is normed over the model width with a weight of its own; the mean of the two."""
    a = block_attention(m["left"], w, p + "left.", h, eps)
    b = constant_decay_mixer(m["right"], w, p + "right.", h, eps)
    return 0.5 * (rms_norm(a, w[p + "left.out"], eps) + rms_norm(b, w[p + "right.out"], eps))


# -- feed-forward -----------------------------------------------------------------------------------------------------

def route(z, correction, top, scale):
    """Router logits z of one token -> (chosen experts, weights): scores are the softmax over ALL logits, the choice goes
    by score + correction (ties: the lower index), the weights are the scores themselves times ``scale``."""
    s = softmax(z)
    order = sorted(range(len(z)), key=lambda e: (-(s[e] + correction[e]), e))[:top]
    return order, [s[e] * scale for e in order]


def expert(w, p, h):
    return gelu(h @ w[p + "up"].T) @ w[p + "down"].T


def mixture(mlp, w, p, h):
    """h [tokens, width].  The last ``identity`` router outputs stand for experts that return their input."""
    r = mlp["router"]
    E, n_id, top, scale = int(r["experts"]), int(r.get("identity") or 0), int(r["top"]), float(r["scale"])
    y = np.zeros_like(h)
    zs = h @ w[p + "router"].T
    for t in range(h.shape[0]):
        chosen, wts = route(zs[t], w[p + "correction"], top, scale)
        for e, c in zip(chosen, wts):
            y[t] += c * (expert(w, f"{p}e{e}.", h[t]) if e < E else h[t])
    if mlp.get("shared"):
        y += expert(w, p + "shared.", h) * sigmoid(h @ w[p + "shared.sg"].T)
    return y


# -- the model --------------------------------------------------------------------------------------------------------

def layer(cfg, lc, w, i, x):
    eps = float(cfg["norm"]["eps"])
    p = f"l{i}."
    h = rms_norm(x, 1.0 + w[p + "norm1"], eps)
    if lc["type"] == "gla":
        y = gla_mixer(lc["mixer"], w, p + "mix.", h, eps)
    elif lc["type"] == "parallel":
        y = side_by_side_mixer(lc["mixer"], w, p + "mix.", h, eps)
    else:
        raise ValueError(lc["type"])
    if lc.get("mlp") is not None:
        y = y + mixture(lc["mlp"], w, p + "mlp.", h)
    return x + float(cfg["residual_mult"]) * y


def forward(cfg, w, tokens, keep_layers=False):
    """-> logits [tokens, vocab] (and the stream behind every layer)."""
    x = w["embed"][np.asarray(tokens)]
    kept = []
    for i, lc in enumerate(cfg["layers"]):
        x = layer(cfg, lc, w, i, x)
        kept.append(x.copy())
    logits = rms_norm(x, 1.0 + w["final.norm"], float(cfg["norm"]["eps"])) @ w["head"].T
    return (logits, kept) if keep_layers else logits


def greedy(cfg, w, prompt, n):
    ids = list(prompt)
    for _ in range(n):
        ids.append(int(np.argmax(forward(cfg, w, ids)[-1])))
    return ids[len(prompt):]
