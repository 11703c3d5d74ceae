"""The Gemosun design restated in numpy (float64), slowly and plainly: one function per mechanism, no cache, no batch,
nothing shared with the library.  A model is a configuration (the dict of config.json) and a dict name -> array.

    tokens -> embedding rows -> layers -> final layer norm -> head

A layer reads the stream x twice through two layer norms (a weight, no bias) and adds both branches at once:
X = x + mixer(ln1(x)) + ff(ln2(x)).  The stream that goes on is a learned mixture of the embedding output and of
every layer's result so far: x <- sum_j dwa[j] X_j.
"""
import math

import numpy as np


# -- small pieces -----------------------------------------------------------------------------------------------------

def layer_norm(x, w, eps):
    mu = x.mean(-1, keepdims=True)
    var = ((x - mu) ** 2).mean(-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def softmax(z):
    e = np.exp(z - z.max())
    return e / e.sum()


# -- positions --------------------------------------------------------------------------------------------------------

def rotation_frequencies(rot):
    """(frequency per pair, factor on cos and sin) of a rotation over ``rot['dims']`` entries, stretched for long
    contexts when ``rot['scaling']`` is given: slow pairs (long wavelengths) are divided by the factor, fast ones stay,
    with a linear ramp over the pair index in between."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=np.float64)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def pair_of(turns):              # the (real-valued) pair index whose wavelength makes `turns` turns over the original context
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(pair_of(float(sc["fast"]))), 0)
    hi = min(math.ceil(pair_of(float(sc["slow"]))), dims - 1)
    ramp = np.clip((np.arange(dims // 2) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_pairs(x, pos, freq, mult, dims):
    """x [.., head size] at position ``pos``: entries (2i, 2i+1), i < dims/2, turn by pos * freq[i]; the rest pass."""
    y = x.copy()
    a = pos * freq
    c, s = np.cos(a) * mult, np.sin(a) * mult
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    y[..., 0:dims:2] = u * c - v * s
    y[..., 1:dims:2] = v * c + u * s
    return y


# -- attention --------------------------------------------------------------------------------------------------------

def visible(i, size, pool):
    """(positions, blocks) that the query at position i sees: the last ``size`` positions, and every block of ``pool``
    positions that lies wholly before them (``pool`` 0 or None: no blocks; ``size`` 0 or None: every position)."""
    if not size:
        return list(range(i + 1)), []
    toks = [j for j in range(i + 1) if i - j < size]
    blocks = []
    if pool:
        b = 0
        while b * pool + pool - 1 <= i - size:
            blocks.append(b)
            b += 1
    return toks, blocks


def attention_mixer(h, m, w, p):
    """h [T, width] of ONE sequence from position 0 -> [T, width].  ``m``: the mixer's sizes; ``w``: name -> array;
    ``p``: the tensors' prefix."""
    T = h.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    rot = m.get("rot") or None
    mask = m.get("mask") or {}
    size, pool = mask.get("size"), mask.get("pool")
    q = (h @ w[p + "q"].T).reshape(T, H, D)
    k = (h @ w[p + "k"].T).reshape(T, G, D)
    v = k.copy()                                   # the values are the keys as projected
    if rot and rot["dims"]:
        f, mult = rotation_frequencies(rot)
        for t in range(T):
            q[t] = rotate_pairs(q[t], t, f, mult, rot["dims"])
            k[t] = rotate_pairs(k[t], t, f, mult, rot["dims"])
    gate = sigmoid(h @ w[p + "g"].T)               # [T, H]
    out = np.zeros((T, H, D))
    for t in range(T):
        toks, blocks = visible(t, size, pool)
        for hh in range(H):
            g = hh // (H // G)
            keys = [k[pool * b:pool * (b + 1), g].mean(0) for b in blocks] + [k[j, g] for j in toks]
            vals = [v[pool * b:pool * (b + 1), g].mean(0) for b in blocks] + [v[j, g] for j in toks]
            sc = np.array([q[t, hh] @ kk for kk in keys]) * m["scale"]
            pr = softmax(sc)
            out[t, hh] = (pr[:, None] * np.array(vals)).sum(0) * gate[t, hh]
    return out.reshape(T, H * D) @ w[p + "o"].T


# -- feed-forwards ----------------------------------------------------------------------------------------------------

def dense_ff(h, w, p):
    return (gelu_tanh(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def small_expert(h, w, p):
    return np.maximum(h @ w[p + "up"].T, 0.0) ** 2 @ w[p + "down"].T


def route(scores, top, groups):
    """One token's scores [experts] -> (chosen experts, their weights).  With ``groups`` = {count, keep}: the experts
    form ``count`` equal runs of neighbours, a run's score is the sum of its two largest scores, and only experts of the
    ``keep`` best runs can be chosen."""
    E = len(scores)
    allowed = np.ones(E, dtype=bool)
    if groups:
        n = int(groups["count"])
        per = E // n
        gs = [np.sort(scores[i * per:(i + 1) * per])[::-1][:2].sum() for i in range(n)]
        best = sorted(range(n), key=lambda i: (-gs[i], i))[:int(groups["keep"])]
        allowed[:] = False
        for i in best:
            allowed[i * per:(i + 1) * per] = True
    order = sorted((e for e in range(E) if allowed[e]), key=lambda e: (-scores[e], e))[:top]
    s = scores[order]
    return order, s / (s.sum() + 1e-20)


def expert_ff(h, mlp, w, p):
    r = mlp["router"]
    out = np.zeros((h.shape[0], w[p + "e0.down"].shape[0]))
    for t in range(h.shape[0]):
        s = sigmoid(w[p + "router"] @ h[t])
        chosen, wt = route(s, int(r["top"]), r.get("groups"))
        for e, a in zip(chosen, wt):
            out[t] += a * small_expert(h[t:t + 1], w, f"{p}e{e}.")[0]
    if mlp.get("shared"):
        out += small_expert(h, w, p + "shared.") * sigmoid(h @ w[p + "shared.sg"].T)
    return out


# -- the model --------------------------------------------------------------------------------------------------------

def forward(cfg, w, tokens, keep_layers=False):
    """tokens of ONE sequence -> logits [T, vocab] (and the stream after every layer if asked)."""
    w = {n: np.asarray(a, dtype=np.float64) for n, a in w.items()}
    eps = cfg["norm"]["eps"]
    x = w["embed"][np.asarray(tokens)]
    hist, after = [x], []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        y = x + attention_mixer(layer_norm(x, w[p + "norm1"], eps), layer["mixer"], w, p + "mix.")
        mlp = layer.get("mlp")
        if mlp:
            h2 = layer_norm(x, w[p + "norm2"], eps)
            y = y + (dense_ff(h2, w, p + "mlp.") if mlp["kind"] == "dense" else expert_ff(h2, mlp, w, p + "mlp."))
        hist.append(y)
        x = sum(w[p + "dwa"][j] * hist[j] for j in range(i + 2))
        after.append(x)
    logits = layer_norm(x, w["final.norm"], eps) @ w["head"].T
    return (logits, np.stack(after)) if keep_layers else logits


def generate_greedy(cfg, w, prompt, n_new):
    """The tokens a greedy loop adds to ``prompt`` (the first largest logit each time), recomputing everything."""
    toks, out = list(prompt), []
    for _ in range(n_new):
        nxt = int(np.argmax(forward(cfg, w, toks)[-1]))
        out.append(nxt)
        toks.append(nxt)
    return out
