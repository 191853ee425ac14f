"""A plain, slow Zamizen: every mechanism as one numpy function over a whole sequence, float64 throughout.

Nothing here is shared with the package: no cache, no state carried between calls, no kernels.  A sequence goes in
whole and every position's result comes out, so that the engine's cuttings (portions, decoding, batches) can be
held against it.  Weights are a dict of numpy arrays by tensor name; the configuration is the plain dict of
config.json.

Notation: T tokens, E the model's width, H query heads, G key/value heads, D key width per head, V value width per
head, C the latent's width, R the rotated width of a latent layer's heads.
"""
import math

import numpy as np

F = np.float64


def layer_norm(x, w, b, eps):
    """(x - mean) / sqrt(var + eps) * w + b with var the mean of squared deviations."""
    x = x.astype(F)
    xc = x - x.mean(axis=-1, keepdims=True)
    return xc / np.sqrt((xc * xc).mean(axis=-1, keepdims=True) + eps) * w.astype(F) + b.astype(F)


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis (eps inside the root), no weight."""
    x = x.astype(F)
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)


def silu(z):
    return z / (1.0 + np.exp(-z))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def causal_filter(u, taps_w):
    """y[t, c] = sum_j w[c, j] u[t - taps + 1 + j, c], u = 0 before the sequence.  u [T, channels]; w [channels, taps]."""
    T, n = u.shape
    taps = taps_w.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, n), dtype=F), u.astype(F)], axis=0)
    y = np.zeros((T, n), dtype=F)
    for j in range(taps):
        y += padded[j:j + T] * taps_w[:, j].astype(F)[None, :]
    return y


def plain_frequencies(base, dims):
    i = np.arange(dims // 2, dtype=F)
    return np.power(F(base), -2.0 * i / dims)


def stretched_frequencies(base, dims, factor, original, fast, slow):
    """Frequencies blended between f_i and f_i / factor by a ramp over the pair index, and the factor that
    multiplies cosines and sines: the ramp runs from the pair whose wavelength makes `fast` turns in `original`
    positions to the one that makes `slow` turns."""
    f = plain_frequencies(base, dims)

    def pair_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_of(fast)), 0)
    hi = min(math.ceil(pair_of(slow)), dims - 1)
    i = np.arange(dims // 2, dtype=F)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_neighbours(x, positions, freq, magnitude=1.0):
    """Pairs (2i, 2i+1) of the first 2 len(freq) entries of the last axis turned by position * freq[i].  x [T, heads, n]."""
    out = x.astype(F).copy()
    n = len(freq)
    angle = np.asarray(positions, dtype=F)[:, None] * freq[None, :]
    c, s = (np.cos(angle) * magnitude)[:, None, :], (np.sin(angle) * magnitude)[:, None, :]
    a, b = out[..., 0:2 * n:2].copy(), out[..., 1:2 * n:2].copy()
    out[..., 0:2 * n:2] = a * c - b * s
    out[..., 1:2 * n:2] = b * c + a * s
    return out


def rotate_halves(x, positions, freq, magnitude=1.0):
    """Pairs (i, i + n), n = len(freq), of the first 2n entries of the last axis turned by position * freq[i]."""
    out = x.astype(F).copy()
    n = len(freq)
    angle = np.asarray(positions, dtype=F)[:, None] * freq[None, :]
    c, s = (np.cos(angle) * magnitude)[:, None, :], (np.sin(angle) * magnitude)[:, None, :]
    a, b = out[..., :n].copy(), out[..., n:2 * n].copy()
    out[..., :n] = a * c - b * s
    out[..., n:2 * n] = b * c + a * s
    return out


def causal_softmax_attention(q, k, v, scale):
    """q [T, H, D], k [T, G, D], v [T, G, V]; head h reads key/value head h // (H / G); position t sees 0..t."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]), dtype=F)
    mask = np.tril(np.ones((T, T), dtype=bool))
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        s = np.where(mask, s, -np.inf)
        p = np.exp(s - s.max(axis=1, keepdims=True))
        out[:, h] = (p / p.sum(axis=1, keepdims=True)) @ v[:, g]
    return out


def attention_mixer(h, w, pre, m, eps, shared=None):
    """Projections with biases, a short causal filter on each of q, k, v, rotation of neighbouring pairs, unit RMS per
    head on q and k after it, causal softmax attention, output projection with bias.  `shared`: (k, v) of another
    layer to read instead of making them.  Returns (output [T, E], (k, v))."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = np.arange(T)
    freq = plain_frequencies(m["rot"]["base"], m["rot"]["dims"]) if m["rot"]["dims"] else np.zeros(0)

    def made(name):
        u = h @ w[pre + name].astype(F).T + w[pre + name + ".b"].astype(F)
        if (pre + name + ".conv") in w:
            u = causal_filter(u, w[pre + name + ".conv"])
        return u

    q = unit_rms(rotate_neighbours(made("q").reshape(T, H, D), pos, freq), eps)
    if shared is None:
        k = unit_rms(rotate_neighbours(made("k").reshape(T, G, D), pos, freq), eps)
        v = made("v").reshape(T, G, V)
    else:
        k, v = shared
    o = causal_softmax_attention(q, k, v, m["scale"]).reshape(T, H * V)
    return o @ w[pre + "o"].astype(F).T + w[pre + "o.b"].astype(F), (k, v)


def latent_mixer(h, w, pre, m, eps):
    """Queries straight from the input; keys and values as linear maps of one normed latent per token, plus one rotated
    key part shared by the heads; rotation of the two-halves pairing with stretched frequencies; a sigmoid gate on the
    concatenated heads; output projection."""
    T = h.shape[0]
    H, D, R, V, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = np.arange(T)
    rot = m["rot"]
    if rot.get("scaling"):
        s = rot["scaling"]
        freq, mag = stretched_frequencies(rot["base"], rot["dims"], s["factor"], s["original"], s["fast"], s["slow"])
    else:
        freq, mag = plain_frequencies(rot["base"], rot["dims"]), 1.0
    q = (h @ w[pre + "q"].astype(F).T).reshape(T, H, D + R)
    down = h @ w[pre + "dkv"].astype(F).T
    c = unit_rms(down[:, :C], eps) * w[pre + "dkv.norm"].astype(F)
    r = rotate_halves(down[:, None, C:], pos, freq, mag)[:, 0]                     # [T, R]
    q_rot = rotate_halves(q[..., D:], pos, freq, mag)
    k_plain = (c @ w[pre + "uk"].astype(F).T).reshape(T, H, D)
    v = (c @ w[pre + "uv"].astype(F).T).reshape(T, H, V)
    mask = np.tril(np.ones((T, T), dtype=bool))
    out = np.zeros((T, H, V), dtype=F)
    for i in range(H):
        s = (q[:, i, :D] @ k_plain[:, i].T + q_rot[:, i] @ r.T) * m["scale"]
        s = np.where(mask, s, -np.inf)
        p = np.exp(s - s.max(axis=1, keepdims=True))
        out[:, i] = (p / p.sum(axis=1, keepdims=True)) @ v[:, i]
    o = out.reshape(T, H * V) * sigmoid(h @ w[pre + "g"].astype(F).T)
    return o @ w[pre + "o"].astype(F).T


def dense_ff(h, w, pre):
    return (silu(h @ w[pre + "gate"].astype(F).T) * (h @ w[pre + "up"].astype(F).T)) @ w[pre + "down"].astype(F).T


def forward(cfg, w, tokens, layers_out=None):
    """Logits [T, vocab] of one sequence.  `layers_out`: a list that receives the stream after every layer."""
    eps, mult = cfg["norm"]["eps"], cfg["residual_mult"]
    x = w["embed"].astype(F)[np.asarray(tokens)]
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        pre = f"l{i}."

        def norm(name, y):
            return layer_norm(y, w[pre + name], w[pre + name + ".b"], eps)

        hin = norm("norm1", x)
        m = layer["mixer"]
        if layer["type"] == "attention":
            shared = kept[m["kv_from"]] if m.get("kv_from") is not None else None
            o, kv = attention_mixer(hin, w, pre + "mix.", m, eps, shared)
            kept[i] = kv
        elif layer["type"] == "latent_attention":
            o = latent_mixer(hin, w, pre + "mix.", m, eps)
        else:
            raise ValueError(layer["type"])
        x = x + mult * norm("norm1b", o)
        if layer.get("mlp") is not None:
            x = x + mult * norm("norm2b", dense_ff(norm("norm2", x), w, pre + "mlp."))
        if layers_out is not None:
            layers_out.append(x.copy())
    x = layer_norm(x, w["final.norm"], w["final.norm.b"], eps)
    return x @ w["head"].astype(F).T
