"""A plain, slow restatement of the Tutunex decoder in float64 numpy: one function per mechanism, token by token
where the mechanism is a recurrence, whole sequences otherwise.  It shares no code with the engine; the tests compare
the engine's kernels, cache and scheduler with it.

Conventions: ``w`` maps a tensor name to a float64 array; a linear weight is stored [out, in]; ``x`` is
[tokens, width] for one sequence whose first token sits at position 0.
"""
from __future__ import annotations

import math

import numpy as np

# ``forward(rounded=True)`` is the same model with what the bfloat16 engine hands from kernel to kernel in 16 bits
# rounded to bfloat16 (the norms' outputs that the projections read, queries, keys and values of the attentions, the
# activations in front of every output product) and nothing else changed: its distance from the unrounded model is
# what eight bits of mantissa at those places cost this very row, the yardstick for the engine's bfloat16 rows.
_ROUND = [False]


def r16(x):
    if not _ROUND[0]:
        return x
    bits = np.asarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    bits = (bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000
    return bits.astype(np.uint32).view(np.float32).astype(np.float64)


def rms(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.log1p(np.exp(-np.abs(z))) + np.maximum(z, 0.0)


# ------------------------------------------------------------------------------ rotation
def rotary_frequencies(rot):
    """(frequency of every pair, what cos and sin are multiplied by)."""
    n, base = rot["dims"], rot["base"]
    i = np.arange(n // 2, dtype=np.float64)
    f = base ** (-2.0 * i / n)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    where = lambda turns: n * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo, hi = max(math.floor(where(sc["fast"])), 0), min(math.ceil(where(sc["slow"])), n - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / sc["factor"] * ramp + f * (1.0 - ramp), 0.1 * math.log(sc["factor"]) + 1.0


def rotate(x, positions, rot):
    """x [T, units, channels]: the first rot['dims'] channels of every unit turn, channel i paired with i + dims/2."""
    f, amp = rotary_frequencies(rot)
    half = rot["dims"] // 2
    a = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]
    c, s = (np.cos(a) * amp)[:, None, :], (np.sin(a) * amp)[:, None, :]
    y = x.copy()
    u, v = x[..., :half], x[..., half:2 * half]
    y[..., :half] = u * c - v * s
    y[..., half:2 * half] = v * c + u * s
    return y


# ------------------------------------------------------------------------------ masks and softmaxes
def visible(T, chunk=None):
    """[query, key]: key j <= query i, and in the same chunk when chunks are given."""
    i = np.arange(T)
    m = i[None, :] <= i[:, None]
    if chunk:
        m &= (i[None, :] // chunk) == (i[:, None] // chunk)
    return m


def softmax_rows(s, mask, sink=False):
    """Softmax over the visible keys of every row; ``sink`` adds one term exp(0) to the denominator only."""
    s = np.where(mask, s, -np.inf)
    top = s.max(-1, keepdims=True)
    if sink:
        top = np.maximum(top, 0.0)
    e = np.exp(s - top)
    return e / (e.sum(-1, keepdims=True) + (np.exp(-top) if sink else 0.0))


# ------------------------------------------------------------------------------ mixers
def difference_lambda(w, p, m):
    return math.exp(float(w[p + ".lq1"] @ w[p + ".lk1"])) - math.exp(float(w[p + ".lq2"] @ w[p + ".lk2"])) + m["diff"]


def differential_attention(h, w, p, m, eps, shared):
    """Two score maps per head over the same values; ``shared`` maps a layer index to the (keys, values) it made."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = np.arange(T)
    q = (h @ w[p + ".q"].T).reshape(T, 2 * H, d)
    if m.get("rot"):
        q = rotate(q, pos, m["rot"])
    q = r16(q)
    if m.get("kv_from") is not None:
        k, v = shared[m["kv_from"]]
    else:
        k = (h @ w[p + ".k"].T).reshape(T, 2 * G, d)
        if m.get("rot"):
            k = rotate(k, pos, m["rot"])
        k, v = r16(k), r16((h @ w[p + ".v"].T).reshape(T, G, dv))
    lam = difference_lambda(w, p, m)
    mask = visible(T, m["mask"]["size"] if m.get("mask") else None)
    out = np.zeros((T, H, dv))
    for head in range(H):
        g = head // (H // G)
        a = [softmax_rows((q[:, 2 * head + i] @ k[:, 2 * g + i].T) * m["scale"], mask) @ v[:, g] for i in range(2)]
        out[:, head] = rms(a[0] - lam * a[1], eps) * (1.0 - m["diff"])
    return r16(out.reshape(T, H * dv)) @ w[p + ".o"].T, (k, v)


def sink_attention(h, w, p, m, eps):
    """Causal attention without positions, queries and keys normalised per head, a sink in the denominator."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = r16(rms((h @ w[p + ".q"].T).reshape(T, H, d), eps) * w[p + ".q.norm"])
    k = r16(rms((h @ w[p + ".k"].T).reshape(T, G, d), eps) * w[p + ".k.norm"])
    v = r16((h @ w[p + ".v"].T).reshape(T, G, dv))
    mask = visible(T)
    out = np.zeros((T, H, dv))
    for head in range(H):
        g = head // (H // G)
        out[:, head] = softmax_rows((q[:, head] @ k[:, g].T) * m["scale"], mask, sink=True) @ v[:, g]
    return r16(out.reshape(T, H * dv)) @ w[p + ".o"].T


def causal_short_conv(x, taps):
    """y[t, c] = sum_j taps[c, j] x[t - (n - 1) + j, c], zeros before the start."""
    T, C = x.shape
    n = taps.shape[1]
    padded = np.concatenate([np.zeros((n - 1, C)), x])
    return sum(padded[j:j + T] * taps[:, j][None, :] for j in range(n))


def gated_delta_rule(q, k, v, beta, decay):
    """Token by token, per head: S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q.
    q, k [T, H, d], v [T, H, dv], beta and decay [T, H]."""
    T, H, d = q.shape
    out = np.zeros_like(v)
    for head in range(H):
        S = np.zeros((d, v.shape[2]))
        for t in range(T):
            S = decay[t, head] * S
            u = beta[t, head] * (v[t, head] - S.T @ k[t, head])
            S = S + np.outer(k[t, head], u)
            out[t, head] = S.T @ q[t, head]
    return out


def delta_mixer(h, w, p, m, eps):
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    unit = lambda x: x / np.sqrt(np.sum(x * x, axis=-1, keepdims=True) + 1e-6)
    q = unit(silu(causal_short_conv(h @ w[p + ".q"].T, w[p + ".q.conv"])).reshape(T, G, d)) * d ** -0.5
    k = unit(silu(causal_short_conv(h @ w[p + ".k"].T, w[p + ".k.conv"])).reshape(T, G, d))
    v = silu(causal_short_conv(h @ w[p + ".v"].T, w[p + ".v.conv"])).reshape(T, H, dv)
    beta = sigmoid(h @ w[p + ".b"].T)
    decay = np.exp(-np.exp(w[p + ".A_log"]) * softplus(h @ w[p + ".a"].T + w[p + ".dt_bias"]))
    rep = H // G
    o = gated_delta_rule(np.repeat(q, rep, axis=1), np.repeat(k, rep, axis=1), v, beta, decay)
    o = rms(o, eps) * w[p + ".norm"] * silu(h @ w[p + ".g"].T).reshape(T, H, dv)
    return r16(o.reshape(T, H * dv)) @ w[p + ".o"].T


def side_by_side(h, w, p, m, eps):
    a = sink_attention(h, w, p + ".left", m["left"], eps)
    b = delta_mixer(h, w, p + ".right", m["right"], eps)
    return 0.5 * (rms(a, eps) * w[p + ".left.out"] + rms(b, eps) * w[p + ".right.out"])


def clamped_ff(h, w, p, c):
    g = np.minimum(h @ w[p + ".gate"].T, c["limit"])
    u = np.clip(h @ w[p + ".up"].T, -c["limit"], c["limit"])
    return r16(g * sigmoid(1.702 * g) * (u + 1.0)) @ w[p + ".down"].T


# ------------------------------------------------------------------------------ the model
def forward(config, w, tokens, layer_outputs=None, rounded=False):
    """Logits [T, vocab] of one whole sequence; ``layer_outputs`` (a list) receives the stream after every layer;
    ``rounded``: see ``r16``."""
    _ROUND[0] = bool(rounded)
    try:
        return _forward(config, w, tokens, layer_outputs)
    finally:
        _ROUND[0] = False


def _forward(config, w, tokens, layer_outputs):
    w = {k: np.asarray(v, dtype=np.float64) for k, v in w.items()}
    eps = config["norm"]["eps"]
    x = w["embed"][np.asarray(tokens)] * config["embedding"]["scale"]
    shared = {}
    for i, L in enumerate(config["layers"]):
        p = f"l{i}"
        h = r16(rms(x, eps) * w[p + ".norm1"])
        if L["type"] == "attention":
            y, shared[i] = differential_attention(h, w, p + ".mix", L["mixer"], eps, shared)
        else:
            y = side_by_side(h, w, p + ".mix", L["mixer"], eps)
        x = x + rms(y, eps) * w[p + ".norm1b"]
        if L.get("mlp") is not None:
            h = r16(rms(x, eps) * w[p + ".norm2"])
            x = x + rms(clamped_ff(h, w, p + ".mlp", L["mlp"]), eps) * w[p + ".norm2b"]
        if layer_outputs is not None:
            layer_outputs.append(x.copy())
    return r16(rms(x, eps) * w["final.norm"]) @ w["head"].T
