"""A plain, slow restatement of the Kapudra decoder in float64 numpy: one function per mechanism, token by
token where the mechanism is a recurrence, whole sequences otherwise.  It shares no code with the engine;
the tests compare the engine's kernels, cache and scheduler with it.

Conventions: ``w`` maps a tensor name to a float64 array; a linear weight is stored [out, in]; ``x`` is
[tokens, width] for one sequence whose first token sits at position 0.
"""
from __future__ import annotations

import math

import numpy as np

# ``forward(rounded=True)`` is the same model with what the bfloat16 engine hands from kernel to kernel in 16 bits
# rounded to bfloat16 (the norm's output that every projection reads, queries, keys and values of the attention, the
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


def log_sigmoid(z):
    return -np.logaddexp(0.0, -z)


def softplus(z):
    return np.logaddexp(0.0, z)


def silu(z):
    return z * sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


# ------------------------------------------------------------------------------ mechanisms
def biased_window_attention(q, k, v, heads, kv_heads, scale, window):
    """q [T, heads, dk], k [T, kv_heads, dk], v [T, kv_heads, dv].  Row i sees the ``window`` keys
    i-window+1..i; a key at distance d loses slope_h * d from its score, slope_h = 2^(-8 (h+1) / heads)."""
    T = q.shape[0]
    out = np.zeros((T, heads, v.shape[-1]))
    per = heads // kv_heads
    for h in range(heads):
        slope = 2.0 ** (-8.0 * (h + 1) / heads)
        g = h // per
        for i in range(T):
            lo = max(0, i - window + 1)
            s = (k[lo:i + 1, g] @ q[i, h]) * scale - slope * (i - np.arange(lo, i + 1))
            p = np.exp(s - s.max())
            out[i, h] = (p / p.sum()) @ v[lo:i + 1, g]
    return out


def causal_short_conv(x, taps):
    """x [T, C], taps [C, n]: y[t, c] = sum_j taps[c, j] x[t - (n-1) + j, c], zeros before the start."""
    T, C = x.shape
    n = taps.shape[1]
    padded = np.concatenate([np.zeros((n - 1, C)), x], axis=0)
    y = np.zeros((T, C))
    for j in range(n):
        y += padded[j:j + T] * taps[:, j]
    return y


def gated_delta_rule(q, k, v, beta, decay):
    """One head.  q, k [T, dk]; v [T, dv]; beta [T]; decay [T, dk] in (0, 1).  Returns o [T, dv]."""
    T, dk = q.shape
    S = np.zeros((dk, v.shape[1]))
    out = np.zeros((T, v.shape[1]))
    for t in range(T):
        S = decay[t][:, None] * S
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + np.outer(k[t], u)
        out[t] = S.T @ q[t]
    return out


def matrix_memory(q, k, v, log_i, log_f):
    """One head of the stabilised matrix memory.  q (already scaled), k [T, dk]; v [T, dv]; log gates [T]."""
    T, dk = q.shape
    S = np.zeros((dk, v.shape[1]))
    n = np.zeros(dk)
    m = 0.0
    out = np.zeros((T, v.shape[1]))
    for t in range(T):
        m_new = max(log_f[t] + m, log_i[t])
        a, b = math.exp(log_f[t] + m - m_new), math.exp(log_i[t] - m_new)
        S = a * S + b * np.outer(k[t], v[t])
        n = a * n + b * k[t]
        m = m_new
        out[t] = (S.T @ q[t]) / (max(abs(n @ q[t]), math.exp(-m)) + 1e-6)
    return out


# ------------------------------------------------------------------------------ mixers
def left_attention(h, w, p, c, eps):
    H, G, dk, dv = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    T = h.shape[0]
    q = rms(h @ w[p + ".q"].T, eps) * w[p + ".q.norm"]
    k = rms(h @ w[p + ".k"].T, eps) * w[p + ".k.norm"]
    v = h @ w[p + ".v"].T
    o = biased_window_attention(r16(q).reshape(T, H, dk), r16(k).reshape(T, G, dk), r16(v).reshape(T, G, dv), H, G,
                                c["scale"], c["mask"]["size"])
    return r16(o.reshape(T, H * dv)) @ w[p + ".o"].T


def right_delta(h, w, p, c, eps):
    H, G, dk, dv = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    T = h.shape[0]
    q = silu(causal_short_conv(h @ w[p + ".q"].T, w[p + ".q.conv"])).reshape(T, G, dk)
    k = silu(causal_short_conv(h @ w[p + ".k"].T, w[p + ".k.conv"])).reshape(T, G, dk)
    v = silu(causal_short_conv(h @ w[p + ".v"].T, w[p + ".v.conv"])).reshape(T, H, dv)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * dk ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    beta = sigmoid(h @ w[p + ".b"].T)                                            # [T, H]
    rate = np.exp(w[p + ".A_log"])                                               # [H]
    step = softplus((h @ w[p + ".a1"].T) @ w[p + ".a2"].T + w[p + ".dt_bias"]).reshape(T, H, dk)
    decay = np.exp(-rate[None, :, None] * step)
    gate = sigmoid((h @ w[p + ".g1"].T) @ w[p + ".g2"].T).reshape(T, H, dv)
    per = H // G
    o = np.stack([gated_delta_rule(q[:, x // per], k[:, x // per], v[:, x], beta[:, x], decay[:, x])
                  for x in range(H)], axis=1)                                    # [T, H, dv]
    o = rms(o, eps) * w[p + ".norm"] * gate
    return r16(o.reshape(T, H * dv)) @ w[p + ".o"].T


def side_by_side(h, w, p, c, eps):
    return (c["left_scale"] * left_attention(h, w, p + ".left", c["left"], eps)
            + c["right_scale"] * right_delta(h, w, p + ".right", c["right"], eps))


def mlstm(h, w, p, c, eps):
    H, dk, dv, cap = c["heads"], c["dim"], c["vdim"], c["gate_cap"]
    T = h.shape[0]
    q = (h @ w[p + ".q"].T).reshape(T, H, dk) * dk ** -0.5
    k = (h @ w[p + ".k"].T).reshape(T, H, dk)
    v = (h @ w[p + ".v"].T).reshape(T, H, dv)
    log_i = cap * np.tanh((h @ w[p + ".i"].T + w[p + ".i.b"]) / cap)
    log_f = log_sigmoid(cap * np.tanh((h @ w[p + ".f"].T + w[p + ".f.b"]) / cap))
    o = np.stack([matrix_memory(q[:, x], k[:, x], v[:, x], log_i[:, x], log_f[:, x]) for x in range(H)], axis=1)
    o = rms(o, eps).reshape(T, H * dv) * w[p + ".norm"] * sigmoid(h @ w[p + ".g"].T)
    return r16(o) @ w[p + ".o"].T


def dense_ff(h, w, p):
    return r16(gelu_tanh(h @ w[p + ".gate"].T) * (h @ w[p + ".up"].T)) @ w[p + ".down"].T


MIXERS = {"parallel": side_by_side, "mlstm": mlstm}


# ------------------------------------------------------------------------------ the model
def layer_order(config):
    """[(layer index, pass number or None when the layer opens no pass)]."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    runs = [(i, None) for i in range(a)]
    for t in range(times):
        runs += [(i, t if i == a else None) for i in range(a, b)]
    return runs + [(i, None) for i in range(b, n)]


def forward(config, w, tokens, layer_outputs=None, rounded=False):
    """Logits [T, vocab] of one whole sequence; ``layer_outputs`` (a list) receives the stream after
    every layer run; ``rounded``: see ``r16``."""
    _ROUND[0] = bool(rounded)
    try:
        return _forward(config, w, tokens, layer_outputs)
    finally:
        _ROUND[0] = False


def _forward(config, w, tokens, layer_outputs):
    w = {k: np.asarray(v, dtype=np.float64) for k, v in w.items()}
    eps = config["norm"]["eps"]
    x0 = w["embed"][np.asarray(tokens)] * config["embedding"]["scale"]
    x = x0.copy()
    for i, opens in layer_order(config):
        if opens is not None:
            if opens > 0:
                x = x + x0
            x = x + w["loop.step"][opens]
        L = config["layers"][i]
        p = f"l{i}"
        h = r16(rms(x, eps) * w[p + ".norm1"])
        y = MIXERS[L["type"]](h, w, p + ".mix", L["mixer"], eps)
        if L.get("mlp") is not None:
            y = y + dense_ff(h, w, p + ".mlp")
        x = x + y
        if layer_outputs is not None:
            layer_outputs.append(x.copy())
    z = r16(rms(x, eps) * w["final.norm"]) @ w["head"].T * config["logit_scale"]
    cap = config["logit_softcap"]
    return cap * np.tanh(z / cap)
