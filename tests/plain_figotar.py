"""A plain, slow implementation of the Figotar design in float64, one function per mechanism.

It shares no code with the engine: it takes a configuration dict (the keys of config.json) and a dict of
tensors by name (numpy arrays), runs one whole sequence, and returns the logits and the residual stream after every
layer.  Everything is written from the design's equations:

* norm: y = x / sqrt(mean(x^2) + eps) * (offset + w); the layers' norms and the final norm store w around zero
  (offset 1), the norms of the latents store it plainly (offset 0);
* a layer: x += post1(mixer(pre1(x))); x += post2(ff(pre2(x)));
* mixers: windowed attention with a distance bias, a query temperature and a gate per head; attention over a
  cached latent with a rotated key part shared by the heads, a sink in the softmax and a gate per head; a matrix
  memory with exponential gates held stable by a running maximum;
* feed-forward: down(gelu_tanh(gate h + b) * (up h + b)) + b.
"""
from __future__ import annotations

import math

import numpy as np


def rms_norm(x, w, eps, offset):
    x = np.asarray(x, dtype=np.float64)
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps) * (offset + np.asarray(w, dtype=np.float64))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def log_sigmoid(z):
    return -np.logaddexp(0.0, -z)


def linear(x, tensors, name, bias=False):
    y = x @ np.asarray(tensors[name], dtype=np.float64).T
    if bias:
        y = y + np.asarray(tensors[name + ".b"], dtype=np.float64)
    return y


def query_temperature(p, coef, every):
    """The factor on the query at position p: 1 + coef * ln(floor((p + 1) / every) + 1)."""
    return 1.0 + coef * math.log((p + 1) // every + 1)


def distance_slopes(heads):
    return np.array([2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)])


def softmax_with_sink(scores, sink=None):
    """Weights of the visible keys; with a sink the denominator also holds exp(sink), which has no value."""
    m = scores.max()
    if sink is not None:
        m = max(m, sink)
    e = np.exp(scores - m)
    den = e.sum() + (math.exp(sink - m) if sink is not None else 0.0)
    return e / den


def attention_rows(q, k, v, scale, window=0, slopes=None, temps=None, sinks=None):
    """q [T, H, D], k [T, G, D], v [T, G, V] of one sequence from position 0; the query at i sees the keys
    max(0, i - window + 1) .. i (window 0: all up to i).  slopes [H]: slope * (i - j) is taken off the score;
    temps [T]: a factor on the query at i; sinks [H].  Returns [T, H, V]."""
    T, H = q.shape[:2]
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]))
    for i in range(T):
        lo = max(0, i - window + 1) if window else 0
        for a in range(H):
            g = a // (H // G)
            s = (k[lo:i + 1, g] @ (q[i, a] * (temps[i] if temps is not None else 1.0))) * scale
            if slopes is not None:
                s = s - slopes[a] * (i - np.arange(lo, i + 1))
            out[i, a] = softmax_with_sink(s, None if sinks is None else sinks[a]) @ v[lo:i + 1, g]
    return out


def windowed_attention(h, tensors, prefix, cfg):
    """h: [T, width] from position 0.  Returns the mixer's output [T, width]."""
    T = h.shape[0]
    H, G, D, V = cfg["heads"], cfg["kv_heads"], cfg["dim"], cfg["vdim"]
    q = linear(h, tensors, prefix + "q", True).reshape(T, H, D)
    k = linear(h, tensors, prefix + "k", True).reshape(T, G, D)
    v = linear(h, tensors, prefix + "v", True).reshape(T, G, V)
    gate = sigmoid(linear(h, tensors, prefix + "g"))               # [T, H]
    temp = cfg.get("q_temp")
    temps = [query_temperature(i, temp["coef"], temp["every"]) for i in range(T)] if temp else None
    out = attention_rows(q, k, v, cfg["scale"], (cfg.get("mask") or {}).get("size", 0), distance_slopes(H), temps)
    out = out * gate[:, :, None]
    return linear(out.reshape(T, H * V), tensors, prefix + "o")


def rotate_half(x, positions, base, dims):
    """x: [T, ..., n]; the first ``dims`` entries of the last axis are rotated, entry i with entry i + dims/2."""
    x = np.array(x, dtype=np.float64)
    half = dims // 2
    f = base ** (-2.0 * np.arange(half) / dims)
    a = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]            # [T, half]
    shape = (x.shape[0],) + (1,) * (x.ndim - 2) + (half,)
    c, s = np.cos(a).reshape(shape), np.sin(a).reshape(shape)
    u, v = x[..., :half].copy(), x[..., half:dims].copy()
    x[..., :half] = u * c - v * s
    x[..., half:dims] = v * c + u * s
    return x


def latent_attention(h, tensors, prefix, cfg, eps):
    T = h.shape[0]
    H, D, R, V, C = cfg["heads"], cfg["dim"], cfg["rot_dim"], cfg["vdim"], cfg["kv_rank"]
    pos = np.arange(T)
    cq = rms_norm(linear(h, tensors, prefix + "dq"), tensors[prefix + "dq.norm"], eps, 0.0)
    q = linear(cq, tensors, prefix + "uq").reshape(T, H, D + R)
    q_plain, q_rot = q[..., :D], rotate_half(q[..., D:], pos, cfg["rot"]["base"], cfg["rot"]["dims"])
    dkv = linear(h, tensors, prefix + "dkv")
    c = rms_norm(dkv[:, :C], tensors[prefix + "dkv.norm"], eps, 0.0)
    k_rot = rotate_half(dkv[:, C:], pos, cfg["rot"]["base"], cfg["rot"]["dims"])       # [T, R], one for all heads
    k_plain = linear(c, tensors, prefix + "uk").reshape(T, H, D)
    v = linear(c, tensors, prefix + "uv").reshape(T, H, V)
    gate = sigmoid(linear(h, tensors, prefix + "g"))
    sinks = np.asarray(tensors[prefix + "sink"], dtype=np.float64)
    # the shared rotated part stands behind every head's own unrotated key
    q_full = np.concatenate([q_plain, q_rot], axis=-1)
    k_full = np.concatenate([k_plain, np.repeat(k_rot[:, None, :], H, axis=1)], axis=-1)
    out = attention_rows(q_full, k_full, v, cfg["scale"], 0, None, None, sinks)
    out = out * gate[:, :, None]
    return linear(out.reshape(T, H * V), tensors, prefix + "o")


def capped_gates(i_raw, f_raw, cap):
    """Log input gate and log forget gate from the raw ones (biases already added)."""
    return cap * np.tanh(i_raw / cap), log_sigmoid(cap * np.tanh(f_raw / cap))


def memory_steps(q, k, v, li, lf, state=None):
    """The recurrence alone: q, k [T, H, D] (q already scaled), v [T, H, V], log gates li, lf [T, H].
    ``state``: None (zeros) or (S [H, D, V], n [H, D], m [H]).  Returns y [T, H, V] and the state after the last row."""
    T, H, D = q.shape
    V = v.shape[2]
    if state is None:
        S, n, m = np.zeros((H, D, V)), np.zeros((H, D)), np.zeros(H)
    else:
        S, n, m = (np.array(a, dtype=np.float64) for a in state)
    y = np.zeros((T, H, V))
    for t in range(T):
        for a in range(H):
            m_new = max(lf[t, a] + m[a], li[t, a])
            keep, take = math.exp(lf[t, a] + m[a] - m_new), math.exp(li[t, a] - m_new)
            S[a] = keep * S[a] + take * np.outer(k[t, a], v[t, a])
            n[a] = keep * n[a] + take * k[t, a]
            m[a] = m_new
            y[t, a] = (S[a].T @ q[t, a]) / (max(abs(n[a] @ q[t, a]), math.exp(-m_new)) + 1e-6)
    return y, (S, n, m)


def mlstm(h, tensors, prefix, cfg, eps, state=None):
    """The matrix memory layer.  Returns the output [T, width] and the state after the last token."""
    T = h.shape[0]
    H, D, V, cap = cfg["heads"], cfg["dim"], cfg["vdim"], cfg["gate_cap"]
    q = linear(h, tensors, prefix + "q").reshape(T, H, D) * D ** -0.5
    k = linear(h, tensors, prefix + "k").reshape(T, H, D)
    v = linear(h, tensors, prefix + "v").reshape(T, H, V)
    li, lf = capped_gates(linear(h, tensors, prefix + "i", True), linear(h, tensors, prefix + "f", True), cap)
    o, state = memory_steps(q, k, v, li, lf, state)
    o = o / np.sqrt(np.mean(o * o, axis=-1, keepdims=True) + eps)
    o = o.reshape(T, H * V) * np.asarray(tensors[prefix + "norm"], dtype=np.float64) * sigmoid(linear(h, tensors, prefix + "g"))
    return linear(o, tensors, prefix + "o"), state


def dense_ff(h, tensors, prefix):
    a = gelu_tanh(linear(h, tensors, prefix + "gate", True)) * linear(h, tensors, prefix + "up", True)
    return linear(a, tensors, prefix + "down", True)


def forward(config, tensors, tokens):
    """Logits [T, vocab] of one whole sequence and the residual stream after every layer [layers, T, width]."""
    eps = config["norm"]["eps"]
    x = np.asarray(tensors["embed"], dtype=np.float64)[np.asarray(tokens)]
    stream = []
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        h = rms_norm(x, tensors[p + "norm1"], eps, 1.0)
        kind = layer["type"]
        if kind == "attention":
            y = windowed_attention(h, tensors, p + "mix.", layer["mixer"])
        elif kind == "latent_attention":
            y = latent_attention(h, tensors, p + "mix.", layer["mixer"], eps)
        elif kind == "mlstm":
            y, _ = mlstm(h, tensors, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(kind)
        x = x + rms_norm(y, tensors[p + "norm1b"], eps, 1.0)
        if layer.get("mlp") is not None:
            y = dense_ff(rms_norm(x, tensors[p + "norm2"], eps, 1.0), tensors, p + "mlp.")
            x = x + rms_norm(y, tensors[p + "norm2b"], eps, 1.0)
        stream.append(x.copy())
    logits = linear(rms_norm(x, tensors["final.norm"], eps, 1.0), tensors, "head")
    return logits, np.stack(stream)
