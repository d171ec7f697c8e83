"""A plain, slow implementation of the Vekedra design in float64 torch, one function per mechanism.

It shares no code with the engine: whole sequences only, no cache, no batching, loops over tokens where
the design is a recurrence.  ``config`` is the dict of a config.json, ``w`` a dict of tensors by name.
"""
import math

import torch


def layer_norm(x, weight, bias, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * weight + bias


def rms_unit(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def gated_feed_forward(h, gate, up, down):
    return (silu(h @ gate.T) * (h @ up.T)) @ down.T


def routed_experts(h, router, experts, top, gaps=None):
    """experts: list of (gate, up, down).  Scores are sigmoids of the router's logits; the ``top`` largest
    are taken as they are; each chosen expert is fed its score times h.  ``gaps`` (a list) takes, per row, how far
    the last chosen logit lies above the first one not chosen (a small gap is a close call that rounding may turn)."""
    z = h @ router.T
    s = torch.sigmoid(z)
    out = torch.zeros(h.shape[0], experts[0][2].shape[0], dtype=h.dtype)
    if gaps is not None:
        ranked = torch.sort(z, dim=1, descending=True).values
        gaps.append(ranked[:, top - 1] - ranked[:, top] if top < z.shape[1] else torch.full((h.shape[0],), float("inf")))
    for t in range(h.shape[0]):
        order = sorted(range(s.shape[1]), key=lambda e: (-s[t, e].item(), e))[:top]
        for e in order:
            out[t] += gated_feed_forward((s[t, e] * h[t])[None], *experts[e])[0]
    return out


def causal_conv_silu(u, taps_weight, bias):
    """u [T, C]; taps_weight [C, K] whose last column meets the current token; zeros before the start."""
    T, C = u.shape
    K = taps_weight.shape[1]
    padded = torch.cat([torch.zeros(K - 1, C, dtype=u.dtype), u])
    out = torch.zeros_like(u)
    for t in range(T):
        out[t] = (padded[t:t + K].T * taps_weight).sum(-1) + bias
    return silu(out)


def mamba2(h, p, m, eps):
    """p: the mixer's tensors by short name; m: the mixer's sizes."""
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    proj = h @ p["in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = causal_conv_silu(xbc, p["conv"], p["conv.b"])
    x = xbc[:, :inner].reshape(-1, H, P)
    B = xbc[:, inner:inner + G * N].reshape(-1, G, N)
    C = xbc[:, inner + G * N:].reshape(-1, G, N)
    dt = softplus(dt + p["dt_bias"])
    decay = torch.exp(-torch.exp(p["A_log"]) * dt)          # [T, H]
    S = torch.zeros(H, N, P, dtype=h.dtype)
    y = torch.zeros(h.shape[0], H, P, dtype=h.dtype)
    per_group = H // G
    for t in range(h.shape[0]):
        for hd in range(H):
            g = hd // per_group
            S[hd] = decay[t, hd] * S[hd] + dt[t, hd] * torch.outer(B[t, g], x[t, hd])
            y[t, hd] = S[hd].T @ C[t, g] + p["D"][hd] * x[t, hd]
    y = y.reshape(-1, inner) * silu(z)
    parts = m["norm_groups"]
    y = rms_unit(y.reshape(-1, parts, inner // parts), eps).reshape(-1, inner) * p["norm"]
    return y @ p["o"].T


def latent(h, p, eps):
    return rms_unit(h @ p["dkv"].T, eps) * p["dkv.norm"]


def latent_attention(h, c, p, m):
    """c: the latents [T, kv_rank] (this layer's own or another layer's)."""
    H, D, V, win = m["heads"], m["dim"], m["vdim"], m["mask"]["size"]
    T = h.shape[0]
    q = (h @ p["q"].T).reshape(T, H, D)
    k = (c @ p["uk"].T).reshape(T, H, D)
    v = (c @ p["uv"].T).reshape(T, H, V)
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for i in range(T):
        lo = max(0, i - win + 1)
        for hd in range(H):
            s = (k[lo:i + 1, hd] @ q[i, hd]) * m["scale"]
            out[i, hd] = torch.softmax(s, 0) @ v[lo:i + 1, hd]
    out = out.reshape(T, H * V) * torch.sigmoid(h @ p["g"].T)
    return out @ p["o"].T


def sub(w, prefix):
    return {k[len(prefix):]: v for k, v in w.items() if k.startswith(prefix)}


def forward(config, w, tokens, residuals=None, gaps=None):
    """Logits [T, vocab] of one whole sequence; ``residuals`` (a list) takes the stream after every layer,
    ``gaps`` (a list) every routed layer's gaps between chosen and not chosen experts."""
    w = {k: v.double() for k, v in w.items()}
    eps = config["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens)] * config["embedding"]["scale"]
    latents = {}
    for i, layer in enumerate(config["layers"]):
        pre = f"l{i}."
        h = layer_norm(x, w[pre + "norm1"], w[pre + "norm1.b"], eps)
        p, m = sub(w, pre + "mix."), layer["mixer"]
        if layer["type"] == "mamba2":
            mixed = mamba2(h, p, m, eps)
        elif layer["type"] == "latent_attention":
            src = m.get("kv_from")
            if src is None:
                latents[i] = latent(h, p, eps)
                src = i
            mixed = latent_attention(h, latents[src], p, m)
        else:
            raise ValueError(layer["type"])
        ff = layer.get("mlp")
        fed = torch.zeros_like(x)
        if ff is not None:
            q = sub(w, pre + "mlp.")
            if ff["kind"] == "dense":
                fed = gated_feed_forward(h, q["gate"], q["up"], q["down"])
            elif ff["kind"] == "moe":
                n = ff["router"]["experts"]
                experts = [(q[f"e{e}.gate"], q[f"e{e}.up"], q[f"e{e}.down"]) for e in range(n)]
                fed = routed_experts(h, q["router"], experts, ff["router"]["top"], gaps)
            else:
                raise ValueError(ff["kind"])
        x = x + (mixed + fed)
        if residuals is not None:
            residuals.append(x.clone())
    h = layer_norm(x, w["final.norm"], w["final.norm.b"], eps)
    return h @ w["head"].T
