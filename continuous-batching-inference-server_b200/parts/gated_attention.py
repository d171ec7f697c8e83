"""Attention over the paged cache with separate projections, a distance bias, a query temperature and a gate per head."""
from __future__ import annotations

import math

import torch

from ..kernels import ops
from ..weights.loader import TensorDecl
from .base import CacheArray, CacheNeed, Delta, Mixer, register_mixer


class GatedAttention(Mixer):
    """q, k, v and a gate come from four matrices stored ``[out, in]`` (q, k, v with biases if ``qkv_bias``), run as
    ONE product.  Keys are ``head_dim`` wide, values ``v_head_dim`` (the two may differ); query head h reads
    key/value head h // (n_head / n_kv_head).  For the query at position p and the key at j <= p:

        score = (q . k) * scale * temperature(p) - slope_h * (p - j)
        temperature(p) = 1 + coef * ln(floor((p + 1) / every) + 1)          (``q_temp`` = (coef, every); None: 1)
        slope_h = 2^(-slope_power * (h + 1) / n_head)                        (``slope_power`` 0: no distance bias)

    inside ``window`` (p - j < window; 0: all keys), ordinary softmax in 32-bit.  Head h's output is multiplied by
    sigmoid(gate_h), one number per token and head read from the mixer's input (``head_gate``), and the heads side by
    side are projected out (no bias).  No rotation: positions enter through the bias and the temperature only.
    ``names``: what follows the layer's prefix in the names of q, k, v, the gate and the output matrix; a bias is
    its matrix's name with ``.b``."""

    def __init__(self, width: int, n_head: int, n_kv_head: int, head_dim: int, v_head_dim: int, scale: float,
                 window: int = 0, qkv_bias: bool = True, slope_power: float = 0.0, q_temp=None, head_gate: bool = True,
                 names=("mix.q", "mix.k", "mix.v", "mix.g", "mix.o")):
        if n_head % n_kv_head:
            raise ValueError(f"n_head={n_head} is not a multiple of n_kv_head={n_kv_head}")
        for what, v in (("head_dim", head_dim), ("v_head_dim", v_head_dim)):
            if not 0 < int(v) <= ops.ATTENTION_MAX_HEAD_DIM:
                raise ValueError(f"{what}={v} is outside 1..{ops.ATTENTION_MAX_HEAD_DIM}, the widest head any "
                                 f"attention kernel takes")
        self.width, self.n_head, self.n_kv_head = int(width), int(n_head), int(n_kv_head)
        self.head_dim, self.v_head_dim = int(head_dim), int(v_head_dim)
        self.scale, self.window, self.own_kv = float(scale), int(window), True
        self.qkv_bias, self.head_gate = bool(qkv_bias), bool(head_gate)
        self.slope_power = float(slope_power)
        self.q_temp = None if q_temp is None else (float(q_temp[0]), int(q_temp[1]))
        if self.q_temp is not None and self.q_temp[1] < 1:
            raise ValueError(f"q_temp: 'every' must be at least 1, got {self.q_temp[1]}")
        self.d_q, self.d_kv, self.d_v = self.n_head * self.head_dim, self.n_kv_head * self.head_dim, self.n_kv_head * self.v_head_dim
        self.names = tuple(names)
        self.w_in = self.b_in = self.w_out = self.slopes = None
        self.sinks = None

    def cache_need(self):
        return CacheNeed((CacheArray("k", self.n_kv_head, self.head_dim), CacheArray("v", self.n_kv_head, self.v_head_dim)),
                         self.window)

    def _shapes(self):
        return [self.d_q, self.d_kv, self.d_v] + ([self.n_head] if self.head_gate else [])

    def tensors(self, prefix):
        n = [prefix + s for s in self.names]
        out = []
        for name, rows, biased in zip(n[:4], self._shapes(), (True, True, True, False)):
            out.append(TensorDecl(name, (rows, self.width)))
            if biased and self.qkv_bias:
                out.append(TensorDecl(name + ".b", (rows,), "vector"))
        return out + [TensorDecl(n[4], (self.width, self.n_head * self.v_head_dim))]

    def load(self, prefix, tensors, dtype, device):
        n = [prefix + s for s in self.names]
        mats, biases = [], []
        for name, rows, biased in zip(n[:4], self._shapes(), (True, True, True, False)):
            mats.append(self._matrix(tensors[name], dtype, device))
            biases.append(self._vector(tensors[name + ".b"], device) if biased and self.qkv_bias
                          else torch.zeros(rows, dtype=torch.float32, device=device))
        self.w_in = torch.cat(mats).contiguous()              # q | k | v | gate: one product
        self.b_in = torch.cat(biases).contiguous() if self.qkv_bias else None
        self.w_out = self._matrix(tensors[n[4]], dtype, device)
        if self.slope_power:
            self.slopes = torch.tensor([2.0 ** (-self.slope_power * (h + 1) / self.n_head) for h in range(self.n_head)],
                                       dtype=torch.float64).to(torch.float32).to(device)

    def streamed_weights(self):
        return [self.w_in, self.w_out]

    def forward(self, ctx, h, cache, state):
        if cache is None:
            raise RuntimeError("attention needs a cache")
        T, HV = h.shape[0], self.n_head * self.v_head_dim
        proj = ops.linear(h, self.w_in, self.b_in)
        out = torch.empty((T, HV), dtype=h.dtype, device=h.device)
        ctx.attention(self, proj, cache, ctx.groups[cache.group], out)     # stores k and v, then attends
        if self.head_gate:
            g0 = self.d_q + self.d_kv + self.d_v
            ops.head_gate_mul(out, proj[:, g0:g0 + self.n_head], self.n_head, out)
        if ops.linear_residual(out, self.w_out, ctx.residual):
            return None
        return Delta(ops.linear(out, self.w_out, None, None, out_dtype=torch.float32))


register_mixer("gated_attention", GatedAttention)
