"""Windowed attention whose keys and values are projections of one cached latent vector per token."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorDecl
from .base import CacheArray, CacheNeed, Delta, Mixer, register_mixer


class LatentAttention(Mixer):
    """q = W_q h per head (``qk_dim`` wide); the latent c = unit_rms(W_dkv h) * weight (``rank`` wide, eps inside the
    root) is the only thing cached per token; per head k = W_uk c, v = W_uv c (``v_dim`` wide).  Scores
    (q . k) * scale over the keys inside ``window`` (0: all), ordinary softmax; the heads' outputs side by side are
    multiplied by sigmoid(W_g h) and projected out.  No position information enters.  With ``own_latent`` False the
    layer has no W_dkv and reads the latents another layer cached (its own W_uk, W_uv, window and the rest).

    The scores never need k: q . (W_uk c) = (W_uk^T q) . c, so queries are carried into the latent space (one
    product per head) and the paged attention kernels run with ONE shared key/value head of ``rank`` dims whose keys
    and values are both the cached latents; their output, still in the latent space, goes through W_uv per head.
    ``names``: what follows the layer's prefix in the tensors' names (q, dkv, the latent's norm weight, uk, uv, the
    output gate, the output projection)."""

    kv_arrays = ("c", "c")      # the pages that stand for keys and for values

    def __init__(self, width: int, n_head: int, qk_dim: int, v_dim: int, rank: int, scale: float, window: int = 0,
                 eps: float = 1e-5, own_latent: bool = True,
                 names=("mix.q", "mix.dkv", "mix.dkv.norm", "mix.uk", "mix.uv", "mix.g", "mix.o")):
        self.width, self.n_head, self.qk_dim, self.v_dim, self.rank = int(width), int(n_head), int(qk_dim), int(v_dim), int(rank)
        if not 0 < self.rank <= ops.ATTENTION_MAX_HEAD_DIM:
            raise ValueError(f"rank={rank} is outside 1..{ops.ATTENTION_MAX_HEAD_DIM}, the widest key any attention "
                             f"kernel takes")
        self.scale, self.window, self.eps, self.own_kv = float(scale), int(window), float(eps), bool(own_latent)
        # what the attention kernels read off a mixer: one key/value head of `rank` dims shared by all query heads
        self.n_kv_head, self.head_dim = 1, self.rank
        self.d_q, self.d_kv = self.n_head * self.rank, self.rank
        self.names = tuple(names)
        self.w_in = self.w_uk_t = self.w_uv = self.w_out = self.norm_w = None

    def cache_need(self):
        return CacheNeed((CacheArray("c", 1, self.rank),), self.window) if self.own_kv else None

    def tensors(self, prefix):
        n = [prefix + s for s in self.names]
        H, D, V, R, W = self.n_head, self.qk_dim, self.v_dim, self.rank, self.width
        own = [TensorDecl(n[1], (R, W)), TensorDecl(n[2], (R,), "norm_weight")] if self.own_kv else []
        return [TensorDecl(n[0], (H * D, W))] + own + [TensorDecl(n[3], (H * D, R)), TensorDecl(n[4], (H * V, R)),
                                                       TensorDecl(n[5], (H * V, W)), TensorDecl(n[6], (W, H * V))]

    def load(self, prefix, tensors, dtype, device):
        n = [prefix + s for s in self.names]
        H, D, V, R = self.n_head, self.qk_dim, self.v_dim, self.rank
        rows = [tensors[n[0]], tensors[n[5]]] + ([tensors[n[1]]] if self.own_kv else [])
        self.w_in = torch.cat([self._matrix(t, dtype, device) for t in rows]).contiguous()       # q | gate | latent
        if self.own_kv:
            self.norm_w = self._vector(tensors[n[2]], device)
        # per head [rank, qk_dim]: carries a head's query into the latent space
        self.w_uk_t = self._matrix(tensors[n[3]], dtype, device).view(H, D, R).transpose(1, 2).contiguous()
        self.w_uv = self._matrix(tensors[n[4]], dtype, device).view(H, V, R).contiguous()
        self.w_out = self._matrix(tensors[n[6]], dtype, device)

    def streamed_weights(self):
        return [self.w_in, self.w_out]

    def forward(self, ctx, h, cache, state):
        if cache is None:
            raise RuntimeError("latent attention needs a cache of latents: its own or the layer's it reads")
        T, H, R = h.shape[0], self.n_head, self.rank
        HD, HV = H * self.qk_dim, H * self.v_dim
        proj = ops.linear(h, self.w_in, None)
        qc = torch.empty((T, self.d_q + (R if self.own_kv else 0)), dtype=h.dtype, device=h.device)
        ops.linear_heads(proj[:, :HD], self.w_uk_t, qc[:, :self.d_q])
        if self.own_kv:
            ops.rms_norm(proj[:, HD + HV:], self.norm_w, self.eps, qc[:, self.d_q:])
        mixed = torch.empty((T, self.d_q), dtype=h.dtype, device=h.device)
        ctx.attention(self, qc, cache, ctx.groups[cache.group], mixed)     # stores the latents (if its own), then attends
        out = torch.empty((T, HV), dtype=h.dtype, device=h.device)
        ops.linear_heads(mixed, self.w_uv, out)
        ops.gate_mul(proj[:, HD:HD + HV], out, "sigmoid", out)
        if ops.linear_residual(out, self.w_out, ctx.residual):      # the product adds into the residual stream itself
            return None
        return Delta(ops.linear(out, self.w_out, None, None, out_dtype=torch.float32))


register_mixer("latent_attention", LatentAttention)
