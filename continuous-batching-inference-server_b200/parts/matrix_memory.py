"""A matrix memory with exponential gates (the mLSTM layer of xLSTM)."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorDecl
from .base import Delta, Mixer, StateNeed, register_mixer


class MatrixMemoryMixer(Mixer):
    """Per head: q (``dim`` wide, times ``q_scale``), k (``dim``) and v (``v_dim``) from the mixer's input, a raw
    input gate and a raw forget gate (one number each, with biases).  In 32-bit, with li = cap tanh(i / cap),
    lf = logsigmoid(cap tanh(f / cap)) (``gate_cap`` 0: no cap) and a running maximum m that starts at 0:

        m' = max(lf + m, li);   S <- exp(lf + m - m') S + exp(li - m') k v^T;   n <- likewise with k alone
        y = S^T q / (max(|n . q|, exp(-m')) + 1e-6)

    Each head's y is divided by its root mean square (eps inside the root); the heads side by side are multiplied by a
    weight and by sigmoid(gate) (a gate as wide as the heads, from the mixer's input), and projected out.

    Per request the mixer keeps S, n and m (zero at the start), 32-bit; a step walks each segment's rows in order from
    that state, so prompt portions cut anywhere, single decoded tokens and whole prompts give the same values.
    Nothing is cached per token.  The two gates' projections are a product of their own with 32-bit results: they
    enter exponentials.  ``names``: what follows the layer's prefix in the tensors' names (q, k, v, the output gate,
    the input gate, the forget gate, the norm's weight, the output matrix); a gate's bias is its name with ``.b``."""

    def __init__(self, width: int, heads: int, dim: int, v_dim: int, gate_cap: float, eps: float, q_scale: float = None,
                 names=("mix.q", "mix.k", "mix.v", "mix.g", "mix.i", "mix.f", "mix.norm", "mix.o")):
        self.width, self.heads, self.dim, self.v_dim = int(width), int(heads), int(dim), int(v_dim)
        if not 0 < self.dim <= ops.MATRIX_MEMORY_MAX_DIM:
            raise ValueError(f"dim={dim} is outside 1..{ops.MATRIX_MEMORY_MAX_DIM}, what the recurrence kernel takes")
        self.gate_cap, self.eps = float(gate_cap), float(eps)
        self.q_scale = float(q_scale) if q_scale is not None else self.dim ** -0.5
        self.den_eps = 1e-6
        self.d_qk, self.d_v = self.heads * self.dim, self.heads * self.v_dim
        self.names = tuple(names)
        self.w_in = self.w_gates = self.i_bias = self.f_bias = self.norm_w = self.w_out = None

    def state_need(self):
        return StateNeed((ops.matrix_memory_state_floats(self.heads, self.dim, self.v_dim),), torch.float32)

    def tensors(self, prefix):
        n = [prefix + s for s in self.names]
        W, H = self.width, self.heads
        return [TensorDecl(n[0], (self.d_qk, W)), TensorDecl(n[1], (self.d_qk, W)), TensorDecl(n[2], (self.d_v, W)),
                TensorDecl(n[3], (self.d_v, W)), TensorDecl(n[4], (H, W)), TensorDecl(n[4] + ".b", (H,), "vector"),
                TensorDecl(n[5], (H, W)), TensorDecl(n[5] + ".b", (H,), "vector"),
                TensorDecl(n[6], (self.d_v,), "norm_weight"), TensorDecl(n[7], (W, self.d_v))]

    def load(self, prefix, tensors, dtype, device):
        n = [prefix + s for s in self.names]
        self.w_in = torch.cat([self._matrix(tensors[k], dtype, device) for k in n[:4]]).contiguous()    # q | k | v | gate
        self.w_gates = torch.cat([self._matrix(tensors[n[4]], dtype, device),
                                  self._matrix(tensors[n[5]], dtype, device)]).contiguous()          # input | forget
        self.i_bias, self.f_bias = self._vector(tensors[n[4] + ".b"], device), self._vector(tensors[n[5] + ".b"], device)
        self.norm_w = self._vector(tensors[n[6]], device)
        self.w_out = self._matrix(tensors[n[7]], dtype, device)

    def streamed_weights(self):
        return [self.w_in, self.w_out]

    def forward(self, ctx, h, cache, state):
        T = h.shape[0]
        proj = ops.linear(h, self.w_in, None)                                            # q | k | v | gate
        gates = ops.linear(h, self.w_gates, None, None, out_dtype=torch.float32)         # raw input | forget gates
        y = torch.empty((T, self.d_v), dtype=torch.float32, device=h.device)
        ops.matrix_memory(proj, 0, self.d_qk, 2 * self.d_qk, gates, self.i_bias, self.f_bias, self.gate_cap, self.q_scale,
                          self.den_eps, state, ctx.seg_slot, ctx.cu_rows, ctx.n_segments, self.heads, self.dim, self.v_dim, y,
                          max_seg_rows=ctx.max_seg_rows)
        g = torch.empty((T, self.d_v), dtype=h.dtype, device=h.device)
        g0 = 2 * self.d_qk + self.d_v
        ops.rms_norm(y, self.norm_w, self.eps, g, parts=self.heads, gate=proj[:, g0:g0 + self.d_v], gate_act="sigmoid",
                     gate_after=True)
        if ops.linear_residual(g, self.w_out, ctx.residual):
            return None
        return Delta(ops.linear(g, self.w_out, None, None, out_dtype=torch.float32))


register_mixer("mlstm", MatrixMemoryMixer)
