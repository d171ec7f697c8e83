"""A selective state-space mixer (the recurrent form of state-space duality)."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorDecl
from .base import Delta, Mixer, StateNeed, register_mixer


class StateSpaceMixer(Mixer):
    """One input projection gives, side by side, a gate z (``heads * head_dim``), the values x (the same), B and C
    (``groups * state`` each) and a raw step size per head.  x | B | C pass a causal convolution per channel
    (``taps`` taps, bias) and silu.  Per head (head h reads group h // (heads / groups)), in 32-bit, with
    dt = softplus(raw + dt_bias): S <- exp(-exp(A_log) dt) S + dt B x^T, y = S^T C + D x.  The heads' y side by side
    are multiplied by silu(z), divided by their root mean square in ``norm_groups`` equal parts (eps inside the root),
    multiplied by a weight, and projected out.

    Per request the mixer keeps S (``heads x head_dim x state`` floats, zero at the start) and the convolution's last
    ``taps - 1`` inputs; a step walks each segment's rows in order from that state, so prompt portions cut anywhere,
    single decoded tokens and whole prompts give the same values.  Nothing is cached per token.
    ``names``: what follows the layer's prefix in the tensors' names (input projection, convolution, its bias,
    dt_bias, A_log, D, the norm's weight, output projection)."""

    def __init__(self, width: int, heads: int, head_dim: int, state: int, groups: int, taps: int, norm_groups: int,
                 eps: float, names=("mix.in", "mix.conv", "mix.conv.b", "mix.dt_bias", "mix.A_log", "mix.D", "mix.norm",
                                    "mix.o")):
        self.width, self.heads, self.head_dim, self.n_state = int(width), int(heads), int(head_dim), int(state)
        self.groups, self.taps, self.norm_groups, self.eps = int(groups), int(taps), int(norm_groups), float(eps)
        if self.heads % self.groups:
            raise ValueError(f"heads={heads} is not a multiple of groups={groups}")
        self.inner = self.heads * self.head_dim
        if self.inner % self.norm_groups:
            raise ValueError(f"heads * head_dim = {self.inner} is not a multiple of norm_groups={norm_groups}")
        if not 1 <= self.taps <= 8:
            raise ValueError(f"taps={taps} is outside 1..8, what the convolution kernel takes")
        if not 1 <= self.n_state <= 256:
            raise ValueError(f"state={state} is outside 1..256, what the recurrence kernel takes")
        self.channels = self.inner + 2 * self.groups * self.n_state
        self.d_proj = 2 * self.inner + 2 * self.groups * self.n_state + self.heads
        self.names = tuple(names)
        self.w_in = self.w_out = self.conv_w = self.conv_b = self.dt_bias = self.a_log = self.d_skip = self.norm_w = None

    def state_need(self):
        return StateNeed((self.inner * self.n_state + (self.taps - 1) * self.channels,), torch.float32)

    def tensors(self, prefix):
        n = [prefix + s for s in self.names]
        return [TensorDecl(n[0], (self.d_proj, self.width)), TensorDecl(n[1], (self.channels, self.taps)),
                TensorDecl(n[2], (self.channels,), "vector"), TensorDecl(n[3], (self.heads,), "vector"),
                TensorDecl(n[4], (self.heads,), "vector"), TensorDecl(n[5], (self.heads,), "vector"),
                TensorDecl(n[6], (self.inner,), "norm_weight"), TensorDecl(n[7], (self.width, self.inner))]

    def load(self, prefix, tensors, dtype, device):
        n = [prefix + s for s in self.names]
        self.w_in = self._matrix(tensors[n[0]], dtype, device)
        # the convolution's few weights and everything of the recurrence are applied in 32-bit
        self.conv_w, self.conv_b, self.dt_bias, self.a_log, self.d_skip, self.norm_w = (
            self._vector(tensors[k], device) for k in n[1:7])
        self.w_out = self._matrix(tensors[n[7]], dtype, device)

    def streamed_weights(self):
        return [self.w_in, self.w_out]

    def forward(self, ctx, h, cache, state):
        T, inner, cut = h.shape[0], self.inner, self.inner * self.n_state
        proj = ops.linear(h, self.w_in, None)                   # z | x B C | raw dt
        ssm_state, conv_state = state[:, :cut], state[:, cut:]
        xbc = torch.empty((T, self.channels), dtype=h.dtype, device=h.device)
        short = ctx.max_seg_rows <= ops.conv_rows_per_block()      # (a decode step) the convolution leaves the state itself
        ops.causal_conv_act(proj, inner, self.channels, self.conv_w, self.conv_b, conv_state, ctx.seg_slot, ctx.cu_rows,
                            ctx.n_segments, ctx.max_seg_rows, "silu", xbc, update_state=short and self.taps > 1)
        if not short:
            ops.conv_state_update(proj, inner, self.channels, self.taps, conv_state, ctx.seg_slot, ctx.cu_rows,
                                  ctx.n_segments)
        y = torch.empty((T, inner), dtype=torch.float32, device=h.device)
        ops.ssm_scan(xbc, proj, self.d_proj - self.heads, self.dt_bias, self.a_log, self.d_skip, ssm_state, ctx.seg_slot,
                     ctx.cu_rows, ctx.n_segments, self.heads, self.head_dim, self.n_state, self.groups, y,
                     max_seg_rows=ctx.max_seg_rows)
        g = torch.empty((T, inner), dtype=h.dtype, device=h.device)
        ops.rms_norm(y, self.norm_w, self.eps, g, parts=self.norm_groups, gate=proj[:, :inner], gate_act="silu")
        if ops.linear_residual(g, self.w_out, ctx.residual):        # the product adds into the residual stream itself
            return None
        return Delta(ops.linear(g, self.w_out, None, None, out_dtype=torch.float32))


register_mixer("mamba2", StateSpaceMixer)
