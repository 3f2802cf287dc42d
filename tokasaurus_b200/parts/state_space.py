"""A selective state space mixer in the state-space-duality form (Mamba-2): a matrix state per head, driven by inputs
that pass a short causal convolution, with a step size per head and token.

One product makes [z | x | B | C | dt] from the input: z and x have ``heads * vdim`` values, B and C ``groups * state``,
dt ``heads``.  x, B and C together pass a causal convolution over time on every channel (``taps`` taps with a bias, the
last tap on the current token, zeros before the request's first token) and SiLU.  Then, per head h of group g,

    dt = softplus(dt + dt_bias_h),   S_t = exp(-exp(A_h) dt) S_(t-1) + dt B_t x_t^T,   y_t = S_t^T C_t + D_h x_t

(S is state x vdim).  y * silu(z) is RMS-normed in ``norm_groups`` equal parts, scaled by a weight vector, and
projected.  What a request carries from token to token, in its slot: the states (float32, zero at admission) and the
convolution's last ``taps - 1`` inputs.  Step sizes, decays, the recurrence, the gate and the norm are float32; the
input product leaves float32 values.
"""

from __future__ import annotations

import torch

from tokasaurus_b200.kernels import ops
from tokasaurus_b200.parts.base import Mixer, StateNeed, WeightSpec
from tokasaurus_b200.parts.recurrent import _rows


class SelectiveStateSpace(Mixer):
    graph_safe = True

    def __init__(self, width: int, n_heads: int, vdim: int, state: int, groups: int, norm_groups: int, taps: int,
                 norm_eps: float, in_name: str, conv_name: str, conv_bias_name: str, dt_bias_name: str, a_log_name: str,
                 d_name: str, norm_name: str, o_name: str):
        if n_heads % groups:
            raise ValueError(f"{n_heads} heads do not divide into {groups} groups")
        if (n_heads * vdim) % norm_groups:
            raise ValueError(f"{n_heads * vdim} inner values do not divide into {norm_groups} norm groups")
        if taps < 1:
            raise ValueError(f"a convolution needs at least one tap, got {taps}")
        self.width, self.n_heads, self.vdim, self.state, self.groups = width, n_heads, vdim, state, groups
        self.norm_groups, self.taps, self.norm_eps = norm_groups, int(taps), float(norm_eps)
        self.inner = n_heads * vdim
        self.channels = self.inner + 2 * groups * state
        self.names = dict(w_in=in_name, conv=conv_name, conv_b=conv_bias_name, dt_bias=dt_bias_name, a_log=a_log_name,
                          d=d_name, norm=norm_name, o=o_name)
        self.defines = ops.decay_recurrence_defines(state, vdim)
        self.walk_builds = ops.decay_walk_modules(state, vdim)

    def weight_specs(self):
        n, H = self.names, self.n_heads
        return (WeightSpec(n["w_in"], (2 * self.inner + 2 * self.groups * self.state + H, self.width)),
                WeightSpec(n["conv"], (self.channels, self.taps), role="vector"),
                WeightSpec(n["conv_b"], (self.channels,), role="vector"),
                WeightSpec(n["dt_bias"], (H,), role="vector"), WeightSpec(n["a_log"], (H,), role="vector"),
                WeightSpec(n["d"], (H,), role="vector"), WeightSpec(n["norm"], (self.inner,), role="vector"),
                WeightSpec(n["o"], (self.width, self.inner)))

    def kernel_modules(self, dtype):
        return tuple(("decay_recurrence.cu", d) for d in self.walk_builds) + (("post_norm.cu", None),)

    def cache_need(self):
        # [S^T of every head: heads x vdim x state | the convolution's last taps - 1 inputs: (taps - 1) x channels]
        return StateNeed((self.n_heads * self.vdim * self.state + (self.taps - 1) * self.channels,), "float32")

    def bind(self, weights, rt) -> None:
        n = self.names
        self.w_in = weights[n["w_in"]].contiguous()
        self.w_o = weights[n["o"]].contiguous()
        self.conv_w, self.conv_b = weights[n["conv"]].contiguous(), weights[n["conv_b"]].contiguous()
        self.dt_bias, self.a_log = weights[n["dt_bias"]].contiguous(), weights[n["a_log"]].contiguous()
        self.d_skip, self.norm_w = weights[n["d"]].contiguous(), weights[n["norm"]].contiguous()

    def forward(self, ctx, h, cache, out_rows=None):
        H, P, N, G = self.n_heads, self.vdim, self.state, self.groups
        T, inner, C = h.shape[0], self.inner, self.channels
        proj = ops.linear(h, self.w_in, out_dtype=torch.float32)
        xbc = torch.empty((T, C), dtype=torch.float32, device=h.device)
        dt_dec = torch.empty((T, 2 * H), dtype=torch.float32, device=h.device)
        ops.ssm_prep(proj, inner, C, self.conv_w, self.conv_b, cache.state, H * P * N, ctx.token_seq, ctx.seq_slot,
                     ctx.seq_q_start, ctx.seq_q_len, ctx.n_seqs, xbc, inner + C, H, self.dt_bias, self.a_log, dt_dec,
                     self.defines, cache.writable)
        raw = torch.empty((T, inner), dtype=torch.float32, device=h.device)
        ops.decay_walk(xbc[:, inner + G * N:], xbc[:, inner:inner + G * N], xbc[:, :inner], H // G, dt_dec, None,
                       self.d_skip, cache.state, raw, ctx.seq_slot, ctx.seq_q_start, ctx.seq_q_len, ctx.n_seqs, H, N, P,
                       cache.writable)
        z = proj[:, :inner]
        if out_rows is not None:
            raw, z = _rows(raw, out_rows), _rows(z.contiguous(), out_rows)
        o = torch.empty(raw.shape, dtype=h.dtype, device=h.device)
        ops.gated_group_norm(raw, z, self.norm_w, o, self.norm_groups, self.norm_eps, gate_first=True)
        return ops.linear_out_f32(o, self.w_o, ctx.status)
