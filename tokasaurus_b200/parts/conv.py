"""A short causal convolution over time on every channel, added to its input:
``g_t = h_t + sum_j w[:, j] * h_(t - taps + 1 + j)`` with zeros before a request's first token.  The last
``taps - 1`` inputs of every request are its state, kept in the request's slot, so a request may be fed in
portions of any size."""

from __future__ import annotations

import torch

from tokasaurus_b200.kernels import ops
from tokasaurus_b200.parts.base import InputStage, StateNeed, WeightSpec
from tokasaurus_b200.parts.norm import LayerNorm


class ShortConv(InputStage):
    def __init__(self, width: int, taps: int, weight_name: str):
        if taps < 1:
            raise ValueError(f"a convolution needs at least one tap, got {taps}")
        self.width = width
        self.taps = int(taps)
        self.weight_name = weight_name
        self.weight: torch.Tensor | None = None

    def weight_specs(self):
        return (WeightSpec(self.weight_name, (self.width, self.taps), role="vector"),)

    def kernel_modules(self, dtype):
        return (("norm_conv.cu", None),)

    def state_need(self):
        return StateNeed((self.taps - 1, self.width), "float32")

    def bind(self, weights, rt) -> None:
        self.weight = weights[self.weight_name].contiguous()

    def forward(self, ctx, h, state):
        out = torch.empty_like(h)
        ops.short_conv(h, out, self.weight, state.state, ctx.token_seq, ctx.seq_slot, ctx.seq_q_start, ctx.seq_q_len,
                       ctx.n_seqs)
        return out

    def forward_with_norm(self, ctx, norm, stream, state):
        """The norm and this stage together.  A step in which every request brings one token runs them as one kernel
        (no token needs a neighbour's normalised row then)."""
        if isinstance(norm, LayerNorm) and ctx.n_tokens == ctx.n_seqs and ctx.single_token_step:
            out = torch.empty(stream.x.shape, dtype=norm.out_dtype, device=stream.x.device)
            ops.add_layernorm_conv1(stream.x, stream.delta, norm.weight, norm.bias, norm.eps, self.weight, state.state,
                                    ctx.token_seq, ctx.seq_slot, out)
            stream.delta = None
            return out
        return self.forward(ctx, norm.forward(ctx, stream), state)
