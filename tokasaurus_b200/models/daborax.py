"""The Daborax decoder put together from parts, and its registry entry.

A decoder whose sublayers read the residual stream itself and are normed on their way OUT
(``parts.block.OutputNormBlock``: ``x += m * ls * norm(sublayer(x))`` with a layer-scale vector ``ls``), over a scaled
embedding plus sinusoidal position vectors.  config.json lists the layers one by one; a layer's mixer is a selective
state space (``parts.state_space.SelectiveStateSpace``), linear attention with a fixed decay a head
(``parts.recurrent.DecayedLinearAttention``) or windowed attention with capped scores and a sink
(``parts.sink_attention.SinkAttention``); its feed-forward is a clamped gated unit (``parts.mlp.ClampedGLU``) or
absent.  A layer may run with an earlier layer's tensors: it is a second call of that block in the run order, with a
cache or state of its own.

Tensor names: ``embed``; per layer i ``l<i>.norm1`` / ``.norm2``, ``l<i>.ls1`` / ``.ls2``, the mixer's ``l<i>.mix.*``
and the feed-forward's ``l<i>.mlp.gate`` / ``.up`` / ``.down``; ``final.norm``; ``head``.
"""

from __future__ import annotations

from tokasaurus_b200.config.daborax_config import DaboraxConfig, LinearAttentionConfig, StateSpaceConfig
from tokasaurus_b200.config.registry import register_architecture
from tokasaurus_b200.parts import (
    ClampedGLU,
    DecayedLinearAttention,
    DecoderModel,
    LayerCall,
    OutputHead,
    OutputNormBlock,
    RMSNorm,
    SelectiveStateSpace,
    SinkAttention,
    SinusoidalPositions,
    TokenEmbedding,
)


def build_daborax(cfg: DaboraxConfig) -> DecoderModel:
    W, eps = cfg.width, cfg.norm_eps
    blocks, order = [], []
    block_of: dict[int, int] = {}
    for i, layer in enumerate(cfg.layers):
        j = layer.weights_of
        if j is not None and (cfg.layers[j].mixer, cfg.layers[j].mlp) == (layer.mixer, layer.mlp):
            order.append(LayerCall(block_of[j]))  # the same block once more, with a cache entry of this call's own
            continue
        # (an entry that names layer j's tensors but other constants: a block of its own over the same tensors)
        p, m = f"l{i if j is None else j}", layer.mixer
        if isinstance(m, StateSpaceConfig):
            mixer = SelectiveStateSpace(W, m.heads, m.vdim, m.state, m.groups, m.norm_groups, m.taps, eps,
                                        in_name=f"{p}.mix.in", conv_name=f"{p}.mix.conv", conv_bias_name=f"{p}.mix.conv.b",
                                        dt_bias_name=f"{p}.mix.dt_bias", a_log_name=f"{p}.mix.A_log", d_name=f"{p}.mix.D",
                                        norm_name=f"{p}.mix.norm", o_name=f"{p}.mix.o")
        elif isinstance(m, LinearAttentionConfig):
            mixer = DecayedLinearAttention(W, m.heads, m.dim, m.vdim, m.decay, eps, q_name=f"{p}.mix.q",
                                           k_name=f"{p}.mix.k", v_name=f"{p}.mix.v", g_name=f"{p}.mix.g",
                                           norm_name=f"{p}.mix.norm", o_name=f"{p}.mix.o")
        else:
            mixer = SinkAttention(W, m.heads, m.kv_heads, m.dim, m.vdim, m.scale, m.softcap, m.window, eps,
                                  q_name=f"{p}.mix.q", k_name=f"{p}.mix.k", v_name=f"{p}.mix.v", o_name=f"{p}.mix.o",
                                  sink_name=f"{p}.mix.sink", bias_names=(f"{p}.mix.q.b", f"{p}.mix.k.b", f"{p}.mix.v.b"),
                                  out_bias_name=f"{p}.mix.o.b", unit_norm=True)
        ff = layer.mlp
        ffn = ClampedGLU(W, ff.ff, ff.limit, f"{p}.mlp.gate", f"{p}.mlp.up", f"{p}.mlp.down") if ff is not None else None
        block_of[i] = len(blocks)
        order.append(LayerCall(len(blocks)))
        blocks.append(OutputNormBlock(
            mixer=mixer, mixer_norm=RMSNorm(W, eps, f"{p}.norm1"), ffn=ffn,
            ffn_norm=RMSNorm(W, eps, f"{p}.norm2") if ffn is not None else None, mult=cfg.residual_mult,
            mixer_scale_name=f"{p}.ls1", ffn_scale_name=f"{p}.ls2"))
    return DecoderModel(
        embedding=TokenEmbedding(cfg.vocab, W, "embed", scale=cfg.embedding_scale, positions=SinusoidalPositions(W)),
        blocks=blocks,
        head=OutputHead(cfg.vocab, W, RMSNorm(W, eps, "final.norm"), "head"),
        run_order=order,
    )


register_architecture("Daborax", DaboraxConfig.from_dict, build_daborax, model_types=("daborax",), replace=True)
