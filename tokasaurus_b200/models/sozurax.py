"""The Sozurax decoder put together from parts, and its registry entry.

A pre-norm decoder whose layers alternate, in the order config.json lists them, between two mixers: a gated linear
recurrence with a matrix state per head (``parts.recurrent.GatedLinearRecurrence``) and latent attention over a
sliding window (``parts.latent_attention.LatentAttention``), some of whose layers read the latent rows an earlier
layer cached instead of making their own.  Every sublayer reads its layer norm through a short causal convolution
(``parts.conv.ShortConv``); feed-forwards are dense with the PolyNorm activation or routed experts with a shared
expert (``parts.mlp``).  The embedding is scaled; the head is a layer norm and a projection.

Tensor names: ``embed``; per layer i ``l<i>.norm1`` / ``.norm1.b`` / ``.norm2`` / ``.norm2.b``, ``l<i>.canon1`` /
``.canon2`` [width, taps], the mixer's ``l<i>.mix.*`` and the feed-forward's ``l<i>.mlp.*``; ``final.norm`` /
``final.norm.b``; ``head``.
"""

from __future__ import annotations

from tokasaurus_b200.config.registry import register_architecture
from tokasaurus_b200.config.sozurax_config import LatentMixerConfig, SozuraxConfig
from tokasaurus_b200.parts import (
    DecoderModel,
    GatedLinearRecurrence,
    GatedMLP,
    LatentAttention,
    LayerCall,
    LayerNorm,
    OutputHead,
    PolyNormMLP,
    PreNormBlock,
    RoutedExperts,
    ShortConv,
    TokenEmbedding,
)


def build_sozurax(cfg: SozuraxConfig) -> DecoderModel:
    W, eps = cfg.width, cfg.norm_eps
    blocks, order = [], []
    # a layer that reads another layer's rows has a window of its own: the entry keeps the widest of its users'
    keep: dict[int, int | None] = {}
    for i, layer in enumerate(cfg.layers):
        if isinstance(layer.mixer, LatentMixerConfig):
            src = i if layer.mixer.kv_from is None else layer.mixer.kv_from
            w = layer.mixer.window
            if src not in keep:
                keep[src] = w
            elif keep[src] is not None:
                keep[src] = None if w is None else max(keep[src], w)
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}", layer.mixer
        cache = i
        if isinstance(m, LatentMixerConfig):
            own = m.kv_from is None
            mixer = LatentAttention(
                W, m.heads, m.dim, m.rot_dim, m.vdim, m.kv_rank, m.q_rank, m.scale, m.rot_base, m.rot_dims, eps, m.window,
                names=dict(dq=f"{p}.mix.dq", dq_norm=f"{p}.mix.dq.norm", uq=f"{p}.mix.uq", dkv=f"{p}.mix.dkv",
                           dkv_norm=f"{p}.mix.dkv.norm", uk=f"{p}.mix.uk", uv=f"{p}.mix.uv", o=f"{p}.mix.o"),
                own_kv=own, cache_window=keep[i if own else m.kv_from])
            if not own:
                cache = m.kv_from
        else:
            own = True
            mixer = GatedLinearRecurrence(W, m.heads, m.dim, m.vdim, eps, q_name=f"{p}.mix.q", f_name=f"{p}.mix.f",
                                          f_bias_name=f"{p}.mix.f.b", lower_name=f"{p}.mix.lower", v_name=f"{p}.mix.v",
                                          norm_name=f"{p}.mix.norm", o_name=f"{p}.mix.o")
        ff = layer.mlp
        if ff is None:
            ffn = None
        elif ff.kind == "dense":
            ffn = PolyNormMLP(W, ff.ff, eps, f"{p}.mlp.up", f"{p}.mlp.down", f"{p}.mlp.act")
        else:
            shared = None
            if ff.shared_ff is not None:
                shared = GatedMLP(W, ff.shared_ff, f"{p}.mlp.shared.gate", f"{p}.mlp.shared.up", f"{p}.mlp.shared.down")
            ffn = RoutedExperts(W, ff.ff, ff.experts, ff.top, f"{p}.mlp.router", f"{p}.mlp.router.b",
                                lambda e, p=p: (f"{p}.mlp.e{e}.gate", f"{p}.mlp.e{e}.up", f"{p}.mlp.e{e}.down"), shared)
        blocks.append(PreNormBlock(
            mixer_norm=LayerNorm(W, eps, f"{p}.norm1", f"{p}.norm1.b"), mixer=mixer,
            ffn_norm=LayerNorm(W, eps, f"{p}.norm2", f"{p}.norm2.b") if ffn is not None else None, ffn=ffn,
            mixer_stage=ShortConv(W, cfg.taps, f"{p}.canon1"),
            ffn_stage=ShortConv(W, cfg.taps, f"{p}.canon2") if ffn is not None else None))
        order.append(LayerCall(i, cache, write_cache=own))
    return DecoderModel(
        embedding=TokenEmbedding(cfg.vocab, W, "embed", scale=cfg.embedding_scale),
        blocks=blocks,
        head=OutputHead(cfg.vocab, W, LayerNorm(W, eps, "final.norm", "final.norm.b"), "head"),
        run_order=order,
    )


register_architecture("Sozurax", SozuraxConfig.from_dict, build_sozurax, model_types=("sozurax",), replace=True)
