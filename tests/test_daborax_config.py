"""The Daborax configuration reader and the model description built from it (no GPU): sizes and constants come from
config.json, a layer that runs with an earlier layer's tensors becomes a second call of that block with a cache entry
of its own, and a configuration that cannot describe a model is refused with the key that is wrong."""

import copy

import pytest

from tokasaurus_b200.config import lookup_architecture
from tokasaurus_b200.config.model_config import ConfigError
from tokasaurus_b200.parts.base import PagedCacheNeed, StateNeed


def base_config():
    ssm = dict(type="mamba2", mixer=dict(heads=4, vdim=24, state=20, groups=2, norm_groups=3, conv=3), mlp=None)
    lin = dict(type="lightning", mixer=dict(heads=3, dim=16, vdim=40, decay=[0.7, 0.95, 0.999]),
               mlp=dict(kind="dense", ff=56, limit=0.8))
    att = dict(type="attention", mixer=dict(heads=6, kv_heads=3, dim=24, vdim=40, mask=dict(size=23), scale=0.4, softcap=8.0),
               mlp=dict(kind="dense", ff=72, limit=1.5))
    return dict(architecture="Daborax", vocab=151, width=96, norm=dict(eps=1e-5), embedding=dict(scale=3.5),
                residual_mult=0.6, layers=[att, ssm, lin, dict(copy.deepcopy(ssm), weights_of=1), dict(copy.deepcopy(att), weights_of=0)])


def test_description_follows_the_configuration():
    d = base_config()
    arch = lookup_architecture(d)
    assert arch.name == "Daborax"
    cfg = arch.parse_config(d)
    assert (cfg.vocab, cfg.width, cfg.embedding_scale, cfg.residual_mult, cfg.norm_eps) == (151, 96, 3.5, 0.6, 1e-5)
    model = arch.build_model(cfg)
    assert len(model.blocks) == 3
    assert [(c.block, c.write_cache) for c in model.run_order] == [(0, True), (1, True), (2, True), (1, True), (0, True)]
    assert len({c.cache for c in model.run_order}) == 5  # every call has a cache or state of its own
    needs = model.cache_entries()
    by_call = [needs[c.cache] for c in model.run_order]
    assert by_call[0] == by_call[4] == PagedCacheNeed(3, 24 + 40, 23, planes=1)
    assert by_call[1] == by_call[3] == StateNeed((4 * 24 * 20 + 2 * (96 + 2 * 2 * 20),), "float32")
    assert by_call[2] == StateNeed((3 * 40 * 16,), "float32")
    names = {s.name: s for s in model.weight_specs()}
    assert not any(n.startswith(("l3.", "l4.")) for n in names)
    assert names["l1.mix.in"].shape == (2 * 96 + 2 * 2 * 20 + 4, 96) and names["l1.mix.conv"].shape == (96 + 80, 3)
    assert names["l1.mix.norm"].shape == (96,) and names["l1.mix.A_log"].shape == (4,) and names["l1.mix.o"].shape == (96, 96)
    assert "l1.norm2" not in names and "l1.ls2" not in names and "l1.ls1" in names
    assert names["l2.mix.g"].shape == (120, 96) and names["l2.mix.q"].shape == (48, 96) and names["l2.mix.norm"].shape == (120,)
    assert names["l0.mix.q"].shape == (144, 96) and names["l0.mix.v"].shape == (120, 96) and names["l0.mix.o"].shape == (96, 240)
    assert names["l0.mix.sink"].shape == (6,) and names["l0.mix.o.b"].shape == (96,) and names["l0.mix.v.b"].shape == (120,)
    assert names["l0.mix.sink"].role == "vector" and names["l1.mix.dt_bias"].role == "vector"  # used in 32-bit
    assert names["l2.mlp.down"].shape == (96, 56)
    mods = {(src, tuple(sorted((dd or {}).items()))) for src, dd in model.kernel_modules("bfloat16")}
    assert ("attention_sink.cu", (("TKB_QK", 24), ("TKB_VD", 40))) in mods
    assert ("decay_recurrence.cu", (("TKB_DR_DPT", 4), ("TKB_DR_LANES", 8))) in mods   # state 20, dim 16: five and four 16-byte pieces
    from tokasaurus_b200.kernels import ops
    assert [d["TKB_DR_LANES"] for d in ops.decay_walk_modules(128, 64)] == [8, 16, 32]
    assert ops.decay_walk_modules(40, 8) == [dict(TKB_DR_LANES=8, TKB_DR_DPT=8), dict(TKB_DR_LANES=16, TKB_DR_DPT=4)]
    att, ssm, lin = (b.mixer for b in model.blocks)
    assert (att.scale, att.softcap, att.window) == (0.4, 8.0, 23) and lin.decay == (0.7, 0.95, 0.999)
    assert model.blocks[0].mult == 0.6 and model.embedding.scale == 3.5 and model.blocks[2].ffn.limit == 0.8


def test_a_layer_may_name_a_layer_that_borrows_itself():
    d = base_config()
    d["layers"].append(dict(copy.deepcopy(d["layers"][3]), weights_of=3))  # layer 3 runs with layer 1's tensors
    arch = lookup_architecture(d)
    cfg = arch.parse_config(d)
    assert cfg.layers[5].weights_of == 1
    model = arch.build_model(cfg)
    assert [c.block for c in model.run_order] == [0, 1, 2, 1, 0, 1] and len({c.cache for c in model.run_order}) == 6


def test_defaults():
    d = base_config()
    d.pop("residual_mult")
    d["layers"][0]["mixer"].pop("softcap")
    d["layers"][0]["mixer"].pop("mask")
    d["layers"][4]["mixer"].pop("softcap")
    d["layers"][4]["mixer"].pop("mask")
    d["layers"][2]["mixer"]["decay"] = 0.9
    arch = lookup_architecture(d)
    cfg = arch.parse_config(d)
    model = arch.build_model(cfg)
    assert cfg.residual_mult == 1.0 and model.blocks[0].mixer.softcap is None and model.blocks[0].mixer.window is None
    assert model.blocks[2].mixer.decay == (0.9, 0.9, 0.9)
    assert model.cache_entries()[model.run_order[0].cache] == PagedCacheNeed(3, 64, None, planes=1)


@pytest.mark.parametrize("change,word", [
    (lambda d: d["layers"][3].update(weights_of=2), "weights_of"),
    (lambda d: d["layers"][3].update(weights_of=7), "weights_of"),
    (lambda d: d["layers"][1]["mixer"].update(groups=3), "groups"),
    (lambda d: d["layers"][1]["mixer"].update(norm_groups=5), "norm groups"),
    (lambda d: d["layers"][1]["mixer"].pop("conv"), "conv"),
    (lambda d: d["layers"][2]["mixer"].update(decay=[0.5, 0.6]), "decay"),
    (lambda d: d["layers"][0]["mixer"].update(kv_heads=4), "kv_heads"),
    (lambda d: d["layers"][0]["mixer"]["mask"].update(size=0), "mask.size"),
    (lambda d: d["layers"][0]["mixer"].update(softcap=-1.0), "softcap"),
    (lambda d: d["layers"][0].update(type="mamba"), "type"),
    (lambda d: d["layers"][2]["mlp"].update(kind="moe"), "kind"),
    (lambda d: d["layers"][2]["mlp"].pop("limit"), "limit"),
    (lambda d: d.pop("width"), "width"),
    (lambda d: d["layers"][2]["mixer"].update(vdim=0), "vdim"),
])
def test_bad_configurations_are_refused(change, word):
    d = base_config()
    change(d)
    arch = lookup_architecture(d)
    with pytest.raises(ConfigError) as e:
        arch.parse_config(d)
    assert word in str(e.value)
