"""The Sozurax configuration reader and the model description built from it (no GPU): sizes and constants come from
config.json, layer order and cache sharing become the run order, input stages get state entries of their own, and a
configuration that cannot describe a model is refused with the key that is wrong."""

import pytest

from tokasaurus_b200.config import lookup_architecture
from tokasaurus_b200.config.model_config import ConfigError
from tokasaurus_b200.parts.base import PagedCacheNeed, StateNeed


def base_config():
    lat = dict(heads=3, dim=20, rot_dim=6, vdim=12, kv_rank=36, q_rank=28, mask=dict(size=19),
               rot=dict(base=500.0, dims=4), scale=0.2)
    return dict(architecture="Sozurax", vocab=97, width=64, norm=dict(eps=1e-5), embedding=dict(scale=2.0),
                canon=dict(taps=3),
                layers=[dict(type="hgrn2", mixer=dict(heads=2, dim=24, vdim=40), mlp=dict(kind="dense", ff=80)),
                        dict(type="latent_attention", mixer=dict(lat), mlp=None),
                        dict(type="latent_attention", mixer=dict(lat, kv_from=1, heads=2, vdim=8),
                             mlp=dict(kind="moe", expert=dict(ff=16), router=dict(experts=4, top=2), shared=dict(ff=24)))])


def test_description_follows_the_configuration():
    d = base_config()
    arch = lookup_architecture(d)
    assert arch.name == "Sozurax"
    cfg = arch.parse_config(d)
    assert (cfg.vocab, cfg.width, cfg.taps, cfg.embedding_scale, cfg.norm_eps) == (97, 64, 3, 2.0, 1e-5)
    model = arch.build_model(cfg)
    assert [(c.block, c.cache, c.write_cache) for c in model.run_order] == [(0, 0, True), (1, 1, True), (2, 1, False)]
    needs = model.cache_entries()
    assert needs[0] == StateNeed((2, 40, 24), "float32")
    assert needs[1] == PagedCacheNeed(1, 42, 19, planes=1)
    # a reader with a wider window than the layer whose rows it reads: the entry keeps the wider one, each mixer
    # masks by its own
    d2 = base_config()
    d2["layers"][2]["mixer"]["mask"] = dict(size=33)
    m2 = arch.build_model(arch.parse_config(d2))
    assert m2.cache_entries()[1] == PagedCacheNeed(1, 42, 33, planes=1)
    assert [b.mixer.window for b in m2.blocks[1:]] == [19, 33]
    # two stages in layers with a feed-forward, one in the layer without
    stage_entries = [e for names in model.stage_entries for e in names.values()]
    assert len(stage_entries) == 5 and all(needs[e] == StateNeed((2, 64), "float32") for e in stage_entries)
    names = {s.name: s for s in model.weight_specs()}
    assert names["l0.canon1"].shape == (64, 3) and names["l0.mlp.act"].shape == (4,)
    assert "l1.norm2" not in names and "l1.canon2" not in names
    assert "l2.mix.dkv" not in names and names["l1.mix.dkv"].shape == (42, 64)
    assert names["l2.mix.uq"].shape == (2 * 26, 28) and names["l2.mix.uv"].shape == (2 * 8, 36)
    assert names["l2.mlp.e3.down"].shape == (64, 16) and names["l2.mlp.shared.gate"].shape == (24, 64)
    assert names["l2.mlp.router"].role == "vector"  # the router works in 32-bit
    mods = dict((src, d) for src, d in model.kernel_modules("float32"))
    assert mods["latent_attention.cu"] == {"TKB_LAT_RANK": 36}
    assert mods["recurrence.cu"] == {"TKB_REC_DPT": 3, "TKB_REC_CPT": 1}


@pytest.mark.parametrize("change,word", [
    (lambda d: d["layers"][2]["mixer"].update(kv_from=0), "kv_from"),
    (lambda d: d["layers"][2]["mixer"].update(kv_rank=40), "kv_rank"),
    (lambda d: d["layers"][1]["mixer"]["rot"].update(dims=8), "rot.dims"),
    (lambda d: d["layers"][0].update(type="mamba"), "type"),
    (lambda d: d["layers"][2]["mlp"]["router"].update(top=5), "top"),
    (lambda d: d["layers"][0]["mlp"].update(kind="glu"), "kind"),
    (lambda d: d.pop("width"), "width"),
    (lambda d: d["layers"][0]["mixer"].update(vdim=0), "vdim"),
])
def test_bad_configurations_are_refused(change, word):
    d = base_config()
    change(d)
    arch = lookup_architecture(d)
    with pytest.raises(ConfigError) as e:
        arch.parse_config(d)
    assert word in str(e.value)


def test_a_block_can_stand_without_a_feed_forward_or_stages():
    from tokasaurus_b200.parts import PreNormBlock, RMSNorm, ShortConv, GatedMLP
    from tokasaurus_b200.parts.base import Mixer

    plain = PreNormBlock(RMSNorm(8, 1e-5, "n1"), Mixer(), RMSNorm(8, 1e-5, "n2"), GatedMLP(8, 16, "g", "u", "d"))
    assert plain.state_needs() == {}
    alone = PreNormBlock(RMSNorm(8, 1e-5, "n1"), Mixer(), None, None, mixer_stage=ShortConv(8, 4, "c"))
    assert alone.state_needs() == {"mixer_stage": StateNeed((3, 8), "float32")}
    assert [s.name for s in alone.weight_specs()] == ["n1", "c"]
    with pytest.raises(ValueError):
        PreNormBlock(RMSNorm(8, 1e-5, "n1"), Mixer(), None, GatedMLP(8, 16, "g", "u", "d"))
