"""The Zisesun configuration reader, its model description and its tensor names (no GPU)."""

import copy

import pytest

from cloud_inference_from_scratch_b200 import models, parts  # noqa: F401  (registries)
from cloud_inference_from_scratch_b200.config import ConfigError, ZisesunConfig, resolve_config
from cloud_inference_from_scratch_b200.models import DecoderModel


def raw_config():
    attention = dict(heads=6, kv_heads=3, dim=8, vdim=12, scale=0.25, mask=dict(size=5))
    lightning = dict(heads=2, dim=4, vdim=6, decay=[0.5, 0.99])
    mlp = dict(kind="moe", expert=dict(ff=10), router=dict(experts=3, top=2))
    return dict(architecture="Zisesun", vocab=50, width=24, max_positions=64, norm=dict(eps=1e-5), streams=2,
                layers=[dict(type="attention", mixer=attention, mlp=mlp),
                        dict(type="lightning", mixer=lightning, mlp=None),
                        dict(type="attention", mixer=attention, mlp=mlp, weights_of=0),
                        dict(type="attention", mixer=attention, mlp=mlp, weights_of=2)])


def test_reads_back_what_it_wrote_and_is_found_by_its_name():
    raw = raw_config()
    arch, config, spec = resolve_config(raw)
    assert arch.name == "Zisesun" and isinstance(config, ZisesunConfig)
    again = config.to_dict()
    assert again["layers"][3]["weights_of"] == 0          # a chain is resolved to the owner
    assert ZisesunConfig.from_dict(again) == config
    assert spec.residual_streams == 2 and spec.position_tensor == "pos" and spec.max_positions == 64
    assert [entry.layer for entry in spec.schedule] == [0, 1, 0, 0] and len(spec.layers) == 2


def test_tensor_names_shapes_and_caches():
    _, _, spec = resolve_config(raw_config())
    model = DecoderModel(spec)
    table = model.tensor_table()
    assert table["embed"].shape == (50, 24) and table["pos"].shape == (64, 24) and table["head"].shape == (50, 24)
    assert table["final.norm"].shape == () and table["l0.norm1"].shape == () and table["l0.norm2"].shape == ()
    assert table["l0.mix.q"].shape == (48, 24) and table["l0.mix.k"].shape == (24, 24) and table["l0.mix.v"].shape == (36, 24)
    assert table["l0.mix.q.b"].shape == (48,) and table["l0.mix.v.b"].shape == (36,)
    assert table["l0.mix.q.norm"].shape == (48,) and table["l0.mix.k.norm"].shape == (24,)
    assert table["l0.mix.r1"].shape == (6,) and table["l0.mix.o"].shape == (24, 72)
    assert table["l0.mlp.router"].shape == (3, 24) and table["l0.mlp.correction"].shape == (3,)
    assert table["l0.mlp.e2.gate"].shape == (10, 24) and table["l0.mlp.e2.down"].shape == (24, 10)
    assert table["l0.hc1.in"].shape == (2,) and table["l0.hc2.mix"].shape == (2, 2)
    assert table["l1.mix.g"].shape == (12, 24) and table["l1.mix.norm"].shape == (12,) and table["l1.mix.o"].shape == (24, 12)
    assert "l1.norm2" not in table and "l1.hc2.in" not in table and not any(name.startswith("l2.") for name in table)
    needs = model.cache_needs()
    assert [need.owner for need in needs] == [0, 1, 2, 3]            # every run keeps a cache of its own
    assert needs[0].pages.window == 5 and needs[0].pages.value_size == 12 and needs[0].state is None
    assert needs[1].pages is None and needs[1].state.shape == (2, 4, 6)


def test_without_streams_there_are_no_connections():
    raw = raw_config()
    del raw["streams"]
    _, _, spec = resolve_config(raw)
    assert spec.residual_streams == 1
    assert not any(".hc" in name for name in DecoderModel(spec).tensor_table())


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].update(type="conv"), "mixer type"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=4), "multiple"),
    (lambda c: c["layers"][1]["mixer"].update(decay=[0.5]), "one number per head"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=4), "exceeds"),
    (lambda c: c["layers"][2].update(weights_of=2), "earlier layer"),
    (lambda c: c["layers"][2].update(weights_of=1), "differs"),
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "not built"),
])
def test_refusals(change, message):
    raw = copy.deepcopy(raw_config())
    change(raw)
    with pytest.raises(ConfigError, match=message):
        ZisesunConfig.from_dict(raw)


def test_pools_keep_keys_and_values_of_different_sizes_apart():
    from cloud_inference_from_scratch_b200.cache.pools import plan_groups

    _, _, spec = resolve_config(raw_config())
    groups, place = plan_groups(DecoderModel(spec).cache_needs(), 2)
    assert len(groups) == 1 and groups[0].window == 5
    assert groups[0].bytes_per_token == 3 * (8 + 12) * 2 * 3          # three runs own pages
    assert sorted(place) == [0, 2, 3]
