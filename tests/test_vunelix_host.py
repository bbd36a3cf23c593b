"""Vunelix without a GPU: the configuration, the run order of a looped span, the manifest, the rotation's frequencies."""
import math

import pytest

import plain_vunelix as plain
from infinicore_infer_b200.config import ConfigError, FrequencyRampSpec, PairRotarySpec, VunelixConfig, config_class_for
from infinicore_infer_b200.parts import cache_needs, model_manifest, state_needs


def cfg(loop=None, cap=7.5):
    layers = [
        {"type": "mamba1", "mixer": {"inner": 24, "state": 6, "dt_rank": 2, "conv": 3}, "mlp": {"kind": "dense", "ff": 20}},
        {"type": "latent_attention", "mlp": {"kind": "moe", "router": {"experts": 3, "top": 2}, "expert": {"ff": 8}, "shared": {"ff": 12}},
         "mixer": {"heads": 2, "dim": 6, "rot_dim": 4, "vdim": 10, "kv_rank": 14, "scale": 0.3,
                   "rot": {"base": 100.0, "dims": 4, "scaling": {"factor": 2.0, "original": 16, "fast": 4.0, "slow": 1.0}}}},
        {"type": "latent_attention", "mlp": None,
         "mixer": {"heads": 1, "dim": 4, "rot_dim": 6, "vdim": 4, "kv_rank": 5, "scale": 0.5, "rot": {"base": 50.0, "dims": 2}}},
    ]
    out = {"architecture": "Vunelix", "norm": {"eps": 1e-5}, "vocab": 40, "width": 16, "layers": layers, "logit_softcap": cap}
    if loop:
        out["loop"] = dict(zip(("start", "stop", "times"), loop))
    return out


def test_the_registry_finds_the_configuration_and_it_reads_back():
    c = config_class_for(cfg())
    assert c is VunelixConfig
    typed = c.from_dict(cfg(loop=(1, 3, 2)), max_tokens=99)
    assert typed.max_positions == 99 and typed.loop == (1, 3, 2) and typed.logit_softcap == 7.5
    again = VunelixConfig.from_dict(typed.to_dict(), max_tokens=99)
    assert again == typed
    assert VunelixConfig.from_dict(cfg(cap=None)).logit_softcap == 0.0


def test_run_order_of_a_span_that_runs_several_times():
    spec = VunelixConfig.from_dict(cfg(loop=(1, 3, 2))).model_spec()
    assert [e.layer for e in spec.order] == [0, 1, 2, 1, 2]
    assert [e.cache for e in spec.order] == [0, 1, 2, 3, 4]
    assert [(e.before.step_index, e.before.steps) if e.before else None for e in spec.order] == [None, (0, 2), None, (1, 2), None]
    assert [(i, t, first) for i, t, first in plain.run_order(cfg(loop=(1, 3, 2)))] == \
        [(i, t, first) for i, t, first in VunelixConfig.from_dict(cfg(loop=(1, 3, 2))).run_order()]
    plain_order = VunelixConfig.from_dict(cfg()).model_spec().order
    assert [e.layer for e in plain_order] == [0, 1, 2] and all(e.before is None for e in plain_order)
    needs, tails = cache_needs(spec), state_needs(spec)
    assert needs[0].shape == (24, 6) and tails[0].shape == (2, 24)
    assert needs[1] == needs[3] and needs[1].head_dim == 18 and needs[1].v_head_dim == 14 and needs[1].values_in_keys
    assert needs[2].head_dim == 11 and tails[1] is None


def test_manifest_names_every_tensor_once():
    names = model_manifest(VunelixConfig.from_dict(cfg(loop=(0, 2, 3))).model_spec())
    assert names["loop.in"].shape == (16, 32) and names["loop.step"].shape == (3, 16)
    assert names["l0.mix.A_log"].shape == (24, 6) and names["l0.mix.x"].shape == (2 + 12, 24) and names["l0.mix.conv.b"].shape == (24,)
    assert names["l1.mix.dkv"].shape == (18, 16) and names["l1.mix.uk"].shape == (12, 14) and names["l1.mix.g"].shape == (20, 16)
    assert names["l1.mlp.e2.down"].shape == (16, 8) and names["l1.mlp.shared.up"].shape == (12, 16) and names["l1.mlp.router"].shape == (3, 16)
    assert "l2.norm2" not in names and "l2.norm1b" in names and names["head"].optional
    assert "loop.in" not in model_manifest(VunelixConfig.from_dict(cfg()).model_spec())


@pytest.mark.parametrize("dims,base,scaling", [(8, 1e4, None), (32, 5e5, (4.0, 256, 16.0, 2.0)), (6, 300.0, (16.0, 8, 2.0, 0.25))])
def test_stretched_frequencies(dims, base, scaling):
    spec = PairRotarySpec(dims=dims, base=base, scaling=None if scaling is None else FrequencyRampSpec(*scaling))
    f, m = spec.frequencies()
    names = None if scaling is None else dict(zip(("factor", "original", "fast", "slow"), scaling))
    pf, pm = plain.rotary_frequencies(dims, base, names)
    assert all(abs(a - b) <= 1e-12 * b for a, b in zip(f, pf.tolist())) and abs(m - pm) < 1e-12
    if scaling:
        assert abs(m - (0.1 * math.log(scaling[0]) + 1.0)) < 1e-12
        plainf = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
        assert all(p / scaling[0] - 1e-15 <= a <= p + 1e-15 for a, p in zip(f, plainf))


@pytest.mark.parametrize("change,what", [
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=6), "rot.dims"),
    (lambda c: c["layers"][0].update(type="mamba2"), "type"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=4), "experts"),
    (lambda c: c.update(loop={"start": 2, "stop": 5, "times": 2}), "loop"),
    (lambda c: c["layers"][0]["mixer"].pop("state"), "state"),
])
def test_what_the_configuration_refuses(change, what):
    c = cfg()
    change(c)
    with pytest.raises(ConfigError, match=what):
        VunelixConfig.from_dict(c)
