"""Nomutar without a GPU: the configuration reader, the layer order, the tensors the builder names, what the cache
manager is asked for, and the frequency tables against the plain implementation's."""
import copy

import numpy as np
import pytest

import plain_nomutar as plain
from llmx_b200.cache.manager import CacheManager, KVSpec, StateSpec
from llmx_b200.config import ConfigError, NomutarConfig
from llmx_b200.parts.rope import banded_frequencies, blended_frequencies
from llmx_b200.registry import architecture_of


def raw_config():
    a1 = {"type": "attention", "mlp": {"kind": "dense", "ff": 40},
          "mixer": {"heads": 6, "kv_heads": 2, "dim": 16, "vdim": 24, "scale": 0.3, "softcap": 4.0, "mask": {"size": 9},
                    "rot": {"base": 300.0, "dims": 8, "scaling": {"factor": 3.0, "low": 0.5, "high": 5.0, "original": 64}}}}
    a2 = {"type": "attention_2", "mlp": {"kind": "moe", "router": {"experts": 6, "top": 2}, "expert": {"ff": 24}, "shared": {"ff": 40}},
          "mixer": {"heads": 4, "kv_heads": 2, "dim": 24, "vdim": 16, "scale": 0.25, "mask": {"size": 13},
                    "rot": {"base": 1000.0, "dims": 12, "scaling": {"factor": 6.0, "original": 64, "fast": 16.0, "slow": 2.0}}}}
    a3 = {"type": "attention_3", "mlp": None, "mixer": {"heads": 3, "kv_heads": 3, "dim": 20, "vdim": 12, "scale": 0.35, "rot": {"base": 50.0, "dims": 20}}}
    return {"architecture": "Nomutar", "vocab": 200, "width": 96, "norm": {"eps": 1e-5, "groups": 3}, "residual_mult": 0.6,
            "canon": {"taps": 3}, "embedding": {"scale": 3.0, "bigram": {"buckets": 53, "mul_prev": 31, "mul_cur": 5}},
            "logit_softcap": 12.0, "loop": {"start": 1, "stop": 3, "times": 2}, "layers": [a1, a2, a3, copy.deepcopy(a2)]}


def test_every_value_is_read_and_written_back():
    cfg = NomutarConfig.from_dict(raw_config())
    assert (cfg.vocab, cfg.width, cfg.norm_groups, cfg.canon_taps, cfg.residual_mult, cfg.logit_softcap) == (200, 96, 3, 3, 0.6, 12.0)
    assert cfg.pair_table.buckets == 53 and cfg.embedding_scale == 3.0 and cfg.ignored == ()
    m = cfg.layers[0].mixer
    assert (m.type, m.heads, m.kv_heads, m.dim, m.vdim, m.window, m.softcap, m.rot_dims) == ("attention", 6, 2, 16, 24, 9, 4.0, 8)
    assert m.rot_scaling.kind == "bands" and cfg.layers[1].mixer.rot_scaling.kind == "ramp" and cfg.layers[2].mixer.rot_scaling is None
    assert cfg.layers[1].mixer.softcap is None and cfg.layers[2].mixer.window is None and cfg.layers[2].mlp is None
    assert cfg.layers[1].mlp.experts == 6 and cfg.layers[1].mlp.top == 2 and cfg.layers[1].mlp.shared_ff == 40
    assert NomutarConfig.from_dict(cfg.to_dict()) == cfg
    assert architecture_of(raw_config()).config_cls is NomutarConfig


def test_what_config_json_does_not_mention_is_not_there():
    raw = raw_config()
    for key in ("canon", "loop", "logit_softcap", "residual_mult"):
        raw.pop(key)
    raw["embedding"] = {}
    raw["norm"] = {"eps": 1e-6}
    raw["something_else"] = 1
    cfg = NomutarConfig.from_dict(raw)
    assert (cfg.canon_taps, cfg.logit_softcap, cfg.residual_mult, cfg.norm_groups, cfg.embedding_scale) == (0, None, 1.0, 1, 1.0)
    assert cfg.pair_table is None and cfg.layer_runs() == [0, 1, 2, 3] and cfg.ignored == ("something_else",)
    model = architecture_of(raw).build(cfg)
    names = set(model.tensor_specs())
    assert "bigram" not in names and not any(n.endswith("canon1") for n in names)
    assert all(isinstance(s, KVSpec) for s in model.cache_entry_specs())


@pytest.mark.parametrize("change, what", [
    (lambda r: r["layers"][0].update(type="attention_4"), "mixer type"),
    (lambda r: r["layers"][0]["mixer"].update(heads=5), "multiple of kv_heads"),
    (lambda r: r["layers"][0]["mixer"]["rot"].update(dims=7), "even"),
    (lambda r: r["layers"][0]["mixer"].update(vdim=23), "vdim must be even"),
    (lambda r: r["layers"][1]["mlp"]["router"].update(top=7), "exceeds"),
    (lambda r: r["layers"][1]["mlp"].update(kind="other"), "not supported"),
    (lambda r: r["norm"].update(groups=5), "multiple of norm.groups"),
    (lambda r: r["loop"].update(stop=9), "loop"),
    (lambda r: r["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda r: r["layers"][0]["mixer"]["rot"]["scaling"].pop("low"), "low"),
    (lambda r: r.update(width="96"), "width"),
])
def test_wrong_values_are_refused_by_name(change, what):
    raw = raw_config()
    change(raw)
    with pytest.raises(ConfigError, match=what):
        NomutarConfig.from_dict(raw)


def test_layer_order_tensors_and_cache_entries():
    raw = raw_config()
    cfg = NomutarConfig.from_dict(raw)
    assert cfg.layer_runs() == [0, 1, 2, 1, 2, 3]
    model = architecture_of(raw).build(cfg)
    names = set(model.tensor_specs())
    for n in ("embed", "bigram", "final.norm", "head", "l0.norm1", "l0.canon1", "l0.mix.q", "l0.mix.q.norm", "l0.mix.k.norm", "l0.mix.sink",
              "l0.mix.o", "l0.mlp.gate", "l1.mix.q.b", "l1.mix.k.b", "l1.mix.v.b", "l1.mlp.router", "l1.mlp.router.b", "l1.mlp.e5.down",
              "l1.mlp.shared.up", "l1.mlp.shared.sg", "l2.mix.k.norm"):
        assert n in names, n
    for n in ("l1.mix.o.b", "l1.mix.sink", "l1.mix.q.norm", "l2.mix.sink", "l2.mlp.gate", "l0.mix.q.b"):
        assert n not in names, n
    specs = model.tensor_specs()
    assert specs["bigram"].shape == (54, 96) and specs["l0.mix.q.norm"].shape == (96,) and specs["l0.mix.k.norm"].shape == (32,)
    assert specs["l0.canon1"].shape == (96, 3) and specs["l1.mlp.shared.sg"].shape == (1, 96) and specs["l0.mix.sink"].shape == (6,)
    entries = model.cache_entry_specs()
    # the token before; then keys and values and the filter's inputs for each of the six layer runs
    assert entries[0] == StateSpec((1,), "int32") and len(entries) == 13
    assert entries[1] == KVSpec(2, 40, 9, planes=1) and entries[2] == StateSpec((2 * 96,), "float32")
    assert entries[3] == entries[7] == KVSpec(2, 40, 13, planes=1) and entries[5] == entries[9] == KVSpec(3, 32, None, planes=1)
    manager = CacheManager(entries, page_size=4, kv_tokens=64, max_requests=2)
    assert len(manager.groups) == 3 and sorted(len(g.members) for g in manager.groups) == [1, 2, 3]
    rc = manager.new_request("r")
    rc.prepare(40)
    rc.commit()
    held = dict(zip([g.spec.window for g in manager.groups], rc.held_pages()))
    assert held[None] == 10 and held[9] <= 4 and held[13] <= 5          # windows give back the pages they have passed
    manager.free_request("r")
    manager.check()


def test_frequency_tables_equal_the_plain_ones():
    for base, dims, factor, low, high, original in ((300.0, 8, 3.0, 0.5, 5.0, 64), (40000.0, 32, 3.0, 1.0, 6.0, 256), (20.0, 6, 2.0, 0.5, 3.0, 16)):
        assert np.allclose(banded_frequencies(base, dims, factor, low, high, original),
                           plain.banded_frequencies(base, dims, factor, low, high, original), rtol=1e-12)
    for base, dims, factor, original, fast, slow in ((1000.0, 12, 6.0, 64, 16.0, 2.0), (300000.0, 48, 6.0, 1024, 24.0, 2.0)):
        f, m = blended_frequencies(base, dims, factor, original, fast, slow)
        pf, pm = plain.ramped_frequencies(base, dims, factor, original, fast, slow)
        assert np.allclose(f, pf, rtol=1e-12) and abs(m - pm) < 1e-12
