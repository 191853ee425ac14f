"""Zamizen without a GPU: its configuration reader, what the builder asks of weights and cache, which cache entry a
layer that borrows keys and values names, the blended frequencies, and the plain implementation's mechanisms against
closed forms."""
import copy
import math

import numpy as np
import pytest

import plain_zamizen as plain

SCALING = {"factor": 4.0, "original": 64, "fast": 32.0, "slow": 1.0}
LATENT = {"heads": 3, "dim": 10, "rot_dim": 6, "vdim": 14, "kv_rank": 20, "scale": 0.25, "rot": {"base": 500.0, "dims": 6, "scaling": SCALING}}
OWN = {"heads": 6, "kv_heads": 2, "dim": 12, "vdim": 10, "scale": 0.3, "conv": 3, "rot": {"base": 10000.0, "dims": 8}}
CFG = {
    "architecture": "Zamizen", "vocab": 130, "width": 48, "norm": {"eps": 1e-6}, "residual_mult": 0.6,
    "layers": [
        {"type": "latent_attention", "mixer": LATENT, "mlp": {"kind": "dense", "ff": 40}},
        {"type": "attention", "mixer": OWN, "mlp": None},
        {"type": "attention", "mixer": dict(OWN, kv_from=1, conv=2), "mlp": {"kind": "dense", "ff": 24}},
        {"type": "attention", "mixer": {"heads": 2, "kv_heads": 1, "dim": 8, "vdim": 16, "scale": 0.5, "rot": {"base": 100.0, "dims": 0}},
         "mlp": {"kind": "dense", "ff": 32}},
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 1, "dim": 8, "vdim": 16, "scale": 0.5, "kv_from": 3, "rot": {"base": 100.0, "dims": 0}},
         "mlp": None},
        {"type": "attention", "mixer": dict(OWN, kv_from=1), "mlp": None},
    ]}


def test_configuration_is_read_written_back_and_refused_by_name():
    from llmx_b200.config import ConfigError, ZamizenConfig
    c = ZamizenConfig.from_dict(CFG)
    assert ZamizenConfig.from_dict(c.to_dict()) == c
    lat, own, reader = c.layers[0].mixer, c.layers[1].mixer, c.layers[2].mixer
    assert (lat.heads, lat.dim, lat.rot_dim, lat.vdim, lat.kv_rank, lat.scale, lat.rot_base, lat.rot_dims) == (3, 10, 6, 14, 20, 0.25, 500.0, 6)
    assert lat.rot_scaling.as_tuple() == (4.0, 64.0, 32.0, 1.0)
    assert (own.heads, own.kv_heads, own.dim, own.vdim, own.conv, own.kv_from, own.rot_dims) == (6, 2, 12, 10, 3, None, 8)
    assert reader.kv_from == 1 and reader.conv == 2 and c.layers[3].mixer.conv == 1 and c.layers[3].mixer.rot_dims == 0
    assert c.layers[1].mlp is None and c.layers[0].mlp.ff == 40 and c.residual_mult == 0.6 and c.norm_eps == 1e-6
    assert ZamizenConfig.from_dict(dict(CFG, note="x")).ignored == ("note",)
    bare = copy.deepcopy(CFG)
    del bare["residual_mult"], bare["layers"][0]["mixer"]["rot"]["scaling"]
    b = ZamizenConfig.from_dict(bare)
    assert b.residual_mult == 1.0 and b.layers[0].mixer.rot_scaling is None

    def broken(path, value):
        raw = copy.deepcopy(CFG)
        node = raw
        for k in path[:-1]:
            node = node[k]
        node[path[-1]] = value
        return raw

    for path, value, word in ((("layers", 0, "type"), "conv", "mixer type"), (("architecture",), "Other", "architecture"),
                              (("layers", 1, "mixer", "kv_heads"), 4, "kv_heads"), (("layers", 1, "mixer", "rot", "dims"), 3, "rot.dims"),
                              (("layers", 1, "mixer", "rot", "dims"), 14, "rot.dims"), (("layers", 0, "mixer", "rot", "dims"), 8, "rot.dims"),
                              (("layers", 1, "mixer", "conv"), 0, "conv"), (("layers", 2, "mixer", "kv_from"), 2, "kv_from"),
                              (("layers", 2, "mixer", "kv_from"), 0, "kv_from"), (("layers", 5, "mixer", "kv_from"), 2, "kv_from"),
                              (("layers", 4, "mixer", "kv_from"), 1, "kv_from"), (("layers", 0, "mlp", "kind"), "moe", "mlp.kind"),
                              (("layers", 0, "mlp", "ff"), 0, "ff"), (("layers", 0, "mixer", "kv_rank"), None, "kv_rank"),
                              (("layers", 0, "mixer", "rot", "scaling"), dict(SCALING, factor=0), "factor"),
                              (("layers", 0, "mixer", "scale"), "1", "scale"), (("width",), 0, "width"), (("layers",), [], "layers"),
                              (("norm",), None, "norm"), (("vocab",), 1.5, "vocab")):
        with pytest.raises(ConfigError) as e:
            ZamizenConfig.from_dict(broken(path, value))
        assert word in str(e.value), (path, str(e.value))


def test_registry_builds_the_model_and_names_its_tensors_cache_needs_and_order():
    from llmx_b200.cache import KVSpec, StateSpec
    from llmx_b200.registry import architecture_of
    entry = architecture_of(CFG)
    model = entry.build(entry.config_cls.from_dict(CFG))
    specs = model.tensor_specs()
    assert specs["embed"].shape == (130, 48) and specs["head"].shape == (130, 48)
    assert specs["final.norm"].shape == (48,) and specs["final.norm.b"].shape == (48,)
    for name in ("norm1", "norm1b", "norm2", "norm2b"):
        assert specs[f"l0.{name}"].shape == specs[f"l0.{name}.b"].shape == (48,)
    assert "l1.norm2" not in specs and "l1.norm2b.b" not in specs and "l1.mlp.gate" not in specs and "l1.norm1b.b" in specs
    assert specs["l0.mix.q"].shape == (3 * 16, 48) and specs["l0.mix.dkv"].shape == (26, 48) and specs["l0.mix.dkv.norm"].shape == (20,)
    assert specs["l0.mix.uk"].shape == (30, 20) and specs["l0.mix.uv"].shape == (42, 20) and specs["l0.mix.g"].shape == (42, 48)
    assert specs["l0.mix.o"].shape == (48, 42) and "l0.mix.q.b" not in specs and "l0.mix.o.b" not in specs and "l0.mix.dq" not in specs
    assert specs["l0.mlp.gate"].shape == specs["l0.mlp.up"].shape == (40, 48) and specs["l0.mlp.down"].shape == (48, 40)
    assert specs["l1.mix.q"].shape == (72, 48) and specs["l1.mix.k"].shape == (24, 48) and specs["l1.mix.v"].shape == (20, 48)
    assert specs["l1.mix.q.b"].shape == (72,) and specs["l1.mix.v.b"].shape == (20,) and specs["l1.mix.o"].shape == (48, 60)
    assert specs["l1.mix.o.b"].shape == (48,) and specs["l1.mix.q.conv"].shape == (72, 3) and specs["l1.mix.k.conv"].shape == (24, 3)
    assert specs["l1.mix.v.conv"].shape == (20, 3) and not any(n.startswith("l1.mix.") and "norm" in n for n in specs)
    # A layer that borrows keys and values has none of their tensors, and a filter of its own length on its queries.
    assert specs["l2.mix.q.conv"].shape == (72, 2) and specs["l2.mix.q.b"].shape == (72,) and specs["l2.mix.o.b"].shape == (48,)
    assert not any(n.startswith("l2.mix.k") or n.startswith("l2.mix.v") for n in specs)
    assert "l3.mix.q.conv" not in specs and specs["l3.mix.k"].shape == (8, 48) and specs["l4.mix.q"].shape == (32, 48)
    # Cache entries: the latent layer one, an attention layer with a filter two (keys and values, the filter's inputs); a
    # borrowing layer names the lender's first entry, does not write it, and has a filter state of its own.
    assert [s.block for s in model.order] == [0, 1, 2, 3, 4, 5]
    assert [s.cache_entry for s in model.order] == [0, (1, 2), (1, 3), 4, 4, (1, 5)]
    assert [s.write_cache for s in model.order] == [True, (True, True), (False, True), True, False, (False, True)]
    needs = model.cache_entry_specs()
    assert needs[0] == KVSpec(1, 20 + 6, None, planes=1)
    assert needs[1] == KVSpec(2, 12 + 10, None, planes=1) and needs[4] == KVSpec(1, 8 + 16, None, planes=1)
    assert needs[2] == StateSpec((2 * (72 + 24 + 20),), "float32")
    assert needs[3] == StateSpec((1 * 72,), "float32") and needs[5] == StateSpec((2 * 72,), "float32")
    assert len(needs) == 6


def test_blended_frequencies_against_the_plain_ones_and_by_hand():
    from llmx_b200.parts.rope import blended_frequencies, power_frequencies
    for base, dims, factor, original, fast, slow in ((500.0, 6, 4.0, 64, 32.0, 1.0), (10000.0, 64, 40.0, 4096, 32.0, 1.0),
                                                     (1e6, 16, 1.0, 128, 8.0, 2.0), (50.0, 2, 8.0, 16, 1.0, 1.0), (300.0, 12, 2.5, 4096, 64.0, 0.5)):
        f, mag = blended_frequencies(base, dims, factor, original, fast, slow)
        g, mag2 = plain.stretched_frequencies(base, dims, factor, original, fast, slow)
        assert np.allclose(f, g, rtol=1e-14) and mag == mag2 == 0.1 * math.log(factor) + 1.0
        assert np.allclose(power_frequencies(base, dims), plain.plain_frequencies(base, dims), rtol=1e-14)
    # By hand: base 500, six rotated values, original 64: the pair making 32 turns is 6 ln(64 / (64 pi)) / (2 ln 500) < 0,
    # so the ramp starts at pair 0; the pair making one turn is 6 ln(64 / (2 pi)) / (2 ln 500) = 1.12..., so it ends at 2.
    f, _ = plain.stretched_frequencies(500.0, 6, 4.0, 64, 32.0, 1.0)
    plain_f = [1.0, 500.0 ** (-1 / 3), 500.0 ** (-2 / 3)]
    assert np.allclose(f, [plain_f[0], plain_f[1] * (0.5 / 4 + 0.5), plain_f[2] / 4])


def test_plain_rotations_pair_neighbours_or_halves_and_leave_the_rest():
    x = np.arange(1.0, 8.0).reshape(1, 1, 7)
    freq = np.array([0.5, 0.1])
    for p in (0, 1, 5):
        n = plain.rotate_neighbours(x, [p], freq)[0, 0]
        h = plain.rotate_halves(x, [p], freq, magnitude=1.2)[0, 0]
        assert np.allclose(n[4:], x[0, 0, 4:]) and np.allclose(h[4:], x[0, 0, 4:])
        for i, f in enumerate(freq):
            c, s = math.cos(p * f), math.sin(p * f)
            u, v = x[0, 0, 2 * i], x[0, 0, 2 * i + 1]
            assert np.isclose(n[2 * i], u * c - v * s) and np.isclose(n[2 * i + 1], v * c + u * s)
            u, v = x[0, 0, i], x[0, 0, i + 2]
            assert np.isclose(h[i], 1.2 * (u * c - v * s)) and np.isclose(h[i + 2], 1.2 * (v * c + u * s))


def test_plain_filter_norms_and_attention_against_closed_forms():
    # The filter's last tap is on the current token; what lies before the sequence is zero.
    u = np.array([[1.0, 10.0], [2.0, 20.0], [3.0, 30.0], [4.0, 40.0]])
    w = np.array([[0.5, 0.25, 2.0], [1.0, 0.0, -1.0]])
    y = plain.causal_filter(u, w)
    assert np.allclose(y[:, 0], [2.0, 4.25, 7.0, 9.75]) and np.allclose(y[:, 1], [-10.0, -20.0, -20.0, -20.0])
    assert np.allclose(plain.causal_filter(u, np.array([[3.0], [0.5]])), u * [3.0, 0.5])
    # The centred norm: a row of equal values norms to the bias; the variance is over the row's width, eps under the root.
    x = np.array([[2.0, 4.0, 6.0, 8.0]])
    ln = plain.layer_norm(x, np.array([1.0, 2.0, 1.0, 1.0]), np.array([0.0, 0.5, 0.0, 1.0]), 0.25)
    assert np.allclose(ln, np.array([[-3.0, -2.0 + 0.5, 1.0, 3.0 + 1.0]]) / math.sqrt(5.25) * [1, 1, 1, 1] + [0, 0.5 - 0.5 / math.sqrt(5.25), 0, 1 - 1 / math.sqrt(5.25)])
    assert np.allclose(plain.layer_norm(np.full((1, 4), 7.0), np.ones(4), np.array([1.0, 2.0, 3.0, 4.0]), 1e-6), [[1.0, 2.0, 3.0, 4.0]])
    assert np.allclose(plain.unit_rms(np.array([[3.0, 4.0]]), 0.5), np.array([[3.0, 4.0]]) / math.sqrt(12.5 + 0.5))
    # Attention: the first position sees itself alone; a query head reads the key/value head of its group; nothing later is seen.
    rng = np.random.default_rng(0)
    q, k, v = rng.normal(size=(5, 4, 3)), rng.normal(size=(5, 2, 3)), rng.normal(size=(5, 2, 6))
    o = plain.causal_softmax_attention(q, k, v, 0.7)
    assert np.allclose(o[0, 0], v[0, 0]) and np.allclose(o[0, 1], v[0, 0]) and np.allclose(o[0, 2], v[0, 1]) and np.allclose(o[0, 3], v[0, 1])
    s = np.array([q[2, 3] @ k[j, 1] for j in range(3)]) * 0.7
    p = np.exp(s) / np.exp(s).sum()
    assert np.allclose(o[2, 3], p @ v[:3, 1])
    k2, v2 = k.copy(), v.copy()
    k2[3], v2[3] = 9.0, 9.0
    o2 = plain.causal_softmax_attention(q, k2, v2, 0.7)
    assert np.array_equal(o[:3], o2[:3]) and not np.allclose(o[3], o2[3])


def test_plain_model_borrowed_keys_and_layers_without_a_feed_forward():
    """The plain model on a tiny configuration: a borrowing layer's result changes with the lender's key weights and not
    with key tensors of its own (it has none), and the stream after each layer comes out one entry a layer."""
    rng = np.random.default_rng(3)
    from llmx_b200.registry import architecture_of
    entry = architecture_of(CFG)
    specs = entry.build(entry.config_cls.from_dict(CFG)).tensor_specs()
    w = {n: rng.normal(size=s.shape) * (0.3 if len(s.shape) == 2 else 1.0) for n, s in specs.items()}
    ids = [int(t) for t in rng.integers(0, 130, size=9)]
    layers = []
    logits = plain.forward(CFG, w, ids, layers_out=layers)
    assert logits.shape == (9, 130) and len(layers) == 6 and all(x.shape == (9, 48) for x in layers)
    w2 = dict(w)
    w2["l1.mix.k"] = w["l1.mix.k"] * 1.5
    layers2 = []
    plain.forward(CFG, w2, ids, layers_out=layers2)
    assert np.array_equal(layers[0], layers2[0]) and not np.allclose(layers[1], layers2[1])
    # With the lender's own attention output muted, only the borrowing layers carry the change.
    w3, w4 = dict(w), dict(w2)
    for d in (w3, w4):
        d["l1.mix.o"] = np.zeros_like(w["l1.mix.o"])
    a, b = [], []
    plain.forward(CFG, w3, ids, layers_out=a)
    plain.forward(CFG, w4, ids, layers_out=b)
    assert np.array_equal(a[1], b[1]) and not np.allclose(a[2], b[2])
    # A prefix's logits do not depend on what follows.
    assert np.allclose(plain.forward(CFG, w, ids[:5]), logits[:5])
