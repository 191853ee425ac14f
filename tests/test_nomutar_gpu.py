"""Nomutar on the GPU against the plain implementation (tests/plain_nomutar.py): every mechanism alone, whole models under
every cutting, the edges of the windows and of the input filter in prompts and in decoding, at page borders and off them,
far keys, slots and pages used again, long decoding, generation through the scheduler, the command line and the replay
program.

The configurations are this file's own: sizes that differ from one another everywhere (head counts, key / value /
rotated widths, windows, caps, taps, groups, experts, layers without a feed-forward), and weights scaled up so that
activations are of order one and attention is far from uniform.
"""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import helpers
import plain_nomutar as plain

pytestmark = pytest.mark.gpu
DEV = "cuda"
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BANDS = {"factor": 3.0, "low": 0.5, "high": 5.0, "original": 64}
RAMP = {"factor": 6.0, "original": 64, "fast": 16.0, "slow": 2.0}


def dense(ff=72):
    return {"kind": "dense", "ff": ff}


def moe(experts=6, top=2, ff=24, shared=40):
    m = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared is not None:
        m["shared"] = {"ff": shared}
    return m


def mixer(kind, heads, kv_heads, dim, vdim, scale, rot_dims, base, scaling, window, cap, mlp):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot_dims is not None:
        m["rot"] = {"base": base, "dims": rot_dims}
        if scaling is not None:
            m["rot"]["scaling"] = dict(scaling)
    if window is not None:
        m["mask"] = {"size": window}
    if cap is not None:
        m["softcap"] = cap
    return {"type": kind, "mixer": m, "mlp": mlp}


def att1(heads=6, kv_heads=2, dim=16, vdim=24, scale=0.3, rot_dims=8, base=300.0, scaling=BANDS, window=9, cap=4.0, mlp=None):
    return mixer("attention", heads, kv_heads, dim, vdim, scale, rot_dims, base, scaling, window, cap, mlp)


def att2(heads=4, kv_heads=2, dim=24, vdim=16, scale=0.25, rot_dims=12, base=1000.0, scaling=RAMP, window=13, cap=6.0, mlp=None):
    return mixer("attention_2", heads, kv_heads, dim, vdim, scale, rot_dims, base, scaling, window, cap, mlp)


def att3(heads=3, kv_heads=3, dim=20, vdim=12, scale=0.35, rot_dims=20, base=50.0, mlp=None):
    return mixer("attention_3", heads, kv_heads, dim, vdim, scale, rot_dims, base, None, None, None, mlp)


def config(layers, width=96, vocab=200, eps=1e-5, groups=3, mult=0.6, taps=3, loop=None, pairs=(53, 31, 5), emb_scale=3.0, cap=12.0):
    cfg = {"architecture": "Nomutar", "vocab": vocab, "width": width, "norm": {"eps": eps, "groups": groups}, "residual_mult": mult,
           "embedding": {"scale": emb_scale}, "layers": layers}
    if taps:
        cfg["canon"] = {"taps": taps}
    if loop is not None:
        cfg["loop"] = dict(zip(("start", "stop", "times"), loop))
    if pairs is not None:
        cfg["embedding"]["bigram"] = dict(zip(("buckets", "mul_prev", "mul_cur"), pairs))
    if cap is not None:
        cfg["logit_softcap"] = cap
    return cfg


# Two whole models.  P: the three mixers with different sizes, dense and routed feed-forwards and none, a looped stretch in
# the middle that runs three times, windows shorter and longer than a page.
MODEL_P = config([att2(mlp=dense()), att1(mlp=moe()), att3(mlp=moe(experts=4, top=3, ff=16, shared=None)), att2(heads=2, kv_heads=1, dim=32, vdim=32,
                                                                                                                  window=40, cap=None, scaling=None),
                  att1(heads=4, kv_heads=4, dim=32, vdim=16, rot_dims=32, window=None, cap=None, scaling=None, mlp=dense(40))],
                 loop=(1, 3, 3))
# Q: a width and a vocabulary that are no multiples of 8 (products off the tensor cores), one head, a residual factor of one, one
# group, a filter of one tap, nothing rotated in one layer, one expert of one, no pair table, no cap on the logits, no loop.
MODEL_Q = config([att2(heads=1, kv_heads=1, dim=10, vdim=14, scale=0.5, rot_dims=None, window=1, mlp=moe(experts=1, top=1, ff=10, shared=6)),
                  att1(heads=3, kv_heads=1, dim=10, vdim=6, scale=0.5, rot_dims=0, window=2, mlp=dense(22)),
                  att3(heads=2, kv_heads=1, dim=6, vdim=10, rot_dims=2, mlp=moe(experts=5, top=5, ff=6, shared=None))],
                 width=50, vocab=101, eps=1e-6, groups=1, mult=1.0, taps=1, pairs=None, cap=None)


def make_folder(tmp, cfg, seed, dtype=torch.float32, gain=5.0, sharpen=1.0):
    """A model folder with random weights of order one: matrices N(0, 0.02) x gain (query maps x sharpen on top), biases of
    order a tenth, sinks of order one, router rows as they come."""
    from llmx_b200.config import NomutarConfig
    from llmx_b200.registry import architecture_of
    from llmx_b200.weights import RandomSource, write_safetensors
    c = NomutarConfig.from_dict(cfg)
    model = architecture_of(cfg).build(c)
    specs = model.tensor_specs()
    src = RandomSource(specs, seed, dtype=torch.float32)
    tensors = {}
    for n in src.names():
        t = src.tensor(n)
        if specs[n].kind in ("matrix", "table") and not n.endswith(("canon1", "router", ".sg")):
            t = t * gain
        if n.endswith(".b") and "router" not in n:
            t = t * 5.0
        if n.endswith("mix.q"):
            t = t * sharpen
        tensors[n] = t.to(dtype)
    os.makedirs(tmp, exist_ok=True)
    with open(os.path.join(tmp, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(tmp, "model.safetensors"), tensors)
    return {n: t.to(torch.float32).numpy() for n, t in tensors.items()}


def engine_of(folder, dtype, kv_tokens, page=4, requests=4):
    from llmx_b200.engine import Engine, EngineOptions
    return Engine.from_dir(folder, EngineOptions(dtype=dtype, kv_tokens=kv_tokens, page_size=page, max_requests=requests))


def worst_error(got, refs, skip=None):
    worst, where = 0.0, None
    for key, row in got.items():
        if skip is not None and skip[key[0]][key[1]]:
            continue
        d = float(np.abs(row - refs[key[0]][key[1]]).max())
        if not np.isfinite(d):
            return float("inf"), key
        if d > worst:
            worst, where = d, key
    return worst, where


def trace_tiny_portions(requests):
    """Portions of one and two tokens from the first token on (shorter than any filter), then larger ones."""
    return helpers.trace_portions(requests, portions=[1, 2, 1, 1, 2, 2, 5, 1, 3, 2, 11, 2, 1, 29, 2])


CUTTINGS = (helpers.trace_whole, helpers.trace_tail_decoded, helpers.trace_portions, trace_tiny_portions, helpers.trace_mixed)


def references(cfg, w, requests, close=None):
    """The plain logits of every request, and (with `close`, a margin) per position whether some router's choice there was
    closer than the margin: the bfloat16 path may choose otherwise at such a position, which is no fault."""
    refs, skip = {}, {}
    for rid, ids in requests.items():
        margins = []
        refs[rid] = plain.forward(cfg, w, ids, margins=margins)
        skip[rid] = np.zeros(len(ids), dtype=bool) if close is None or not margins else np.min(np.stack(margins), axis=0) < close
    return refs, skip


def run_cuttings(folder, cfg, w, dtype, lengths, tol, page=4, seed=0, close=None):
    requests = {f"r{i}": helpers.random_ids(cfg["vocab"], n, seed=seed + i) for i, n in enumerate(lengths)}
    refs, skip = references(cfg, w, requests, close)
    assert sum(int(s.sum()) for s in skip.values()) <= 0.4 * sum(lengths)
    scale = max(float(np.abs(r).max()) for r in refs.values())
    measured = {}
    for make in CUTTINGS:
        steps = make(requests)
        engine = engine_of(folder, dtype, helpers.tokens_needed(steps), page)
        got = helpers.run_trace(engine, steps)
        engine.cache.check()
        assert all(u == 0 for u in engine.cache.used_pages())
        assert engine.cache.state_slots.free_slots == engine.cache.state_slots.num_slots
        worst, where = worst_error(got, refs, skip)
        measured[make.__name__] = worst / scale
        assert len(got) == sum(lengths)
        assert worst <= tol * scale, f"{make.__name__}: {worst:.3e} at {where} (scale {scale:.3f})"
    return measured


# ---- every mechanism alone: models of one or two layers ---------------------------------------------------------------
SMALL = {
    "attention": config([att1()]),
    "attention_no_window_no_cap_plain_frequencies": config([att1(window=None, cap=None, scaling=None)]),
    "attention_groups_are_heads_all_rotated": config([att1(heads=3, kv_heads=3, dim=20, vdim=12, rot_dims=20, window=5)], groups=1),
    "attention_one_kv_head_nothing_rotated": config([att1(heads=5, kv_heads=1, dim=12, vdim=36, rot_dims=0, window=33)], taps=0),
    "attention_wide_heads": config([att1(heads=2, kv_heads=1, dim=160, vdim=72, scale=0.08, rot_dims=64, window=70)]),
    "attention_tensor_core_sizes": config([att1(heads=8, kv_heads=2, dim=64, vdim=128, scale=0.12, rot_dims=32, window=90, base=2e5)]),
    "attention_2": config([att2()]),
    "attention_2_no_window_no_cap_plain_frequencies": config([att2(window=None, cap=None, scaling=None)], taps=5),
    "attention_2_one_head": config([att2(heads=1, kv_heads=1, dim=8, vdim=40, rot_dims=8, window=4)], groups=2, pairs=None),
    "attention_2_tensor_core_sizes": config([att2(heads=8, kv_heads=2, dim=128, vdim=128, scale=0.09, rot_dims=32, window=100, base=2e5)]),
    "attention_3": config([att3()]),
    "attention_3_tensor_core_sizes": config([att3(heads=4, kv_heads=2, dim=64, vdim=96, scale=0.11, rot_dims=48, base=2e4)], taps=2, groups=2),
    "attention_3_partly_rotated_with_bands": config([mixer("attention_3", 4, 2, 16, 8, 0.3, 6, 20.0, BANDS, None, None, None)], taps=2),
    "dense_feed_forward": config([att3(heads=2, kv_heads=2, dim=8, vdim=8, rot_dims=8, mlp=dense(264))]),
    "routed_experts_with_shared": config([att3(heads=2, kv_heads=2, dim=8, vdim=8, rot_dims=8, mlp=moe())], mult=0.5),
    "routed_experts_alone_top_one": config([att3(heads=2, kv_heads=2, dim=8, vdim=8, rot_dims=8, mlp=moe(experts=9, top=1, ff=32, shared=None))]),
    "looped_twice": config([att1(mlp=dense(24)), att2(mlp=moe(experts=3, top=2, ff=8, shared=16))], loop=(0, 2, 2)),
    "ten_layers_with_windows_of_their_own": config([att2(heads=2, kv_heads=1, dim=8, vdim=8, rot_dims=8, window=w) for w in range(3, 13)], taps=2),
    "no_pair_table_no_caps_no_filter": config([att2(cap=None)], pairs=None, cap=None, taps=0, emb_scale=1.0, mult=1.0),
}


@pytest.mark.parametrize("name", sorted(SMALL))
def test_one_mechanism_under_every_cutting_float32(tmp_path, name):
    cfg = SMALL[name]
    w = make_folder(str(tmp_path), cfg, seed=7)
    run_cuttings(str(tmp_path), cfg, w, "float32", [50, 3, 77, 20, 1, 64], 1e-4)


@pytest.mark.parametrize("name", ["attention_tensor_core_sizes", "attention_2_tensor_core_sizes", "attention_3_tensor_core_sizes", "attention",
                                  "attention_2_one_head"])
def test_one_mixer_under_every_cutting_bfloat16(tmp_path, name):
    """The tiled attention (prompt portions) and the plain one (decoded rows) on the bfloat16 path, sizes it takes and not."""
    cfg = SMALL[name]
    w = make_folder(str(tmp_path), cfg, seed=7, dtype=torch.bfloat16)
    measured = run_cuttings(str(tmp_path), cfg, w, "bfloat16", [50, 3, 77, 20, 1, 150], 1.2e-2, page=16)
    print("bfloat16 error / scale:", name, measured)


def test_row_kernels_against_the_plain_functions():
    from llmx_b200 import ops
    g = torch.Generator().manual_seed(3)
    for width, groups in ((50, 1), (96, 3), (1032, 4), (4096, 8)):
        x = torch.randn(5, width, generator=g) * 3.0 + 1.5
        wt = torch.rand(width, generator=g) + 0.5
        ref = plain.grouped_rms_norm(x.numpy(), wt.numpy(), 1e-5, groups)
        out = torch.empty(5, width, dtype=torch.float32, device=DEV)
        spare = torch.full((8,), 3.0, dtype=torch.float32, device=DEV)
        ops.group_norm_conv(x.to(DEV), wt.to(DEV), 1e-5, groups, out, zero=spare)
        assert np.abs(out.cpu().numpy() - ref).max() <= 1e-5 * np.abs(ref).max() and float(spare.abs().max()) == 0.0
        rows = torch.tensor([4, 0, 4], dtype=torch.int32, device=DEV)
        half = torch.empty(3, width, dtype=torch.bfloat16, device=DEV)
        ops.group_norm_conv(x.to(DEV), wt.to(DEV), 1e-5, groups, half, row_index=rows)
        assert np.abs(half.float().cpu().numpy() - ref[[4, 0, 4]]).max() <= 2 ** -7 * np.abs(ref).max()
        # A filter of one tap keeps no state: hm = h (1 + w).
        tap = torch.randn(1, width, generator=g)
        both = torch.empty(2, 5, width, dtype=torch.float32, device=DEV)
        ops.group_norm_conv(x.to(DEV), wt.to(DEV), 1e-5, groups, both[0], taps_w=tap.to(DEV), filtered=both[1])
        assert np.abs(both[1].cpu().numpy() - ref * (1.0 + tap.numpy()[0])).max() <= 1e-5 * np.abs(ref).max()
    z = torch.randn(7, 33, generator=g) * 40
    assert np.abs(ops.softcap_(z.clone().to(DEV), 30.0).cpu().numpy() - plain.soft_cap(z.numpy().astype(np.float64), 30.0)).max() <= 1e-5
    x, y, f = torch.randn(7, 33, generator=g), torch.randn(7, 33, generator=g), torch.rand(7, generator=g)
    assert torch.allclose(ops.add_rows_(x.clone().to(DEV), y.to(DEV), 0.7).cpu(), x + 0.7 * y, atol=1e-6)
    assert torch.allclose(ops.add_rows_(x.clone().to(DEV), y.to(DEV), 1.0, f.to(DEV)).cpu(), x + f[:, None] * y, atol=1e-6)


def test_the_router_chooses_and_weighs_as_the_plain_one():
    from llmx_b200 import ops
    g = torch.Generator().manual_seed(5)
    for rows, width, experts, top in ((9, 50, 7, 3), (4, 96, 1, 1), (130, 64, 16, 16), (3, 40, 33, 5)):
        h = torch.randn(rows, width, generator=g)
        wr, b, sg = torch.randn(experts, width, generator=g), torch.randn(experts, generator=g), torch.randn(1, width, generator=g)
        z = h.double().numpy() @ wr.double().numpy().T + b.double().numpy()
        choice = torch.empty(rows, top, dtype=torch.int32, device=DEV)
        weight = torch.empty(rows, top, dtype=torch.float32, device=DEV)
        gate = torch.empty(rows, dtype=torch.float32, device=DEV)
        ops.moe_router(h.to(DEV), torch.cat([wr, sg]).to(DEV), b.to(DEV), experts, top, choice, weight, gate)
        order = np.argsort(-z, axis=1, kind="stable")[:, :top]
        assert np.array_equal(choice.cpu().numpy(), order)
        p = np.exp(np.take_along_axis(z, order, 1) - z.max(axis=1, keepdims=True))
        assert np.abs(weight.cpu().numpy() - p / p.sum(axis=1, keepdims=True)).max() <= 1e-5
        assert np.abs(gate.cpu().numpy() - plain.sigmoid(h.double().numpy() @ sg.double().numpy()[0])).max() <= 1e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads, kv_heads, D, V", [(6, 2, 64, 80), (8, 1, 32, 32), (16, 1, 16, 24), (4, 4, 128, 256), (5, 5, 8, 512)])
def test_the_staged_attention_kernel_against_a_plain_sum(dtype, heads, kv_heads, D, V):
    """Rows of several requests at positions of their own over pages in no order, key ranges of 1, 3 and 7, with and without a
    window, a cap, a sink and rotated values: the staged form and the form of one block a (row, head), both against sums in
    double precision over the same cached rows."""
    from llmx_b200 import ops
    g = torch.Generator().manual_seed(heads * 1000 + D)
    page, n_pages, requests = 16, 40, 3
    cache = (torch.randn(n_pages, 1, kv_heads, page, D + V, generator=g) * 0.7).to(dtype).to(DEV)
    tables = torch.stack([torch.randperm(n_pages, generator=g)[:12] for _ in range(requests)]).to(torch.int32).to(DEV)
    positions = [0, 1, 15, 16, 17, 100, 190, 191]
    row_request = [0, 1, 2, 0, 1, 2, 0, 1]
    q = (torch.randn(len(positions), heads * D, generator=g)).to(dtype).to(DEV)
    sink = torch.randn(heads, generator=g).to(DEV)
    vfreq = torch.from_numpy(np.power(100.0, -2.0 * np.arange(V // 2) / V).astype(np.float32)).to(DEV)
    pos_t, req_t = torch.tensor(positions, dtype=torch.int32, device=DEV), torch.tensor(row_request, dtype=torch.int32, device=DEV)
    c64, q64, scale = cache.double().cpu().numpy(), q.double().cpu().numpy().reshape(len(positions), heads, D), 0.3
    for window, cap, sk, turn in ((None, None, None, False), (37, 5.0, "learned", True), (1, None, "zero", False), (150, 2.0, None, True)):
        ref = np.zeros((len(positions), heads, V))
        for r, (p, rq) in enumerate(zip(positions, row_request)):
            lo = 0 if window is None else max(0, p - window + 1)
            rows = np.stack([c64[int(tables[rq, t // page]), 0, :, t % page] for t in range(lo, p + 1)])       # [keys, G, D + V]
            for h in range(heads):
                kvh = h // (heads // kv_heads)
                sc = rows[:, kvh, :D] @ q64[r, h] * scale
                sc = plain.soft_cap(sc, cap) if cap else sc
                extra = [] if sk is None else [float(sink[h]) if sk == "learned" else 0.0]
                m = max([sc.max()] + extra)
                e = np.exp(sc - m)
                o = (e / (e.sum() + sum(np.exp(x - m) for x in extra))) @ rows[:, kvh, D:]
                ref[r, h] = plain.rotate(o[None, None], [p], vfreq.double().cpu().numpy(), "halves", sign=-1.0)[0, 0] if turn else o
        extras = ops.SoftmaxExtras(cap, sink if sk == "learned" else sk, vfreq if turn else None, False)
        for staged in (True, False):
            for splits in (1, 3, 7):
                out = torch.empty(len(positions), heads * V, dtype=dtype, device=DEV)
                ops.attention_split(q, cache, out, req_t, pos_t, tables, heads, kv_heads, D, V, window, None, scale, splits=splits,
                                    extras=extras, staged=staged and ops.attention_staged_fits(dtype, dtype, heads, kv_heads, D, V))
                err = np.abs(out.double().cpu().numpy().reshape(ref.shape) - ref).max()
                assert err <= (2e-5 if dtype is torch.float32 else 2e-2) * max(np.abs(ref).max(), 1.0), (window, staged, splits, err)
    assert ops.attention_staged_fits(dtype, dtype, heads, kv_heads, D, V) or D % 8


# ---- whole models ----------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("which", ["P", "Q"])
def test_whole_models_under_every_cutting_float32(tmp_path, which):
    cfg = MODEL_P if which == "P" else MODEL_Q
    w = make_folder(str(tmp_path), cfg, seed=11)
    run_cuttings(str(tmp_path), cfg, w, "float32", [50, 3, 77, 20, 1, 64, 133], 1e-4, page=4 if which == "P" else 8)


# About twice the error measured when the budget was frozen, as a fraction of the logit scale (the plain implementation is
# exact; the path rounds the inputs of products and the cached keys and values to bfloat16).  Positions where a router's
# choice is closer than a twentieth of the spread of its logits are left out: rounding may turn the choice there.
BF16_BUDGET = {"P": 5e-2, "Q": 1.2e-2}


@pytest.mark.parametrize("which", ["P", "Q"])
def test_whole_models_under_every_cutting_bfloat16(tmp_path, which):
    cfg = MODEL_P if which == "P" else MODEL_Q
    w = make_folder(str(tmp_path), cfg, seed=11, dtype=torch.bfloat16)
    measured = run_cuttings(str(tmp_path), cfg, w, "bfloat16", [50, 3, 77, 20, 1, 64, 133], BF16_BUDGET[which], page=16, close=0.05)
    print("bfloat16 error / scale:", which, measured)


def test_a_request_in_a_batch_equals_the_request_alone(tmp_path):
    """Unequal requests in one step (a long portion, a short one, single tokens after history) against each alone."""
    from llmx_b200.engine import StepEntry
    cfg = MODEL_P
    make_folder(str(tmp_path), cfg, seed=5)
    ids = {r: helpers.random_ids(cfg["vocab"], n, seed=40 + i) for i, (r, n) in enumerate({"a": 90, "b": 31, "c": 12, "d": 2}.items())}
    alone = {}
    for r, t in ids.items():
        e = engine_of(str(tmp_path), "float32", 256)
        cut = len(t) // 2
        e.step([StepEntry(r, t[:cut], [])])
        alone[r] = e.step([StepEntry(r, t[cut:], list(range(len(t) - cut)))]).cpu().numpy()
    e = engine_of(str(tmp_path), "float32", 512)
    e.step([StepEntry(r, t[:len(t) // 2], []) for r, t in ids.items()])
    got = e.step([StepEntry(r, t[len(t) // 2:], list(range(len(t) - len(t) // 2))) for r, t in ids.items()]).cpu().numpy()
    at = 0
    for r, t in ids.items():
        n = len(t) - len(t) // 2
        assert np.abs(got[at:at + n] - alone[r]).max() <= 1e-5 * np.abs(alone[r]).max(), r
        at += n


# ---- the edges: what a position sees, at page borders and off them ---------------------------------------------------------
EDGES = {"attention": (att1, 9), "attention_2": (att2, 6), "attention_wide_window": (att1, 21)}


@pytest.mark.parametrize("kind", sorted(EDGES))
@pytest.mark.parametrize("page", [4, 16])
def test_a_token_is_seen_from_its_own_position_to_the_window_s_end_and_no_further(tmp_path, kind, page):
    """One layer with a window of w keys, an input filter of t taps and the pair table.  Token j enters position i through
    the pair row of j and j + 1, the filter's taps and the window: the logits at i differ for j <= i <= j + w + t - 1 and are
    bit for bit the same before j and from j + w + t on; in a prompt taken whole, in portions cut around j and around the far
    edge, and decoded; j at page borders and off them.  (Attention is flat here, so every visible key carries weight.)"""
    from llmx_b200.engine import StepEntry
    make, window = EDGES[kind]
    taps = 3
    cfg = config([make(window=window, cap=50.0)], taps=taps, cap=None)
    make_folder(str(tmp_path), cfg, seed=3, sharpen=0.3)
    reach = window + taps - 1                     # the last position token j reaches is j + reach
    n = 3 * page + reach + 9
    base = helpers.random_ids(cfg["vocab"], n, seed=1)
    for j in (0, 1, page - 1, page, 2 * page + 1):
        other = list(base)
        other[j] = (base[j] + 1) % cfg["vocab"]
        for how in ("whole", "portions", "decoded"):
            rows = []
            for ids in (base, other):
                e = engine_of(str(tmp_path), "float32", 256, page)
                if how == "whole":
                    out = e.step([StepEntry("r", ids, list(range(n)))]).cpu().numpy()
                elif how == "portions":
                    cuts, out, at, k = [max(j, 1), 1, 2, reach - 3, 2, 1, 7], [], 0, 0
                    while at < n:
                        p = max(1, min(cuts[k % len(cuts)], n - at))
                        out.append(e.step([StepEntry("r", ids[at:at + p], list(range(p)))]).cpu().numpy())
                        at, k = at + p, k + 1
                    out = np.concatenate(out)
                else:
                    head = max(min(j - 1, n), 1)
                    out = [e.step([StepEntry("r", ids[:head], list(range(head)))]).cpu().numpy()]
                    out += [e.step([StepEntry("r", [t], [0])]).cpu().numpy() for t in ids[head:]]
                    out = np.concatenate(out)
                e.cache.check()
                rows.append(out)
            a, b = rows
            assert np.array_equal(a[:j], b[:j]), (how, j, "a later token was seen")
            for i in range(j, j + reach + 1):
                assert np.abs(a[i] - b[i]).max() > 1e-6 * np.abs(a).max(), (how, j, i, "a position must see the token")
            assert np.array_equal(a[j + reach + 1:], b[j + reach + 1:]), (how, j, "a token beyond the window was seen")


def test_the_filter_and_the_pair_table_across_portions(tmp_path):
    """A filter of five taps and the pair table across portions of one, two and three rows from the first token on, and
    across requests that share a step: every portion begins with rows whose earlier inputs lie in the state."""
    from llmx_b200.engine import StepEntry
    cfg = config([att3(heads=2, kv_heads=2, dim=8, vdim=8, rot_dims=0)], taps=5)
    w = make_folder(str(tmp_path), cfg, seed=13)
    ids = helpers.random_ids(cfg["vocab"], 40, seed=2)
    ref = plain.forward(cfg, w, ids)
    for portions in ([40], [1] * 40, [2] * 20, [3, 1, 2, 1, 1, 5, 2, 25], [37, 1, 1, 1]):
        e = engine_of(str(tmp_path), "float32", 128, 4)
        out, at = [], 0
        for p in portions:
            # a second request beside it, so that the rows' requests differ within a step
            got = e.step([StepEntry("s", ids[at:at + p][::-1], []), StepEntry("r", ids[at:at + p], list(range(p)))]).cpu().numpy()
            out.append(got)
            at += p
        assert np.abs(np.concatenate(out) - ref).max() <= 1e-4 * np.abs(ref).max(), portions


@pytest.mark.parametrize("kind", ["attention_3", "attention_window", "attention_2_window"])
def test_far_keys_decide(tmp_path, kind):
    """Prompts of several hundred tokens with sharpened queries: attention is concentrated on a few keys, far back for the
    causal layer and anywhere in a window of hundreds for the others, so one page read from the wrong place, a range of
    keys dropped or a window one key off moves the logits far beyond the bound."""
    layers = {"attention_3": [att3(), att3(heads=4, kv_heads=1, dim=32, vdim=16, scale=0.2, rot_dims=16, mlp=dense(40))],
              "attention_window": [att1(window=300, cap=30.0), att1(heads=4, kv_heads=1, dim=32, vdim=16, window=129, cap=None)],
              "attention_2_window": [att2(window=200, cap=30.0), att2(heads=3, kv_heads=3, window=257, scaling=dict(RAMP, original=32))]}[kind]
    cfg = config(layers)
    w = make_folder(str(tmp_path), cfg, seed=9, sharpen=6.0)
    run_cuttings(str(tmp_path), cfg, w, "float32", [700, 333, 517], 1e-4, page=16)


def test_a_sink_takes_its_share(tmp_path):
    """The same model with its sinks moved far down (no share) and far up (nearly all of it): both agree with the plain
    implementation, and they differ from one another, so the sink is neither left out nor counted twice."""
    from llmx_b200.engine import StepEntry
    cfg = config([att1(window=7)])
    ids = helpers.random_ids(cfg["vocab"], 30, seed=4)
    outs = []
    for shift in (-30.0, 0.0, 6.0):
        folder = str(tmp_path / f"s{shift}")
        w = make_folder(folder, cfg, seed=21)
        w["l0.mix.sink"] = w["l0.mix.sink"] + np.float32(shift)
        from llmx_b200.weights import write_safetensors
        write_safetensors(os.path.join(folder, "model.safetensors"), {n: torch.from_numpy(np.ascontiguousarray(t)) for n, t in w.items()})
        ref = plain.forward(cfg, w, ids)
        got = engine_of(folder, "float32", 64).step([StepEntry("r", ids, list(range(30)))]).cpu().numpy()
        assert np.abs(got - ref).max() <= 1e-4 * np.abs(ref).max(), shift
        outs.append(got)
    assert np.abs(outs[0] - outs[1]).max() > 1e-3 * np.abs(outs[1]).max() and np.abs(outs[2] - outs[1]).max() > 1e-3 * np.abs(outs[1]).max()


# ---- slots and pages used again, long decoding -------------------------------------------------------------------------
def test_slots_and_pages_used_again_start_from_nothing(tmp_path):
    """Requests follow one another through the same state slots and the same few pages; each equals the plain
    implementation from its first token (the filter sees zeros and the pair table its last row at a request's start,
    whatever the slot held)."""
    from llmx_b200.engine import StepEntry
    cfg = MODEL_P
    w = make_folder(str(tmp_path), cfg, seed=2)
    e = engine_of(str(tmp_path), "float32", 64, page=4, requests=1)
    for i in range(5):
        ids = helpers.random_ids(cfg["vocab"], 40 + 5 * i, seed=90 + i)
        ref = plain.forward(cfg, w, ids)
        got = np.concatenate([e.step([StepEntry(i, ids[:2], [0, 1])]).cpu().numpy(),
                              e.step([StepEntry(i, ids[2:], list(range(len(ids) - 2)))]).cpu().numpy()])
        e.end(i)
        e.cache.check()
        assert np.abs(got - ref).max() <= 1e-4 * np.abs(ref).max(), i
    assert all(u == 0 for u in e.cache.used_pages())


@pytest.mark.parametrize("which", ["P", "Q"])
def test_long_decoding_with_windows_passing_over_decoded_tokens(tmp_path, which):
    cfg = MODEL_P if which == "P" else MODEL_Q
    w = make_folder(str(tmp_path), cfg, seed=4)
    ids = helpers.random_ids(cfg["vocab"], 300, seed=8)
    ref = plain.forward(cfg, w, ids)
    steps = helpers.trace_tail_decoded({"r": ids}, tail=290)
    e = engine_of(str(tmp_path), "float32", 320, page=16)
    got = helpers.run_trace(e, steps)
    worst, where = worst_error(got, {"r": ref})
    assert worst <= 1e-4 * np.abs(ref).max(), where


# ---- the framework's entry points ------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_scheduler(tmp_path, dtype):
    from llmx_b200.engine.generate import LLM
    from llmx_b200.sampling import SamplingParams
    cfg = MODEL_P
    w = make_folder(str(tmp_path), cfg, seed=6, dtype=torch.bfloat16 if dtype == "bfloat16" else torch.float32)
    prompts = [helpers.random_ids(cfg["vocab"], n, seed=n) for n in (5, 17, 33, 60)]
    llm = LLM(str(tmp_path), dtype=dtype, kv_tokens=512, page_size=16, ubatch=24, max_seqs=3)
    outs = llm.generate(prompts, SamplingParams(max_tokens=24, temp=0.0, top_k=0, top_p=1.0, ignore_eos=True))
    assert [len(o.tokens) for o in outs] == [24] * 4
    for p, o in zip(prompts, outs):
        ids = list(p)
        for t in o.tokens:
            logits = plain.forward(cfg, w, ids)[-1]
            best = int(np.argmax(logits))
            gap = 2 * BF16_BUDGET["P"] if dtype == "bfloat16" else 1e-4
            assert t == best or logits[best] - logits[t] <= gap * np.abs(logits).max(), (len(ids), t, best)
            ids.append(t)
    assert all(u == 0 for u in llm.engine.cache.used_pages())
    assert llm.engine.cache.state_slots.free_slots == llm.engine.cache.state_slots.num_slots


def test_recorded_steps_equal_plain_steps(tmp_path):
    """Steps whose shape keeps coming are recorded as CUDA graphs and replayed: the same logits as the plain
    implementation, the filter's state, the token before and the routing included."""
    from llmx_b200.engine import Engine, EngineOptions
    cfg = MODEL_P
    w = make_folder(str(tmp_path), cfg, seed=14)
    requests = {f"r{i}": helpers.random_ids(cfg["vocab"], n, seed=30 + i) for i, n in enumerate([70, 70, 70, 41])}
    refs = {rid: plain.forward(cfg, w, ids) for rid, ids in requests.items()}
    steps = helpers.trace_portions(requests, portions=[7, 7, 7, 7, 7, 7, 7, 7, 7, 1, 1, 1, 1, 1, 1, 1])
    engine = Engine.from_dir(str(tmp_path), EngineOptions(dtype="float32", kv_tokens=256, page_size=16, max_requests=2, record_after=1))
    assert engine.model.recordable
    got = helpers.run_trace(engine, steps, record=True)
    assert len(engine.step_recordings) >= 2          # the portion of seven rows and the single row, at least
    worst, where = worst_error(got, refs)
    assert worst <= 1e-4 * max(float(np.abs(r).max()) for r in refs.values()), where
    engine.cache.check()


def test_command_line_generates_from_a_folder(tmp_path):
    cfg = MODEL_Q
    w = make_folder(str(tmp_path), cfg, seed=15, dtype=torch.bfloat16)
    run = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "llmx"), "generate", str(tmp_path), "5,17,3,99", "-n", "6", "--temp", "0",
                          "--ignore-eos", "--dtype", "f32"], capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stderr[-2000:]
    ids = next(l for l in run.stdout.splitlines() if l.startswith("ids: "))
    tokens = [int(t) for t in ids[5:].split(",")]
    assert len(tokens) == 6
    seq = [5, 17, 3, 99]
    for t in tokens:
        logits = plain.forward(cfg, w, seq)[-1]
        best = int(np.argmax(logits))
        assert t == best or logits[best] - logits[t] <= 1e-4 * np.abs(logits).max()
        seq.append(t)


def test_trace_run_program(tmp_path):
    cfg = MODEL_Q
    w = make_folder(str(tmp_path / "m"), cfg, seed=12, dtype=torch.bfloat16)
    requests = {f"q{i}": helpers.random_ids(cfg["vocab"], n, seed=50 + i) for i, n in enumerate([45, 3, 80, 20, 64])}
    steps = helpers.trace_mixed(requests, tail=5)
    for dtype, tol in (("float32", 1e-4), ("bfloat16", BF16_BUDGET["Q"])):
        out = tmp_path / ("out_" + dtype)
        proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", str(tmp_path / "m"), "--dtype", dtype,
                               "--out", str(out), "--max-tokens", str(helpers.tokens_needed(steps))],
                              input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
        assert proc.returncode == 0, proc.stderr[-2000:]
        assert [l for l in proc.stdout.splitlines() if l.startswith("done ")] == [f"done {s['step']}" for s in steps]
        got = helpers.read_trace_output(steps, str(out), cfg["vocab"])
        refs = {rid: plain.forward(cfg, w, ids) for rid, ids in requests.items()}
        worst, where = worst_error(got, refs)
        assert worst <= tol * max(float(np.abs(r).max()) for r in refs.values()), (dtype, worst, where)
