"""Zamizen on the GPU against the plain implementation (tests/plain_zamizen.py): every mechanism alone, whole models
under every cutting, the causal edge at and off page borders, the filter's state across portions of one and two
tokens, borrowed keys and values, far keys, slots and pages used again, long decoding, generation through the scheduler.

The configurations are this file's own: sizes that differ from one another everywhere (head counts, key / value /
latent / rotated widths, filter lengths, groups, layers without a feed-forward, without a filter, without rotation,
lenders with several borrowers), and weights scaled up so that activations are of order one and attention is far from
uniform.
"""
import copy
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import helpers
import plain_zamizen as plain

pytestmark = pytest.mark.gpu
DEV = "cuda"
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
STRETCH = {"factor": 4.0, "original": 64, "fast": 32.0, "slow": 1.0}


def dense(ff=72):
    return None if ff is None else {"kind": "dense", "ff": ff}


def latent(heads=3, dim=24, rot_dim=8, vdim=20, kv_rank=40, scale=0.2, base=10000.0, scaling=STRETCH, ff=72):
    rot = {"base": base, "dims": rot_dim}
    if scaling is not None:
        rot["scaling"] = dict(scaling)
    return {"type": "latent_attention", "mlp": dense(ff),
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale, "rot": rot}}


def attention(heads=6, kv_heads=2, dim=16, vdim=24, scale=0.3, conv=3, rot_dims=8, base=10000.0, kv_from=None, ff=72):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": {"base": base, "dims": rot_dims}}
    if conv is not None:
        m["conv"] = conv
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m, "mlp": dense(ff)}


def config(layers, width=96, vocab=200, eps=1e-5, mult=0.7):
    return {"architecture": "Zamizen", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult, "layers": layers}


# Two whole models.  P: both mixers with different sizes, a lender with two borrowers (one with a filter length of its own, one
# across other layers), a second lender without a filter, layers without a feed-forward, a latent layer with plain frequencies.
MODEL_P = config([latent(), attention(), latent(heads=2, dim=16, rot_dim=16, vdim=8, kv_rank=24, scale=0.4, base=300.0, scaling=None, ff=None),
                  attention(kv_from=1, conv=2), attention(heads=4, kv_heads=4, dim=24, vdim=8, scale=0.25, conv=None, rot_dims=24, base=500.0, ff=40),
                  attention(kv_from=1, ff=None), attention(heads=4, kv_heads=4, dim=24, vdim=8, scale=0.5, conv=None, rot_dims=24, base=500.0, kv_from=4),
                  latent(heads=5, dim=8, rot_dim=4, vdim=32, kv_rank=16, scale=0.3, scaling=dict(STRETCH, factor=16.0, original=32))])
# Q: a width and a vocabulary that are no multiples of 8 (products off the tensor cores), one head, a residual factor of one,
# nothing rotated in one layer and everything in another, a filter of five taps and one of a single tap.
MODEL_Q = config([attention(heads=1, kv_heads=1, dim=10, vdim=14, scale=0.5, conv=5, rot_dims=0, ff=30),
                  latent(heads=1, dim=9, rot_dim=6, vdim=7, kv_rank=11, scale=0.35, base=50.0, scaling=dict(STRETCH, slow=2.0), ff=None),
                  attention(heads=3, kv_heads=1, dim=10, vdim=14, scale=0.5, conv=1, rot_dims=10, kv_from=0, ff=22)],
                 width=50, vocab=101, eps=1e-6, mult=1.0)


def make_folder(tmp, cfg, seed, dtype=torch.float32, gain=5.0, sharpen=1.0, mute=()):
    """A model folder with random weights of order one: matrices N(0, 0.02) x gain (query maps x sharpen on top), biases
    of order a tenth, norm biases of order a fifth.  `mute`: tensor-name endings whose tensors are zeroed."""
    from llmx_b200.config import ZamizenConfig
    from llmx_b200.registry import architecture_of
    from llmx_b200.weights import RandomSource, write_safetensors
    c = ZamizenConfig.from_dict(cfg)
    model = architecture_of(cfg).build(c)
    specs = model.tensor_specs()
    src = RandomSource(specs, seed, dtype=torch.float32)
    tensors = {}
    for n in src.names():
        t = src.tensor(n)
        if specs[n].kind in ("matrix", "table") and not n.endswith(".conv"):
            t = t * gain
        if n.endswith(".b"):
            t = t * (10.0 if ".norm" in n else 5.0)
        if n.endswith("mix.q"):
            t = t * sharpen
        if any(n.endswith(m) for m in mute):
            t = t * 0.0
        tensors[n] = t.to(dtype)
    os.makedirs(tmp, exist_ok=True)
    with open(os.path.join(tmp, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(tmp, "model.safetensors"), tensors)
    return {n: t.to(torch.float32).numpy() for n, t in tensors.items()}


def engine_of(folder, dtype, kv_tokens, page=4, requests=4):
    from llmx_b200.engine import Engine, EngineOptions
    return Engine.from_dir(folder, EngineOptions(dtype=dtype, kv_tokens=kv_tokens, page_size=page, max_requests=requests))


def worst_error(got, refs):
    worst, where = 0.0, None
    for key, row in got.items():
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


def run_cuttings(folder, cfg, w, dtype, lengths, tol, page=4, seed=0):
    requests = {f"r{i}": helpers.random_ids(cfg["vocab"], n, seed=seed + i) for i, n in enumerate(lengths)}
    refs = {rid: plain.forward(cfg, w, ids) for rid, ids in requests.items()}
    scale = max(float(np.abs(r).max()) for r in refs.values())
    measured = {}
    for make in CUTTINGS:
        steps = make(requests)
        engine = engine_of(folder, dtype, helpers.tokens_needed(steps), page)
        got = helpers.run_trace(engine, steps)
        engine.cache.check()
        assert all(u == 0 for u in engine.cache.used_pages())
        assert engine.cache.state_slots.free_slots == engine.cache.state_slots.num_slots
        worst, where = worst_error(got, refs)
        measured[make.__name__] = worst / scale
        assert len(got) == sum(lengths)
        assert worst <= tol * scale, f"{make.__name__}: {worst:.3e} at {where} (scale {scale:.3f})"
    return measured


# ---- every mechanism alone: one- and two-layer models ----------------------------------------------------------------
SMALL = {
    "latent": [latent()],
    "latent_plain_frequencies": [latent(scaling=None, ff=None)],
    "latent_one_head_wide_rotation": [latent(heads=1, dim=8, rot_dim=32, vdim=8, kv_rank=12, scale=0.3, scaling=dict(STRETCH, factor=2.0, original=256), ff=None)],
    "latent_values_wider_than_keys": [latent(heads=4, dim=8, rot_dim=2, vdim=48, kv_rank=72, scale=0.5, base=7.0, ff=None)],
    "latent_full_size_heads": [latent(heads=2, dim=128, rot_dim=64, vdim=128, kv_rank=256, scale=0.07, ff=None)],
    "latent_nothing_rotated": [latent(heads=2, dim=16, rot_dim=0, vdim=16, kv_rank=24, scale=0.25, scaling=None, ff=None)],
    "attention": [attention()],
    "attention_without_filter": [attention(conv=None, ff=None)],
    "attention_groups_are_heads_long_filter": [attention(heads=3, kv_heads=3, dim=20, vdim=12, conv=6, rot_dims=20, ff=None)],
    "attention_one_kv_head_nothing_rotated": [attention(heads=5, kv_heads=1, dim=12, vdim=36, conv=2, rot_dims=0, ff=None)],
    "attention_wide_heads": [attention(heads=2, kv_heads=1, dim=160, vdim=72, scale=0.08, conv=4, rot_dims=64, ff=None)],
    "attention_heads_wider_than_256": [attention(heads=2, kv_heads=1, dim=320, vdim=272, scale=0.06, conv=2, rot_dims=32, ff=None)],
    "borrowed_keys_next_layer": [attention(ff=None), attention(kv_from=0, ff=None)],
    "borrowed_keys_other_filter_lengths": [attention(conv=None, ff=None), attention(kv_from=0, conv=4, ff=None), attention(kv_from=0, conv=None, ff=None)],
    "feed_forward_wide": [attention(heads=2, kv_heads=2, dim=8, vdim=8, conv=None, ff=264)],
}


@pytest.mark.parametrize("name", sorted(SMALL))
def test_one_mixer_under_every_cutting_float32(tmp_path, name):
    cfg = config(SMALL[name])
    w = make_folder(str(tmp_path), cfg, seed=7)
    run_cuttings(str(tmp_path), cfg, w, "float32", [50, 3, 77, 20, 1, 64], 1e-4)


def test_row_kernels_against_the_plain_functions():
    from llmx_b200 import ops
    g = torch.Generator().manual_seed(3)
    for width in (50, 96, 1030, 4096):
        x = torch.randn(5, width, generator=g) * 3.0 + 1.5
        wt, b, pre = torch.rand(width, generator=g) + 0.5, torch.randn(width, generator=g), torch.randn(width, generator=g)
        ref = plain.layer_norm(x.numpy(), wt.numpy(), b.numpy(), 1e-5)
        out = torch.empty(5, width, dtype=torch.float32, device=DEV)
        spare = torch.full((8,), 3.0, dtype=torch.float32, device=DEV)
        ops.layernorm(x.to(DEV), wt.to(DEV), 1e-5, out, zero=spare, bias=b.to(DEV))
        assert np.abs(out.cpu().numpy() - ref).max() <= 1e-5 and float(spare.abs().max()) == 0.0
        half = torch.empty(5, width, dtype=torch.bfloat16, device=DEV)
        ops.layernorm(x.to(DEV), wt.to(DEV), 1e-5, half, bias=b.to(DEV))
        assert np.abs(half.float().cpu().numpy() - ref).max() <= 2 ** -7 * np.abs(ref).max()
        # The norm after a sublayer: the stream takes factor * norm(y + the bias the sublayer's last product left).
        stream = torch.randn(5, width, generator=g)
        got = ops.layernorm_add_(stream.clone().to(DEV), x.to(DEV), wt.to(DEV), b.to(DEV), 1e-5, 0.7, in_bias=pre.to(DEV)).cpu().numpy()
        assert np.abs(got - (stream.numpy() + 0.7 * plain.layer_norm(x.numpy() + pre.numpy(), wt.numpy(), b.numpy(), 1e-5))).max() <= 1e-5
        # A row of equal values norms to the bias whatever the value (the variance is of deviations, not of the values).
        flat = torch.full((2, width), 1000.0)
        ops.layernorm(flat.to(DEV), wt.to(DEV), 1e-5, out[:2], bias=b.to(DEV))
        assert np.abs(out[:2].cpu().numpy() - b.numpy()).max() <= 1e-4
    o, wide = torch.randn(6, 40, generator=g), torch.randn(6, 100, generator=g) * 3
    for dtype, tol in ((torch.float32, 1e-6), (torch.bfloat16, 2 ** -7)):
        got = ops.sigmoid_gate_(o.to(dtype).to(DEV), wide.to(DEV)[:, 30:70]).float().cpu().numpy()
        ref = o.to(dtype).float().numpy() * plain.sigmoid(wide[:, 30:70].numpy().astype(np.float64))
        assert np.abs(got - ref).max() <= tol * 4
    x = torch.randn(7, 33, generator=g)
    bias = torch.randn(33, generator=g)
    assert torch.allclose(ops.add_bias_(x.clone().to(DEV), bias.to(DEV)).cpu(), x + bias)


# ---- whole models ----------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("which", ["P", "Q"])
def test_whole_models_under_every_cutting_float32(tmp_path, which):
    cfg = MODEL_P if which == "P" else MODEL_Q
    w = make_folder(str(tmp_path), cfg, seed=11)
    run_cuttings(str(tmp_path), cfg, w, "float32", [50, 3, 77, 20, 1, 64, 133], 1e-4, page=4 if which == "P" else 8)


# Twice the error measured when the budget was frozen, as a fraction of the logit scale (the plain implementation is
# exact; the path rounds the inputs of products and the cached keys, values and latents to bfloat16).
BF16_BUDGET = {"P": 6e-2, "Q": 6e-2}


@pytest.mark.parametrize("which", ["P", "Q"])
def test_whole_models_under_every_cutting_bfloat16(tmp_path, which):
    cfg = MODEL_P if which == "P" else MODEL_Q
    w = make_folder(str(tmp_path), cfg, seed=11, dtype=torch.bfloat16)
    measured = run_cuttings(str(tmp_path), cfg, w, "bfloat16", [50, 3, 77, 20, 1, 64, 133], BF16_BUDGET[which], page=16)
    print("bfloat16 error / scale:", which, measured)


# R: attention whose keys and values are equally wide, of the widths (64 and 128) for which the framework has kernels
# that round softmax weights to bfloat16.  Zamizen keeps its weights in 32-bit, so those kernels must not serve it on
# either path; a lender and a borrower among the layers, a latent layer between.
MODEL_R = config([attention(heads=4, kv_heads=2, dim=64, vdim=64, scale=0.2, conv=3, rot_dims=32),
                  latent(ff=None),
                  attention(heads=4, kv_heads=2, dim=64, vdim=64, scale=0.2, conv=2, rot_dims=32, kv_from=0, ff=None),
                  attention(heads=3, kv_heads=1, dim=128, vdim=128, scale=0.15, conv=None, rot_dims=128, base=700.0, ff=40)])


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_equally_wide_keys_and_values_under_every_cutting(tmp_path, dtype):
    from llmx_b200.engine import Engine, EngineOptions
    cfg = MODEL_R
    w = make_folder(str(tmp_path), cfg, seed=21, dtype=torch.bfloat16 if dtype == "bfloat16" else torch.float32)
    engine = Engine.from_dir(str(tmp_path), EngineOptions(dtype=dtype, kv_tokens=64, page_size=16, max_requests=2))
    assert [b.mixer.paged for b in engine.model.blocks if hasattr(b.mixer, "paged")] == [False] * 3
    del engine
    measured = run_cuttings(str(tmp_path), cfg, w, dtype, [50, 3, 77, 20, 1, 64, 133], BF16_BUDGET["P"] if dtype == "bfloat16" else 1e-4, page=16)
    print(dtype, "error / scale:", measured)


def test_the_attention_part_with_rounded_weights_runs_the_paged_kernels(tmp_path, monkeypatch):
    """`MaskedAttention(rounded_weights=True)`, which no design sets: the same model built with it keeps keys and values
    in planes and runs the paged kernels in bfloat16; it agrees with the plain implementation to the bfloat16 budget."""
    import functools
    import llmx_b200.models.zamizen as builder
    from llmx_b200.engine import Engine, EngineOptions
    from llmx_b200.parts import MaskedAttention
    monkeypatch.setattr(builder, "MaskedAttention", functools.partial(MaskedAttention, rounded_weights=True))
    cfg = MODEL_R
    w = make_folder(str(tmp_path), cfg, seed=21, dtype=torch.bfloat16)
    engine = Engine.from_dir(str(tmp_path), EngineOptions(dtype="bfloat16", kv_tokens=64, page_size=16, max_requests=2))
    assert [b.mixer.paged for b in engine.model.blocks if hasattr(b.mixer, "paged")] == [True] * 3
    del engine
    run_cuttings(str(tmp_path), cfg, w, "bfloat16", [50, 3, 77, 20, 1, 64, 133], BF16_BUDGET["P"], page=16)


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


# ---- the causal edge, at page borders and off them --------------------------------------------------------------------
LAST = {"latent": [latent(ff=None)], "attention": [attention(conv=None, ff=None)], "filtered": [attention(conv=4, ff=None)],
        "borrowed": [attention(conv=3, ff=None), attention(kv_from=0, conv=2, ff=None)]}


@pytest.mark.parametrize("kind", sorted(LAST))
@pytest.mark.parametrize("page", [4, 16])
def test_a_token_is_seen_from_its_own_position_on_and_not_before(tmp_path, kind, page):
    """Changing token j changes the logits at j and at every later position and leaves all earlier ones bit for bit as they
    were: in a prompt taken whole, in portions cut right before, at and after j, and decoded; j at page borders and off
    them, the first token and the last.  (Attention is flat here, so every visible key carries weight.)"""
    from llmx_b200.engine import StepEntry
    cfg = config(LAST[kind])
    make_folder(str(tmp_path), cfg, seed=3, sharpen=0.3)
    n = 3 * page + 7
    base = helpers.random_ids(cfg["vocab"], n, seed=1)
    for j in (0, 1, page - 1, page, 2 * page + 1, n - 1):
        other = list(base)
        other[j] = (base[j] + 1) % cfg["vocab"]
        for how in ("whole", "portions", "decoded"):
            rows = []
            for ids in (base, other):
                e = engine_of(str(tmp_path), "float32", 256, page)
                if how == "whole":
                    out = e.step([StepEntry("r", ids, list(range(n)))]).cpu().numpy()
                elif how == "portions":
                    cuts, out, at, k = [max(j, 1), 1, 2, 1, 7], [], 0, 0
                    while at < n:
                        p = max(1, min(cuts[k % 5], n - at))
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
            for i in range(j, n):
                assert np.abs(a[i] - b[i]).max() > 1e-6 * np.abs(a).max(), (how, j, i, "a position must see the token")


def test_the_filter_reads_exactly_its_taps(tmp_path):
    """A layer whose attention sees only the current token (the first key is made to win by nothing: one position) shows
    the filter alone: with the score scale at zero attention averages the values, so instead the test compares two prompts
    that differ at token j through a model whose query and key weights are muted: logits from j on differ, and the
    difference made by the filter's own reach (taps - 1 further tokens) is larger than the one made by the average."""
    from llmx_b200.engine import StepEntry
    taps = 4
    cfg = config([attention(heads=2, kv_heads=2, dim=8, vdim=8, conv=taps, rot_dims=0, ff=None)])
    w = make_folder(str(tmp_path), cfg, seed=13, mute=("mix.q", "mix.q.b"))
    ids = helpers.random_ids(cfg["vocab"], 40, seed=2)
    ref = plain.forward(cfg, w, ids)
    for portions in ([40], [1] * 40, [2] * 20, [3, 1, 2, 1, 1, 5, 2, 25], [37, 1, 1, 1]):
        e = engine_of(str(tmp_path), "float32", 64, 4)
        out, at = [], 0
        for p in portions:
            out.append(e.step([StepEntry("r", ids[at:at + p], list(range(p)))]).cpu().numpy())
            at += p
        assert np.abs(np.concatenate(out) - ref).max() <= 1e-4 * np.abs(ref).max(), portions


@pytest.mark.parametrize("kind", ["latent", "attention", "borrowed"])
def test_one_far_key_decides(tmp_path, kind):
    """A prompt of several hundred tokens in which one token, far back and at a page's last slot, first slot or in its
    middle, carries a key that the last positions' queries prefer by a wide margin (the query weights are sharpened and the
    marked token is looked for among random ones): the plain implementation's attention there is concentrated on a few
    far keys, so one page read from the wrong place, or a range of keys dropped, moves the logits far beyond the bound."""
    layers = {"latent": [latent(ff=None), latent(heads=2, dim=32, rot_dim=16, vdim=24, kv_rank=64, scale=0.15)],
              "attention": [attention(ff=None), attention(heads=4, kv_heads=1, dim=32, vdim=16, scale=0.2, conv=2, rot_dims=16)],
              "borrowed": [attention(ff=None), latent(), attention(kv_from=0, conv=None)]}[kind]
    cfg = config(layers)
    w = make_folder(str(tmp_path), cfg, seed=9, sharpen=6.0)
    run_cuttings(str(tmp_path), cfg, w, "float32", [700, 333, 517], 1e-4, page=16)


# ---- slots and pages used again, long decoding -------------------------------------------------------------------------
def test_slots_and_pages_used_again_start_from_nothing(tmp_path):
    """Requests follow one another through the same filter-state slot and the same few pages; each equals the plain
    implementation from its first token (the filter sees zeros before the start, whatever the slot held, and a borrower
    reads only what its lender wrote for this request)."""
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
def test_long_decoding(tmp_path, which):
    cfg = MODEL_P if which == "P" else MODEL_Q
    w = make_folder(str(tmp_path), cfg, seed=4)
    ids = helpers.random_ids(cfg["vocab"], 400, seed=8)
    ref = plain.forward(cfg, w, ids)
    steps = helpers.trace_tail_decoded({"r": ids}, tail=390)
    e = engine_of(str(tmp_path), "float32", 512, page=16)
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
    implementation, the filter's state and the borrowed entries included."""
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
