"""Nomutar put together from the parts, and its registration.

A layer is a parallel block: one RMS norm in groups (every part of the row by its own root mean square), and a mixer
and a feed-forward (or none) that both read the norm's output; a factor times their sum joins the float32 residual.
The mixer reads the norm's output plus a short causal filter of it over time; the block keeps the filter's inputs.
The mixer is one of three softmax attentions, as the configuration's layer list says, in any order:
  * `attention`: one RMS norm over all of a row's queries and one over all of its keys, rotation in the two-halves
    pairing with frequencies changed by wavelength, values rotated by their position and outputs turned back, capped
    scores, a sliding window, a learned sink per head in the softmax's denominator;
  * `attention_2`: biases on q, k and v, rotation of neighbouring pairs with frequencies ramped over the pair index and
    a factor on cosines and sines, capped scores, a sliding window, one added to the softmax's denominator;
  * `attention_3`: the norms of the first, two-halves rotation, causal over everything, plain softmax.
The feed-forward is a gated unit or a mixture of experts with a router (softmax over the chosen logits) beside a shared
unit under a sigmoid gate.  A stretch of the layers may run several times with the same weights (`loop`), every pass on
cache entries of its own.  The embedding carries a factor and adds a row of a hashed table of token pairs; the logits
are capped.
Tensor names: `embed`, `bigram`, `l<i>.norm1`, `l<i>.canon1`, `l<i>.mix.<role>`, `l<i>.mlp.<role>`, `final.norm`, `head`.

The design has no context limit of its own; positions are int32 and their angles 32-bit floats, exact up to 2^24.
"""
from __future__ import annotations

from ..config.nomutar import AttentionMixer, DenseMlp, NomutarConfig, RoutedMlp
from ..parts import (GatedMLP, GroupedRMSNorm, InputFilter, LogitsHead, MaskedAttention, PairHashEmbedding, ParallelBlock,
                     RoutedExperts, TokenEmbedding)
from ..parts.rope import banded_frequencies, blended_frequencies
from ..registry import register_architecture
from .model import LayerStep, Model, _as_tuple

MAX_POSITIONS = 1 << 24


def _mixer(cfg: NomutarConfig, m: AttentionMixer) -> MaskedAttention:
    freq, magnitude = None, 1.0
    sc = m.rot_scaling
    if sc is not None and m.rot_dims:
        if sc.kind == "bands":
            freq = banded_frequencies(m.rot_base, m.rot_dims, sc.factor, sc.a, sc.b, sc.original)
        else:
            freq, magnitude = blended_frequencies(m.rot_base, m.rot_dims, sc.factor, sc.original, sc.a, sc.b)
    common = dict(scale=m.scale, rot_dims=m.rot_dims, rot_base=m.rot_base, rot_freq=freq, rot_magnitude=magnitude,
                  window=m.window, softcap=m.softcap)
    if m.type == "attention_2":
        return MaskedAttention(cfg.width, m.heads, m.kv_heads, m.dim, m.vdim, bias=True, output_bias=False, pairing="neighbours",
                               sink="zero", **common)
    if m.type == "attention":
        return MaskedAttention(cfg.width, m.heads, m.kv_heads, m.dim, m.vdim, qk_norm_eps=cfg.norm_eps, qk_norm="whole",
                               sink="learned", rotate_values=True, **common)
    return MaskedAttention(cfg.width, m.heads, m.kv_heads, m.dim, m.vdim, qk_norm_eps=cfg.norm_eps, qk_norm="whole", **common)


def _feed_forward(cfg: NomutarConfig, m):
    if m is None:
        return None
    if isinstance(m, DenseMlp):
        return GatedMLP(cfg.width, m.ff, names=("gate", "up", "down"))
    if isinstance(m, RoutedMlp):
        shared = None if m.shared_ff is None else GatedMLP(cfg.width, m.shared_ff, names=("gate", "up", "down"))
        return RoutedExperts(cfg.width, m.experts, m.top, m.ff, shared=shared, shared_gate=True)
    raise TypeError(type(m).__name__)


def build_nomutar(cfg: NomutarConfig) -> Model:
    E = cfg.width
    blocks = []
    for layer in cfg.layers:
        filt = InputFilter(E, cfg.canon_taps, role="") if cfg.canon_taps > 0 else None
        blocks.append(ParallelBlock(GroupedRMSNorm(E, cfg.norm_eps, cfg.norm_groups, role=""), _mixer(cfg, layer.mixer),
                                    _feed_forward(cfg, layer.mlp), names=("norm1", "mix", "mlp", "canon1"),
                                    factor=cfg.residual_mult, input_filter=filt))
    if cfg.pair_table is not None:
        p = cfg.pair_table
        embedding = PairHashEmbedding(cfg.vocab, E, p.buckets, p.mul_prev, p.mul_cur, scale=cfg.embedding_scale, role="", pair_role="/bigram")
    else:
        embedding = TokenEmbedding(cfg.vocab, E, scale=cfg.embedding_scale, role="")
    # The order: entry 0 is the embedding's (the token before), then every run of a layer has entries of its own.
    at = 0 if cfg.pair_table is None else 1
    order = []
    for i in cfg.layer_runs():
        n = len(_as_tuple(blocks[i].cache_spec()))
        entries = tuple(range(at, at + n))
        at += n
        order.append(LayerStep(i, entries[0] if n == 1 else (entries or None), True))
    head = LogitsHead(GroupedRMSNorm(E, cfg.norm_eps, cfg.norm_groups, role=""), cfg.vocab, E, role="", softcap=cfg.logit_softcap)
    return Model(embedding=embedding, blocks=blocks, head=head, order=order, vocab_size=cfg.vocab, max_positions=MAX_POSITIONS,
                 block_prefix=lambda i: f"l{i}.", embedding_prefix="embed.", head_norm_prefix="final.norm.", head_prefix="head.",
                 embedding_entry=None if cfg.pair_table is None else 0)


register_architecture(("Nomutar", "nomutar"), NomutarConfig, build_nomutar)
