"""Zamizen put together from the parts, and its registration.

A layer is a sandwich block: a centred norm (weight and bias) before and after each sublayer, and a factor on what
enters the float32 residual: x += m * norm1b(mixer(norm1(x))); x += m * norm2b(ff(norm2(x))).  The mixer is one of
two, as the configuration's layer list says, in any order:
  * `attention`: grouped-query softmax attention with biases on its four products, a short causal filter on q, k and
    v, a rotation of neighbouring pairs and a unit RMS norm per head after it; a layer may read the keys and values an
    earlier such layer cached (`kv_from`) instead of making its own;
  * `latent_attention`: queries straight from the input, keys and values through one normed latent per token plus a
    rotated key part shared by the heads, two-halves rotation with frequencies blended for long contexts, a sigmoid
    gate on the heads' outputs.
The feed-forward is the gated unit with silu.  The final norm is the centred one with a bias.
Tensor names: `embed`, `l<i>.norm1|norm1b|norm2|norm2b` (+ `.b`), `l<i>.mix.<role>`, `l<i>.mlp.gate|up|down`,
`final.norm` (+ `.b`), `head`.

The design has no context limit of its own; positions are int32 and their angles 32-bit floats, exact up to 2^24.
"""
from __future__ import annotations

from ..config.zamizen import AttentionMixer, LatentMixer, ZamizenConfig
from ..parts import GatedMLP, LatentAttention, LayerNorm, LogitsHead, MaskedAttention, SandwichBlock, TokenEmbedding
from ..registry import register_architecture
from .model import LayerStep, Model, _as_tuple

MAX_POSITIONS = 1 << 24


def _mixer(cfg: ZamizenConfig, m):
    E, eps = cfg.width, cfg.norm_eps
    if isinstance(m, AttentionMixer):
        return MaskedAttention(E, m.heads, m.kv_heads, m.dim, m.vdim, scale=m.scale, qk_norm_eps=eps, rot_dims=m.rot_dims,
                               rot_base=m.rot_base, bias=True, taps=m.conv, pairing="neighbours", qk_norm="after",
                               qk_norm_weight=False, shared_kv=m.kv_from is not None)
    if isinstance(m, LatentMixer):
        return LatentAttention(E, m.heads, m.dim, m.rot_dim, m.vdim, None, m.kv_rank, m.scale, m.rot_base, m.rot_dims, eps,
                               pairing="halves", rot_scaling=m.rot_scaling.as_tuple() if m.rot_scaling else None, gate=True)
    raise TypeError(type(m).__name__)


def build_zamizen(cfg: ZamizenConfig) -> Model:
    E, eps = cfg.width, cfg.norm_eps

    def norm():
        return LayerNorm(E, eps, role="", bias="b")

    blocks = []
    for layer in cfg.layers:
        ffn = None if layer.mlp is None else GatedMLP(E, layer.mlp.ff, names=("gate", "up", "down"))
        blocks.append(SandwichBlock(norm(), _mixer(cfg, layer.mixer), norm(), norm() if ffn else None, ffn, norm() if ffn else None,
                                    factor=cfg.residual_mult))
    # The order: every layer has cache entries of its own, but a layer that reads another's keys and values names that
    # layer's entry (and does not write it) beside its own filter state.
    order, at, kv_entry = [], 0, {}
    for i, layer in enumerate(cfg.layers):
        specs = _as_tuple(blocks[i].cache_spec())
        source = getattr(layer.mixer, "kv_from", None)
        entries, writes = [], []
        for k, _ in enumerate(specs):
            if k == 0 and source is not None:
                entries.append(kv_entry[source])
                writes.append(False)
            else:
                entries.append(at)
                writes.append(True)
                at += 1
        kv_entry[i] = entries[0]
        if len(entries) == 1:
            order.append(LayerStep(i, entries[0], writes[0]))
        else:
            order.append(LayerStep(i, tuple(entries), tuple(writes)))
    embedding = TokenEmbedding(cfg.vocab, E, role="")
    head = LogitsHead(norm(), cfg.vocab, E, role="")
    return Model(embedding=embedding, blocks=blocks, head=head, order=order, vocab_size=cfg.vocab, max_positions=MAX_POSITIONS,
                 block_prefix=lambda i: f"l{i}.", embedding_prefix="embed.", head_norm_prefix="final.norm.", head_prefix="head.")


register_architecture(("Zamizen", "zamizen"), ZamizenConfig, build_zamizen)
