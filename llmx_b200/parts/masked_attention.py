"""Grouped-query softmax attention whose keys and values have widths of their own, under a window, inside chunks, or
over everything.

For the rows of a step, with H query heads, G key/value heads (query head h reads key/value head h // (H / G)), key
width D and value width V:
    q, k, v = h Wq^T, h Wk^T, h Wv^T            (one product over the stacked weight; no biases)
    q, k    = RMSNorm per head over D with one weight of D values shared by the heads (optional), then
              rotated by position on the first `rot_dims` values of every head: value i pairs with value
              i + rot_dims / 2, the pair (u, v) at position p becomes (u cos a - v sin a, v cos a + u sin a),
              a = p * base^(-2i / rot_dims) / rot_factor   (32-bit; `rot_factor`: linear scaling of the frequencies)
    [k ; v] -> the row's cache slot             (one row of D + V values per token and key/value head)
    o       = softmax(q K^T * scale) V over the keys lo..p of the request, where lo is the larger of
              p - window + 1 (under a window) and floor(p / chunk) * chunk (inside chunks, counted from the
              request's first token whatever way its prompt was cut), or 0
    residual += o Wo^T
Sizes, the scale, whether q/k are normed, the rotation's constants, window and chunk are constructor arguments, and so
are the tensors' roles.  The cache keeps what later rows can still see: pages wholly below the window or the chunk
of the next position are given back.  Kernels: csrc/attention_split.cu.

Options for designs that vary it (any of them makes the rows go through the general finishing kernel, `llmx_qkv_finish`):
    bias True             q, k, v and the output product have biases (the tensor's role with ".b" added)
    taps n > 1            a causal filter of n taps on each channel of q, k and v right after the product (roles
                          "<q>.conv" ..., [channels, taps], last tap on the current token, zeros before the request's first
                          token); the last n - 1 product rows of a request are its state (a second cache entry, a state
                          slot of (n - 1) * channels floats)
    pairing "neighbours"  rotation pair i is (2i, 2i + 1) instead of (i, i + rot_dims / 2)
    qk_norm "after"       the per-head RMS norm comes after the rotation instead of before it
    qk_norm_weight False  the norm has no weight
    shared_kv True        the mixer has no key and value tensors: it reads the cache entry another layer's mixer of the
                          same geometry wrote (the layer order names that entry and does not write it), with queries,
                          filter state and everything else of its own
    output_bias False     with `bias`, the output product has none (biases on q, k and v alone)
    qk_norm "whole"       one RMS norm over all of a row's queries and one over all of its keys, before they are split into
                          heads and rotated, with weights of heads * D and kv_heads * D values
    rot_freq, rot_magnitude   the rotation's frequencies [rot_dims / 2] as the design scales them (float64 or float32, rounded
                          once to 32-bit; default base^(-2i / rot_dims) / rot_factor) and a factor on cosines and sines
    softcap c             score <- c tanh(score / c), after the scale
    sink "learned" | "zero"   exp(sink_h) joins head h's softmax denominator, a learned number per head (role "sink") that has
                          no key and no value; "zero": a sink of 0 (one is added to the denominator)
    rotate_values True    the value of position j is rotated by j over all of V (pair m by j * rot_base^(-2m / V), no scaling,
                          in the q/k pairing) and cached so; a row's output is turned back by its own position
With a filter the mixer's cache need is a pair (keys and values, filter state) and `forward` is handed a pair of entries.

    rounded_weights True  the design lets softmax weights enter the product with the values rounded to bfloat16 (the
                          kernels here keep them to 24 bits: the plain form in 32-bit arithmetic, the tiled form as three
                          bfloat16 parts).  Then, where keys and values are equally wide (64 or 128), nothing cuts the keys
                          into chunks and the path is bfloat16, the mixer keeps keys and values in planes of their own,
                          [pages, 2, kv_heads, page, D], and its attention is the paged kernels' (split-KV decode, tcgen05
                          prompt tiles: `ops_attn.paged_attention`), whatever finished its queries; a layer that reads
                          another's keys decides the same way, having the same geometry.  Off by default.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import numpy as np
import torch

from .. import ops, runtime
from ..cache.manager import KVSpec, StateSpec
from ..weights.spec import TensorSpec
from .base import Part, Precision, StepBatch
from .linear import Linear, stored_product


class MaskedAttention(Part):
    def __init__(self, hidden: int, heads: int, kv_heads: int, key_dim: int, value_dim: int, scale: Optional[float] = None,
                 qk_norm_eps: Optional[float] = None, rot_dims: int = 0, rot_base: float = 10000.0, rot_factor: float = 1.0,
                 window: Optional[int] = None, chunk: Optional[int] = None,
                 names=("q", "k", "v", "o", "q.norm", "k.norm"), bias: bool = False, taps: int = 1, pairing: str = "halves",
                 qk_norm: str = "before", qk_norm_weight: bool = True, shared_kv: bool = False, rounded_weights: bool = False,
                 output_bias: Optional[bool] = None, rot_freq=None, rot_magnitude: float = 1.0, softcap: Optional[float] = None,
                 sink: Optional[str] = None, rotate_values: bool = False, sink_role: str = "sink"):
        if heads % kv_heads:
            raise ValueError("attention: head count must be divisible by the key/value head count")
        if rot_dims % 2 or rot_dims > key_dim or rot_dims < 0:
            raise ValueError("attention: the rotated width must be even and at most the key width")
        self.hidden, self.heads, self.kv_heads = int(hidden), int(heads), int(kv_heads)
        self.key_dim, self.value_dim = int(key_dim), int(value_dim)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.key_dim)
        self.qk_norm_eps = qk_norm_eps
        self.rot_dims, self.rot_base, self.rot_factor = int(rot_dims), float(rot_base), float(rot_factor)
        self.window, self.chunk, self.names = window, chunk, tuple(names)
        self.q_width, self.k_width, self.v_width = self.heads * self.key_dim, self.kv_heads * self.key_dim, self.kv_heads * self.value_dim
        self.o_width = self.heads * self.value_dim
        if pairing not in ("halves", "neighbours") or qk_norm not in ("before", "after", "whole") or taps < 1:
            raise ValueError("attention: pairing is halves or neighbours, qk_norm before, after or whole, the filter has at least one tap")
        if sink not in (None, "learned", "zero") or (softcap is not None and not softcap > 0):
            raise ValueError("attention: sink is learned, zero or None; a cap on the scores is positive")
        if rotate_values and self.value_dim % 2:
            raise ValueError("attention: rotated values need an even value width")
        if rot_freq is not None and len(rot_freq) != rot_dims // 2:
            raise ValueError("attention: one frequency for each rotated pair")
        self.has_output_bias = bool(bias) if output_bias is None else bool(output_bias) and bool(bias)
        self.rot_freq = None if rot_freq is None else np.asarray(rot_freq, dtype=np.float64)
        self.rot_magnitude, self.softcap, self.sink, self.sink_role = float(rot_magnitude), softcap, sink, sink_role
        self.rotate_values = bool(rotate_values)
        self.bias, self.taps, self.pairing, self.qk_norm = bool(bias), int(taps), pairing, qk_norm
        self.qk_norm_weight, self.shared_kv = bool(qk_norm_weight), bool(shared_kv)
        self.general = (self.bias or self.taps > 1 or pairing != "halves" or qk_norm != "before" or not self.qk_norm_weight or self.shared_kv
                        or self.rot_magnitude != 1.0 or self.rotate_values)
        plain_softmax = softcap is None and sink is None and not self.rotate_values
        self.channels = self.q_width + (0 if self.shared_kv else self.k_width + self.v_width)
        # Whether the paged kernels can serve this geometry (decided for good in `load`, which knows the path's type).
        self.paged_shape = None
        if rounded_weights and plain_softmax and self.key_dim == self.value_dim and self.chunk is None and self.key_dim in (64, 128) and self.heads // self.kv_heads <= 16:
            from .attention import AttentionShape
            self.paged_shape = AttentionShape(self.heads, self.kv_heads, self.key_dim, self.window)
        self.paged = False
        self.defer_output_bias = False       # a block that reads the output through a kernel of its own may add the bias there
        self.output_bias: Optional[torch.Tensor] = None

    def stored_products(self):
        return (self.qkv,)

    def children(self):
        return {"paged": self.paged_shape} if self.paged_shape is not None else {}

    def cache_spec(self):
        kv = KVSpec(self.kv_heads, self.key_dim, self.window) if self.paged else KVSpec(self.kv_heads, self.key_dim + self.value_dim, self.window, planes=1, chunk=self.chunk)
        if self.taps > 1:
            return (kv, StateSpec(((self.taps - 1) * self.channels,), "float32"))
        return kv

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        q, k, v, o, qn, kn = self.names
        made = {q: self.q_width} if self.shared_kv else {q: self.q_width, k: self.k_width, v: self.v_width}
        specs = {o: TensorSpec((self.hidden, self.o_width))}
        for name, width in made.items():
            specs[name] = TensorSpec((width, self.hidden))
            if self.bias:
                specs[name + ".b"] = TensorSpec((width,), "vector", init="normal", std=0.02)
            if self.taps > 1:
                specs[name + ".conv"] = TensorSpec((width, self.taps), std=0.3)
        if self.has_output_bias:
            specs[o + ".b"] = TensorSpec((self.hidden,), "vector", init="normal", std=0.02)
        if self.qk_norm_eps is not None and self.qk_norm_weight:
            whole = self.qk_norm == "whole"
            specs[qn] = TensorSpec((self.q_width if whole else self.key_dim,), "vector", init="one_plus_normal", std=0.01)
            if not self.shared_kv:
                specs[kn] = TensorSpec((self.k_width if whole else self.key_dim,), "vector", init="one_plus_normal", std=0.01)
        if self.sink == "learned":
            specs[self.sink_role] = TensorSpec((self.heads,), "vector", init="normal", std=1.0)
        return specs

    def frequencies(self) -> np.ndarray:
        """base^(-2i / rot_dims) / rot_factor, i < rot_dims / 2, or the frequencies the design gave, rounded once to 32-bit."""
        if self.rot_freq is not None:
            return self.rot_freq.astype(np.float32)
        i = np.arange(self.rot_dims // 2, dtype=np.float64)
        return (np.power(self.rot_base, -2.0 * i / max(self.rot_dims, 1)) / self.rot_factor).astype(np.float32)

    def load(self, tensors, precision: Precision) -> None:
        super().load(tensors, precision)
        self.cleared_outputs = {}
        self._staged = {}                    # by the cache's type: whether the staged form of the plain attention takes these sizes
        q, k, v, o, qn, kn = self.names
        made = [q] if self.shared_kv else [q, k, v]
        self.qkv = Linear(torch.cat([tensors[n] for n in made], dim=0), precision)
        self.o = Linear(tensors[o], precision)
        self.q_norm = self.k_norm = None
        if self.qk_norm_eps is not None and self.qk_norm_weight:
            self.q_norm = tensors[qn].to(torch.float32).contiguous()
            self.k_norm = None if self.shared_kv else tensors[kn].to(torch.float32).contiguous()
        self.in_bias = torch.cat([tensors[n + ".b"] for n in made]).to(torch.float32).contiguous() if self.bias else None
        self.output_bias = tensors[o + ".b"].to(torch.float32).contiguous() if self.has_output_bias else None
        dev = self.o.weight.device
        self.vfreq = None
        if self.rotate_values:
            m = np.arange(self.value_dim // 2, dtype=np.float64)
            self.vfreq = torch.from_numpy(np.power(np.float64(self.rot_base), -2.0 * m / self.value_dim).astype(np.float32)).to(dev)
        sink = tensors[self.sink_role].to(torch.float32).contiguous() if self.sink == "learned" else self.sink
        self.extras = None
        if self.softcap is not None or self.sink is not None or self.rotate_values:
            self.extras = ops.SoftmaxExtras(self.softcap, sink, self.vfreq, self.pairing == "neighbours")
        self.taps_w = torch.cat([tensors[n + ".conv"] for n in made], dim=0).to(torch.float32).contiguous() if self.taps > 1 else None
        self.freq = torch.from_numpy(self.frequencies()).to(self.o.weight.device) if self.rot_dims else None
        self.paged = self.paged_shape is not None and precision.act is torch.bfloat16 and not precision.invariant
        self.tiled = precision.act is torch.bfloat16 and not precision.invariant and \
            ops.attention_tiled_fits(self.heads, self.kv_heads, self.key_dim, self.value_dim)

    def forward(self, h: torch.Tensor, step: StepBatch, cache_entry, residual: torch.Tensor, write_cache=True) -> None:
        """`cache_entry`: the entry of keys and values, or with a filter the pair (keys and values, filter state);
        `write_cache` likewise one flag or a pair (the filter's state is always written: it is the mixer's own)."""
        rows = h.shape[0]
        state_entry = None
        if isinstance(cache_entry, (tuple, list)):
            cache_entry, state_entry = cache_entry
        if isinstance(write_cache, (tuple, list)):
            write_cache = write_cache[0]
        write_cache = bool(write_cache) and not self.shared_kv
        if not (h.is_cuda and h.is_contiguous() and h.dtype is self.precision.act and tuple(h.shape) == (rows, self.hidden)
                and residual.dtype is torch.float32 and residual.is_contiguous() and tuple(residual.shape) == (rows, self.hidden)):
            raise runtime.KernelError("attention: rows of the path's type and the mixer's width, a float32 residual")
        group, cache = step.kv(cache_entry)
        proj = stored_product(self, self.qkv, h)                             # [rows, q | k | v], 32-bit
        q = torch.empty((rows, self.q_width), dtype=self.precision.act, device=h.device)
        slots = group.slots if write_cache else torch.full_like(group.slots, -1)
        if self.general or self.paged:
            ops.qkv_finish(proj, self.heads, 0 if self.shared_kv else self.kv_heads, self.key_dim, self.value_dim, step, q,
                           cache=None if self.shared_kv else cache, slots=None if self.shared_kv else slots, bias=self.in_bias,
                           taps_w=self.taps_w, state=step.state(state_entry) if self.taps > 1 else None,
                           norm="none" if self.qk_norm_eps is None else self.qk_norm, q_weight=self.q_norm, k_weight=self.k_norm,
                           eps=float(self.qk_norm_eps or 0.0), freq=self.freq, neighbours=self.pairing == "neighbours",
                           rot_mag=self.rot_magnitude, vfreq=self.vfreq)
        else:
            ops.qk_norm_rope_write(proj, self.heads, self.kv_heads, self.key_dim, self.value_dim, self.q_norm, self.k_norm,
                                   float(self.qk_norm_eps or 0.0), self.freq, step.positions, slots, q, cache)
        o = torch.empty((rows, self.o_width), dtype=self.precision.act, device=h.device)
        # Which kernel is a matter of speed only.  Steps that bring some request more than a few rows run the tiled
        # form (bfloat16, sizes it takes); others run the plain form, a row's keys cut into ranges when the rows alone
        # would not fill the device.
        if self.paged:
            from .. import ops_attn
            ops_attn.paged_attention(q, o, step, cache_entry, self.heads, self.kv_heads, self.key_dim, self.window, self.scale)
        elif self.tiled and step.max_row_count > 4 and cache.dtype is torch.bfloat16:
            ops.attention_tiled(q, cache, o, step, group.block_tables, self.heads, self.kv_heads, self.key_dim, self.value_dim,
                                self.window, self.chunk, self.scale, extras=self.extras)
        else:
            span = min(x for x in (step.max_context, self.window, self.chunk) if x)
            staged = self._staged.get(cache.dtype)
            if staged is None:
                staged = self._staged[cache.dtype] = not self.precision.invariant and ops.attention_staged_fits(
                    q.dtype, cache.dtype, self.heads, self.kv_heads, self.key_dim, self.value_dim)
            if staged:
                # A block a (row, key/value head, range of keys): enough ranges to fill the device three blocks an SM.
                splits = max(1, min(64, span // 128, 444 // max(rows * self.kv_heads, 1)))
            else:
                splits = 1 if self.precision.invariant else max(1, min(32, span // 128, 2368 // max(rows * self.heads, 1)))
            ops.attention_split(q, cache, o, step.row_request, step.positions, group.block_tables, self.heads, self.kv_heads,
                                self.key_dim, self.value_dim, self.window, self.chunk, self.scale, splits=splits, extras=self.extras,
                                staged=staged)
        self.o(o, out=residual, accumulate=True)
        if self.output_bias is not None and not self.defer_output_bias:
            ops.add_bias_(residual, self.output_bias)
