"""How a layer's parts are arranged.  PreNormBlock: x += mixer(norm(x)); x += ffn(norm(x)).
ParallelBlock: x += mixer(norm(x)) + ffn(norm(x)).  SandwichBlock: a norm before and after each sublayer and a factor
on what enters the stream: x += m * norm_b(mixer(norm_a(x))); x += m * norm_d(ffn(norm_c(x))).

The names of the four parts (the prefixes of their tensors) are arguments, so
the arrangement knows no architecture's tensor names.  When all four parts have a twin in the native runtime
the block has one too and runs as a single native call; with a part written in Python the block walks its parts
here.
"""
from __future__ import annotations

import ctypes
import inspect
from typing import Dict, Optional

import torch

from .. import runtime
from .base import NativeHandle, Part, StepBatch
from .linear import call_struct


def _cleared(part: Part, rows: int, device, step: StepBatch):
    """The buffer `part` wants zeroed before its forward, if it says so."""
    clear = getattr(part, "wants_cleared", None)
    if clear is None:
        return None
    if "step" in inspect.signature(clear).parameters:
        return clear(rows, device, step)
    return clear(rows, device)


class PreNormBlock(Part):
    def __init__(self, mixer_norm: Part, mixer: Part, ffn_norm: Part, ffn: Part,
                 names=("input_layernorm", "self_attn", "post_attention_layernorm", "mlp")):
        self.mixer_norm, self.mixer, self.ffn_norm, self.ffn = mixer_norm, mixer, ffn_norm, ffn
        self.names = tuple(names)
        self._native: Optional[NativeHandle] = None
        self._native_tried = False

    def children(self) -> Dict[str, Part]:
        return dict(zip(self.names, (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn)))

    def cache_spec(self):
        return self.mixer.cache_spec()

    def load(self, tensors, precision) -> None:
        super().load(tensors, precision)
        self._native, self._native_tried = None, False

    @property
    def native(self):
        if not self._native_tried:
            self._native_tried = True
            handles = [p.native for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn)]
            if all(handles):
                self._native = NativeHandle(runtime.lib().llmx_prenorm_block_create(*handles),
                                            keep=(self.mixer_norm, self.mixer, self.ffn_norm, self.ffn))
        return self._native.handle if self._native is not None else None

    def forward(self, x: torch.Tensor, step: StepBatch, cache_entry: Optional[int], write_cache: bool = True) -> None:
        """x: the float32 residual stream [rows, hidden], updated in place."""
        rows = x.shape[0]
        if self.native is not None:
            rt = runtime.lib()
            probe = step.struct_for(self)
            need = rt.llmx_part_workspace(self.native, ctypes.byref(probe), rows, -1 if cache_entry is None else int(cache_entry))
            runtime.bind_missing()
            s = step.struct_for(self, need)
            runtime.check(rt.llmx_block_forward(self.native, ctypes.byref(s), x.data_ptr(), rows,
                                                -1 if cache_entry is None else int(cache_entry), 1 if write_cache else 0), "block")
            return
        # A part may ask for a buffer to be zeroed before it runs; the norm in front of it does that in passing.
        h = self.mixer_norm.forward(x, zero=_cleared(self.mixer, rows, x.device, step))
        self.mixer.forward(h, step, cache_entry, x, write_cache)
        h = self.ffn_norm.forward(x, zero=_cleared(self.ffn, rows, x.device, step))
        self.ffn.forward(h, step, x)


class InputFilter(Part):
    """The taps of a short causal filter over time on every channel of a mixer's input, [width, taps] (the last tap lies on
    the row itself); the block that holds it applies it (`ParallelBlock(input_filter=)`) and keeps its state."""

    def __init__(self, width: int, taps: int, role: str = ""):
        if taps < 1:
            raise ValueError("input filter: at least one tap")
        self.width, self.taps, self.role = int(width), int(taps), role
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self):
        from ..weights.spec import TensorSpec
        return {self.role: TensorSpec((self.width, self.taps), std=0.3)}

    def load(self, tensors, precision) -> None:
        super().load(tensors, precision)
        self.weight = tensors[self.role].to(torch.float32).t().contiguous()       # [taps, width]: a tap of neighbouring channels is one piece


class ParallelBlock(Part):
    """x += factor * (mixer(norm(x)) + ffn(norm(x))): one norm, and both parts read its output.  `ffn` may be None (a layer
    with a mixer only).  `names`: the prefixes of the parts' tensors (norm, mixer, feed-forward, input filter).

    With `factor` 1 and no filter both parts add straight into the float32 residual.  Otherwise their outputs are
    gathered in a float32 buffer that the norm's launch clears in passing, and one kernel adds `factor` times the buffer
    into the stream.  `input_filter`: the mixer reads h + filter(h) instead of h = norm(x), a causal filter over the
    request's rows on each channel (the feed-forward reads h as it is); the norm must offer `forward_filtered`, and the
    block's cache need is then the mixer's entries and, last, a state entry of (taps - 1) * width floats (the last
    normed rows of the request; none for a filter of one tap)."""

    def __init__(self, norm: Part, mixer: Part, ffn: Optional[Part], names=("norm", "mixer", "mlp", "filter"), factor: float = 1.0,
                 input_filter: Optional[InputFilter] = None):
        self.norm, self.mixer, self.ffn = norm, mixer, ffn
        self.names = tuple(names)
        self.factor, self.input_filter = float(factor), input_filter
        if input_filter is not None and (len(self.names) < 4 or not hasattr(norm, "forward_filtered")):
            raise ValueError("parallel block: an input filter needs a name and a norm that can apply it")
        self.gathered = self.factor != 1.0 or input_filter is not None

    def children(self) -> Dict[str, Part]:
        out = {self.names[0]: self.norm, self.names[1]: self.mixer}
        if self.ffn is not None:
            out[self.names[2]] = self.ffn
        if self.input_filter is not None:
            out[self.names[3]] = self.input_filter
        return out

    def cache_spec(self):
        spec = self.mixer.cache_spec()
        if self.input_filter is None or self.input_filter.taps == 1:     # one tap reads the row itself: nothing to keep
            return spec
        from ..cache.manager import StateSpec
        mine = StateSpec(((self.input_filter.taps - 1) * self.input_filter.width,), "float32")
        return (() if spec is None else tuple(spec) if isinstance(spec, (tuple, list)) else (spec,)) + (mine,)

    def forward(self, x: torch.Tensor, step: StepBatch, cache_entry: Optional[int], write_cache: bool = True) -> None:
        """x: the float32 residual stream [rows, hidden], updated in place."""
        rows = x.shape[0]
        # Products that store their result and add their pieces with atomics want their outputs cleared first: one
        # buffer for all of the block's, cleared by the norm's launch in passing, handed back in pieces.
        wanted = []
        for part in (self.mixer, self.ffn):
            for lin in (getattr(part, "stored_products", lambda: ())() if part is not None else ()):
                n = rows * lin.out_features
                if lin.adds_pieces(rows) and n % 4 == 0:
                    wanted.append((part, lin, n))
        # A part may also ask for cleared scratch of its own (`cleared_scratch(rows)` floats, handed over as `part.scratch`).
        scratch = [(p, (p.cleared_scratch(rows) + 3) & ~3) for p in (self.mixer, self.ffn) if p is not None and hasattr(p, "cleared_scratch")]
        gathered = ((rows * x.shape[1] + 3) & ~3) if self.gathered else 0
        total = gathered + sum(n for _, _, n in wanted) + sum(n for _, n in scratch)
        flat = torch.empty(total, dtype=torch.float32, device=x.device) if total else None
        # Parts with the older way of asking (`wants_cleared`) get theirs cleared by a call of its own.
        others = [_cleared(p, rows, x.device, step) for p in (self.mixer, self.ffn) if p is not None and not hasattr(p, "stored_products")]
        filter_entry = None
        if self.input_filter is not None:
            state = None
            if self.input_filter.taps > 1:
                entries = tuple(cache_entry) if isinstance(cache_entry, (tuple, list)) else (cache_entry,)
                writes = tuple(write_cache) if isinstance(write_cache, (tuple, list)) else (write_cache,) * len(entries)
                filter_entry, entries, writes = entries[-1], entries[:-1], writes[:-1]
                cache_entry = None if not entries else entries[0] if len(entries) == 1 else entries
                write_cache = True if not writes else writes[0] if len(writes) == 1 else writes
                state = step.state(filter_entry)
            h, hm = self.norm.forward_filtered(x, self.input_filter.weight, state, step, zero=flat)
        else:
            h = hm = self.norm.forward(x, zero=flat)
        for z in others:
            if z is not None:
                z.zero_()
        at = gathered
        for part, lin, n in wanted:
            part.cleared_outputs[id(lin)] = flat[at:at + n].view(rows, lin.out_features)
            at += n
        for part, n in scratch:
            part.scratch = flat[at:at + n]
            at += n
        out = flat[:rows * x.shape[1]].view(rows, x.shape[1]) if self.gathered else x
        self.mixer.forward(hm, step, cache_entry, out, write_cache)
        if self.ffn is not None:
            self.ffn.forward(h, step, out)
        if self.gathered:
            from .. import ops
            ops.add_rows_(x, out, self.factor)


class SandwichBlock(Part):
    """x += factor * post_mixer_norm(mixer(pre_mixer_norm(x))); then, with a feed-forward,
    x += factor * post_ffn_norm(ffn(pre_ffn_norm(x))).  A sublayer's output is gathered in a float32 buffer of its own
    (cleared by the launch of the norm before the sublayer), and the norm after it adds into the stream in the same
    kernel that norms (`add_into(residual, y, factor, in_bias)` of the norm part).  A mixer that says so
    (`defer_output_bias`) leaves the bias of its output projection to that kernel.  `ffn` and its two norms may be None.
    `names`: the prefixes of the six parts' tensors."""

    def __init__(self, pre_mixer_norm: Part, mixer: Part, post_mixer_norm: Part, pre_ffn_norm: Optional[Part], ffn: Optional[Part],
                 post_ffn_norm: Optional[Part], factor: float = 1.0,
                 names=("norm1", "mix", "norm1b", "norm2", "mlp", "norm2b")):
        if (ffn is None) != (pre_ffn_norm is None) or (ffn is None) != (post_ffn_norm is None):
            raise ValueError("sandwich block: a feed-forward comes with both of its norms, or none of the three")
        self.pre_mixer_norm, self.mixer, self.post_mixer_norm = pre_mixer_norm, mixer, post_mixer_norm
        self.pre_ffn_norm, self.ffn, self.post_ffn_norm = pre_ffn_norm, ffn, post_ffn_norm
        self.factor, self.names = float(factor), tuple(names)
        if hasattr(mixer, "defer_output_bias"):
            mixer.defer_output_bias = True

    def children(self) -> Dict[str, Part]:
        parts = (self.pre_mixer_norm, self.mixer, self.post_mixer_norm, self.pre_ffn_norm, self.ffn, self.post_ffn_norm)
        return {n: p for n, p in zip(self.names, parts) if p is not None}

    def cache_spec(self):
        return self.mixer.cache_spec()

    def forward(self, x: torch.Tensor, step: StepBatch, cache_entry, write_cache=True) -> None:
        """x: the float32 residual stream [rows, hidden], updated in place."""
        rows, width = x.shape
        both = self.ffn is not None
        n = rows * width
        pad = (n + 3) & ~3                                  # the second buffer starts on a 16-byte boundary
        flat = torch.empty(pad * (2 if both else 1), dtype=torch.float32, device=x.device)
        out = flat[:n].view(rows, width)
        h = self.pre_mixer_norm.forward(x, zero=flat[:pad])
        self.mixer.forward(h, step, cache_entry, out, write_cache)
        pending = getattr(self.mixer, "output_bias", None) if getattr(self.mixer, "defer_output_bias", False) else None
        self.post_mixer_norm.add_into(x, out, self.factor, in_bias=pending)
        if both:
            out = flat[pad:pad + n].view(rows, width)
            h = self.pre_ffn_norm.forward(x, zero=flat[pad:])
            self.ffn.forward(h, step, out)
            self.post_ffn_norm.add_into(x, out, self.factor)
