"""The two ends of a model: token embedding and the logits head."""
from __future__ import annotations

import ctypes
from typing import Dict, Optional

import torch

from .. import runtime
from ..weights.spec import TensorSpec
from .base import NativeHandle, Part, Precision, StepBatch
from .linear import Linear, bare_step


class TokenEmbedding(Part):
    """x[r, :] = table[ids[r], :] widened to 32-bit (src/model/arch/blocks.hpp:95-97), times `scale` when the
    architecture has a factor on its embedding (the product is made in 32-bit).  `role`: the table's tensor role."""

    def __init__(self, vocab: int, hidden: int, scale: float = 1.0, role: str = "weight"):
        self.vocab, self.hidden = int(vocab), int(hidden)
        self.scale, self.role = float(scale), role
        self.table: Optional[torch.Tensor] = None
        self._native: Optional[NativeHandle] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self.role: TensorSpec((self.vocab, self.hidden), "table")}

    def load(self, tensors, precision: Precision) -> None:
        super().load(tensors, precision)
        self.table = tensors[self.role].to(precision.act).contiguous()
        self._native = None

    @property
    def native(self):
        if self.scale != 1.0:
            return None               # the runtime's embedding has no factor: the kernel with one is called from here
        if self._native is None:
            runtime.need("rowwise")
            self._native = NativeHandle(runtime.lib().llmx_embedding_create(self.table.data_ptr(), runtime.code(self.table.dtype),
                                                                           self.vocab, self.hidden), keep=(self.table,))
        return self._native.handle

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        if not (ids.is_cuda and ids.dtype is torch.int32 and ids.is_contiguous()):
            raise runtime.KernelError("embed: ids must be int32 on the device")
        x = torch.empty((ids.numel(), self.hidden), dtype=torch.float32, device=ids.device)
        if self.scale != 1.0:
            from .. import ops
            return ops.embed_scaled(self.table, ids, x, self.scale)
        s = bare_step(ids.device)
        runtime.check(runtime.lib().llmx_embedding_forward(self.native, ctypes.byref(s), ids.data_ptr(), x.data_ptr(), ids.numel()),
                      "embed")
        return x


class PairHashEmbedding(TokenEmbedding):
    """x[r] = table[id] * scale + pairs[(id before * mul_prev + id * mul_cur) mod buckets]; a request's first token takes
    row `buckets` (the last) of the pair table.  The id before a step's first row is the request's state: one int32 in a
    state slot (`cache_spec`), read at the slot the step reads and written, with the step's last id, at the slot it
    writes.  `pair_role`: the pair table's tensor role (with a leading "/" a name of its own)."""

    def __init__(self, vocab: int, hidden: int, buckets: int, mul_prev: int, mul_cur: int, scale: float = 1.0, role: str = "weight",
                 pair_role: str = "pairs"):
        super().__init__(vocab, hidden, scale, role)
        self.buckets, self.mul_prev, self.mul_cur, self.pair_role = int(buckets), int(mul_prev), int(mul_cur), pair_role
        self.pairs: Optional[torch.Tensor] = None

    def cache_spec(self):
        from ..cache.manager import StateSpec
        return StateSpec((1,), "int32")

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self.role: TensorSpec((self.vocab, self.hidden), "table"),
                self.pair_role: TensorSpec((self.buckets + 1, self.hidden), "table")}

    def load(self, tensors, precision: Precision) -> None:
        super().load(tensors, precision)
        self.pairs = tensors[self.pair_role].to(precision.act).contiguous()

    @property
    def native(self):
        return None

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        raise runtime.KernelError("a pair embedding needs the step (the token before a request's rows): forward_step")

    def forward_step(self, step: StepBatch, cache_entry: int) -> torch.Tensor:
        from .. import ops
        ids = step.token_ids
        x = torch.empty((ids.numel(), self.hidden), dtype=torch.float32, device=ids.device)
        return ops.embed_pairs(self.table, self.pairs, ids, x, self.scale, self.buckets, self.mul_prev, self.mul_cur,
                               step.state(cache_entry), step)


class LogitsHead(Part):
    """Logits for the rows that want them: gather, norm, product (src/model/arch/blocks.hpp:267-272).

    The product's weight is the model's own `weight` tensor, or, when `tied_to`
    is given, the embedding's table (the reference's alias, src/model/runtime.hpp:46-53).
    """

    def __init__(self, norm: Part, vocab: int, hidden: int, tied_to: Optional[TokenEmbedding] = None, scale: float = 1.0,
                 role: str = "weight", softcap: Optional[float] = None):
        """`scale`: a factor on the logits (applied to the float32 product); `role`: the weight's tensor role; `softcap` c:
        logits <- c tanh(logits / c), last."""
        self.norm, self.vocab, self.hidden, self.tied_to = norm, int(vocab), int(hidden), tied_to
        self.scale, self.role = float(scale), role
        self.softcap = float(softcap) if softcap else None
        self.linear: Optional[Linear] = None
        self._native: Optional[NativeHandle] = None
        self._native_tried = False

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {} if self.tied_to is not None else {self.role: TensorSpec((self.vocab, self.hidden))}

    def load(self, tensors, precision: Precision) -> None:
        super().load(tensors, precision)
        if self.tied_to is None:
            self.linear = Linear(tensors[self.role], precision)
        self._native, self._native_tried = None, False

    def bind_tied(self) -> None:
        if self.tied_to is not None:
            self.linear = Linear(self.tied_to.table, self.precision)
            self.linear.weight = self.tied_to.table  # the same memory, not a copy
            self._native, self._native_tried = None, False

    @property
    def native(self):
        if not self._native_tried:
            self._native_tried = True
            norm = self.norm.native if self.scale == 1.0 and self.softcap is None else None
            if norm:
                d = self.linear.desc()
                self._native = NativeHandle(runtime.lib().llmx_head_create(norm, ctypes.byref(d)), keep=(self.norm, self.linear.weight))
        return self._native.handle if self._native is not None else None

    def forward(self, x: torch.Tensor, logit_rows: torch.Tensor) -> torch.Tensor:
        rows = logit_rows.numel()
        out = self.linear.output_to_clear(rows, x.device)          # cleared by the norm's launch when the product adds pieces
        h = self.norm.forward(x, row_index=logit_rows, zero=out)
        logits = self.linear(h, out=out, cleared=True) if out is not None else self.linear(h)
        if self.scale != 1.0:
            from .. import ops
            ops.scale_(logits, self.scale)
        if self.softcap is not None:
            from .. import ops
            ops.softcap_(logits, self.softcap)
        return logits
