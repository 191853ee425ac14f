"""Feed-forward parts.  GatedMLP: residual += (act(h Wg^T) * (h Wu^T)) Wd^T.

With act = silu this is the SwiGLU block (src/model/arch/blocks.hpp:101-106):
silu(g) = g / (1 + exp(-g)) in 32-bit.  Gate and up weights are stacked by rows
so one product gives both.  The forward pass is the native runtime's (`GatedMlp` in csrc/runtime/runtime.cpp).
"""
from __future__ import annotations

import ctypes
from typing import Dict, Optional

import torch

from .. import runtime
from ..weights.spec import TensorSpec
from .base import NativeHandle, Part, Precision, StepBatch
from .linear import Linear, call_struct, stored_product


class GatedMLP(Part):
    def __init__(self, hidden: int, intermediate: int, activation: str = "silu",
                 names=("gate_proj.weight", "up_proj.weight", "down_proj.weight")):
        """`names`: the roles of the gate, up and down weights."""
        if activation != "silu":
            raise ValueError(f"activation {activation!r} has no kernel here (silu)")
        self.hidden, self.intermediate, self.activation = int(hidden), int(intermediate), activation
        self.names = tuple(names)
        self._native: Optional[NativeHandle] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        g, u, d = self.names
        return {g: TensorSpec((self.intermediate, self.hidden)), u: TensorSpec((self.intermediate, self.hidden)),
                d: TensorSpec((self.hidden, self.intermediate))}

    def load(self, tensors, precision: Precision) -> None:
        super().load(tensors, precision)
        g, u, d = self.names
        self.gate_up = Linear(torch.cat([tensors[g], tensors[u]], dim=0), precision)
        self.down = Linear(tensors[d], precision)
        self._native = None

    @property
    def native(self) -> int:
        if self._native is None:
            runtime.need("rowwise")
            d = runtime.MlpDesc(self.hidden, self.intermediate, self.gate_up.desc(), self.down.desc(), self.precision.flags)
            self._native = NativeHandle(runtime.lib().llmx_gated_mlp_create(ctypes.byref(d)),
                                        keep=(self.gate_up.weight, self.down.weight))
        return self._native.handle

    def wants_cleared(self, rows: int, device, step: Optional[StepBatch] = None):
        """A float32 buffer this part wants zeroed before `forward` (the norm before it clears it in passing)."""
        s = step.struct_for(self) if step is not None else None
        n = runtime.lib().llmx_part_wants_cleared(self.native, ctypes.byref(s), rows) if s is not None else 0
        self._cleared = torch.empty(int(n), dtype=torch.float32, device=device) if n else None
        return self._cleared

    def forward(self, h: torch.Tensor, step: StepBatch, residual: torch.Tensor) -> None:
        rows = h.shape[0]
        cleared, self._cleared = getattr(self, "_cleared", None), None
        if not (h.is_cuda and h.is_contiguous() and h.dtype is self.precision.act and tuple(h.shape) == (rows, self.hidden)
                and residual.dtype is torch.float32 and residual.is_contiguous() and tuple(residual.shape) == (rows, self.hidden)):
            raise runtime.KernelError("feed-forward: rows of the path's type and the part's width, a float32 residual")
        rt = runtime.lib()
        s, _keep = call_struct(step, self, h.device, lambda p: rt.llmx_part_workspace(self.native, ctypes.byref(p), rows, -1))
        runtime.check(rt.llmx_ffn_forward(self.native, ctypes.byref(s), h.data_ptr(), rows, residual.data_ptr(), runtime.ptr(cleared)),
                      "feed-forward")


class ClampedGLU(Part):
    """residual += (g sigmoid(alpha g) (u + 1)) Wd^T with g = min(h Wg^T, limit), u = clamp(h Wu^T, -limit, limit).

    The gate is cut from above only, the linear branch on both sides and shifted by one; `limit` and `alpha` are
    arguments.  Gate and up weights are stacked so one product gives both; the activation is `llmx_clamped_glu`
    (csrc/rowwise.cu) in 32-bit.  `names`: the three tensors' roles."""

    def __init__(self, hidden: int, intermediate: int, limit: float, alpha: float = 1.702, names=("gate", "up", "down")):
        self.hidden, self.intermediate = int(hidden), int(intermediate)
        self.limit, self.alpha, self.names = float(limit), float(alpha), tuple(names)

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        g, u, d = self.names
        return {g: TensorSpec((self.intermediate, self.hidden)), u: TensorSpec((self.intermediate, self.hidden)),
                d: TensorSpec((self.hidden, self.intermediate))}

    def stored_products(self):
        return (self.gate_up,)

    def load(self, tensors, precision: Precision) -> None:
        super().load(tensors, precision)
        self.cleared_outputs = {}
        g, u, d = self.names
        self.gate_up = Linear(torch.cat([tensors[g], tensors[u]], dim=0), precision)
        self.down = Linear(tensors[d], precision)

    def forward(self, h: torch.Tensor, step: Optional[StepBatch], residual: torch.Tensor) -> None:
        from .. import ops
        rows = h.shape[0]
        if not (h.is_cuda and h.is_contiguous() and h.dtype is self.precision.act and tuple(h.shape) == (rows, self.hidden)
                and residual.dtype is torch.float32 and residual.is_contiguous() and tuple(residual.shape) == (rows, self.hidden)):
            raise runtime.KernelError("feed-forward: rows of the path's type and the part's width, a float32 residual")
        gu = stored_product(self, self.gate_up, h)
        act = torch.empty((rows, self.intermediate), dtype=self.precision.act, device=h.device)
        ops.clamped_glu(gu, act, self.limit, self.alpha)
        self.down(act, out=residual, accumulate=True)


class TableRoutedExperts(Part):
    """A mixture of experts without a router: an integer table [vocab, top] gives each token id its `top` experts
    (the entries of a row differ), each weighing 1 / top.
        residual += (1 / top) * sum over the token's experts e of (silu(h Wg_e^T) * (h Wu_e^T)) Wd_e^T  [+ shared(h)]
    `shared`: a feed-forward part that runs for every token beside the experts (or None).  The experts' weights are
    stacked ([experts, 2 ff, E] gate rows then up rows, and [experts, E, ff]); the step's (row, expert) pairs are sorted
    by expert on the device and the products run a tile of one expert's pairs at a time (csrc/moe.cu), so nothing of
    the routing is read on the host.  Tensor roles: `table`, `e<i>.gate|up|down`; the shared part's under `shared.`."""

    few_pairs = 64          # up to this many (row, expert) pairs a step, the products run the form for a few pairs

    def __init__(self, hidden: int, vocab: int, experts: int, top: int, intermediate: int, shared: Optional[Part] = None,
                 names=("gate", "up", "down"), table_role: str = "table", shared_name: str = "shared"):
        if not 1 <= top <= experts:
            raise ValueError("experts: a token uses between one and all of the experts")
        self.hidden, self.vocab, self.experts, self.top = int(hidden), int(vocab), int(experts), int(top)
        self.intermediate, self.shared, self.names = int(intermediate), shared, tuple(names)
        self.table_role, self.shared_name = table_role, shared_name

    def children(self) -> Dict[str, Part]:
        return {} if self.shared is None else {self.shared_name: self.shared}

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        g, u, d = self.names
        specs = {self.table_role: TensorSpec((self.vocab, self.top), "int_table", init="distinct_rows", bound=self.experts)}
        for e in range(self.experts):
            specs[f"e{e}.{g}"] = TensorSpec((self.intermediate, self.hidden))
            specs[f"e{e}.{u}"] = TensorSpec((self.intermediate, self.hidden))
            specs[f"e{e}.{d}"] = TensorSpec((self.hidden, self.intermediate))
        return specs

    def load(self, tensors, precision: Precision) -> None:
        super().load(tensors, precision)
        g, u, d = self.names
        self.table = tensors[self.table_role].to(torch.int32).contiguous()
        if int(self.table.min()) < 0 or int(self.table.max()) >= self.experts:
            raise ValueError(f"experts: the table names an expert outside 0..{self.experts - 1}")
        act = precision.act
        self.w_gate_up = torch.stack([torch.cat([tensors[f"e{e}.{g}"], tensors[f"e{e}.{u}"]], dim=0) for e in range(self.experts)]).to(act).contiguous()
        self.w_down = torch.stack([tensors[f"e{e}.{d}"] for e in range(self.experts)]).to(act).contiguous()
        from .. import ops
        self.tensor_cores = not precision.invariant and ops.moe_tensor_cores_fit(act, self.hidden, self.intermediate)

    def forward(self, h: torch.Tensor, step: StepBatch, residual: torch.Tensor) -> None:
        from .. import ops
        rows = h.shape[0]
        if not (h.is_cuda and h.is_contiguous() and h.dtype is self.precision.act and tuple(h.shape) == (rows, self.hidden)
                and residual.dtype is torch.float32 and residual.is_contiguous() and tuple(residual.shape) == (rows, self.hidden)):
            raise runtime.KernelError("experts: rows of the path's type and the part's width, a float32 residual")
        pairs = rows * self.top
        dev = h.device
        act = torch.empty((pairs, self.intermediate), dtype=self.precision.act, device=dev)
        y = torch.empty((pairs, self.hidden), dtype=torch.float32, device=dev)
        if self.tensor_cores and pairs <= self.few_pairs:
            # A few pairs (decoding): the experts' weights streamed once a pair; which form runs follows the step's rows alone.
            ops.moe_product_few(h, self.top, self.w_gate_up, step.token_ids, self.table, pairs, act, gated=True)
            ops.moe_product_few(act, 1, self.w_down, step.token_ids, self.table, pairs, y, gated=False)
        else:
            lists = torch.empty((self.experts, pairs), dtype=torch.int32, device=dev)
            counts = torch.empty((self.experts,), dtype=torch.int32, device=dev)
            tiles = torch.empty((ops.moe_tiles_len(pairs, self.experts),), dtype=torch.int32, device=dev)
            tc = self.tensor_cores
            ops.moe_route(step.token_ids, self.table, self.experts, lists, counts, tiles, tensor_cores=tc)
            ops.moe_product(h, self.top, self.w_gate_up, lists, counts, tiles, pairs, act, gated=True, tensor_cores=tc)
            ops.moe_product(act, 1, self.w_down, lists, counts, tiles, pairs, y, gated=False, tensor_cores=tc)
        ops.moe_combine_(residual, y, self.top, 1.0 / self.top)
        if self.shared is not None:
            self.shared.forward(h, step, residual)


class RoutedExperts(Part):
    """A mixture of experts with a router: logits z = h Wr^T + b in 32-bit, the `top` experts with the largest logits,
    weighted by the softmax over the chosen logits alone.
        residual += sum over the row's experts e of p_e (silu(h Wg_e^T) * (h Wu_e^T)) Wd_e^T  [+ g * shared(h)]
    `shared`: a feed-forward part that runs for every row beside the experts (or None); with `shared_gate` its output is
    multiplied by g = sigmoid(h . w_sg), one number a row (the gate's weight [1, width] is one more row of the router's
    product).  The experts' weights are stacked as `TableRoutedExperts` stacks them and the same kernels run the
    products (csrc/moe.cu); the router writes its choice as a table [rows, top] on the device, so nothing of the routing
    is read on the host.  Tensor roles: `router`, `router.b`, `e<i>.gate|up|down`; the shared part's under `shared.`,
    its gate `shared.sg`."""

    few_pairs = 64

    def __init__(self, hidden: int, experts: int, top: int, intermediate: int, shared: Optional[Part] = None, shared_gate: bool = False,
                 names=("gate", "up", "down"), router_role: str = "router", router_bias_role: Optional[str] = "router.b",
                 shared_name: str = "shared", shared_gate_role: str = "sg"):
        if not 1 <= top <= experts:
            raise ValueError("experts: a token uses between one and all of the experts")
        self.hidden, self.experts, self.top, self.intermediate = int(hidden), int(experts), int(top), int(intermediate)
        self.shared, self.shared_gate, self.names = shared, bool(shared_gate) and shared is not None, tuple(names)
        self.router_role, self.router_bias_role, self.shared_name = router_role, router_bias_role, shared_name
        self.gate_role = f"{shared_name}.{shared_gate_role}"
        self.scratch: Optional[torch.Tensor] = None

    def children(self) -> Dict[str, Part]:
        return {} if self.shared is None else {self.shared_name: self.shared}

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        g, u, d = self.names
        specs = {self.router_role: TensorSpec((self.experts, self.hidden), std=0.5)}
        if self.router_bias_role is not None:
            specs[self.router_bias_role] = TensorSpec((self.experts,), "vector", init="normal", std=0.5)
        if self.shared_gate:
            specs[self.gate_role] = TensorSpec((1, self.hidden), std=0.1)
        for e in range(self.experts):
            specs[f"e{e}.{g}"] = TensorSpec((self.intermediate, self.hidden))
            specs[f"e{e}.{u}"] = TensorSpec((self.intermediate, self.hidden))
            specs[f"e{e}.{d}"] = TensorSpec((self.hidden, self.intermediate))
        return specs

    def cleared_scratch(self, rows: int) -> int:
        """Floats of cleared scratch a step of `rows` rows needs (the gated shared part's output)."""
        return rows * self.hidden if self.shared_gate else 0

    def load(self, tensors, precision: Precision) -> None:
        super().load(tensors, precision)
        g, u, d = self.names
        rows = [tensors[self.router_role]] + ([tensors[self.gate_role].reshape(1, self.hidden)] if self.shared_gate else [])
        self.router_w = torch.cat([r.to(torch.float32) for r in rows], dim=0).contiguous()
        self.router_b = tensors[self.router_bias_role].to(torch.float32).contiguous() if self.router_bias_role is not None else None
        act = precision.act
        self.w_gate_up = torch.stack([torch.cat([tensors[f"e{e}.{g}"], tensors[f"e{e}.{u}"]], dim=0) for e in range(self.experts)]).to(act).contiguous()
        self.w_down = torch.stack([tensors[f"e{e}.{d}"] for e in range(self.experts)]).to(act).contiguous()
        from .. import ops
        self.tensor_cores = not precision.invariant and ops.moe_tensor_cores_fit(act, self.hidden, self.intermediate)

    def forward(self, h: torch.Tensor, step: StepBatch, residual: torch.Tensor) -> None:
        from .. import ops
        rows = h.shape[0]
        if not (h.is_cuda and h.is_contiguous() and h.dtype is self.precision.act and tuple(h.shape) == (rows, self.hidden)
                and residual.dtype is torch.float32 and residual.is_contiguous() and tuple(residual.shape) == (rows, self.hidden)):
            raise runtime.KernelError("experts: rows of the path's type and the part's width, a float32 residual")
        pairs = rows * self.top
        dev = h.device
        choice = torch.empty((rows, self.top), dtype=torch.int32, device=dev)
        weight = torch.empty((rows, self.top), dtype=torch.float32, device=dev)
        gate = torch.empty((rows,), dtype=torch.float32, device=dev) if self.shared_gate else None
        ops.moe_router(h, self.router_w, self.router_b, self.experts, self.top, choice, weight, gate)
        act = torch.empty((pairs, self.intermediate), dtype=self.precision.act, device=dev)
        y = torch.empty((pairs, self.hidden), dtype=torch.float32, device=dev)
        if self.tensor_cores and pairs <= self.few_pairs:
            # A few pairs (decoding): the experts' weights streamed once a pair; which form runs follows the step's rows alone.
            ops.moe_product_few(h, self.top, self.w_gate_up, None, choice, pairs, act, gated=True)
            ops.moe_product_few(act, 1, self.w_down, None, choice, pairs, y, gated=False)
        else:
            lists = torch.empty((self.experts, pairs), dtype=torch.int32, device=dev)
            counts = torch.empty((self.experts,), dtype=torch.int32, device=dev)
            tiles = torch.empty((ops.moe_tiles_len(pairs, self.experts),), dtype=torch.int32, device=dev)
            tc = self.tensor_cores
            ops.moe_route(None, choice, self.experts, lists, counts, tiles, tensor_cores=tc)
            ops.moe_product(h, self.top, self.w_gate_up, lists, counts, tiles, pairs, act, gated=True, tensor_cores=tc)
            ops.moe_product(act, 1, self.w_down, lists, counts, tiles, pairs, y, gated=False, tensor_cores=tc)
        ops.moe_combine_weighted_(residual, y, weight, self.top)
        if self.shared is None:
            return
        if not self.shared_gate:
            self.shared.forward(h, step, residual)
            return
        scratch, self.scratch = self.scratch, None
        if scratch is None or scratch.numel() < rows * self.hidden:
            scratch = torch.zeros(rows * self.hidden, dtype=torch.float32, device=dev)
        out = scratch[:rows * self.hidden].view(rows, self.hidden)
        self.shared.forward(h, step, out)
        ops.add_rows_(residual, out, 1.0, gate)
