"""Latent attention: queries, keys and values through low-rank latents, and a cache of the latents alone.

For the rows of a step, with H heads, D unrotated and R rotated query/key values per head, V value values per head,
a query latent of `q_rank` and a key/value latent of C = `kv_rank` values:
    cq = RMSNorm(h Wdq^T) * w_dq;   q = cq Wuq^T, per head [D unrotated | R rotated]
    [c_raw | r_raw] = h Wdkv^T (C + R values; one product with Wdq over the stacked weight);   c = RMSNorm(c_raw) * w_dkv;   r = rotate(r_raw) (one part for all heads)
    per head: k = [Wuk_h c | r],  v = Wuv_h c,   s = (q_plain . Wuk_h c + rotate(q_rot) . r) * scale
    o = softmax over the keys lo..p (lo = 0, or p - window + 1 under a sliding window) of s, times v
    residual += o Wo^T
Only [c | r] is cached, one vector per token (a cache entry of one plane).  The rotation pairs neighbours
(2i, 2i + 1) of the first `rot_dims` values of the rotated part by the angle p * base^(-2i / rot_dims).  The kernels
(csrc/latent_attention.cu) never make keys or values of cached tokens: the query goes through Wuk once, the weighted
sum of latents through Wuv once.

Options for designs that vary it:
    q_rank None        no query latent: q = h Wq^T straight from the input (tensor role `q` instead of dq, dq.norm, uq)
    pairing "halves"   rotation pair i is (i, i + rot_dims / 2) instead of neighbours
    rot_scaling        (factor, original, fast, slow): frequencies blended for contexts longer than the original one and
                       a factor on cosines and sines (`parts.rope.blended_frequencies`); the score scale stays as given
    gate True          the concatenated heads are multiplied by sigmoid(h Wg^T) before the output product (role `g`)
Whatever reads h is one product over the stacked weight.
"""
from __future__ import annotations

from typing import Dict, Optional

import numpy as np
import torch

from .. import ops, runtime
from ..cache.manager import KVSpec
from ..weights.spec import TensorSpec
from .base import Part, PartPlan, Precision, StepBatch, StepShape
from .linear import Linear, stored_product
from .rope import blended_frequencies, power_frequencies


class _TilePlan(PartPlan):
    """The row tiles of a step for the tiled kernels: (first row, rows) per tile, rows of one request each.  They follow
    the step's row counts alone, so a recorded step's plan never changes."""

    def __init__(self, tiles):
        self.tiles = np.asarray(tiles, dtype=np.int32).reshape(-1)
        self.ints = int(self.tiles.size)

    def fill(self, histories, out: np.ndarray) -> None:
        out[:self.ints] = self.tiles


class LatentAttention(Part):
    def __init__(self, hidden: int, heads: int, key_dim: int, rot_dim: int, value_dim: int, q_rank: Optional[int], kv_rank: int,
                 scale: float, rot_base: float, rot_dims: int, norm_eps: float, window: Optional[int] = None,
                 pairing: str = "neighbours", rot_scaling=None, gate: bool = False):
        if rot_dims % 2 or rot_dims > rot_dim or rot_dims < 0:
            raise ValueError("latent attention: the rotated width must be even and at most the rotated part's width")
        if pairing not in ("neighbours", "halves"):
            raise ValueError("latent attention: rotation pairs are neighbours or halves")
        self.hidden, self.heads, self.key_dim, self.rot_dim, self.value_dim = int(hidden), int(heads), int(key_dim), int(rot_dim), int(value_dim)
        self.q_rank, self.kv_rank, self.scale = int(q_rank or 0), int(kv_rank), float(scale)
        self.pairing, self.gate = pairing, bool(gate)
        self.rot_scaling = tuple(float(x) for x in rot_scaling) if rot_scaling is not None else None
        self.rot_magnitude = 1.0
        self.rot_base, self.rot_dims, self.norm_eps = float(rot_base), int(rot_dims), float(norm_eps)
        self.window = int(window) if window else None
        self.q_width = self.heads * (self.key_dim + self.rot_dim)
        self.v_width = self.heads * self.value_dim
        self.freq: Optional[torch.Tensor] = None
        self.plain_cores = False      # True: the tiled scores stay on the CUDA cores also where the tensor-core form would run

    def stored_products(self):
        """The products whose result is stored (not added to the residual): a block may clear their outputs in passing."""
        return (self.down, self.uq) if self.q_rank else (self.down,)

    def cache_spec(self):
        return KVSpec(1, self.kv_rank + self.rot_dim, self.window, planes=1)

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        E, C, R = self.hidden, self.kv_rank, self.rot_dim
        specs = {"dkv": TensorSpec((C + R, E)), "dkv.norm": TensorSpec((C,), "vector", init="one_plus_normal", std=0.01),
                 "uk": TensorSpec((self.heads * self.key_dim, C)), "uv": TensorSpec((self.v_width, C)),
                 "o": TensorSpec((E, self.v_width))}
        if self.q_rank:
            specs.update({"dq": TensorSpec((self.q_rank, E)), "dq.norm": TensorSpec((self.q_rank,), "vector", init="one_plus_normal", std=0.01),
                          "uq": TensorSpec((self.q_width, self.q_rank))})
        else:
            specs["q"] = TensorSpec((self.q_width, E))
        if self.gate:
            specs["g"] = TensorSpec((self.v_width, E))
        return specs

    def frequencies(self):
        """(float32 frequencies [rot_dims / 2] rounded once from double, the factor on cosines and sines)."""
        if self.rot_scaling is not None and self.rot_dims:
            f, magnitude = blended_frequencies(self.rot_base, self.rot_dims, *self.rot_scaling)
        else:
            f, magnitude = power_frequencies(self.rot_base, self.rot_dims), 1.0
        return f.astype(np.float32), float(magnitude)

    def load(self, tensors, precision: Precision) -> None:
        super().load(tensors, precision)
        self.cleared_outputs = {}
        t = tensors
        # One product for everything that reads h: [query latent | key/value latent | rotated part], or without a query
        # latent [key/value latent | rotated part | queries], then the gate's input.
        stacked = [t["dq"], t["dkv"]] if self.q_rank else [t["dkv"], t["q"]]
        if self.gate:
            stacked.append(t["g"])
        self.down = Linear(torch.cat(stacked, dim=0), precision)
        self.o = Linear(t["o"], precision)
        self.uq = Linear(t["uq"], precision) if self.q_rank else None
        self.dq_norm = t["dq.norm"].to(torch.float32).contiguous() if self.q_rank else None
        self.dkv_norm = t["dkv.norm"].to(torch.float32).contiguous()
        self.w_uk = t["uk"].to(precision.act).contiguous()
        self.w_uv = t["uv"].to(precision.act).contiguous()
        # Frequencies in double precision, rounded once; the angle is the float product with the position.
        freq, self.rot_magnitude = self.frequencies()
        self.freq = torch.from_numpy(freq).to(self.w_uk.device)
        self._sms = torch.cuda.get_device_properties(self.w_uk.device).multi_processor_count if self.w_uk.is_cuda else 148

    # -- how the tiled kernels cut a step (the same on the host when the plan is made and when the step runs) -------
    def _tiling(self, counts, max_context: int):
        """(tiles [(first row, rows)], ranges a tile's keys are cut into so that the blocks fill the device twice)."""
        ht, rt = ops.latent_tile_shape(self.heads)
        tiles, start = [], 0
        for n in counts:
            tiles += [(start + i, min(rt, n - i)) for i in range(0, n, rt)]
            start += n
        keys = max(int(max_context), 1) if self.window is None else min(max(int(max_context), 1), self.window + rt - 1)
        blocks = len(tiles) * -(-self.heads // ht)
        splits = max(1, min(-(-2 * self._sms // blocks), keys // 128))
        return tiles, splits

    def plan_step(self, shape: StepShape) -> Optional[PartPlan]:
        if getattr(self, "precision", None) is None or self.precision.invariant:
            return None
        context = shape.room if shape.room > 0 else max(h + c for h, c in zip(shape.histories, shape.counts))
        return _TilePlan(self._tiling(shape.counts, context)[0])

    def forward(self, h: torch.Tensor, step: StepBatch, cache_entry: int, residual: torch.Tensor,
                write_cache: bool = True) -> None:
        rows = h.shape[0]
        if not (h.is_cuda and h.is_contiguous() and h.dtype is self.precision.act and tuple(h.shape) == (rows, self.hidden)
                and residual.dtype is torch.float32 and residual.is_contiguous() and tuple(residual.shape) == (rows, self.hidden)):
            raise runtime.KernelError("latent attention: rows of the path's type and the mixer's width, a float32 residual")
        group, cache = step.kv(cache_entry)
        slots = group.slots if write_cache else torch.full((rows,), -1, dtype=torch.int32, device=h.device)
        halves, mag = self.pairing == "halves", self.rot_magnitude
        proj = stored_product(self, self.down, h)
        latents = self.q_rank + self.kv_rank + self.rot_dim
        if self.q_rank:
            cq = torch.empty((rows, self.q_rank), dtype=self.precision.act, device=h.device)
            ops.latent_write(proj[:, :latents], self.q_rank, self.dq_norm, cq, self.dkv_norm, self.norm_eps, self.freq, step.positions,
                             slots, cache, self.kv_rank, self.rot_dim, halves=halves, magnitude=mag)
            q = stored_product(self, self.uq, cq)
            gate_at = latents
        else:
            ops.latent_write(proj[:, :latents], 0, None, None, self.dkv_norm, self.norm_eps, self.freq, step.positions,
                             slots, cache, self.kv_rank, self.rot_dim, halves=halves, magnitude=mag)
            q = proj[:, latents:latents + self.q_width]
            gate_at = latents + self.q_width
        o = torch.empty((rows, self.v_width), dtype=self.precision.act, device=h.device)
        # The tiled kernels hold a cache row in a warp's registers: rows of up to 768 values.
        tiles = None if self.precision.invariant or self.kv_rank + self.rot_dim > 768 else step.plan_ints(self)
        if tiles is not None:
            # The tiled kernels: 16 (row, head) pairs share the keys they read; key ranges fill the device when rows are few.
            host_tiles, splits = self._tiling(step.host_row_count, step.max_context)
            ops.latent_attention_tiled(q, cache, self.w_uk, self.w_uv, o, self.freq, step.row_request, step.positions,
                                       group.block_tables, tiles, len(host_tiles), splits, self.heads, self.key_dim, self.rot_dim,
                                       self.value_dim, self.kv_rank, group.page_size, self.window, self.scale, plain_cores=self.plain_cores,
                                       halves=halves, magnitude=mag)
        else:
            # One block per (row, head): the schedule follows the sizes alone (an invariant path, or a step without a plan).
            ops.latent_attention(q, cache, self.w_uk, self.w_uv, o, self.freq, step.row_request, step.positions, group.block_tables,
                                 self.heads, self.key_dim, self.rot_dim, self.value_dim, self.kv_rank, group.page_size, self.window,
                                 self.scale, halves=halves, magnitude=mag)
        if self.gate:
            ops.sigmoid_gate_(o, proj[:, gate_at:gate_at + self.v_width])
        self.o(o, out=residual, accumulate=True)
