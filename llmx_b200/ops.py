"""Python faces of single CUDA kernels.

The model's forward pass calls the kernels from the native runtime (llmx_b200/runtime.py, csrc/runtime/); the
functions here call one kernel each, for tests that hold a kernel to its plain reference and for parts written
in Python.  Every function launches hand-written sm_100a kernels from `csrc/` on the
current CUDA stream and returns at once.  Arguments are torch tensors on one
CUDA device; shapes, types and contiguity are checked here, on the host, before
a launch, so that a kernel is never handed memory it would read out of bounds.
There is no CPU path and no library fallback: without a GPU or a working nvcc
these functions raise.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .csrc import build as _build

F32, BF16 = 0, 1
_CODE = {torch.float32: F32, torch.bfloat16: BF16}


from .runtime import KernelError      # noqa: E402  (one error type for kernels and runtime)


def _code(t: torch.Tensor) -> int:
    try:
        return _CODE[t.dtype]
    except KeyError:
        raise KernelError(f"element type {t.dtype} is not one the kernels take (float32, bfloat16)") from None


def _ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> ctypes.c_void_p:
    """The current stream of the current device (the raw handle: this runs before every launch)."""
    if _raw_stream is not None and _raw_device is not None:
        return ctypes.c_void_p(_raw_stream(_raw_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _need(cond: bool, what: str) -> None:
    if not cond:
        raise KernelError(what)


def _cuda(*tensors: Optional[torch.Tensor]) -> None:
    for t in tensors:
        if t is not None:
            _need(t.is_cuda, "kernel arguments must be CUDA tensors (there is no CPU path)")
            _need(t.is_contiguous(), "kernel arguments must be contiguous")


_ERRORS = {10001: "bad argument", 10002: "shape or type not supported by this kernel",
           10003: "TMA descriptor could not be encoded", 10004: "size beyond the stated maximum"}


_launches = 0


def launch_count() -> int:
    """Kernels of this package launched so far: by the native runtime (the model's forward pass, replayed
    recordings included) and by the single-kernel functions of this module."""
    from . import runtime
    return _launches + runtime.launches()


def count_launches(n: int) -> None:
    """Adds the kernels a replayed recording launches."""
    global _launches
    _launches += n


def _check(status: int, what: str, launches: int = 1) -> None:
    global _launches
    _launches += launches
    if status != 0:
        why = _ERRORS.get(status, f"CUDA error {status}")
        raise KernelError(f"{what}: {why}")


_i, _f, _p = ctypes.c_int, ctypes.c_float, ctypes.c_void_p
_SIGNATURES = {
    ("rowwise", "llmx_embed"): [_p, _i, _p, _p, _i, _i, _i, _p],
    ("rowwise", "llmx_rmsnorm"): [_p, _p, _p, _i, _p, _i, _i, _f, _p, ctypes.c_longlong, _p],
    ("rowwise", "llmx_head_norm_rope_kv"): [_p, _i, _i, _i, _p, _p, _f, _p, _p, _i, _p, _p, _p, _i, _p, _i,
                                            _i, _i, _i, _i, _i, _p],
    ("rowwise", "llmx_swiglu"): [_p, _p, _i, _i, _i, _p],
    ("rowwise", "llmx_embed_scaled"): [_p, _i, _p, _p, _i, _i, _i, _f, _p],
    ("rowwise", "llmx_scale"): [_p, ctypes.c_longlong, _f, _p],
    ("rowwise", "llmx_layernorm"): [_p, _p, _p, _i, _p, _i, _i, _f, _p, ctypes.c_longlong, _p],
    ("rowwise", "llmx_layernorm_affine"): [_p, _p, _p, _p, _p, _i, _p, _f, _p, _i, _i, _f, _p, ctypes.c_longlong, _p],
    ("rowwise", "llmx_sigmoid_gate"): [_p, _i, _p, _i, _i, _i, _p],
    ("rowwise", "llmx_add_bias"): [_p, _p, _i, _i, _p],
    ("rowwise", "llmx_clamped_glu"): [_p, _p, _i, _i, _i, _f, _f, _p],
    ("rowwise", "llmx_silu_columns"): [_p, _i, _i, _i, _i, _p],
    ("rowwise", "llmx_gated_rmsnorm"): [_p, _p, _i, _p, _i, _p, _i, _i, _i, _i, _f, _i, _i, _p],
    ("rowwise", "llmx_pair_norm_add"): [_p, _p, _p, _p, _p, _i, _i, _f, _f, _p],
    ("rowwise", "llmx_add"): [_p, _p, ctypes.c_longlong, _p],
    ("recurrence", "llmx_linear_recurrence"): [_p, _p, _p, _i, _i, _i, _i, _p, _p, _p, _i, _i, _p, _p, ctypes.c_longlong, _p, _p,
                                               _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _p],
    ("recurrence", "llmx_conv_prepare"): [_p, _i, _i, _i, _i, _i, _p, _p, _i, _p, _p, _p, _i, _i, _i, _p, _i, _p, _i, _i, _i, _f,
                                          _p, ctypes.c_longlong, ctypes.c_longlong, _p, _p, _p, _p, _p, _p, _i, _i, _p],
    ("attention_split", "llmx_qk_norm_rope_write"): [_p, _i, _p, _p, _f, _p, _i, _p, _p, _p, _i, _p, _i, _i, _i, _i, _i, _i, _i, _p],
    ("attention_split", "llmx_qkv_finish"): [_p, _i, _p, _p, _i, _p, ctypes.c_longlong, ctypes.c_longlong, _p, _p, _p, _p, _p, _p, _p, _p, _i,
                                             _f, _p, _i, _i, _p, _p, _p, _i, _p, _i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _p, _p],
    ("attention_split", "llmx_attention_split"): [_p, _i, _p, _i, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _i, _p,
                                                  _f, _p, _i, _p, _i, _p],
    ("attention_split", "llmx_attention_staged"): [_p, _i, _p, _i, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _i, _p,
                                                   _f, _p, _i, _p, _i, _p],
    ("attention_split", "llmx_attention_staged_fits"): [_i, _i, _i, _i, _i, _i],
    ("attention_split", "llmx_attention_tiled_fits"): [_i, _i, _i, _i],
    ("attention_split", "llmx_attention_tiled"): [_p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _f,
                                                  _f, _p, _i, _p, _i, _p],
    ("moe", "llmx_moe_route"): [_p, _p, _i, _i, _i, _i, _p, _p, _p, _i, _p],
    ("moe", "llmx_moe_product_few"): [_p, _i, _p, _p, _p, _i, _i, _i, _i, _p, _i, _i, _i, _i, _p],
    ("moe", "llmx_moe_product"): [_p, _i, _p, _i, _p, _p, _p, _i, _i, _p, _i, _i, _i, _i, _i, _p],
    ("moe", "llmx_moe_combine"): [_p, _p, _i, _i, _i, _f, _p],
    ("moe", "llmx_moe_router"): [_p, _i, _p, _p, _i, _i, _i, _i, _i, _p, _p, _p, _p],
    ("moe", "llmx_moe_combine_weighted"): [_p, _p, _p, _i, _i, _i, _f, _p],
    ("rowwise", "llmx_group_norm_conv"): [_p, _p, _i, _i, _f, _p, _i, _p, _p, _i, _p, _i, _p, ctypes.c_longlong, ctypes.c_longlong,
                                          _p, _p, _p, _p, _p, _p, _i, _p, ctypes.c_longlong, _p],
    ("rowwise", "llmx_embed_pairs"): [_p, _p, _i, _p, _p, _i, _i, _i, _f, _i, ctypes.c_longlong, ctypes.c_longlong, _p, _p, _p, _p, _p,
                                      ctypes.c_longlong, _p, _p, _i, _p],
    ("rowwise", "llmx_add_rows"): [_p, _p, _p, _f, _i, _i, _p],
    ("rowwise", "llmx_softcap"): [_p, ctypes.c_longlong, _f, _p],
    ("latent_attention", "llmx_latent_write"): [_p, _i, _i, _p, _p, _i, _p, _f, _p, _i, _i, _f, _p, _p, _p, _i, _i, _i, _i, _p],
    ("latent_attention", "llmx_latent_attention"): [_p, _i, _p, _i, _p, _p, _i, _p, _p, _i, _i, _f, _p, _p, _p, _i, _i, _i, _i,
                                                    _i, _i, _i, _i, _i, _f, _p],
    ("latent_attention", "llmx_latent_query"): [_p, _i, _p, _i, _p, _p, _i, _i, _f, _p, _i, _i, _i, _i, _i, _f, _p],
    ("latent_attention", "llmx_latent_scores"): [_p, _p, _i, _p, _p, _i, _i, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _p],
    ("latent_attention", "llmx_latent_merge"): [_p, _p, _i, _p, _i, _i, _i, _i, _i, _p],
    ("gemm_plain", "llmx_gemm_plain"): [_p, _i, _p, _i, _p, _i, _i, _i, _i, _p],
    ("attention_plain", "llmx_attention_plain"): [_p, _i, _p, _i, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _f, _p],
}
_fns = {}


_timed_calls = None       # while `kernel_times` is open: [(exported function, start event, end event)]


def _fn(lib: str, name: str):
    key = (lib, name)
    f = _fns.get(key)
    if f is None:
        f = getattr(_build.load(lib), name)
        f.argtypes = _SIGNATURES[key]
        f.restype = ctypes.c_int
        _fns[key] = f
    if _timed_calls is None:
        return f

    def timed(*args):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        status = f(*args)
        end.record()
        _timed_calls.append((name, start, end))
        return status
    return timed


class kernel_times:
    """Device time of every kernel call made inside the `with` block, by exported function (the reference's
    `bench --profile`, src/cli/main.cpp:1326-1352): CUDA events around each call on its stream, in the native
    runtime (the model's forward pass) and in this module's single-kernel functions.  For plain
    steps only: a step that replays a recording makes no calls, and events must not be recorded into one.
    The events keep a kernel from starting while the one before drains, so the times are those of kernels alone."""

    def __enter__(self) -> "kernel_times":
        global _timed_calls
        from . import runtime
        if _timed_calls is not None:
            raise KernelError("kernel_times is already open")
        _timed_calls = []
        runtime.profile(True)
        return self

    def __exit__(self, *exc) -> None:
        global _timed_calls
        from . import runtime
        calls, _timed_calls = _timed_calls, None
        runtime.profile(False)                   # synchronises
        torch.cuda.synchronize()
        native = runtime.profile_results()
        self.calls = len(calls) + len(native)
        self.by_function = {}
        for name, start, end in calls:
            n, ms = self.by_function.get(name, (0, 0.0))
            self.by_function[name] = (n + 1, ms + start.elapsed_time(end))
        for name, ms_one, _ in native:
            n, ms = self.by_function.get(name, (0, 0.0))
            self.by_function[name] = (n + 1, ms + ms_one)
        self.total_ms = sum(ms for _, ms in self.by_function.values())
        self.idle_ms = sum(max(0.0, calls[i][2].elapsed_time(calls[i + 1][1])) for i in range(len(calls) - 1)) \
            + sum(idle for _, _, idle in native)

    def lines(self, what: str):
        """The report, most expensive first."""
        out = [f"profile {what}: {self.total_ms:.3f} ms of device time over {self.calls} kernel calls"]
        for name, (n, ms) in sorted(self.by_function.items(), key=lambda kv: -kv[1][1]):
            share = 100.0 * ms / self.total_ms if self.total_ms > 0 else 0.0
            out.append(f"profile:   {name} x{n} {ms:.3f} ms ({share:.1f}%)")
        out.append(f"profile {what}: idle {self.idle_ms:.3f} ms between timed calls")
        return out


def register_signature(lib: str, name: str, argtypes) -> None:
    _SIGNATURES[(lib, name)] = list(argtypes)


# ---------------------------------------------------------------------------
def embed(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[r, :] = table[ids[r], :] widened to float32.  ids int32 [rows]; out float32 [rows, width]."""
    _cuda(table, ids, out)
    rows, width = out.shape
    _need(ids.dtype == torch.int32 and ids.numel() == rows, "embed: ids must be int32, one per output row")
    _need(out.dtype == torch.float32 and table.dim() == 2 and table.shape[1] == width, "embed: shapes do not fit")
    _check(_fn("rowwise", "llmx_embed")(_ptr(table), _code(table), _ptr(ids), _ptr(out), rows, width,
                                        table.shape[0], _stream()), "embed")
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
            row_index: Optional[torch.Tensor] = None, zero: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[i] = x[row_index[i] or i] * (rsqrt(mean x^2 + eps) * weight); x float32, out float32 or bfloat16.

    `zero` (optional): a float32 tensor the same launch clears (the output of a product that follows and
    adds its pieces with atomics)."""
    _cuda(x, weight, out, row_index, zero)
    if zero is not None:
        _need(zero.dtype == torch.float32 and zero.numel() % 4 == 0, "rmsnorm: the buffer to clear must be float32, a multiple of 4 long")
    rows, width = out.shape
    _need(x.dtype == torch.float32 and weight.dtype == torch.float32, "rmsnorm: input and weight must be float32")
    _need(x.dim() == 2 and x.shape[1] == width and weight.numel() == width, "rmsnorm: widths do not fit")
    if row_index is None:
        _need(x.shape[0] >= rows, "rmsnorm: fewer input rows than output rows")
    else:
        _need(row_index.dtype == torch.int32 and row_index.numel() == rows, "rmsnorm: row_index must be int32 per row")
    _check(_fn("rowwise", "llmx_rmsnorm")(_ptr(x), _ptr(weight), _ptr(out), _code(out), _ptr(row_index), rows, width,
                                          float(eps), _ptr(zero), 0 if zero is None else zero.numel(), _stream()),
           "rmsnorm")
    return out


def head_norm_rope_kv(qkv: torch.Tensor, heads: int, kv_heads: int, head_dim: int,
                      q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                      cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], positions: torch.Tensor,
                      slots: torch.Tensor, q_out: torch.Tensor, cache: torch.Tensor) -> None:
    """Per-head norm, rotation and the cache write for one layer.

    qkv float32 [rows, (heads + 2 kv_heads) * head_dim] (queries, keys, values);
    q_out [rows, heads * head_dim]; cache [pages, 2, kv_heads, page_size, head_dim];
    cos/sin float32 [positions, rot_half] or None (no rotation); slots int32 [rows],
    negative to skip a row's cache write.
    """
    _cuda(qkv, q_weight, k_weight, cos, sin, positions, slots, q_out, cache)
    rows = qkv.shape[0]
    q_w, kv_w = heads * head_dim, kv_heads * head_dim
    _need(qkv.dtype == torch.float32 and qkv.shape[1] == q_w + 2 * kv_w, "head_norm_rope_kv: qkv width does not fit")
    _need(tuple(q_out.shape) == (rows, q_w), "head_norm_rope_kv: q_out shape does not fit")
    _need(cache.dim() == 5 and cache.shape[1] == 2 and cache.shape[2] == kv_heads and cache.shape[4] == head_dim,
          "head_norm_rope_kv: cache layout does not fit")
    _need(positions.dtype == torch.int32 and slots.dtype == torch.int32 and positions.numel() >= rows
          and slots.numel() >= rows, "head_norm_rope_kv: positions and slots must be int32 per row")
    rot_half = 0
    if cos is not None:
        _need(sin is not None and cos.shape == sin.shape and cos.dtype == torch.float32 and cos.dim() == 2,
              "head_norm_rope_kv: cos and sin tables do not fit")
        rot_half = cos.shape[1]
        _need(2 * rot_half <= head_dim, "head_norm_rope_kv: rotated width exceeds the head width")
    for w in (q_weight, k_weight):
        _need(w is None or (w.dtype == torch.float32 and w.numel() == head_dim), "head_norm_rope_kv: norm weight")
    page_size = cache.shape[3]
    _check(_fn("rowwise", "llmx_head_norm_rope_kv")(
        _ptr(qkv), qkv.shape[1], q_w, q_w + kv_w, _ptr(q_weight), _ptr(k_weight), float(eps), _ptr(cos), _ptr(sin),
        rot_half, _ptr(positions), _ptr(slots), _ptr(q_out), _code(q_out), _ptr(cache), _code(cache), rows, heads,
        kv_heads, head_dim, page_size, _stream()), "head_norm_rope_kv")


def swiglu(gu: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out = silu(gu[:, :F]) * gu[:, F:]; gu float32 [rows, 2F]."""
    _cuda(gu, out)
    rows, width = out.shape
    _need(gu.dtype == torch.float32 and tuple(gu.shape) == (rows, 2 * width), "swiglu: shapes do not fit")
    _check(_fn("rowwise", "llmx_swiglu")(_ptr(gu), _ptr(out), _code(out), rows, width, _stream()), "swiglu")
    return out


def gemm_plain(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> torch.Tensor:
    """out (+)= a @ w.T on the CUDA cores; a [M, K], w [N, K] of one type, out float32 [M, N]."""
    _cuda(a, w, out)
    m, k = a.shape
    n = w.shape[0]
    _need(w.shape[1] == k and tuple(out.shape) == (m, n) and out.dtype == torch.float32, "gemm: shapes do not fit")
    _need(a.dtype == w.dtype, "gemm: inputs and weights must have one element type")
    _check(_fn("gemm_plain", "llmx_gemm_plain")(_ptr(a), _code(a), _ptr(w), _code(w), _ptr(out), m, n, k,
                                                1 if accumulate else 0, _stream()), "gemm_plain")
    return out


def attention_plain(q: torch.Tensor, cache: torch.Tensor, out: torch.Tensor, row_request: torch.Tensor,
                    positions: torch.Tensor, block_tables: torch.Tensor, heads: int, kv_heads: int, head_dim: int,
                    window: Optional[int], scale: float) -> torch.Tensor:
    """Paged attention, one block per (row, head); q/out [rows, heads * head_dim] of one element type, the cache of
    its own (float32 or bfloat16 each)."""
    _cuda(q, cache, out, row_request, positions, block_tables)
    rows = q.shape[0]
    _need(q.shape == out.shape and q.shape[1] == heads * head_dim, "attention: q and out shapes do not fit")
    _need(q.dtype == out.dtype, "attention: q and out must have one element type")
    _need(cache.dim() == 5 and cache.shape[1] == 2 and cache.shape[2] == kv_heads and cache.shape[4] == head_dim,
          "attention: cache layout does not fit")
    for t in (row_request, positions, block_tables):
        _need(t.dtype == torch.int32, "attention: metadata must be int32")
    _need(block_tables.dim() == 2 and row_request.numel() >= rows and positions.numel() >= rows,
          "attention: metadata shapes do not fit")
    _check(_fn("attention_plain", "llmx_attention_plain")(
        _ptr(q), _code(q), _ptr(cache), _code(cache), _ptr(out), _ptr(row_request), _ptr(positions), _ptr(block_tables),
        block_tables.shape[1], rows, heads, kv_heads, head_dim, cache.shape[3], int(window or 0), float(scale),
        _stream()), "attention_plain")
    return out


# ---------------------------------------------------------------------------
# Row-wise kernels of models with a centred norm, factors on embedding and logits, and a clamped gated unit.
def embed_scaled(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, scale: float) -> torch.Tensor:
    """out[r, :] = table[ids[r], :] * scale in float32."""
    _cuda(table, ids, out)
    rows, width = out.shape
    _need(ids.dtype == torch.int32 and ids.numel() == rows, "embed: ids must be int32, one per output row")
    _need(out.dtype == torch.float32 and table.dim() == 2 and table.shape[1] == width, "embed: shapes do not fit")
    _check(_fn("rowwise", "llmx_embed_scaled")(_ptr(table), _code(table), _ptr(ids), _ptr(out), rows, width, table.shape[0],
                                               float(scale), _stream()), "embed_scaled")
    return out


def scale_(x: torch.Tensor, factor: float) -> torch.Tensor:
    """x *= factor in place; x float32."""
    _cuda(x)
    _need(x.dtype == torch.float32, "scale: a float32 tensor")
    _check(_fn("rowwise", "llmx_scale")(_ptr(x), x.numel(), float(factor), _stream()), "scale")
    return x


def layernorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
              row_index: Optional[torch.Tensor] = None, zero: Optional[torch.Tensor] = None,
              bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[i] = (x - mean) / sqrt(var + eps) * weight (+ bias) over row (row_index[i] or i); x float32, out float32 or bfloat16.
    `zero` (optional): a float32 tensor the same launch clears (outputs of products that follow and add their pieces)."""
    _cuda(x, weight, out, row_index, zero, bias)
    if zero is not None:
        _need(zero.dtype == torch.float32 and zero.numel() % 4 == 0, "layernorm: the buffer to clear must be float32, a multiple of 4 long")
    rows, width = out.shape
    _need(x.dtype == torch.float32 and weight.dtype == torch.float32, "layernorm: input and weight must be float32")
    _need(x.dim() == 2 and x.shape[1] == width and weight.numel() == width, "layernorm: widths do not fit")
    _need(bias is None or (bias.dtype == torch.float32 and bias.numel() == width), "layernorm: bias float32 of the row's width")
    if row_index is None:
        _need(x.shape[0] >= rows, "layernorm: fewer input rows than output rows")
    else:
        _need(row_index.dtype == torch.int32 and row_index.numel() == rows, "layernorm: row_index must be int32 per row")
    _check(_fn("rowwise", "llmx_layernorm_affine")(_ptr(x), None, _ptr(weight), _ptr(bias), _ptr(out), _code(out), None, 0.0,
                                                   _ptr(row_index), rows, width, float(eps), _ptr(zero),
                                                   0 if zero is None else zero.numel(), _stream()), "layernorm")
    return out


def layernorm_add_(residual: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], eps: float,
                   factor: float, in_bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """residual += factor * ((z - mean) / sqrt(var + eps) * weight + bias), z = y + in_bias, row by row; all float32.
    The norm after a sublayer and the sublayer's weighted entry into the stream in one kernel; `in_bias`: a bias the
    sublayer's last product left for whoever reads its output."""
    _cuda(residual, y, weight, bias, in_bias)
    rows, width = residual.shape
    _need(residual.dtype == torch.float32 and y.dtype == torch.float32 and tuple(y.shape) == (rows, width),
          "layernorm_add: float32 tensors of one shape")
    for t in (weight, bias, in_bias):
        _need(t is None or (t.dtype == torch.float32 and t.numel() == width), "layernorm_add: float32 vectors of the row's width")
    _need(weight is not None, "layernorm_add: a weight")
    _check(_fn("rowwise", "llmx_layernorm_affine")(_ptr(y), _ptr(in_bias), _ptr(weight), _ptr(bias), None, F32, _ptr(residual),
                                                   float(factor), None, rows, width, float(eps), None, 0, _stream()), "layernorm_add")
    return residual


def add_bias_(x: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """x[r, :] += bias; float32."""
    _cuda(x, bias)
    _need(x.dtype == torch.float32 and bias.dtype == torch.float32 and x.dim() == 2 and bias.numel() == x.shape[1],
          "add_bias: float32 rows and a bias of their width")
    _check(_fn("rowwise", "llmx_add_bias")(_ptr(x), _ptr(bias), x.shape[0], x.shape[1], _stream()), "add_bias")
    return x


def sigmoid_gate_(o: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    """o *= sigmoid(gate) in place; o [rows, width] of the path's type, contiguous; gate float32 [rows, width], a view whose
    rows may be strided."""
    _need(o.is_cuda and gate.is_cuda, "kernel arguments must be CUDA tensors (there is no CPU path)")
    rows, width = o.shape
    _need(o.is_contiguous() and gate.dtype == torch.float32 and tuple(gate.shape) == (rows, width) and gate.stride(1) == 1,
          "sigmoid_gate: contiguous rows and a float32 gate of the same shape")
    _check(_fn("rowwise", "llmx_sigmoid_gate")(_ptr(o), _code(o), _ptr(gate), gate.stride(0) if rows > 1 else width, rows, width,
                                               _stream()), "sigmoid_gate")
    return o


def clamped_glu(gu: torch.Tensor, out: torch.Tensor, limit: float, alpha: float) -> torch.Tensor:
    """out = g sigmoid(alpha g) (u + 1), g = min(gu[:, :F], limit), u = clamp(gu[:, F:], -limit, limit); gu float32 [rows, 2F]."""
    _cuda(gu, out)
    rows, width = out.shape
    _need(gu.dtype == torch.float32 and tuple(gu.shape) == (rows, 2 * width), "clamped_glu: shapes do not fit")
    _check(_fn("rowwise", "llmx_clamped_glu")(_ptr(gu), _ptr(out), _code(out), rows, width, float(limit), float(alpha),
                                              _stream()), "clamped_glu")
    return out


def silu_columns_(x: torch.Tensor, first: int, count: int) -> torch.Tensor:
    """x[:, first:first + count] = silu(...) in place; x float32 [rows, width]."""
    _cuda(x)
    _need(x.dtype == torch.float32 and x.dim() == 2 and 0 <= first and first + count <= x.shape[1], "silu_columns: range does not fit")
    _check(_fn("rowwise", "llmx_silu_columns")(_ptr(x), x.shape[0], x.shape[1], int(first), int(count), _stream()), "silu_columns")
    return x


def gated_rmsnorm(o: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float, group: int, gate_kind: str,
                  out: torch.Tensor, gate_first: bool = False) -> torch.Tensor:
    """out = o / sqrt(mean over each group of `group` values of o^2 + eps) * weight * act(gate); act sigmoid or silu.
    `gate_first`: the gate comes before the norm: z = o * act(gate), out = z / sqrt(mean z^2 + eps) * weight.
    o float32 [rows, width] contiguous; gate float32 [rows, width], a view whose rows may be strided; weight float32 of
    the row's width, or of one group's width and shared by the groups."""
    _need(o.is_cuda and gate.is_cuda and weight.is_cuda and out.is_cuda, "kernel arguments must be CUDA tensors (there is no CPU path)")
    rows, width = o.shape
    _need(o.is_contiguous() and out.is_contiguous() and weight.is_contiguous(), "gated_rmsnorm: contiguous input, weight and output")
    _need(o.dtype == torch.float32 and gate.dtype == torch.float32 and weight.dtype == torch.float32, "gated_rmsnorm: float32 inputs")
    _need(tuple(out.shape) == (rows, width) and tuple(gate.shape) == (rows, width) and gate.stride(1) == 1, "gated_rmsnorm: shapes do not fit")
    _need(group > 0 and width % group == 0 and weight.numel() in (group, width), "gated_rmsnorm: the group must divide the row; weight of a group or of the row")
    _need(gate_kind in ("sigmoid", "silu"), "gated_rmsnorm: gate must be sigmoid or silu")
    _check(_fn("rowwise", "llmx_gated_rmsnorm")(_ptr(o), _ptr(gate), gate.stride(0) if rows > 1 else width, _ptr(weight),
                                                weight.numel(), _ptr(out), _code(out), rows, width // group, group,
                                                float(eps), 0 if gate_kind == "sigmoid" else 1, 1 if gate_first else 0, _stream()),
           "gated_rmsnorm")
    return out


def pair_norm_add_(x: torch.Tensor, a: torch.Tensor, b: torch.Tensor, wa: torch.Tensor, wb: torch.Tensor, eps: float,
                   factor: float) -> torch.Tensor:
    """x += factor * (a / rms(a) * wa + b / rms(b) * wb), each row of a and b normed over its whole width; all float32."""
    _cuda(x, a, b, wa, wb)
    rows, width = x.shape
    _need(all(t.dtype == torch.float32 for t in (x, a, b, wa, wb)), "pair_norm_add: float32 tensors")
    _need(tuple(a.shape) == (rows, width) and tuple(b.shape) == (rows, width) and wa.numel() == width and wb.numel() == width,
          "pair_norm_add: shapes do not fit")
    _check(_fn("rowwise", "llmx_pair_norm_add")(_ptr(a), _ptr(b), _ptr(wa), _ptr(wb), _ptr(x), rows, width, float(eps),
                                                float(factor), _stream()), "pair_norm_add")
    return x


def add_(x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    """x += y; float32 tensors of one shape."""
    _cuda(x, y)
    _need(x.dtype == torch.float32 and y.dtype == torch.float32 and x.shape == y.shape, "add: float32 tensors of one shape")
    _check(_fn("rowwise", "llmx_add")(_ptr(x), _ptr(y), x.numel(), _stream()), "add")
    return x


# ---------------------------------------------------------------------------
# Matrix-state recurrences.
def group_norm_conv(x: torch.Tensor, weight: torch.Tensor, eps: float, groups: int, out: torch.Tensor,
                    row_index: Optional[torch.Tensor] = None, zero: Optional[torch.Tensor] = None,
                    taps_w: Optional[torch.Tensor] = None, filtered: Optional[torch.Tensor] = None,
                    state: Optional[torch.Tensor] = None, step=None, state_off: int = 0) -> torch.Tensor:
    """RMS norm in `groups` equal consecutive parts of a row (each part by its own root mean square), times the weight, to
    `out`; with `taps_w` float32 [taps, width] (tap by tap) also `filtered` = out + a causal filter of out over the request's
    rows (last tap on the row itself, zeros before the request), whose earlier inputs lie in `state` float32 [slots, floats] at
    `state_off` ([taps - 1][width], read at the request's slot, written at its spare).  `step`: the StepBatch."""
    _cuda(x, weight, out, row_index, zero, taps_w, filtered, state)
    rows = x.shape[0] if row_index is None else row_index.numel()
    width = x.shape[1]
    _need(x.dtype == torch.float32 and weight.dtype == torch.float32 and weight.numel() == width and width % groups == 0,
          "group_norm: float32 rows and weight, a width the groups divide")
    _need(tuple(out.shape) == (rows, width), "group_norm: output shape does not fit")
    _need(row_index is None or row_index.dtype == torch.int32, "group_norm: row_index must be int32")
    _need(zero is None or (zero.dtype == torch.float32 and zero.numel() % 4 == 0 and zero.data_ptr() % 16 == 0), "group_norm: zero buffer float32, 16-byte pieces")
    taps = 1
    if taps_w is not None:
        taps = taps_w.shape[0]
        _need(taps_w.dtype == torch.float32 and tuple(taps_w.shape) == (taps, width) and taps >= 1, "group_norm: taps float32 [taps, width]")
        _need(filtered is not None and filtered.dtype == out.dtype and tuple(filtered.shape) == (rows, width) and row_index is None,
              "group_norm: the filter wants a second output")
    if taps > 1:
        _need(step is not None and rows == step.rows, "group_norm: the filter wants the step")
        _need(state is not None and state.dtype == torch.float32 and state.dim() == 2 and state_off + (taps - 1) * width <= state.shape[1],
              "group_norm: state slots too small for the filter's inputs")
    s = step if taps > 1 else None
    _check(_fn("rowwise", "llmx_group_norm_conv")(
        _ptr(x), _ptr(weight), width, int(groups), float(eps), _ptr(row_index), rows, _ptr(out), _ptr(filtered if taps_w is not None else None),
        _code(out), _ptr(taps_w), taps, _ptr(state if taps > 1 else None), 0 if s is None else state.shape[1],
        int(state_off), _ptr(s.row_request if s else None), _ptr(s.row_start if s else None), _ptr(s.row_count if s else None),
        _ptr(s.history if s else None), _ptr(s.state_slots if s else None), _ptr(s.state_slots_out if s else None),
        s.requests if s else 0, _ptr(zero), 0 if zero is None else zero.numel(), _stream()), "group_norm_conv")
    return out


def embed_pairs(table: torch.Tensor, pair_table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, scale: float, buckets: int,
                mul_prev: int, mul_cur: int, state: torch.Tensor, step) -> torch.Tensor:
    """out[r] = table[id] * scale + pair_table[(id before * mul_prev + id * mul_cur) mod buckets], row `buckets` of the pair
    table for a request's first token; the id before a step's first row is read from `state` int32 [slots, 1] at the
    request's slot, and the step's last id goes to its spare."""
    _cuda(table, pair_table, ids, out, state)
    rows, width = ids.numel(), table.shape[1]
    _need(table.dtype == pair_table.dtype and pair_table.shape[1] == width and pair_table.shape[0] == buckets + 1, "embed_pairs: tables do not fit")
    _need(ids.dtype == torch.int32 and out.dtype == torch.float32 and tuple(out.shape) == (rows, width) and rows == step.rows, "embed_pairs: ids int32, out float32 [rows, width]")
    _need(state.dtype == torch.int32 and state.dim() == 2, "embed_pairs: state int32 [slots, ints]")
    _check(_fn("rowwise", "llmx_embed_pairs")(
        _ptr(table), _ptr(pair_table), _code(table), _ptr(ids), _ptr(out), rows, width, table.shape[0], float(scale), int(buckets),
        int(mul_prev), int(mul_cur), _ptr(step.row_request), _ptr(step.row_start), _ptr(step.row_count), _ptr(step.history),
        _ptr(state), state.shape[1], _ptr(step.state_slots), _ptr(step.state_slots_out), step.requests, _stream()), "embed_pairs")
    return out


def add_rows_(x: torch.Tensor, y: torch.Tensor, factor: float = 1.0, row_factor: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x[r] += factor * row_factor[r] * y[r] (row_factor None: 1); float32 rows."""
    _cuda(x, y, row_factor)
    _need(x.dtype == torch.float32 and y.dtype == torch.float32 and x.shape == y.shape and x.dim() == 2, "add_rows: float32 rows of one shape")
    _need(row_factor is None or (row_factor.dtype == torch.float32 and row_factor.numel() == x.shape[0]), "add_rows: a float32 factor per row")
    _check(_fn("rowwise", "llmx_add_rows")(_ptr(x), _ptr(y), _ptr(row_factor), float(factor), x.shape[0], x.shape[1], _stream()), "add_rows")
    return x


def softcap_(x: torch.Tensor, cap: float) -> torch.Tensor:
    """x <- cap * tanh(x / cap), float32, in place."""
    _cuda(x)
    _need(x.dtype == torch.float32 and cap > 0, "softcap: float32 values, a positive cap")
    _check(_fn("rowwise", "llmx_softcap")(_ptr(x), x.numel(), float(cap), _stream()), "softcap")
    return x


def _strided_rows(t: torch.Tensor, what: str) -> int:
    _need(t.is_cuda and t.dtype == torch.float32 and t.dim() == 2 and t.stride(1) == 1, f"{what}: float32 rows, contiguous within a row")
    return t.stride(0) if t.shape[0] > 1 else t.shape[1]


def linear_recurrence(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, state: torch.Tensor, step, out: torch.Tensor,
                      heads: int, qk_heads: int, key_dim: int, value_dim: int, decay: Optional[torch.Tensor] = None,
                      gate: Optional[torch.Tensor] = None, beta: Optional[torch.Tensor] = None, form: Optional[str] = None,
                      skip: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Per (request, head): S <- a S + k u^T, o = S^T q over the step's rows in order, S [D, V] float32 carried in the
    request's state slot.  `form` (default: "decay" with `decay`, else "delta"):
      "decay"          a = decay_h [heads], u = v
      "delta"          a = gate, u = beta (v - a S^T k); gate, beta [rows, heads] (views)
      "scaled"         a = gate, u = beta v, o += skip_h v; gate, beta [rows, heads], skip [heads] or None
      "delta_channel"  S <- diag(gate) S first, gate [rows, heads * D]; then u = beta (v - S^T k), S <- S + k u^T
    q, k [rows, qk_heads * D], v [rows, heads * V]: float32 views whose rows may be strided.  state [slots, floats]: the
    recurrence's values first, [H][V][D].  `step`: the StepBatch (row ranges, histories and slots are read on the device)."""
    rows = q.shape[0]
    qs, ks, vs = _strided_rows(q, "recurrence q"), _strided_rows(k, "recurrence k"), _strided_rows(v, "recurrence v")
    _need(q.shape[1] == qk_heads * key_dim and k.shape[1] == qk_heads * key_dim and v.shape[1] == heads * value_dim
          and k.shape[0] == rows and v.shape[0] == rows, "recurrence: q, k, v shapes do not fit")
    _cuda(state, out, decay, skip)
    _need(state.dtype == torch.float32 and state.dim() == 2 and state.shape[1] >= heads * key_dim * value_dim, "recurrence: state slots too small")
    _need(out.dtype == torch.float32 and tuple(out.shape) == (rows, heads * value_dim), "recurrence: output shape does not fit")
    if form is None:
        form = "delta" if gate is not None else "decay"
    _need(form in ("decay", "delta", "scaled", "delta_channel"), "recurrence: unknown form")
    mode = ("decay", "delta", "scaled", "delta_channel").index(form)
    gs = bs = 0
    if mode == 0:
        _need(decay is not None and decay.dtype == torch.float32 and decay.numel() == heads and gate is None, "recurrence: decay float32 [heads]")
    else:
        _need(gate is not None and beta is not None and decay is None, "recurrence: this form takes gate and beta and no constant decay")
        gs, bs = _strided_rows(gate, "recurrence gate"), _strided_rows(beta, "recurrence beta")
        _need(tuple(gate.shape) == (rows, heads * key_dim if mode == 3 else heads) and tuple(beta.shape) == (rows, heads),
              "recurrence: gate [rows, heads] (or [rows, heads * D] per key channel) and beta [rows, heads]")
    if skip is not None:
        _need(mode == 2 and skip.dtype == torch.float32 and skip.numel() == heads, "recurrence: skip float32 [heads], scaled form only")
    _check(_fn("recurrence", "llmx_linear_recurrence")(
        _ptr(q), _ptr(k), _ptr(v), qs, ks, vs, mode, _ptr(decay), _ptr(gate), _ptr(beta), gs, bs, _ptr(skip), _ptr(state),
        state.shape[1], _ptr(step.row_start), _ptr(step.row_count), _ptr(step.history), _ptr(step.state_slots),
        _ptr(step.state_slots_out), _ptr(out), step.requests, heads, qk_heads, key_dim, value_dim, int(step.max_row_count),
        _stream()), "linear_recurrence")
    return out


def conv_prepare(proj: torch.Tensor, channels: int, q_channels: int, k_channels: int, taps_w: torch.Tensor,
                 ready: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor, b_off: int, a_off: int,
                 gates: torch.Tensor, heads: int, key_dim: int, q_factor: float, state: torch.Tensor, conv_off: int,
                 step, first: int = 0, bias: Optional[torch.Tensor] = None, gate_kind: str = "delta",
                 decay_in: Optional[torch.Tensor] = None) -> None:
    """The short causal convolution (+ `bias`), silu, unit q/k heads and the gates of a recurrent mixer
    (csrc/recurrence.cu).  The filtered channels are columns first .. first + channels - 1 of `proj`.  `gate_kind`:
    "delta": gates [rows, 2 heads] = g, beta;  "step": gates [rows, 2 heads] = g, dt with dt = softplus(a + dt_bias);
    "delta_channel": gates [rows, heads + heads * D] = beta, then g per key channel made from `decay_in`
    [rows, heads * D] and dt_bias [heads * D].  The request's slot read and the slot written must differ (a step reads
    one and writes its spare)."""
    _cuda(proj, taps_w, ready, a_log, dt_bias, gates, state, bias, decay_in)
    rows = proj.shape[0]
    taps = taps_w.shape[1]
    kind = ("delta", "step", "delta_channel").index(gate_kind)
    _need(proj.dtype == torch.float32 and proj.dim() == 2 and proj.shape[1] >= first + channels, "conv_prepare: projections float32 [rows, >= channels]")
    _need(taps_w.dtype == torch.float32 and tuple(taps_w.shape) == (channels, taps), "conv_prepare: taps float32 [channels, taps]")
    _need(bias is None or (bias.dtype == torch.float32 and bias.numel() == channels), "conv_prepare: bias float32 [channels]")
    _need(ready.dtype == torch.float32 and tuple(ready.shape) == (rows, channels), "conv_prepare: output shape does not fit")
    per_row = heads + heads * key_dim if kind == 2 else 2 * heads
    _need(gates.dtype == torch.float32 and tuple(gates.shape) == (rows, per_row), "conv_prepare: gates float32 of the kind's width")
    _need(a_log.dtype == torch.float32 and dt_bias.dtype == torch.float32 and a_log.numel() == heads
          and dt_bias.numel() == (heads * key_dim if kind == 2 else heads), "conv_prepare: A_log [heads] and dt_bias float32")
    _need((kind == 2 or a_off + heads <= proj.shape[1]) and (kind == 1 or b_off + heads <= proj.shape[1]),
          "conv_prepare: gate columns outside the projections")
    ds = 0
    if kind == 2:
        _need(decay_in is not None and decay_in.dtype == torch.float32 and tuple(decay_in.shape) == (rows, heads * key_dim),
              "conv_prepare: decay_in float32 [rows, heads * D]")
        ds = decay_in.shape[1]
    _need(state.dtype == torch.float32 and state.dim() == 2 and conv_off + (taps - 1) * channels <= state.shape[1],
          "conv_prepare: state slots too small")
    _check(_fn("recurrence", "llmx_conv_prepare")(
        _ptr(proj), proj.shape[1], int(first), channels, q_channels, k_channels, _ptr(taps_w), _ptr(bias), taps, _ptr(ready),
        _ptr(a_log), _ptr(dt_bias), int(b_off), int(a_off), kind, _ptr(decay_in), ds, _ptr(gates), gates.shape[1], heads, key_dim,
        float(q_factor), _ptr(state), state.shape[1], int(conv_off), _ptr(step.row_request), _ptr(step.row_start),
        _ptr(step.row_count), _ptr(step.history), _ptr(step.state_slots), _ptr(step.state_slots_out), rows, step.requests,
        _stream()), "conv_prepare")


# ---------------------------------------------------------------------------
# Softmax attention over [key ; value] rows; experts chosen by a table.
def qk_norm_rope_write(proj: torch.Tensor, heads: int, kv_heads: int, key_dim: int, value_dim: int,
                       q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                       freq: Optional[torch.Tensor], positions: torch.Tensor, slots: torch.Tensor, q_out: torch.Tensor,
                       cache: torch.Tensor) -> None:
    """Rows of the stacked product [q (heads * D) | k (kv_heads * D) | v (kv_heads * V)], float32: per-head RMS norm of q
    and k (weights [D] or None), rotation of the first 2 * len(freq) values of each q and k head (value i with value
    i + len(freq), angle position * freq[i]), queries to q_out [rows, heads * D], [k ; v] to cache [pages, 1, kv_heads,
    page, D + V] at the rows' slots."""
    _cuda(proj, q_weight, k_weight, freq, positions, slots, q_out, cache)
    rows = proj.shape[0]
    _need(proj.dtype == torch.float32 and proj.shape[1] == (heads + kv_heads) * key_dim + kv_heads * value_dim, "qk_write: product width does not fit")
    _need(tuple(q_out.shape) == (rows, heads * key_dim), "qk_write: q_out shape does not fit")
    _need(cache.dim() == 5 and cache.shape[1] == 1 and cache.shape[2] == kv_heads and cache.shape[4] == key_dim + value_dim,
          "qk_write: cache layout does not fit")
    for w in (q_weight, k_weight):
        _need(w is None or (w.dtype == torch.float32 and w.numel() == key_dim), "qk_write: norm weight float32 [D]")
    half = 0 if freq is None else freq.numel()
    _need(freq is None or freq.dtype == torch.float32, "qk_write: frequencies float32")
    _need(positions.dtype == torch.int32 and slots.dtype == torch.int32 and positions.numel() >= rows and slots.numel() >= rows,
          "qk_write: positions and slots must be int32 per row")
    _check(_fn("attention_split", "llmx_qk_norm_rope_write")(
        _ptr(proj), proj.shape[1], _ptr(q_weight), _ptr(k_weight), float(eps), _ptr(freq), half, _ptr(positions), _ptr(slots),
        _ptr(q_out), _code(q_out), _ptr(cache), _code(cache), rows, heads, kv_heads, key_dim, value_dim, cache.shape[3],
        _stream()), "qk_norm_rope_write")


def qkv_finish(proj: torch.Tensor, heads: int, kv_heads: int, key_dim: int, value_dim: int, step, q_out: torch.Tensor,
               cache: Optional[torch.Tensor] = None, slots: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
               taps_w: Optional[torch.Tensor] = None, state: Optional[torch.Tensor] = None, conv_off: int = 0,
               norm: str = "none", q_weight: Optional[torch.Tensor] = None, k_weight: Optional[torch.Tensor] = None, eps: float = 0.0,
               freq: Optional[torch.Tensor] = None, neighbours: bool = False, rot_mag: float = 1.0,
               vfreq: Optional[torch.Tensor] = None) -> None:
    """The general finishing of a stacked q/k/v product's rows (csrc/attention_split.cu, `QkvFinish`): proj float32 [rows, q
    (heads * D) | k (kv_heads * D) | v (kv_heads * V)] (a view whose rows may be strided; kv_heads 0: queries alone) plus
    `bias` [channels]; a causal filter `taps_w` [channels, taps] per channel whose earlier inputs lie in `state`
    [slots, floats] at `conv_off` ([taps - 1][channels], read at the request's slot, written at its spare); an RMS norm
    per q and k head `norm` = "none" | "before" | "after" the rotation, with weights [D] or without; a rotation of the
    first 2 * len(freq) values of a head by position * freq[i], pairs (i, i + len(freq)) or `neighbours` (2i, 2i + 1);
    queries to q_out [rows, heads * D], [k ; v] to cache [pages, 1, kv_heads, page, D + V] at `slots`, or, where the cache
    has planes of keys and of values, [pages, 2, kv_heads, page, D] (D = V), to those.  `step`: the StepBatch.
    `norm` "whole": one RMS norm over all of a row's queries and one over all of its keys, before they are split into
    heads, with weights [heads * D] and [kv_heads * D].  `rot_mag`: a factor on the rotation's cosines and sines.  `vfreq`
    float32 [V / 2]: the values are rotated too, over all of V, pair m by position * vfreq[m], in the same pairing."""
    _cuda(bias, taps_w, state, q_weight, k_weight, freq, slots, q_out, cache, vfreq)
    rows = proj.shape[0]
    channels = (heads + kv_heads) * key_dim + kv_heads * value_dim
    _need(proj.is_cuda and proj.dtype == torch.float32 and proj.dim() == 2 and proj.shape[1] == channels and proj.stride(1) == 1,
          "qkv_finish: product rows float32 [rows, q | k | v]")
    _need(tuple(q_out.shape) == (rows, heads * key_dim) and rows == step.rows, "qkv_finish: q_out shape or the step's rows do not fit")
    _need(norm in ("none", "before", "after", "whole"), "qkv_finish: norm is none, before, after or whole")
    qn, kn = (heads * key_dim, kv_heads * key_dim) if norm == "whole" else (key_dim, key_dim)
    for t, n in ((bias, channels), (q_weight, qn), (k_weight, kn)):
        _need(t is None or (t.dtype == torch.float32 and t.numel() == n), "qkv_finish: float32 bias [channels], norm weights [D] (whole: [heads * D])")
    _need(vfreq is None or (vfreq.dtype == torch.float32 and 2 * vfreq.numel() == value_dim), "qkv_finish: value frequencies float32 [V / 2]")
    taps = 1
    if taps_w is not None:
        taps = taps_w.shape[1]
        _need(taps_w.dtype == torch.float32 and tuple(taps_w.shape) == (channels, taps), "qkv_finish: taps float32 [channels, taps]")
    if taps > 1:
        _need(state is not None and state.dtype == torch.float32 and state.dim() == 2
              and conv_off + (taps - 1) * channels <= state.shape[1], "qkv_finish: state slots too small for the filter's inputs")
    if kv_heads:
        _need(cache is not None and slots is not None and cache.dim() == 5 and cache.shape[2] == kv_heads and cache.is_contiguous()
              and ((cache.shape[1] == 1 and cache.shape[4] == key_dim + value_dim)
                   or (cache.shape[1] == 2 and key_dim == value_dim and cache.shape[4] == key_dim))
              and slots.dtype == torch.int32 and slots.numel() >= rows, "qkv_finish: cache layout or slots do not fit")
    _need(freq is None or (freq.dtype == torch.float32 and 2 * freq.numel() <= key_dim), "qkv_finish: frequencies float32 [<= D / 2]")
    _check(_fn("attention_split", "llmx_qkv_finish")(
        _ptr(proj), proj.stride(0) if rows > 1 else proj.shape[1], _ptr(bias), _ptr(taps_w), taps, _ptr(state),
        0 if state is None else state.shape[1], int(conv_off), _ptr(step.row_request), _ptr(step.row_start), _ptr(step.row_count),
        _ptr(step.history), _ptr(step.state_slots), _ptr(step.state_slots_out), _ptr(q_weight), _ptr(k_weight),
        ("none", "before", "after", "whole").index(norm), float(eps), _ptr(freq), 0 if freq is None else freq.numel(), 1 if neighbours else 0,
        _ptr(step.positions), _ptr(slots), _ptr(q_out), _code(q_out), _ptr(cache), _code(cache) if cache is not None else F32, rows,
        step.requests, heads, kv_heads, key_dim, value_dim, cache.shape[3] if cache is not None else 1,
        cache.shape[1] if cache is not None else 1, float(rot_mag), _ptr(vfreq), _stream()), "qkv_finish")


class SoftmaxExtras:
    """What a design may add to the softmax of `attention_split` / `attention_tiled` (csrc/attention_split.cu, `AttnExtras`):
    `softcap` c > 0: score <- c tanh(score / c) after the scale; `sink`: a float32 tensor [heads] whose exp joins each head's
    denominator (it has no key and no value), or the string "zero" for a sink of 0 (one is added to the denominator);
    `vfreq` float32 [V / 2]: the cached values were rotated by their positions, and a row's output is turned back by its
    own (`v_neighbours`: pairs (2m, 2m + 1) instead of (m, m + V / 2))."""

    def __init__(self, softcap: Optional[float] = None, sink=None, vfreq: Optional[torch.Tensor] = None, v_neighbours: bool = False):
        self.softcap, self.sink, self.vfreq, self.v_neighbours = softcap, sink, vfreq, bool(v_neighbours)

    def checked(self, heads: int, value_dim: int):
        learned = isinstance(self.sink, torch.Tensor)
        if learned:
            _cuda(self.sink)
            _need(self.sink.dtype == torch.float32 and self.sink.numel() == heads, "attention: a sink per head, float32")
        else:
            _need(self.sink in (None, "zero"), "attention: sink is a tensor [heads], \"zero\" or None")
        if self.vfreq is not None:
            _cuda(self.vfreq)
            _need(self.vfreq.dtype == torch.float32 and 2 * self.vfreq.numel() == value_dim, "attention: value frequencies float32 [V / 2]")
        _need(self.softcap is None or self.softcap > 0, "attention: the cap on the scores must be positive")
        return (float(self.softcap or 0.0), _ptr(self.sink if learned else None), 1 if learned else 2 if self.sink == "zero" else 0,
                _ptr(self.vfreq), 1 if self.v_neighbours else 0)


NO_EXTRAS = SoftmaxExtras()


def attention_split(q: torch.Tensor, cache: torch.Tensor, out: torch.Tensor, row_request: torch.Tensor,
                    positions: torch.Tensor, block_tables: torch.Tensor, heads: int, kv_heads: int, key_dim: int,
                    value_dim: int, window: Optional[int], chunk: Optional[int], scale: float, splits: int = 1,
                    extras: Optional["SoftmaxExtras"] = None, staged: bool = False) -> torch.Tensor:
    """Paged softmax attention, one block per (row, head); q [rows, heads * D] and out [rows, heads * V] of one type;
    cache [pages, 1, kv_heads, page, D + V].  A row at position p reads keys max(p - window + 1, floor(p / chunk) * chunk,
    0) .. p.  `splits` > 1: a row's keys are cut into that many ranges, a block each, merged by a second kernel in
    range order (for steps of few rows over long histories; the result is the same up to the order of sums).
    `staged` (where `attention_staged_fits`): one block per (row, key/value head, range) that copies tiles of keys and
    values into shared memory once for all heads of the group (a matter of speed: the same sums in another order)."""
    _cuda(q, cache, out, row_request, positions, block_tables)
    rows = q.shape[0]
    _need(q.shape[1] == heads * key_dim and tuple(out.shape) == (rows, heads * value_dim) and q.dtype == out.dtype,
          "attention: q and out shapes do not fit")
    _need(cache.dim() == 5 and cache.shape[1] == 1 and cache.shape[2] == kv_heads and cache.shape[4] == key_dim + value_dim,
          "attention: cache layout does not fit")
    for t in (row_request, positions, block_tables):
        _need(t.dtype == torch.int32, "attention: metadata must be int32")
    _need(block_tables.dim() == 2 and row_request.numel() >= rows and positions.numel() >= rows, "attention: metadata shapes do not fit")
    splits = max(1, min(int(splits), 64))
    partial = torch.empty((rows, heads, splits, value_dim + 2), dtype=torch.float32, device=q.device) if splits > 1 else None
    x = (extras or NO_EXTRAS).checked(heads, value_dim)
    if staged:
        if partial is None:
            partial = torch.empty((rows, heads, 1, value_dim + 2), dtype=torch.float32, device=q.device)
        _check(_fn("attention_split", "llmx_attention_staged")(
            _ptr(q), _code(q), _ptr(cache), _code(cache), _ptr(out), _ptr(row_request), _ptr(positions), _ptr(block_tables),
            block_tables.shape[1], rows, heads, kv_heads, key_dim, value_dim, cache.shape[3], int(window or 0), int(chunk or 0),
            float(scale), splits, _ptr(partial), *x, _stream()), "attention_staged", 2)
        return out
    _check(_fn("attention_split", "llmx_attention_split")(
        _ptr(q), _code(q), _ptr(cache), _code(cache), _ptr(out), _ptr(row_request), _ptr(positions), _ptr(block_tables),
        block_tables.shape[1], rows, heads, kv_heads, key_dim, value_dim, cache.shape[3], int(window or 0), int(chunk or 0),
        float(scale), splits, _ptr(partial), *x, _stream()), "attention_split", 2 if splits > 1 else 1)
    return out


def attention_staged_fits(q_dtype: torch.dtype, cache_dtype: torch.dtype, heads: int, kv_heads: int, key_dim: int, value_dim: int) -> bool:
    """Whether `attention_split(staged=True)` takes these types and sizes."""
    if q_dtype not in _CODE or cache_dtype not in _CODE:
        return False
    f = _fn("attention_split", "llmx_attention_staged_fits")
    return bool(f(_CODE[q_dtype], _CODE[cache_dtype], int(heads), int(kv_heads), int(key_dim), int(value_dim)))


def attention_tiled_fits(heads: int, kv_heads: int, key_dim: int, value_dim: int) -> bool:
    """Whether the tiled form of `attention_split` takes these sizes (it also wants bfloat16 queries and cache)."""
    f = _fn("attention_split", "llmx_attention_tiled_fits")
    return bool(f(int(heads), int(kv_heads), int(key_dim), int(value_dim)))


def attention_tiled(q: torch.Tensor, cache: torch.Tensor, out: torch.Tensor, step, block_tables: torch.Tensor, heads: int,
                    kv_heads: int, key_dim: int, value_dim: int, window: Optional[int], chunk: Optional[int], scale: float,
                    extras: Optional["SoftmaxExtras"] = None) -> torch.Tensor:
    """`attention_split` on the tensor cores (csrc/attention_split.cu): bfloat16 q [rows, heads * D], out [rows, heads * V]
    and cache; 64 rows that share their keys a block, keys in tiles of 64; softmax weights enter the second product
    as sums of three bfloat16 values.  `step`: the StepBatch (row ranges and histories are read on the device)."""
    _cuda(q, cache, out, block_tables)
    rows = q.shape[0]
    _need(q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and cache.dtype == torch.bfloat16, "attention_tiled: bfloat16 queries, output and cache")
    _need(q.shape[1] == heads * key_dim and tuple(out.shape) == (rows, heads * value_dim), "attention: q and out shapes do not fit")
    _need(cache.dim() == 5 and cache.shape[1] == 1 and cache.shape[2] == kv_heads and cache.shape[4] == key_dim + value_dim,
          "attention: cache layout does not fit")
    _need(block_tables.dtype == torch.int32 and block_tables.dim() == 2 and rows == step.rows, "attention: metadata does not fit")
    _check(_fn("attention_split", "llmx_attention_tiled")(
        _ptr(q), _ptr(cache), _ptr(out), _ptr(step.row_start), _ptr(step.row_count), _ptr(step.history), _ptr(block_tables),
        block_tables.shape[1], rows, step.requests, heads, kv_heads, key_dim, value_dim, cache.shape[3], int(window or 0),
        int(chunk or 0), float(scale), *(extras or NO_EXTRAS).checked(heads, value_dim), _stream()), "attention_tiled")
    return out


def moe_tiles_len(pairs: int, experts: int) -> int:
    """Ints the tiles of a routing take at most (tiles of 32 pairs; tiles of 128 are fewer)."""
    return 2 + 2 * ((pairs + 31) // 32 + experts)


_moe_tile_rows = {}


def moe_tensor_cores_fit(dtype: torch.dtype, *inner_widths: int) -> bool:
    """Whether the experts' products of this type over these inner widths can all run the tensor-core form."""
    f = getattr(_build.load("moe"), "llmx_moe_tensor_cores_fit")
    f.argtypes, f.restype = [_i, _i], _i
    return dtype in _CODE and all(bool(f(_CODE[dtype], int(k))) for k in inner_widths)


def moe_product_few(a: torch.Tensor, a_div: int, w: torch.Tensor, token_ids: torch.Tensor, table: torch.Tensor, pairs: int,
                    out: torch.Tensor, gated: bool) -> torch.Tensor:
    """`moe_product` for steps of a few pairs (bfloat16, inner width a multiple of 8): a block a pair and 16 output
    columns, the pair's expert read from the table, no lists."""
    _cuda(a, w, token_ids, table, out)
    experts, wn, K = w.shape
    N = wn // 2 if gated else wn
    vocab, top = table.shape
    # No ids: the table has a row for each row of the step (a router wrote it).
    _need(a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.dim() == 2 and a.shape[1] == K and a.shape[0] * a_div >= pairs,
          "moe_product_few: bfloat16 rows that fit the weights")
    _need(table.dtype == torch.int32 and (vocab * top >= pairs if token_ids is None else
                                          token_ids.dtype == torch.int32 and token_ids.numel() * top >= pairs),
          "moe_product_few: int32 ids and table")
    _need(tuple(out.shape) == (pairs, N), "moe_product_few: output shape does not fit")
    _check(_fn("moe", "llmx_moe_product_few")(_ptr(a), int(a_div), _ptr(w), _ptr(token_ids), _ptr(table), top, vocab, pairs, experts,
                                              _ptr(out), _code(out), N, K, 1 if gated else 0, _stream()), "moe_product_few")
    return out


def moe_route(token_ids: torch.Tensor, table: torch.Tensor, experts: int, lists: torch.Tensor, counts: torch.Tensor,
              tiles: torch.Tensor, tensor_cores: bool = False) -> None:
    """Sort the step's (row, k) pairs by the expert the table gives them: lists int32 [experts, rows * top] (pairs in
    order), counts int32 [experts], tiles int32 [moe_tiles_len] (their number, their size, then (expert, first place) of
    every tile).  `tensor_cores`: the form of `moe_product` that will run (it sets the tiles' size: 128 pairs, else 32)."""
    _cuda(token_ids, table, lists, counts, tiles)
    vocab, top = table.shape
    rows = vocab if token_ids is None else token_ids.numel()      # no ids: the table has a row for each row of the step
    for t in (token_ids, table, lists, counts, tiles):
        _need(t is None or t.dtype == torch.int32, "moe_route: int32 tensors")
    _need(lists.numel() >= experts * rows * top and counts.numel() >= experts and tiles.numel() >= moe_tiles_len(rows * top, experts),
          "moe_route: outputs too small")
    tile_rows = _moe_tile_rows.get(bool(tensor_cores))
    if tile_rows is None:
        f = getattr(_build.load("moe"), "llmx_moe_tile_rows")
        f.argtypes, f.restype = [_i], _i
        tile_rows = _moe_tile_rows[bool(tensor_cores)] = f(1 if tensor_cores else 0)
    _check(_fn("moe", "llmx_moe_route")(_ptr(token_ids), _ptr(table), top, rows, experts, vocab, _ptr(lists), _ptr(counts),
                                        _ptr(tiles), tile_rows, _stream()), "moe_route", 2)


def moe_product(a: torch.Tensor, a_div: int, w: torch.Tensor, lists: torch.Tensor, counts: torch.Tensor, tiles: torch.Tensor,
                pairs: int, out: torch.Tensor, gated: bool, tensor_cores: bool = False) -> torch.Tensor:
    """out[pair] = a[pair // a_div] W_e^T for the expert e whose list holds the pair; w [experts, N (gated: 2 N, gate rows
    then up rows), K] of a's type.  gated: out = silu(gate) * up in out's type; else float32.  `tensor_cores` as the
    routing was told."""
    _cuda(a, w, lists, counts, tiles, out)
    experts, wn, K = w.shape
    N = wn // 2 if gated else wn
    _need(a.dtype == w.dtype and a.dim() == 2 and a.shape[1] == K and a.shape[0] * a_div >= pairs, "moe_product: rows do not fit the weights")
    _need(tuple(out.shape) == (pairs, N), "moe_product: output shape does not fit")
    _check(_fn("moe", "llmx_moe_product")(_ptr(a), int(a_div), _ptr(w), _code(w), _ptr(lists), _ptr(counts), _ptr(tiles), pairs,
                                          experts, _ptr(out), _code(out), N, K, 1 if gated else 0, 1 if tensor_cores else 0,
                                          _stream()), "moe_product")
    return out


def moe_router(h: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], experts: int, top: int, choice: torch.Tensor,
               weight: torch.Tensor, gate: Optional[torch.Tensor] = None) -> None:
    """A router on the device: logits h w[:experts]^T + bias in 32-bit (w float32 [experts + extra, K]), the `top` largest to
    choice int32 [rows, top] (the lower index first among equals), the softmax over the chosen logits to weight float32
    [rows, top]; the `extra` rows of w after the experts' give gate float32 [rows, extra] through a sigmoid."""
    _cuda(h, w, bias, choice, weight, gate)
    rows, K = h.shape
    extra = w.shape[0] - experts
    _need(w.dtype == torch.float32 and w.dim() == 2 and w.shape[1] == K and extra >= 0, "moe_router: float32 weights [experts + extra, K]")
    _need(bias is None or (bias.dtype == torch.float32 and bias.numel() == experts), "moe_router: float32 bias [experts]")
    _need(choice.dtype == torch.int32 and tuple(choice.shape) == (rows, top) and weight.dtype == torch.float32
          and tuple(weight.shape) == (rows, top), "moe_router: choice int32 and weight float32 [rows, top]")
    _need(extra == 0 or (gate is not None and gate.dtype == torch.float32 and gate.numel() == rows * extra), "moe_router: gate float32 [rows, extra]")
    _check(_fn("moe", "llmx_moe_router")(_ptr(h), _code(h), _ptr(w), _ptr(bias), rows, K, experts, top, extra, _ptr(choice), _ptr(weight),
                                         _ptr(gate), _stream()), "moe_router")


def moe_combine_weighted_(x: torch.Tensor, y: torch.Tensor, pair_weight: torch.Tensor, top: int, factor: float = 1.0) -> torch.Tensor:
    """x[row] += factor * sum_k pair_weight[row, k] * y[row * top + k], k in increasing order; float32."""
    _cuda(x, y, pair_weight)
    rows, width = x.shape
    _need(x.dtype == torch.float32 and y.dtype == torch.float32 and tuple(y.shape) == (rows * top, width)
          and pair_weight.dtype == torch.float32 and pair_weight.numel() == rows * top, "moe_combine: shapes do not fit")
    _check(_fn("moe", "llmx_moe_combine_weighted")(_ptr(y), _ptr(x), _ptr(pair_weight), rows, top, width, float(factor), _stream()),
           "moe_combine_weighted")
    return x


def moe_combine_(x: torch.Tensor, y: torch.Tensor, top: int, weight: float) -> torch.Tensor:
    """x[row] += weight * sum_k y[row * top + k], k in increasing order; float32."""
    _cuda(x, y)
    rows, width = x.shape
    _need(x.dtype == torch.float32 and y.dtype == torch.float32 and tuple(y.shape) == (rows * top, width), "moe_combine: shapes do not fit")
    _check(_fn("moe", "llmx_moe_combine")(_ptr(y), _ptr(x), rows, top, width, float(weight), _stream()), "moe_combine")
    return x


# ---------------------------------------------------------------------------
# Attention over a cache of latents.
def latent_write(down: torch.Tensor, q_rank: int, q_weight: Optional[torch.Tensor], cq: Optional[torch.Tensor], weight: torch.Tensor,
                 eps: float, freq: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor, cache: torch.Tensor, latent: int,
                 rot: int, halves: bool = False, magnitude: float = 1.0) -> None:
    """Rows of the stacked down projections [query latent | key/value latent | rotated key part]:
    cq = rmsnorm(query latent) * q_weight (in cq's type; `q_rank` 0: the rows hold no query latent), and
    cache[slot] = [rmsnorm(key/value latent) * weight ; rotate(rotated part)]; cache [pages, 1, 1, page, latent + rot].
    `down` may be a view of the first columns of a wider product's output.  `halves`: rotation pair i is (i, i + pairs)
    instead of neighbours; `magnitude`: a factor on cosines and sines."""
    _need(all(t is None or t.is_cuda for t in (down, q_weight, cq, weight, freq, positions, slots, cache)), "kernel arguments must be CUDA tensors (there is no CPU path)")
    rows = down.shape[0]
    _need(down.dtype == torch.float32 and down.dim() == 2 and down.shape[1] == q_rank + latent + rot and down.stride(1) == 1,
          "latent_write: down projections float32 [rows, q_rank + latent + rot]")
    if q_rank:
        _need(q_weight is not None and cq is not None and q_weight.dtype == torch.float32 and q_weight.numel() == q_rank
              and tuple(cq.shape) == (rows, q_rank), "latent_write: query latent weight [q_rank] and output [rows, q_rank]")
    _need(weight.dtype == torch.float32 and weight.numel() == latent and freq.dtype == torch.float32 and 2 * freq.numel() <= rot,
          "latent_write: weight [latent], frequencies [<= rot / 2]")
    _need(cache.shape[-1] == latent + rot, "latent_write: cache rows do not fit")
    _need(positions.dtype == torch.int32 and slots.dtype == torch.int32 and positions.numel() >= rows and slots.numel() >= rows,
          "latent_write: positions and slots must be int32 per row")
    _check(_fn("latent_attention", "llmx_latent_write")(_ptr(down), down.stride(0) if rows > 1 else down.shape[1], int(q_rank), _ptr(q_weight), _ptr(cq),
                                                        _code(cq) if cq is not None else F32, _ptr(weight), float(eps), _ptr(freq),
                                                        freq.numel(), 1 if halves else 0, float(magnitude), _ptr(positions), _ptr(slots),
                                                        _ptr(cache), _code(cache), rows, latent, rot, _stream()), "latent_write")


def latent_attention(q: torch.Tensor, cache: torch.Tensor, w_uk: torch.Tensor, w_uv: torch.Tensor, out: torch.Tensor,
                     freq: torch.Tensor, row_request: torch.Tensor, positions: torch.Tensor, block_tables: torch.Tensor,
                     heads: int, key_dim: int, rot: int, value_dim: int, latent: int, page_size: int,
                     window: Optional[int], scale: float, halves: bool = False, magnitude: float = 1.0) -> torch.Tensor:
    """Softmax attention of query heads [key_dim unrotated ; rot rotated] over cached [latent ; rotated key part] rows, the
    keys and values of a head being linear maps of the latent (csrc/latent_attention.cu).  q float32 [rows, heads *
    (key_dim + rot)]; w_uk [heads * key_dim, latent], w_uv [heads * value_dim, latent] and out [rows, heads * value_dim]
    of one type.  q may be a view of columns of a wider product's output."""
    _cuda(cache, w_uk, w_uv, out, freq, row_request, positions, block_tables)
    rows = q.shape[0]
    _need(q.is_cuda and q.dtype == torch.float32 and q.shape[1] == heads * (key_dim + rot) and q.stride(1) == 1,
          "latent_attention: queries float32 [rows, heads * (key_dim + rot)]")
    _need(tuple(w_uk.shape) == (heads * key_dim, latent) and tuple(w_uv.shape) == (heads * value_dim, latent)
          and w_uk.dtype == w_uv.dtype == out.dtype, "latent_attention: key and value maps do not fit")
    _need(tuple(out.shape) == (rows, heads * value_dim) and cache.shape[-1] == latent + rot, "latent_attention: output or cache rows do not fit")
    for t in (row_request, positions, block_tables):
        _need(t.dtype == torch.int32, "latent_attention: metadata must be int32")
    _check(_fn("latent_attention", "llmx_latent_attention")(
        _ptr(q), q.stride(0) if rows > 1 else q.shape[1], _ptr(cache), _code(cache), _ptr(w_uk), _ptr(w_uv), _code(w_uk), _ptr(out),
        _ptr(freq), freq.numel(), 1 if halves else 0, float(magnitude), _ptr(row_request), _ptr(positions), _ptr(block_tables), block_tables.shape[1], rows, heads, key_dim, rot, value_dim,
        latent, page_size, int(window or 0), float(scale), _stream()), "latent_attention")
    return out


def latent_tile_shape(heads: int):
    """(heads a block of the tiled form holds, rows a tile holds): 16 (row, head) pairs share every key they read."""
    ht = min((heads + 1) & ~1, 16)
    while 16 % ht:
        ht += 2
    return ht, 16 // ht


def latent_attention_tiled(q: torch.Tensor, cache: torch.Tensor, w_uk: torch.Tensor, w_uv: torch.Tensor, out: torch.Tensor,
                           freq: torch.Tensor, row_request: torch.Tensor, positions: torch.Tensor, block_tables: torch.Tensor,
                           tiles: torch.Tensor, n_tiles: int, splits: int, heads: int, key_dim: int, rot: int, value_dim: int,
                           latent: int, page_size: int, window: Optional[int], scale: float, plain_cores: bool = False,
                           halves: bool = False, magnitude: float = 1.0) -> torch.Tensor:
    """`latent_attention` in its tiled form (csrc/latent_attention.cu): `tiles` int32 [n_tiles, 2] on the device, the
    first row and the row count of every tile (rows of one request, at most `latent_tile_shape`'s); `splits` ranges
    of a tile's keys run as blocks of their own and are merged.  With a bfloat16 cache and a latent of 128, 256 or 512
    values the scores run on the tensor cores, 32-bit factors as sums of three bfloat16 values; `plain_cores` keeps
    them on the CUDA cores."""
    _cuda(cache, w_uk, w_uv, out, freq, row_request, positions, block_tables, tiles)
    rows = q.shape[0]
    _need(q.is_cuda and q.dtype == torch.float32 and q.shape[1] == heads * (key_dim + rot) and q.stride(1) == 1,
          "latent_attention: queries float32 [rows, heads * (key_dim + rot)]")
    _need(tuple(w_uk.shape) == (heads * key_dim, latent) and tuple(w_uv.shape) == (heads * value_dim, latent)
          and w_uk.dtype == w_uv.dtype == out.dtype, "latent_attention: key and value maps do not fit")
    _need(tuple(out.shape) == (rows, heads * value_dim) and cache.shape[-1] == latent + rot, "latent_attention: output or cache rows do not fit")
    for t in (row_request, positions, block_tables, tiles):
        _need(t.dtype == torch.int32, "latent_attention: metadata must be int32")
    _need(tiles.numel() >= 2 * n_tiles and n_tiles > 0 and splits > 0, "latent_attention: tiles do not fit")
    qk = torch.empty((rows, heads, latent + rot), dtype=torch.float32, device=q.device)
    part = torch.empty((rows, heads, splits, latent + 2), dtype=torch.float32, device=q.device)
    _check(_fn("latent_attention", "llmx_latent_query")(_ptr(q), q.stride(0) if rows > 1 else q.shape[1], _ptr(w_uk), _code(w_uk), _ptr(qk),
                                                        _ptr(freq), freq.numel(), 1 if halves else 0, float(magnitude),
                                                        _ptr(positions), rows, heads, key_dim, rot, latent, float(scale), _stream()),
           "latent_query")
    _check(_fn("latent_attention", "llmx_latent_scores")(_ptr(qk), _ptr(cache), _code(cache), _ptr(part), _ptr(tiles), int(n_tiles),
                                                         int(splits), _ptr(row_request), _ptr(positions), _ptr(block_tables),
                                                         block_tables.shape[1], heads, latent, rot, page_size, int(window or 0),
                                                         1 if plain_cores else 0, _stream()), "latent_scores")
    _check(_fn("latent_attention", "llmx_latent_merge")(_ptr(part), _ptr(w_uv), _code(w_uv), _ptr(out), rows, heads, value_dim, latent,
                                                        int(splits), _stream()), "latent_merge")
    return out
