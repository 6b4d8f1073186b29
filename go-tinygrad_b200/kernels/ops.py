"""Tensor-level entry points of the hand-written kernels.

Each function checks shapes, dtypes and layout on the host, then calls the C
launcher of the compiled library on the current CUDA stream.  A size that a
kernel does not take is refused here with a `KernelError` that says why; there
is no other route for the same work (no library attention, no CPU path).
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_ulonglong, c_void_p
from typing import Optional

import torch

from . import build

PAGE_TOKENS = 64

_P, _I, _L, _F, _U = c_void_p, c_int, c_longlong, c_float, c_ulonglong

# library, symbol -> argument types (the stream is always last)
_SIGNATURES = {
    "gtg_embed": ("elementwise", [_I, _P, _P, _P, _I, _I, _I, _P]),
    "gtg_add_rmsnorm": ("elementwise", [_I, _P, _P, _P, _F, _P, _P, _I, _I, _P]),
    "gtg_swiglu": ("elementwise", [_I, _P, _P, _I, _I, _P]),
    "gtg_rope_table": ("elementwise", [_P, _P, _P, _I, _I, _P]),
    "gtg_rope_kv_store": ("elementwise", [_I, _P, _I, _P, _I, _I, _I, _I, _I, _P, _P, _L, _P, _I, _P, _P, _P, _I, _P]),
    "gtg_advance": ("elementwise", [_P, _P, _P, _P, _I, _P]),
    "gtg_check_cache_access": ("elementwise", [_I, _I, _P, _P, _P, _P, _P, _I, _P, _I, _I, _I, _P, _P]),
    "gtg_gemm_f32": ("gemm_f32", [_P, _I, _P, _I, _P, _I, _I, _I, _I, _P]),
    "gtg_gemm_bf16_mma": ("gemm_bf16_mma", [_P, _I, _P, _I, _P, _I, _I, _I, _I, _I, _P]),
    "gtg_gemm_bf16_skinny": ("gemm_bf16_skinny", [_P, _I, _P, _I, _P, _I, _I, _I, _I, _I, _I, _P]),
    "gtg_gemm_bf16_skinny_status": ("gemm_bf16_skinny", []),
    "gtg_gemm_bf16_skinny_test_hooks": ("gemm_bf16_skinny", [_I]),
    "gtg_gemm_bf16_tcgen05_test_hooks": ("gemm_bf16_tcgen05", [_I]),
    "gtg_gemm_bf16_swapab_test_hooks": ("gemm_bf16_swapab", [_I]),
    "gtg_attention_tcgen05_test_hooks": ("attention_tcgen05", [_I]),
    "gtg_gemm_bf16_tcgen05": ("gemm_bf16_tcgen05", [_P, _I, _P, _I, _P, _I, _I, _I, _I, _I, _I, _P]),
    "gtg_gemm_bf16_tcgen05_add": ("gemm_bf16_tcgen05", [_P, _I, _P, _I, _P, _I, _I, _I, _I, _P]),
    "gtg_gemm_bf16_tcgen05_status": ("gemm_bf16_tcgen05", []),
    "gtg_gemm_bf16_tcgen05_qkv_rope": ("gemm_bf16_tcgen05", [_P, _I, _P, _I, _P, _I, _I, _I, _P, _P, _P, _P, _P, _I,
                                                             _P, _P, _L, _I, _I, _P]),
    "gtg_gemm_bf16_swapab": ("gemm_bf16_swapab", [_P, _I, _P, _I, _P, _I, _I, _I, _I, _I, _I, _P, _P]),
    "gtg_gemm_bf16_swapab_scratch_floats": ("gemm_bf16_swapab", [_I, _I, _I]),
    "gtg_gemm_bf16_swapab_status": ("gemm_bf16_swapab", []),
    "gtg_attention_simple": ("attention_simple", [_I, _P, _I, _P, _I, _P, _P, _L, _P, _I, _P, _P, _P,
                                                  _I, _I, _I, _I, _F, _I, _P]),
    "gtg_attention_bf16_supports": ("attention_bf16", [_I]),
    "gtg_attention_decode_scratch_floats": ("attention_bf16", [_I, _I, _I, _I]),
    "gtg_attention_decode_plan": ("attention_bf16", [_I, _I, _I, _I, _I, _L, _I, _P, _P]),
    "gtg_attention_prefill_bf16": ("attention_bf16", [_P, _I, _P, _I, _P, _P, _L, _P, _I, _P, _P, _P,
                                                      _I, _I, _I, _I, _I, _F, _I, _P]),
    "gtg_attention_decode_rope_bf16": ("attention_bf16", [_P, _I, _P, _I, _P, _P, _L, _P, _I, _P, _P,
                                                          _I, _I, _I, _I, _F, _I, _I, _P, _P, _P, _P, _I, _I, _I, _P]),
    "gtg_attention_decode_bf16": ("attention_bf16", [_P, _I, _P, _I, _P, _P, _L, _P, _I, _P, _P,
                                                     _I, _I, _I, _I, _F, _I, _I, _P, _I, _I, _P]),
    "gtg_attention_tcgen05_supports": ("attention_tcgen05", [_I]),
    "gtg_attention_tcgen05_status": ("attention_tcgen05", []),
    "gtg_attention_prefill_tcgen05": ("attention_tcgen05", [_P, _I, _I, _P, _I, _P, _P, _L, _I, _P, _I, _P, _P, _P,
                                                            _I, _I, _I, _I, _I, _F, _I, _P]),
    "gtg_argmax": ("sampling", [_P, _I, _I, _I, _P, _P]),
    "gtg_sample_temperature": ("sampling", [_P, _I, _I, _I, _F, _U, _P, _P, _P, _P]),
}
_RESTYPES = {"gtg_attention_decode_scratch_floats": c_longlong,
             "gtg_gemm_bf16_swapab_scratch_floats": c_longlong}

_FUNCS = {}


class KernelError(RuntimeError):
    """A kernel refused its arguments or its launch failed."""


_chained = False


def _apply_chained(lib) -> None:
    setter = getattr(lib, "gtg_set_chained_launch", None)
    if setter is not None:
        setter.argtypes, setter.restype = [c_int], None
        setter(1 if _chained else 0)


class chained_launches:
    """Within this context the small kernels of a step are launched so that each
    may begin (up to the point where it needs its predecessor's results) while
    the one before it is still running -- programmatic dependent launch.  It is
    meant for decode steps, where launch and drain gaps are a large share of the
    time; the launches may be recorded into a CUDA graph."""

    def __init__(self, on: bool = True):
        self.on = bool(on)

    def __enter__(self):
        global _chained
        self.before = _chained
        _chained = self.on
        for lib in build._LOADED.values():
            _apply_chained(lib)
        return self

    def __exit__(self, *exc):
        global _chained
        _chained = self.before
        for lib in build._LOADED.values():
            _apply_chained(lib)


def _fn(symbol: str):
    f = _FUNCS.get(symbol)
    if f is None:
        lib_name, argtypes = _SIGNATURES[symbol]
        if not torch.cuda.is_available():
            raise KernelError(f"{symbol}: no CUDA device; this library runs on the GPU only "
                              f"and has no CPU path")
        lib = build.library(lib_name)
        _apply_chained(lib)
        f = getattr(lib, symbol)
        f.argtypes = argtypes
        f.restype = _RESTYPES.get(symbol, c_int)
        _FUNCS[symbol] = f
    return f


_CODES = {-1: "bad argument", -2: "size not supported by this kernel"}


_launches = 0


def launch_count() -> int:
    """How many kernel launchers of this library have been called so far (a
    launcher that is recorded into a CUDA graph counts once, when recorded)."""
    return _launches


def _check(code: int, what: str) -> None:
    global _launches
    _launches += 1
    if code != 0:
        if code in _CODES:
            raise KernelError(f"{what}: {_CODES[code]}")
        raise KernelError(f"{what}: CUDA error {code} (cudaError_t)")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current stream's handle.  Called once per launch: the direct binding
    costs a fraction of a microsecond, `torch.cuda.current_stream()` many."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return 0
    if t.dtype == torch.bfloat16:
        return 1
    raise KernelError(f"dtype {t.dtype} is not supported (float32 or bfloat16)")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


def _rows2d(t: torch.Tensor, name: str) -> None:
    _need(t.dim() == 2 and t.stride(1) == 1, f"{name} must be 2-D with a unit inner stride, "
                                             f"got shape {tuple(t.shape)} strides {t.stride()}")


# ------------------------------------------------- the debug pass over cache addresses
_checked = False
_ACCESS_FAULTS = {1: "a token names a sequence outside the batch", 2: "a sequence's slot is outside the cache",
                  3: "a position or a run of tokens is negative", 4: "a position lies beyond the block table's row",
                  5: "the block table names a page outside the cache"}


class checked_access:
    """Within this context every kernel that finds keys and values through the block
    table is preceded by a pass over the same indices (sequence -> slot -> table row
    -> page); the first index that would leave its array is reported as a
    `KernelError` and the kernel is not launched.  The stand-in for a memory
    checker: it costs a kernel and a synchronisation per call, so it is for
    debugging, not for serving, and a step under it is not recorded as a graph."""

    def __init__(self, on: bool = True):
        self.on = bool(on)

    def __enter__(self):
        global _checked
        self.before, _checked = _checked, self.on
        return self

    def __exit__(self, *exc):
        global _checked
        _checked = self.before


def _check_access(what: str, mode: int, kv, slots, positions=None, token_seq=None, start_pos=None,
                  cu_seqlens=None, n_items: Optional[int] = None) -> None:
    if not _checked or kv is None:
        return
    n_seqs = slots.numel()
    if n_items is None:
        n_items = n_seqs
    flag = torch.zeros(2, dtype=torch.int32, device=slots.device)
    code = _fn("gtg_check_cache_access")(mode, int(n_items), _ptr(token_seq), _ptr(slots), _ptr(positions),
                                         _ptr(start_pos), _ptr(cu_seqlens), n_seqs, _ptr(kv.block_table),
                                         kv.table_stride, kv.block_table.shape[0], kv.k.shape[0], _ptr(flag), _stream())
    if code != 0:
        raise KernelError(f"{what}: the access check could not run (code {code})")
    bad, item = flag.tolist()
    if bad:
        unit = "token" if mode == 0 else "sequence"
        raise KernelError(f"{what}: {_ACCESS_FAULTS.get(bad, bad)} ({unit} {item} of the step); the kernel was not launched")


# ------------------------------------------------------------------ elementwise
def embed(tokens: torch.Tensor, table: torch.Tensor, out: torch.Tensor) -> None:
    """out[n,:] (float32) = table[tokens[n],:]."""
    N, (V, H) = tokens.numel(), table.shape
    _need(tokens.dtype == torch.int32 and tokens.is_contiguous(), "embed: tokens must be contiguous int32")
    _need(table.is_contiguous() and out.is_contiguous() and out.dtype == torch.float32
          and tuple(out.shape) == (N, H), "embed: out must be contiguous float32 [N, H]")
    _check(_fn("gtg_embed")(_dt(table), _ptr(tokens), _ptr(table), _ptr(out), N, H, V, _stream()), "embed")


def add_rmsnorm(residual: torch.Tensor, pending: Optional[torch.Tensor], weight: torch.Tensor,
                eps: float, out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
    """residual (+= pending); out = rmsnorm(residual) * weight.  With `rows` only
    those rows are read (nothing is written back) and out has len(rows) rows."""
    H = residual.shape[1]
    R = rows.numel() if rows is not None else residual.shape[0]
    _need(residual.dtype == torch.float32 and residual.is_contiguous(), "add_rmsnorm: residual must be contiguous float32")
    _need(weight.dtype == torch.float32 and weight.is_contiguous() and weight.numel() == H,
          "add_rmsnorm: weight must be float32 [H]")
    _need(out.is_contiguous() and tuple(out.shape) == (R, H), "add_rmsnorm: out must be contiguous [rows, H]")
    if pending is not None:
        _need(pending.dtype == out.dtype and pending.is_contiguous() and pending.shape == residual.shape,
              "add_rmsnorm: pending must match the residual's shape and out's dtype")
    if rows is not None:
        _need(rows.dtype == torch.int32 and rows.is_contiguous(), "add_rmsnorm: rows must be contiguous int32")
    _check(_fn("gtg_add_rmsnorm")(_dt(out), _ptr(residual), _ptr(pending), _ptr(weight), float(eps),
                                  _ptr(out), _ptr(rows), R, H, _stream()), "add_rmsnorm")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[m,i] = silu(gate_up[m,i]) * gate_up[m,I+i]."""
    M, two_i = gate_up.shape
    _need(two_i % 2 == 0 and gate_up.is_contiguous() and out.is_contiguous()
          and tuple(out.shape) == (M, two_i // 2) and out.dtype == gate_up.dtype,
          "swiglu: gate_up [M, 2I] and out [M, I] must be contiguous and of one dtype")
    _check(_fn("gtg_swiglu")(_dt(out), _ptr(gate_up), _ptr(out), M, two_i // 2, _stream()), "swiglu")


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor, out: torch.Tensor) -> None:
    """out[n,i] = (cos, sin)(positions[n] * inv_freq[i]), angle and functions in float64."""
    N, half = positions.numel(), inv_freq.numel()
    _need(positions.dtype == torch.int32 and positions.is_contiguous(), "rope_table: positions must be int32")
    _need(inv_freq.dtype == torch.float64 and inv_freq.is_contiguous(), "rope_table: inv_freq must be float64")
    _need(out.dtype == torch.float32 and out.is_contiguous() and tuple(out.shape) == (N, half, 2),
          "rope_table: out must be float32 [N, half, 2]")
    _check(_fn("gtg_rope_table")(_ptr(positions), _ptr(inv_freq), _ptr(out), N, half, _stream()), "rope_table")


ROTARY_PAIRINGS = {"half": 0, "interleaved": 1}


def rope_kv_store(qkv: torch.Tensor, cos_sin: Optional[torch.Tensor], n_heads: int, n_kv_store: int,
                  head_dim: int, kv, token_seq: torch.Tensor, slots: torch.Tensor,
                  positions: torch.Tensor, pairing: str = "half", rotary_dim: Optional[int] = None) -> None:
    """Rotate the query heads of qkv in place; rotate the key heads and copy the
    value heads into the cache `kv` at each token's (slot, position).  With
    n_kv_store == 0 only queries are rotated and `kv` may be None.  `pairing`:
    "half" rotates channel i with i + rotary_dim/2, "interleaved" 2i with 2i+1;
    the first `rotary_dim` channels of a head rotate (default: all), the rest
    pass unchanged.  Any other layout is refused."""
    _rows2d(qkv, "rope_kv_store: qkv")
    N = qkv.shape[0]
    _need(head_dim % 2 == 0, "rope_kv_store: head_dim must be even")
    _need(pairing in ROTARY_PAIRINGS, f"rope_kv_store: pairing {pairing!r} is not supported; "
                                      f"supported: {sorted(ROTARY_PAIRINGS)}")
    rot = head_dim if rotary_dim is None else int(rotary_dim)
    _need(rot % 2 == 0 and 0 < rot <= head_dim,
          f"rope_kv_store: rotary_dim {rot} must be even and between 2 and head_dim {head_dim}")
    _need(qkv.shape[1] >= (n_heads + 2 * n_kv_store) * head_dim, "rope_kv_store: qkv is too narrow")
    if cos_sin is not None:
        _need(cos_sin.dtype == torch.float32 and cos_sin.is_contiguous()
              and tuple(cos_sin.shape) == (N, rot // 2, 2), "rope_kv_store: cos_sin must be float32 [N, rotary_dim/2, 2]")
    for name, t in (("token_seq", token_seq), ("slots", slots), ("positions", positions)):
        _need(t.dtype == torch.int32 and t.is_contiguous(), f"rope_kv_store: {name} must be contiguous int32")
    if n_kv_store > 0:
        _need(kv is not None and kv.k.dtype == qkv.dtype and kv.head_dim == head_dim
              and kv.n_kv_heads == n_kv_store, "rope_kv_store: cache entry does not match the heads to store")
        _check_access("rope_kv_store", 0, kv, slots, positions, token_seq, n_items=N)
        args = (_ptr(kv.k), _ptr(kv.v), kv.page_stride, _ptr(kv.block_table), kv.table_stride)
    else:
        args = (None, None, 0, None, 0)
    _check(_fn("gtg_rope_kv_store")(_dt(qkv), _ptr(qkv), qkv.stride(0), _ptr(cos_sin), n_heads, n_kv_store,
                                    head_dim, rot, ROTARY_PAIRINGS[pairing], *args, _ptr(token_seq), _ptr(slots), _ptr(positions),
                                    N, _stream()), "rope_kv_store")


def advance(tokens: torch.Tensor, positions: torch.Tensor, steps: torch.Tensor,
            sampled: torch.Tensor) -> None:
    """tokens <- sampled; positions += 1; steps += 1 (between decode steps that stay on the device)."""
    B = tokens.numel()
    for name, t in (("tokens", tokens), ("positions", positions), ("steps", steps), ("sampled", sampled)):
        _need(t.dtype == torch.int32 and t.is_contiguous() and t.numel() >= B, f"advance: {name} must be int32 [B]")
    _check(_fn("gtg_advance")(_ptr(tokens), _ptr(positions), _ptr(steps), _ptr(sampled), B, _stream()), "advance")


# ---------------------------------------------------------------- matrix products
SKINNY_MAX_ROWS = 128         # most rows the weight-streaming kernels take (beyond: the prompt-sized product)
STREAM_MAX_ROWS = 16          # up to here: warp-level MMA fed by bulk copies; beyond: tcgen05 with swapped operands
WARP_LEVEL_MAX_ROWS = 64      # most rows the warp-level kernel takes when asked for by name
TILED_KIND = "tcgen05"        # what "auto" uses beyond SKINNY_MAX_ROWS rows


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """The weight layout of the fused SwiGLU epilogue: rows in blocks of 8 gate
    features followed by the same 8 up features.  gate, up: [I, K] with I % 8 == 0."""
    i, k = gate.shape
    _need(up.shape == gate.shape and i % 8 == 0, "interleave_gate_up: equal shapes with a multiple of 8 rows")
    return torch.stack([gate.reshape(i // 8, 8, k), up.reshape(i // 8, 8, k)], dim=1).reshape(2 * i, k).contiguous()


def linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, kind: str = "auto",
           epilogue: str = "none") -> None:
    """out[M,N] = x[M,K] . w[N,K]^T.  float32 operands take the true 32-bit
    kernel; bfloat16 operands accumulate in float and write bfloat16 or float32.
    `kind` picks the bfloat16 kernel: "auto" (by the number of rows), "skinny"
    (weight streaming, up to 64 rows), "swapab" (weight streaming on tcgen05 with
    the tokens as the N dimension, up to 128 rows), "tcgen05" (TMA + tensor memory)
    or "tiled" (warp-level MMA).  epilogue="swiglu" (bfloat16, not "tiled"): w is laid out by
    `interleave_gate_up` and out[M, N/2] = silu(gate) * up, computed from the
    float accumulators."""
    _rows2d(x, "linear: x"); _rows2d(w, "linear: w"); _rows2d(out, "linear: out")
    M, K = x.shape
    N = w.shape[0]
    _need(epilogue in ("none", "swiglu"), f"linear: unknown epilogue {epilogue!r}")
    n_out = N // 2 if epilogue == "swiglu" else N
    _need(w.shape[1] == K and tuple(out.shape) == (M, n_out),
          f"linear: shapes {tuple(x.shape)} x {tuple(w.shape)} -> {tuple(out.shape)} (epilogue {epilogue})")
    if x.dtype == torch.float32:
        _need(epilogue == "none", "linear: the float32 product has no fused epilogue")
        _need(w.dtype == torch.float32 and out.dtype == torch.float32, "linear: float32 x needs float32 w and out")
        _check(_fn("gtg_gemm_f32")(_ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(out), out.stride(0),
                                   M, N, K, _stream()), "linear(float32)")
        return
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "linear: operands must both be bfloat16 or both float32")
    _need(out.dtype in (torch.bfloat16, torch.float32), "linear: out must be bfloat16 or float32")
    _need(K % 8 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0,
          f"linear(bfloat16): the inner size {K} and the row strides must be multiples of 8")
    # few rows (a decode step): stream the weights once; many rows: tiled product
    if kind == "auto":
        kind = "skinny" if M <= STREAM_MAX_ROWS else "swapab" if M <= SKINNY_MAX_ROWS else TILED_KIND
    symbol = {"skinny": "gtg_gemm_bf16_skinny", "tiled": "gtg_gemm_bf16_mma", "swapab": "gtg_gemm_bf16_swapab",
              "tcgen05": "gtg_gemm_bf16_tcgen05"}.get(kind)
    _need(symbol is not None, f"linear: unknown kind {kind!r}")
    if kind in ("skinny", "swapab"):
        most = WARP_LEVEL_MAX_ROWS if kind == "skinny" else SKINNY_MAX_ROWS
        _need(M <= most, f"linear: the weight-streaming kernel {kind!r} takes at most {most} rows")
    out_f32 = 1 if out.dtype == torch.float32 else 0
    if kind == "tiled":
        _need(epilogue == "none", "linear: the warp-level kernel has no fused epilogue")
        code = _fn(symbol)(_ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(out), out.stride(0),
                           out_f32, M, N, K, _stream())
    elif kind == "swapab":
        if epilogue == "swiglu":
            _need(N % 16 == 0, f"linear: the fused SwiGLU needs a multiple of 16 rows of w, got {N}")
        scratch = torch.empty(int(_fn("gtg_gemm_bf16_swapab_scratch_floats")(M, N, K)), dtype=torch.float32,
                              device=x.device)
        code = _fn(symbol)(_ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(out), out.stride(0),
                           out_f32, M, N, K, 1 if epilogue == "swiglu" else 0, _ptr(scratch), _stream())
    else:
        if epilogue == "swiglu":
            _need(N % 16 == 0, f"linear: the fused SwiGLU needs a multiple of 16 rows of w, got {N}")
        code = _fn(symbol)(_ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(out), out.stride(0),
                           out_f32, M, N, K, 1 if epilogue == "swiglu" else 0, _stream())
    _check(code, "linear(bfloat16)")


def linear_add_residual(x: torch.Tensor, w: torch.Tensor, residual: torch.Tensor) -> bool:
    """residual[M,N] += bfloat16(x[M,K] . w[N,K]^T): the product of a prompt step
    adds its result to a float32 residual stream in its epilogue (tensor reductions,
    each element once), rounded as it would be if it were stored first -- what
    `linear` into a bfloat16 update followed by the norm kernel's addition gives,
    without the update's trip through memory.  False, with nothing done, for
    operands the tensor-memory kernel does not take this way (few rows, float32
    operands, rows the tensor copies cannot address); the caller then uses `linear`."""
    if not (x.dim() == 2 and w.dim() == 2 and residual.dim() == 2):
        return False
    M, K = x.shape
    N = w.shape[0]
    if not (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and residual.dtype == torch.float32
            and M > SKINNY_MAX_ROWS and w.shape[1] == K and tuple(residual.shape) == (M, N)
            and x.stride(1) == 1 and w.stride(1) == 1 and residual.stride(1) == 1
            and K % 8 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and residual.stride(0) % 4 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and residual.data_ptr() % 16 == 0):
        return False
    code = _fn("gtg_gemm_bf16_tcgen05_add")(_ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(residual),
                                            residual.stride(0), M, N, K, _stream())
    if code == -2:
        return False
    _check(code, "linear_add_residual")
    return True


def qkv_rope_fused_supports(x: torch.Tensor, w: torch.Tensor, qkv: torch.Tensor, cos_sin, n_heads: int,
                            n_kv_heads: int, head_dim: int, kv) -> bool:
    """Whether `linear_qkv_rope` takes these operands: a prompt-sized bfloat16
    product (more rows than the weight-streaming kernels take), heads of 64
    channels, a rotation table, and operands the tensor copies can address."""
    return (cos_sin is not None and kv is not None and head_dim == 64 and x.shape[0] > SKINNY_MAX_ROWS
            and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and qkv.dtype == torch.bfloat16
            and kv.k.dtype == torch.bfloat16 and kv.head_dim == 64 and kv.n_kv_heads == n_kv_heads
            and w.shape[0] == (n_heads + 2 * n_kv_heads) * 64 and qkv.shape[1] == w.shape[0]
            and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and qkv.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and qkv.data_ptr() % 16 == 0
            and kv.page_stride % 8 == 0)


def linear_qkv_rope(x: torch.Tensor, w: torch.Tensor, qkv: torch.Tensor, cos_sin: torch.Tensor, n_heads: int,
                    n_kv_heads: int, kv, token_seq: torch.Tensor, slots: torch.Tensor,
                    positions: torch.Tensor) -> None:
    """The query/key/value projection of a prompt with rotation and cache store in
    its epilogue (heads of 64 channels): qkv[:, :n_heads*64] = rotated queries;
    rotated keys and the values go into `kv` at each token's (slot, position); the
    key and value columns of qkv are not written.  What `linear` followed by
    `rope_kv_store` computes, with the rotation applied to the float accumulators."""
    _rows2d(x, "linear_qkv_rope: x"); _rows2d(w, "linear_qkv_rope: w"); _rows2d(qkv, "linear_qkv_rope: qkv")
    _need(qkv_rope_fused_supports(x, w, qkv, cos_sin, n_heads, n_kv_heads, 64, kv),
          "linear_qkv_rope: operands not supported (see qkv_rope_fused_supports)")
    M, K = x.shape
    _need(w.shape[1] == K and qkv.shape[0] == M, "linear_qkv_rope: shapes do not agree")
    _need(cos_sin.dtype == torch.float32 and cos_sin.is_contiguous() and tuple(cos_sin.shape) == (M, 32, 2),
          "linear_qkv_rope: cos_sin must be float32 [M, 32, 2]")
    for name, t in (("token_seq", token_seq), ("slots", slots), ("positions", positions)):
        _need(t.dtype == torch.int32 and t.is_contiguous(), f"linear_qkv_rope: {name} must be contiguous int32")
    _check_access("linear_qkv_rope", 0, kv, slots, positions, token_seq, n_items=M)
    _check(_fn("gtg_gemm_bf16_tcgen05_qkv_rope")(
        _ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(qkv), qkv.stride(0), M, K, _ptr(cos_sin),
        _ptr(token_seq), _ptr(slots), _ptr(positions), _ptr(kv.block_table), kv.table_stride,
        _ptr(kv.k), _ptr(kv.v), kv.page_stride, n_heads, n_kv_heads, _stream()), "linear_qkv_rope")


def bounded_wait_failures() -> int:
    """Non-zero if a kernel ever gave up a bounded wait on its own asynchronous
    copies (it then returned without a result).  Reading it synchronises."""
    total = 0
    for symbol in ("gtg_gemm_bf16_skinny_status", "gtg_gemm_bf16_tcgen05_status", "gtg_gemm_bf16_swapab_status",
                   "gtg_attention_tcgen05_status"):
        if _SIGNATURES[symbol][0] in build._LOADED:        # only libraries that have run can have failed
            total += int(_fn(symbol)())
    return total


WAITING_LIBRARIES = ("gemm_bf16_skinny", "gemm_bf16_tcgen05", "gemm_bf16_swapab", "attention_tcgen05")


def wait_test_hooks(library: str, test_waits: bool) -> None:
    """For tests of the give-up path only.  While set, every launch of `library`
    (one of WAITING_LIBRARIES) takes the test form of its kernel: the same code
    compiled so that it issues none of its asynchronous copies -- the barriers it
    waits on then never complete -- and so that a wait polls a thousand times
    before it gives up.  A kernel launched so returns without a result and
    `bounded_wait_failures()` reads non-zero.  The call synchronises the device and
    clears the library's status word; False restores normal operation."""
    _need(library in WAITING_LIBRARIES, f"wait_test_hooks: {library!r} has no bounded waits; known: {WAITING_LIBRARIES}")
    code = int(_fn(f"gtg_{library}_test_hooks")(1 if test_waits else 0))
    if code != 0:
        raise KernelError(f"wait_test_hooks({library}): CUDA error {code}")


# ----------------------------------------------------------------------- attention
def attention_bf16_supports(head_dim: int) -> bool:
    return bool(_fn("gtg_attention_bf16_supports")(head_dim))


def attention_simple(q: torch.Tensor, out: torch.Tensor, kv, token_seq, slots, positions,
                     n_heads: int, scale: float, window: int = 0) -> None:
    """One warp per (token, head): the float32 path's attention, for prompts and
    decode steps alike."""
    _rows2d(q, "attention: q"); _rows2d(out, "attention: out")
    N = q.shape[0]
    _need(kv.k.dtype == q.dtype == out.dtype, "attention: q, out and the cache must share a dtype")
    _need(kv.head_dim <= 256, f"attention: head_dim {kv.head_dim} exceeds 256")
    _check_access("attention_simple", 0, kv, slots, positions, token_seq, n_items=N)
    _check(_fn("gtg_attention_simple")(_dt(q), _ptr(q), q.stride(0), _ptr(out), out.stride(0),
                                       _ptr(kv.k), _ptr(kv.v), kv.page_stride, _ptr(kv.block_table),
                                       kv.table_stride, _ptr(token_seq), _ptr(slots), _ptr(positions),
                                       N, n_heads, kv.n_kv_heads, kv.head_dim, float(scale), int(window),
                                       _stream()), "attention_simple")


def attention_prefill_bf16(q, out, kv, cu_seqlens, slots, start_pos, n_seqs: int, max_q_len: int,
                           n_heads: int, scale: float, window: int = 0) -> None:
    _rows2d(q, "attention: q"); _rows2d(out, "attention: out")
    _need(q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and kv.k.dtype == torch.bfloat16,
          "attention_prefill_bf16: bfloat16 only")
    _need(attention_bf16_supports(kv.head_dim),
          f"attention_prefill_bf16: head_dim {kv.head_dim} is not a multiple of 16 up to 128")
    _check_access("attention_prefill_bf16", 2, kv, slots, start_pos=start_pos, cu_seqlens=cu_seqlens, n_items=n_seqs)
    _check(_fn("gtg_attention_prefill_bf16")(_ptr(q), q.stride(0), _ptr(out), out.stride(0),
                                             _ptr(kv.k), _ptr(kv.v), kv.page_stride, _ptr(kv.block_table),
                                             kv.table_stride, _ptr(cu_seqlens), _ptr(slots), _ptr(start_pos),
                                             n_seqs, max_q_len, n_heads, kv.n_kv_heads, kv.head_dim,
                                             float(scale), int(window), _stream()), "attention_prefill_bf16")


def attention_tcgen05_supports(kv) -> bool:
    """The tensor-core prompt attention serves heads of 64 or 128 channels whose
    keys and values lie page by page as [k|v][head][token][channel]."""
    hd = kv.head_dim
    return (kv.k.dtype == torch.bfloat16 and hd in (64, 128)
            and kv.page_stride == 2 * kv.n_kv_heads * 64 * hd
            and kv.v.data_ptr() - kv.k.data_ptr() == kv.n_kv_heads * 64 * hd * 2)


def attention_prefill_tcgen05(q, out, kv, cu_seqlens, slots, start_pos, n_seqs: int, max_q_len: int,
                              n_heads: int, scale: float, window: int = 0) -> None:
    """Prompt attention on tcgen05 (128 queries x one head per thread block)."""
    _rows2d(q, "attention: q"); _rows2d(out, "attention: out")
    _need(q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16, "attention_prefill_tcgen05: bfloat16 only")
    _need(attention_tcgen05_supports(kv),
          "attention_prefill_tcgen05: needs head_dim 64 or 128 and keys and values of a page side by side")
    _check_access("attention_prefill_tcgen05", 2, kv, slots, start_pos=start_pos, cu_seqlens=cu_seqlens, n_items=n_seqs)
    _check(_fn("gtg_attention_prefill_tcgen05")(_ptr(q), q.stride(0), q.shape[0], _ptr(out), out.stride(0),
                                                _ptr(kv.k), _ptr(kv.v), kv.page_stride, kv.k.shape[0],
                                                _ptr(kv.block_table), kv.table_stride, _ptr(cu_seqlens),
                                                _ptr(slots), _ptr(start_pos), n_seqs, max_q_len, n_heads,
                                                kv.n_kv_heads, kv.head_dim, float(scale), int(window), _stream()),
           "attention_prefill_tcgen05")


def attention_decode_plan(n_seqs: int, n_heads: int, n_kv_heads: int, head_dim: int, max_kv_len: int,
                          window: int = 0, total_kv_len: int = 0):
    """(n_splits, chunk_pages, ring_pages) for `attention_decode_bf16`: into how
    many thread blocks the keys of the longest sequence's (sequence, key/value
    head) pairs are split, how many pages one split takes (a shorter sequence
    then takes as many splits as its own pages need), and which form of the
    kernel runs: the one with three pages in its ring and more blocks to an SM,
    or, for a batch that brings about one block per place on the device, the one
    with four.  `total_kv_len` is the batch's keys altogether (0: all sequences
    as long as the longest).  The library estimates, for every chunk size, the
    waves of blocks on this device (its multiprocessor count and the kernel's
    own occupancy, from the runtime) and the time the memory needs, and takes
    the least.  The choice depends on the batch's lengths and the window, never
    on the data."""
    chunk, ring = c_int(0), c_int(0)
    n = int(_fn("gtg_attention_decode_plan")(n_seqs, n_heads, n_kv_heads, head_dim, int(max_kv_len),
                                             int(total_kv_len), int(window), ctypes.byref(chunk), ctypes.byref(ring)))
    if n < 1:
        raise KernelError(f"attention_decode_plan: {_CODES.get(n, n)}")
    return n, int(chunk.value), int(ring.value)


def attention_decode_scratch_floats(n_seqs: int, n_heads: int, head_dim: int, n_splits: int) -> int:
    return int(_fn("gtg_attention_decode_scratch_floats")(n_seqs, n_heads, head_dim, n_splits))


def attention_decode_bf16(q, out, kv, slots, positions, n_heads: int, scale: float, window: int,
                          n_splits: int, scratch: Optional[torch.Tensor], unrotated=None,
                          chunk_pages: int = 0, ring_pages: int = 0) -> None:
    """Attention of one new token per sequence over the cache (keys split over
    `n_splits` thread blocks per head group).  Normally q is rotated and the new
    keys and values are in the cache (`rope_kv_store`).  With
    unrotated=(cos_sin, k_new, v_new, store) the kernel does that work itself: q
    and k_new come as the projection wrote them, cos_sin float32 [B, hd/2, 2] or
    None rotates them, and the new key and value are attended to and, if `store`,
    written to the cache; k_new None for a layer that reads another's cache.
    With `chunk_pages` (from `attention_decode_plan`; 0: every sequence is cut into
    n_splits equal parts) a sequence is cut into as many equal parts as give parts
    of about that many pages, at most n_splits: shorter sequences take fewer splits.
    Blocks start sequence by sequence in batch order: with very unequal lengths, put
    the long sequences first.  `ring_pages` (from the plan; 0: the default) picks
    the form of the kernel; the result does not depend on it."""
    _rows2d(q, "attention: q"); _rows2d(out, "attention: out")
    B = q.shape[0]
    _need(chunk_pages >= 0, "attention_decode_bf16: chunk_pages must not be negative")
    _need(q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and kv.k.dtype == torch.bfloat16,
          "attention_decode_bf16: bfloat16 only")
    _need(attention_bf16_supports(kv.head_dim),
          f"attention_decode_bf16: head_dim {kv.head_dim} is not a multiple of 16 up to 128")
    _check_access("attention_decode_bf16", 1, kv, slots, positions, n_items=B)
    if n_splits > 1:
        need = attention_decode_scratch_floats(B, n_heads, kv.head_dim, n_splits)
        _need(scratch is not None and scratch.dtype == torch.float32 and scratch.is_contiguous()
              and scratch.numel() >= need, f"attention_decode_bf16: scratch needs {need} floats")
    if unrotated is not None:
        cos_sin, k_new, v_new, store = unrotated
        hd = kv.head_dim
        if cos_sin is not None:
            _need(cos_sin.dtype == torch.float32 and cos_sin.is_contiguous() and tuple(cos_sin.shape) == (B, hd // 2, 2),
                  "attention_decode_bf16: cos_sin must be float32 [B, hd/2, 2]")
        if k_new is not None:
            for name, t in (("k_new", k_new), ("v_new", v_new)):
                _need(t is not None and t.dtype == torch.bfloat16 and t.dim() == 2 and t.stride(1) == 1
                      and t.stride(0) == q.stride(0) and tuple(t.shape) == (B, kv.n_kv_heads * hd),
                      f"attention_decode_bf16: {name} must be bfloat16 [B, n_kv * hd] with q's row stride")
        _check(_fn("gtg_attention_decode_rope_bf16")(
            _ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(kv.k), _ptr(kv.v), kv.page_stride,
            _ptr(kv.block_table), kv.table_stride, _ptr(slots), _ptr(positions), B, n_heads, kv.n_kv_heads,
            kv.head_dim, float(scale), int(window), int(n_splits), _ptr(scratch), _ptr(cos_sin),
            _ptr(k_new), _ptr(v_new) if k_new is not None else None, 1 if store else 0,
            int(chunk_pages), int(ring_pages), _stream()),
            "attention_decode_bf16")
        return
    _check(_fn("gtg_attention_decode_bf16")(_ptr(q), q.stride(0), _ptr(out), out.stride(0),
                                            _ptr(kv.k), _ptr(kv.v), kv.page_stride, _ptr(kv.block_table),
                                            kv.table_stride, _ptr(slots), _ptr(positions), B, n_heads,
                                            kv.n_kv_heads, kv.head_dim, float(scale), int(window),
                                            int(n_splits), _ptr(scratch), int(chunk_pages), int(ring_pages),
                                            _stream()),
           "attention_decode_bf16")


# ------------------------------------------------------------------------ sampling
def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] = first index of the maximum of logits[r,:]."""
    _rows2d(logits, "argmax: logits")
    R, V = logits.shape
    _need(logits.dtype == torch.float32 and out.dtype == torch.int32 and out.numel() >= R and out.is_contiguous(),
          "argmax: logits float32, out int32 [R]")
    _check(_fn("gtg_argmax")(_ptr(logits), logits.stride(0), R, V, _ptr(out), _stream()), "argmax")


def sample_temperature(logits: torch.Tensor, temperature: float, seed: int, sequence_ids: torch.Tensor,
                       steps: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] ~ softmax(logits[r,:] / temperature), drawn with the uniform that
    (seed, sequence_ids[r], steps[r]) determine."""
    _rows2d(logits, "sample: logits")
    R, V = logits.shape
    _need(temperature > 0, "sample_temperature: the temperature must be positive (0 means greedy: use argmax)")
    for name, t in (("sequence_ids", sequence_ids), ("steps", steps), ("out", out)):
        _need(t.dtype == torch.int32 and t.is_contiguous() and t.numel() >= R, f"sample: {name} must be int32 [R]")
    _check(_fn("gtg_sample_temperature")(_ptr(logits), logits.stride(0), R, V, float(temperature),
                                         int(seed) & (2**64 - 1), _ptr(sequence_ids), _ptr(steps),
                                         _ptr(out), _stream()), "sample_temperature")
