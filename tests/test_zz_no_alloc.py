"""The allocation-free decode-attention entry point, called through its exported
C symbol, against the regular entry point that takes a scratch buffer from the
caller.  It is for users who cannot call cudaMalloc where their code runs (a
plugin inside someone else's allocator, a loop that must not allocate after
start-up): see csrc/attention_decode_static.h.  The file sorts last so that a
run that stops at the first failure has already run everything else."""
import ctypes
import math

import pytest
import torch

import go_tinygrad_b200  # noqa: F401
from go_tinygrad_b200.kernels import build, ops
from test_kernels_gpu import attention_case

pytestmark = pytest.mark.gpu
P, I, L, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float


def static_entry():
    lib = build.library("attention_decode_static")
    fn = lib.gtg_attention_decode_bf16_static
    fn.argtypes = [P, I, P, I, P, P, L, P, I, P, P, I, I, I, I, F, I, I, P]
    fn.restype = I
    cap = lib.gtg_static_scratch_capacity_floats
    cap.argtypes, cap.restype = [], L
    return fn, int(cap())


def call_static(fn, q, out, kv, slots, positions, n_heads, scale, window, splits):
    return fn(q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), kv.k.data_ptr(), kv.v.data_ptr(),
              kv.page_stride, kv.block_table.data_ptr(), kv.table_stride, slots.data_ptr(),
              positions.data_ptr(), q.shape[0], n_heads, kv.n_kv_heads, kv.head_dim, scale, window,
              splits, torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("n_heads,n_kv,hd,splits,window", [(8, 8, 64, 4, 0), (6, 2, 128, 3, 37), (3, 1, 48, 1, 0)])
def test_static_scratch_matches_the_regular_entry_point(n_heads, n_kv, hd, splits, window):
    fn, capacity = static_entry()
    assert capacity == 1 << 20
    lens_before = [0, 63, 64, 700, 129]
    cache, q, want, m, scale = attention_case(torch.bfloat16, n_heads, n_kv, hd, lens_before,
                                              [1] * len(lens_before), window)
    kv = cache.handles[0].kv
    regular = torch.empty_like(q)
    n = ops.attention_decode_scratch_floats(len(lens_before), n_heads, hd, splits)
    scratch = torch.empty(max(n, 1), dtype=torch.float32, device="cuda")
    ops.attention_decode_bf16(q, regular, kv, m["slots"], m["positions"], n_heads, scale, window, splits, scratch)
    torch.testing.assert_close(regular.float(), want, rtol=2e-2, atol=2e-2)
    outs = [torch.full_like(q, float("nan")) for _ in range(3)]
    # the first call on a device loads the module and looks up the array's address
    assert call_static(fn, q, outs[0], kv, m["slots"], m["positions"], n_heads, scale, window, splits) == 0
    torch.cuda.synchronize()
    # From here on nothing may be taken from the device: the driver's own count of free
    # bytes, which sees every cudaMalloc of the process whoever makes it (PyTorch's
    # counters see only PyTorch's allocator), stays where it is over the calls.
    free_before, _ = torch.cuda.mem_get_info()
    for out in outs[1:]:             # calls in a row share the array
        assert call_static(fn, q, out, kv, m["slots"], m["positions"], n_heads, scale, window, splits) == 0
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, f"the entry point took {free_before - free_after} bytes from the device"
    for call, out in enumerate(outs):
        assert torch.equal(out, regular), f"call {call}"
        torch.testing.assert_close(out.float(), want, rtol=2e-2, atol=2e-2)


def test_static_scratch_refuses_what_it_cannot_hold():
    fn, capacity = static_entry()
    n_heads, hd, splits = 32, 64, 16
    B = capacity // (n_heads * splits * (hd + 2)) + 1        # one sequence too many
    cache, q, want, m, scale = attention_case(torch.bfloat16, 2, 1, 16, [5], [1], 0)
    kv = cache.handles[0].kv
    out = torch.zeros(1, 16, dtype=torch.bfloat16, device="cuda")
    code = fn(q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), kv.k.data_ptr(), kv.v.data_ptr(),
              kv.page_stride, kv.block_table.data_ptr(), kv.table_stride, m["slots"].data_ptr(),
              m["positions"].data_ptr(), B, n_heads, n_heads, hd, scale, 0, splits,
              torch.cuda.current_stream().cuda_stream)
    assert code == -3
    torch.cuda.synchronize()
    assert float(out.abs().sum()) == 0.0
