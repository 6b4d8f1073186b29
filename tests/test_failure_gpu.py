"""Failure detection on the device, without a fault: every wait of the kernels that
copy asynchronously (TMA, bulk copies) and compute on tensor memory is bounded.
Here the waits are made to run out -- a test hook makes a library launch the test
form of its kernels, the same code compiled to issue none of its copies, so that
the barriers it waits on never complete, and to poll a thousand times instead of
millions -- and the test checks what must follow:
the launch returns, the library's status word says that a wait gave up, the context
stays usable, tensor memory has been given back (the next launch of the same kernel
gets its columns and computes the right result), and the status reads zero again.
Nothing here traps, faults or spins without a limit."""
import math

import pytest
import torch

import go_tinygrad_b200  # noqa: F401
from go_tinygrad_b200.kernels import ops
from test_kernels_gpu import attention_case, rnd

pytestmark = pytest.mark.gpu
DEV = "cuda"
BF16 = torch.bfloat16


def product(kind, M, N, K):
    x, w = rnd(M, K, dtype=BF16, seed=1), rnd(N, K, dtype=BF16, seed=2, scale=0.5)
    want = (x.double() @ w.double().T).float().to(BF16).float()

    def run():
        out = torch.full((M, N), 7.0, dtype=BF16, device=DEV)
        ops.linear(x, w, out, kind=kind)
        return out.float()
    return run, want, dict(rtol=1.6e-2, atol=1e-2 * math.sqrt(K / 64))


def residual_product():
    M, N, K = 300, 256, 512
    x, w = rnd(M, K, dtype=BF16, seed=1), rnd(N, K, dtype=BF16, seed=2, scale=0.5)
    before = rnd(M, N, seed=3)
    want = before + (x.double() @ w.double().T).float().to(BF16).float()

    def run():
        residual = before.clone()
        assert ops.linear_add_residual(x, w, residual)
        return residual
    return run, want, dict(rtol=1.6e-2, atol=5e-2)


def prompt_attention():
    n_heads, n_kv, hd = 4, 2, 64
    cache, q, want, m, scale = attention_case(BF16, n_heads, n_kv, hd, [0, 70], [200, 60], 0)

    def run():
        out = torch.full_like(q, 7.0)
        ops.attention_prefill_tcgen05(q, out, cache.handles[0].kv, m["cu"], m["slots"], m["start"], 2, 200,
                                      n_heads, scale, 0)
        return out.float()
    return run, want, dict(rtol=2e-2, atol=2e-2)


CASES = {
    # library -> what runs its kernels: (how to build the case)
    "gemm_bf16_tcgen05": [lambda: product("tcgen05", 300, 520, 1024), residual_product],
    "gemm_bf16_swapab": [lambda: product("swapab", 40, 2048, 2048),      # clusters of eight slices
                         lambda: product("swapab", 64, 16384, 512)],     # one slice a tile, more CTAs than fit at once
    "gemm_bf16_skinny": [lambda: product("skinny", 4, 2048, 8192),       # a cluster of four ranks per row
                         lambda: product("skinny", 16, 6144, 2048),
                         lambda: product("skinny", 3, 50, 8200),         # an inner size that takes the row-copy kernel,
                         lambda: product("skinny", 5, 96, 264)],         # ... with a cluster of ranks and with one
    "attention_tcgen05": [prompt_attention],
}


@pytest.mark.parametrize("library", list(CASES))
def test_a_wait_that_runs_out_returns_and_says_so(library):
    for build in CASES[library]:
        run, want, close = build()
        torch.testing.assert_close(run(), want, **close)              # the case itself is sound
        assert ops.bounded_wait_failures() == 0
        try:
            ops.wait_test_hooks(library, True)
            run()                                                     # no copy arrives: every wait runs out
            torch.cuda.synchronize()                                  # ... and the kernel has returned, with no error
            assert ops.bounded_wait_failures() != 0, "the kernel did not report that its wait gave up"
        finally:
            ops.wait_test_hooks(library, False)
        assert ops.bounded_wait_failures() == 0                       # the word is clear again
        for _ in range(2):                                            # tensor memory and barriers are as good as new
            torch.testing.assert_close(run(), want, **close)
        assert ops.bounded_wait_failures() == 0


# ------------------------------------------------------------------ addresses checked before they are used
def test_a_bad_block_table_is_found_before_the_kernel_runs():
    """The debug pass that stands in for a memory checker: with `ops.checked_access`
    a kernel that reads the cache is preceded by a walk over the same indices on the
    device; a table entry, slot or position that would leave its array is reported
    and the kernel is not launched -- the bad access never happens."""
    n_heads, n_kv, hd = 4, 2, 64
    lens_before = [100, 63, 200]
    cache, q, want, m, scale = attention_case(BF16, n_heads, n_kv, hd, lens_before, [1, 1, 1], 0)
    kv = cache.handles[0].kv
    n_pages = kv.k.shape[0]

    def decode(slots=m["slots"], positions=m["positions"]):
        out = torch.full_like(q, 7.0)
        ops.attention_decode_bf16(q, out, kv, slots, positions, n_heads, scale, 0, 1, None)
        return out
    with ops.checked_access():
        torch.testing.assert_close(decode().float(), want, rtol=2e-2, atol=2e-2)       # sound as it is
        slot = int(m["slots"][2])
        good = int(kv.block_table[slot, 1])
        for bad_page in (n_pages + 3, -1):
            kv.block_table[slot, 1] = bad_page
            with pytest.raises(ops.KernelError, match="page outside the cache.*sequence 2.*not launched"):
                decode()
        kv.block_table[slot, 1] = good
        with pytest.raises(ops.KernelError, match="slot is outside the cache"):
            decode(slots=torch.tensor([0, 1, 99], dtype=torch.int32, device=DEV))
        with pytest.raises(ops.KernelError, match="beyond the block table"):
            decode(positions=torch.tensor([100, 63, 64 * kv.table_stride], dtype=torch.int32, device=DEV))
        with pytest.raises(ops.KernelError, match="negative"):
            decode(positions=torch.tensor([100, -5, 200], dtype=torch.int32, device=DEV))
        torch.testing.assert_close(decode().float(), want, rtol=2e-2, atol=2e-2)       # and sound again
    # prompt kernels and the per-token kernels take the same pass
    cache, q, want, m, scale = attention_case(BF16, n_heads, n_kv, hd, [10, 64], [70, 5], 0)
    kv = cache.handles[0].kv
    out = torch.full_like(q, 7.0)
    with ops.checked_access():
        ops.attention_prefill_tcgen05(q, out, kv, m["cu"], m["slots"], m["start"], 2, 70, n_heads, scale, 0)
        torch.testing.assert_close(out.float(), want, rtol=2e-2, atol=2e-2)
        slot = int(m["slots"][0])
        good = int(kv.block_table[slot, 0])
        kv.block_table[slot, 0] = kv.k.shape[0]
        for call in (lambda: ops.attention_prefill_tcgen05(q, out, kv, m["cu"], m["slots"], m["start"], 2, 70, n_heads, scale, 0),
                     lambda: ops.attention_prefill_bf16(q, out, kv, m["cu"], m["slots"], m["start"], 2, 70, n_heads, scale, 0),
                     lambda: ops.attention_simple(q, out, kv, m["token_seq"], m["slots"], m["positions"], n_heads, scale, 0)):
            with pytest.raises(ops.KernelError, match="page outside the cache"):
                call()
        kv.block_table[slot, 0] = good
    # outside the context nothing is checked and nothing synchronises; the engine turns it on per model
    assert not ops._checked


def test_the_engine_runs_under_access_checks(tmp_path):
    import go_tinygrad_b200 as lib
    from conftest import TINY, make_prompts
    folder = str(tmp_path / "m")
    lib.write_random_model(folder, TINY["A"], seed=2, dtype="bfloat16", std=0.12, norm_std=0.05)
    model = lib.Model.load(folder, dtype="bfloat16", device="cuda")
    prompts = make_prompts("A", [70, 5], seed=3)
    plain = [r.tokens for r in lib.generate(model, prompts, max_new_tokens=5, stop=[])]
    model.rt.check_access = True
    assert not model.capturable
    checked = [r.tokens for r in lib.generate(model, prompts, max_new_tokens=5, stop=[])]
    assert checked == plain
