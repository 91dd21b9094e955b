"""GPU test of fmha_i8_sm100_quantize_f32_noalloc, the quantisation entry point for hosts that cannot
let a library allocate device memory (their own pool owns the whole GPU, or their loop cannot take the
device-wide synchronisation an allocation implies).  It must give bit-for-bit the result of
fmha_i8_sm100_quantize_f32 -- same kernels, only the scratch lives in the library's device image --
on two calls in a row that share that scratch, the second smaller than the first so that stale
partial maxima of the first call would show if they were ever read.

This file sorts last on purpose: a run that stops at the first failure has then already run every
other test."""
import ctypes

import numpy as np
import pytest

pytestmark = [pytest.mark.gpu, pytest.mark.timeout(300)]

NOALLOC = "fmha_i8_sm100_quantize_f32_noalloc"
MAX_ELEMENTS = 4096 * 65536


def _quantize(pkg, torch, tx, entry):
    out = torch.full((tx.numel() + 64,), 0x5A, dtype=torch.int8, device="cuda")
    amax = torch.zeros(1, dtype=torch.float32, device="cuda")
    pkg.quantize_f32(None, tx, out, amax, n=tx.numel(), entry=entry)
    torch.cuda.synchronize()
    assert bool((out[tx.numel():] == 0x5A).all()), "wrote past the end of the output"
    return out[:tx.numel()].clone(), float(amax.item())


def test_noalloc_matches_allocating_entry_twice_in_a_row(pkg):
    import torch
    torch.cuda.set_device(0)
    g = torch.Generator(device="cuda")
    g.manual_seed(99)
    big = torch.randn(5 * 65536 + 1234, generator=g, device="cuda", dtype=torch.float32) * 40.0   # 6 chunks, large amax
    small = torch.randn(65536 + 77, generator=g, device="cuda", dtype=torch.float32) * 0.01       # 2 chunks, tiny amax
    want_big = _quantize(pkg, torch, big, "fmha_i8_sm100_quantize_f32")
    want_small = _quantize(pkg, torch, small, "fmha_i8_sm100_quantize_f32")
    got_big = _quantize(pkg, torch, big, NOALLOC)          # first call: also looks up the scratch address
    got_small = _quantize(pkg, torch, small, NOALLOC)      # second call shares the scratch the first one filled
    for got, want in ((got_big, want_big), (got_small, want_small)):
        assert got[1] == want[1]                           # amax, bit for bit
        assert torch.equal(got[0], want[0])                # int8 output, bit for bit
    st, words = pkg.device_status()
    assert st == pkg.OK, words


def test_noalloc_leaves_free_device_memory_unchanged(pkg):
    """The property the entry point exists for: after its one-time set-up, calls of several sizes change the
    amount of free device memory by nothing (cudaMemGetInfo before and after, inputs and outputs allocated up
    front), while the allocating entry point may grow its scratch."""
    import torch
    torch.cuda.set_device(0)
    sizes = [65536 + 5, 9 * 65536, 3 * 65536 + 1, 40 * 65536]
    xs = [torch.randn(n, device="cuda", dtype=torch.float32) for n in sizes]
    outs = [torch.empty(n, dtype=torch.int8, device="cuda") for n in sizes]
    amax = torch.zeros(1, dtype=torch.float32, device="cuda")
    pkg.quantize_f32(None, xs[0], outs[0], amax, n=sizes[0], entry=NOALLOC)      # warm call: set-up happens here
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for rep in range(3):
        for x, o, n in zip(xs, outs, sizes):
            pkg.quantize_f32(None, x, o, amax, n=n, entry=NOALLOC)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, f"free device memory changed by {free_before - free_after} bytes"
    # the results are still right
    for x, o, n in zip(xs, outs, sizes):
        want = torch.empty_like(o)
        pkg.quantize_f32(None, x, want, amax, n=n, entry="fmha_i8_sm100_quantize_f32")
        torch.cuda.synchronize()
        assert torch.equal(o, want)


def test_noalloc_size_limit_is_exact(pkg):
    """n == the maximum passes the size check (the call then fails on its NULL input, before any launch);
    n == maximum + 1 is refused as too large whatever the other arguments are."""
    import torch
    torch.cuda.set_device(0)
    o = torch.zeros(64, dtype=torch.int8, device="cuda")
    L = pkg.lib()
    vp = ctypes.c_void_p
    fn = getattr(L, NOALLOC)
    assert fn(None, None, MAX_ELEMENTS, vp(o.data_ptr()), None) == pkg.ERR_NULL_POINTER
    x = torch.zeros(64, dtype=torch.float32, device="cuda")
    assert fn(None, vp(x.data_ptr() + 4), MAX_ELEMENTS, vp(o.data_ptr()), None) == pkg.ERR_MISALIGNED
    assert fn(None, vp(x.data_ptr()), MAX_ELEMENTS + 1, vp(o.data_ptr()), None) == pkg.ERR_TOO_LARGE


def test_noalloc_refuses_sizes_beyond_its_scratch(pkg):
    import torch
    torch.cuda.set_device(0)
    x = torch.zeros(64, dtype=torch.float32, device="cuda")
    o = torch.zeros(64, dtype=torch.int8, device="cuda")
    L = pkg.lib()
    vp = ctypes.c_void_p
    fn = getattr(L, NOALLOC)
    assert fn(None, vp(x.data_ptr()), MAX_ELEMENTS + 1, vp(o.data_ptr()), None) == pkg.ERR_TOO_LARGE   # refused before any launch
    assert fn(None, None, 64, vp(o.data_ptr()), None) == pkg.ERR_NULL_POINTER
    assert "maximum" in pkg.status_string(pkg.ERR_TOO_LARGE)
