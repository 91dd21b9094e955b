"""GPU test of the failure-reporting path: a device-side wait that runs out must surface as a status the
host can read, leave the context usable, and be reported ONCE by the next forward call that can see it (the
kernels themselves never look at the status words, so one failure cannot switch the library off).  The wait that
runs out belongs to a one-warp debug kernel waiting on a barrier nothing arrives on, with a limit of about two
milliseconds: no fault, no trap, no unbounded spin."""
import numpy as np
import pytest

pytestmark = [pytest.mark.gpu, pytest.mark.timeout(300)]

DEV_WAIT_DEBUG = 10


def test_wait_that_runs_out_is_reported_and_the_context_survives(pkg, wl, oracle):
    import torch
    torch.cuda.set_device(0)
    st, words = pkg.device_status()
    assert st == pkg.OK, words

    # a small forward problem, result known
    B, H, S, D = 1, 2, 128, 64
    w = wl.Workload("t", B, H, S, D)
    q, k, v, m = wl.make_fp32_np(w, 5)
    q8, qa = wl.quantize_np(q)
    k8, ka = wl.quantize_np(k)
    v8, va = wl.quantize_np(v)
    o, _ = oracle.fp32_attention(q, k, v, m)
    amax = [qa, ka, va, float(np.abs(o).max())]
    want = oracle.q128(q8, k8, v8, m, amax)
    tq, tk, tv, tm = (torch.from_numpy(x).cuda() for x in (q8, k8, v8, m))
    prm, desc = pkg.FMHAParamI8(*amax, 1.0), pkg.AttnDataDescriptor(B, S, H, D)

    pkg.debug_wait_probe(None, 4_000_000)                 # about two milliseconds of SM cycles
    # a forward pass enqueued behind it, before the failure is visible on the host, runs normally
    to = torch.full_like(tq, 0x5A)
    pkg.FMHAInferI8(None, prm, desc, tq, tk, tv, tm, to, True)
    torch.cuda.synchronize()
    d = np.abs(to.cpu().numpy().astype(np.int32) - want.astype(np.int32))
    assert d.max() <= 1, "a forward pass behind a failed kernel must still compute"

    # by now the kernel has written the host-visible word: the next call reports the failure once, without launching
    to2 = torch.full_like(tq, 0x5A)
    L = pkg.lib()
    before = pkg.launch_count()
    pkg.FMHAInferI8(None, prm, desc, tq, tk, tv, tm, to2, True, check=False)
    assert L.fmha_i8_sm100_last_status() == pkg.ERR_DEVICE
    assert pkg.launch_count() == before
    torch.cuda.synchronize()
    assert bool((to2 == 0x5A).all())
    assert "wait" in pkg.status_string(pkg.ERR_DEVICE)
    # ... once: the call after that runs
    pkg.FMHAInferI8(None, prm, desc, tq, tk, tv, tm, to2, True)
    torch.cuda.synchronize()
    d = np.abs(to2.cpu().numpy().astype(np.int32) - want.astype(np.int32))
    assert d.max() <= 1

    # the details stay in the status words until they are read
    st, words = pkg.device_status()
    assert st == pkg.ERR_DEVICE
    assert words[0] == DEV_WAIT_DEBUG and words[1] == 0 and words[2] == 0 and words[3] == 4, words
    st, words = pkg.device_status()
    assert st == pkg.OK and words[0] == 0
    pkg.FMHAInferI8(None, prm, desc, tq, tk, tv, tm, to, True)
    st, words = pkg.device_status()
    assert st == pkg.OK, words


def test_probe_limit_is_checked_on_the_host(pkg):
    L = pkg.lib()
    assert L.fmha_i8_sm100_debug_wait_probe(None, 10) == pkg.ERR_TOO_LARGE
    assert L.fmha_i8_sm100_debug_wait_probe(None, 10**12) == pkg.ERR_TOO_LARGE
