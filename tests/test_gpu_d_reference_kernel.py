"""The reference project's own CUDA kernel, rebuilt unchanged for sm_100a (oracle/_ref/libref_gpu.so),
run beside the new kernel on the same inputs.  Skipped where that library was not built.  Only
shapes the reference launches with a thread count that matches its tile size are run (seq_len a
multiple of 128).

The reference kernel indexes WMMA accumulator fragments by a register layout that the WMMA API
leaves unspecified (inc/fmha_i8.cuh:183-196,239-253).  Where its output agrees with the quantised CPU
oracle to +-1 LSB it pins both the oracle and the new kernel; where it does not (the case on B200:
most of its int8 outputs are off by more than one step) it cannot serve as a pin, and the test only
requires that the oracle and the new kernel meet the reference's own acceptance criterion (mean
relative deviation from the fp32 golden < 20 %, inc/utils.hpp:59-89) on the very same inputs and are
no further from that golden than the reference kernel is."""
import ctypes

import numpy as np
import pytest

from _util import assert_parity, parity_stats

pytestmark = [pytest.mark.gpu, pytest.mark.timeout(600)]


def _reference_style(B, H, S, D, seed):
    """test_fmha_i8.cpp:74-89: Q,K ~ U(-.5,.5), V ~ |U(-.5,.5)|, mask ~ Bernoulli(0.2)."""
    rng = np.random.Generator(np.random.Philox(key=seed))
    mask = (rng.random((B, S)) < 0.2).astype(np.int8)
    q = (rng.random((B, H, S, D), dtype=np.float32) - np.float32(0.5)).astype(np.float32)
    k = (rng.random((B, H, S, D), dtype=np.float32) - np.float32(0.5)).astype(np.float32)
    v = np.abs(rng.random((B, H, S, D), dtype=np.float32) - np.float32(0.5)).astype(np.float32)
    return q, k, v, mask


@pytest.mark.parametrize("B,H,S,D,kind", [(1, 1, 128, 64, "reftest"), (1, 1, 512, 128, "reftest"), (2, 2, 256, 128, "normal"),
                                          (2, 3, 512, 64, "normal_valid"), (1, 2, 1024, 128, "normal_valid")])
def test_reference_kernel_beside_new_kernel(pkg, wl, oracle, B, H, S, D, kind):
    import torch
    if not oracle.ref_gpu_available():
        pytest.skip("oracle/_ref/libref_gpu.so not built")
    R = oracle.ref_gpu()
    assert R.ref_gpu_shape_ok(S, D) == 1
    torch.cuda.set_device(0)
    if kind == "reftest":
        q, k, v, m = _reference_style(B, H, S, D, seed=2023)
    else:
        w = wl.Workload("t", B, H, S, D, valid_choices=(S // 2, S - 64, S) if kind == "normal_valid" else None)
        q, k, v, m = wl.make_fp32_np(w, seed=S + D)
    q8, qa = wl.quantize_np(q)
    k8, ka = wl.quantize_np(k)
    v8, va = wl.quantize_np(v)
    o, _ = oracle.fp32_attention(q, k, v, m)
    oa = float(np.abs(o).max())
    amax = [qa, ka, va, oa]
    want = oracle.q128(q8, k8, v8, m, amax)

    tq, tk, tv, tm = (torch.from_numpy(x).cuda() for x in (q8, k8, v8, m))
    t_ref = torch.zeros_like(tq)
    a5 = (ctypes.c_float * 5)(*amax, 1.0)
    d4 = (ctypes.c_int * 4)(B, S, H, D)
    torch.cuda.synchronize()
    rc = R.ref_gpu_fmha(None, a5, d4, tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), tm.data_ptr(), t_ref.data_ptr())
    torch.cuda.synchronize()
    assert rc == 0
    ref = t_ref.cpu().numpy()

    t_new = torch.zeros_like(tq)
    pkg.FMHAInferI8(None, pkg.FMHAParamI8(*amax, 1.0), pkg.AttnDataDescriptor(B, S, H, D), tq, tk, tv, tm, t_new, True)
    st, words = pkg.device_status()
    assert st == pkg.OK, words
    new = t_new.cpu().numpy()

    dev_ref = oracle.mean_rel_deviation(ref, o, oa)
    dev_new = oracle.mean_rel_deviation(new, o, oa)
    dev_orc = oracle.mean_rel_deviation(want, o, oa)
    mx_o, f1_o, f0_o = parity_stats(ref, want)
    print(f"B{B}H{H}S{S}D{D} {kind}: mean rel. deviation from fp32 golden: reference kernel {dev_ref:.2f} %, "
          f"new kernel {dev_new:.2f} %, oracle {dev_orc:.2f} %; reference kernel vs oracle max={mx_o} within1={f1_o:.4f}")
    assert dev_new < 20.0 and dev_orc < 20.0
    assert_parity(new, want, "new kernel vs oracle")
    if f1_o >= 0.999 and mx_o <= 2:
        # the reference kernel is right on this GPU: it pins the oracle and the new kernel
        assert_parity(new, ref, "new kernel vs reference kernel")
    else:
        # Observed on B200: the rebuilt reference kernel is far from its own fp32 golden element by
        # element (it indexes WMMA fragments by an unspecified register layout), so it cannot pin
        # anything.  The new kernel must then at least be no further from the golden than it is.
        assert dev_new <= dev_ref
