"""The reference project's own CUDA kernel, rebuilt unchanged for sm_100a (oracle/_ref/libref_gpu.so),
run beside the new kernel on the same inputs.  Skipped where that library was not built.  Only
shapes the reference launches with a thread count that matches its tile size are run (seq_len a
multiple of 128).

What these tests establish:
  * the WMMA register layouts on this GPU are the ones the reference's hand indexing assumes
    (inc/fmha_i8.cuh:183-196,239-253), dumped by a one-warp probe kernel;
  * a CPU emulation of the reference kernel AS WRITTEN (oracle_refkernel_emulate) reproduces the bytes
    the reference kernel really produces, within exp-approximation noise.  The emulation is the
    quantised CPU oracle (tier C) plus two switches: masked keys enter the tile maximum as int(-1e6)
    (:191-193), and the accumulator-to-A-operand relayout of P (:239-253) behaves as __shfl_sync
    really does -- every lane publishes the element ITS OWN lane id selects -- which drops keys 4-11
    of every block of 16 from P.V and counts keys 0-3 and 12-15 twice.  That pins the arithmetic the
    oracle shares with the emulation (scale order, rounding, tile merge, epilogue) to real reference
    output, and it shows why the reference kernel's output is far from its own fp32 golden on
    anything but near-uniform attention: the defect is in its source, not in the GPU it runs on;
  * the new kernel agrees with tier C (the emulation with both switches off) to +-1 LSB."""
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
    emu = oracle.refkernel_emulate(q8, k8, v8, m, amax, mask_minus_1e6=True, shuffle_as_written=True)
    intended = oracle.refkernel_emulate(q8, k8, v8, m, amax, mask_minus_1e6=True, shuffle_as_written=False)
    mx_o, f1_o, f0_o = parity_stats(ref, want)
    mx_e, f1_e, f0_e = parity_stats(ref, emu)
    mx_i, f1_i, f0_i = parity_stats(intended, want)
    print(f"B{B}H{H}S{S}D{D} {kind}: mean rel. deviation from fp32 golden: reference kernel {dev_ref:.2f} %, "
          f"new kernel {dev_new:.2f} %, oracle {dev_orc:.2f} %; reference kernel vs oracle max={mx_o} within1={f1_o:.4f}; "
          f"reference kernel vs its emulation max={mx_e} within1={f1_e:.5f} exact={f0_e:.5f}; "
          f"emulation with the intended relayout vs oracle max={mx_i} within1={f1_i:.5f}")
    assert dev_new < 20.0 and dev_orc < 20.0
    assert_parity(new, want, "new kernel vs oracle")
    # the pin: real reference output == the emulation of the kernel as written (same tolerance as everywhere)
    assert_parity(ref, emu, "reference kernel vs its CPU emulation")
    # and the emulation differs from tier C only through the two documented switches: with the relayout the
    # code intends, what is left is the masked-key treatment, which stays inside the tolerance on these inputs
    assert_parity(intended, want, "emulation (intended relayout) vs tier C")


def test_wmma_register_layout_is_the_one_the_reference_assumes(oracle):
    """One-warp probe (oracle/wmma_probe.cu): element (r, c) of a 16x16 matrix holds 16 r + c."""
    import torch
    if not oracle.ref_gpu_available():
        pytest.skip("oracle/_ref/libref_gpu.so not built")
    R = oracle.ref_gpu()
    if not hasattr(R, "wmma_layout_probe"):
        pytest.skip("oracle/_ref/libref_gpu.so was built without the probe")
    torch.cuda.set_device(0)
    acc = torch.full((32, 8), -7, dtype=torch.int32, device="cuda")
    a = torch.full((32, 8), -7, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    assert R.wmma_layout_probe(acc.data_ptr(), a.data_ptr()) == 0
    torch.cuda.synchronize()
    acc, a = acc.cpu().numpy(), a.cpu().numpy()
    want_acc = np.empty((32, 8), np.int32)
    want_a = np.empty((32, 8), np.int32)
    for lane in range(32):
        for tc_xi in range(2):
            for tc_yi in range(2):
                for e in range(2):      # inc/fmha_i8.cuh:183-196
                    want_acc[lane, tc_xi * 4 + tc_yi * 2 + e] = 16 * (lane // 4 + 8 * tc_yi) + 8 * tc_xi + 2 * (lane % 4) + e
        for tc_yi in range(2):
            for t in range(4):          # inc/fmha_i8.cuh:239-253
                want_a[lane, tc_yi * 4 + t] = 16 * (lane // 4 + 8 * tc_yi) + 4 * (lane % 4) + t
    print("accumulator fragment, lanes 0-3:", acc[:4].tolist())
    print("matrix_a fragment,    lanes 0-3:", a[:4].tolist())
    assert (acc == want_acc).all(), "accumulator layout differs from the one the reference indexes by"
    assert (a == want_a).all(), "matrix_a layout differs from the one the reference indexes by"
