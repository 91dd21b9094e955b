"""Generates tests/golden/*.npz from the REFERENCE project's own CPU code.

Runs only where oracle/_ref/libref_cpu.so exists (built by oracle/Makefile from a checkout of
jundaf2/INT8-Flash-Attention-FMHA-Quantization); the resulting files are committed so the tests
can run without the reference.  Every array named ref_* below is an output of unmodified
reference code:
    ref_q8/k8/v8  float_quant2_int8 (inc/utils.hpp:23-29) with amax from abs_max (:31-39)
    ref_s_int32   cpuGEMM<int32_t,int32_t,int8_t,int32_t> on the int8 Q,K (inc/cpuGEMM.hpp:8-31)
    ref_o_fp32    cpuGEMM<float> -> cpuAttentionMaskedSoftmax<float,float> -> cpuGEMM<float>,
                  called as in test_fmha_i8.cpp:142-159;  ref_s_max = abs_max(P) (:152)
    ref_dev_pct   compareResultsWithGoldenI8 (inc/utils.hpp:59-89) applied to the int8 array
                  `probe_o8` against ref_o_fp32
The file cross_b1h2q96k192d64.npz holds the same reference outputs for a problem with 96 query rows
against 192 keys (the reference CPU templates take both lengths; its test never uses that).
`oracle_o8` is NOT a reference output: it is the tier-C restatement's result at generation time,
kept to notice drift of the restatement.

    python tests/golden/make_golden.py            # every fixture
    python tests/golden/make_golden.py cross      # only the Sq != Sk fixture
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import __graft_entry__ as ge  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def reference_style_inputs(B, H, S, D, seed):
    """Value distributions of the reference test (test_fmha_i8.cpp:74-89): Q,K ~ U(-.5,.5),
    V ~ |U(-.5,.5)|, mask ~ Bernoulli(0.2)."""
    rng = np.random.Generator(np.random.Philox(key=seed))
    mask = (rng.random((B, S)) < 0.2).astype(np.int8)
    q = (rng.random((B, H, S, D), dtype=np.float32) - np.float32(0.5)).astype(np.float32)
    k = (rng.random((B, H, S, D), dtype=np.float32) - np.float32(0.5)).astype(np.float32)
    v = np.abs(rng.random((B, H, S, D), dtype=np.float32) - np.float32(0.5)).astype(np.float32)
    return q, k, v, mask


def main():
    oracle = ge.load_oracle()
    oracle.build()
    assert oracle.ref_cpu_available(), "oracle/_ref/libref_cpu.so missing: run `make -C oracle` with the reference present"
    ge.load_package()
    import importlib
    wl = importlib.import_module("int8_fmha_b200.workloads")
    R = oracle.ref_cpu()

    cases = {}
    # C1 of the benchmark list: plumbing shape, no padding
    cases["c1_b1h2s64d64"] = wl.make_fp32_np(wl.CONFIGS["C1"], seed=2023)
    # the reference test's own distributions, random 20 % key mask, ragged S (64-wide last tile)
    cases["reftest_b1h2s192d64"] = reference_style_inputs(1, 2, 192, 64, seed=2023)
    # head_dim 128, valid-length padding ending inside a tile
    w = wl.Workload("g3", 2, 1, 128, 128, valid_choices=(64, 128))
    q, k, v, _ = wl.make_fp32_np(w, seed=11)
    cases["valid_b2h1s128d128"] = (q, k, v, wl.mask_from_valid(np.array([64, 128]), 128))
    # one key tile entirely masked in the middle, random mask elsewhere
    q, k, v, mask = reference_style_inputs(1, 1, 320, 64, seed=77)
    mask[:, 128:256] = 1
    cases["hole_b1h1s320d64"] = (q, k, v, mask)

    make_cross(oracle, R)
    if "cross" in sys.argv[1:]:
        return
    for name, (q, k, v, mask) in cases.items():
        B, H, S, D = q.shape
        qa = float(R.ref_abs_max(q.ravel(), q.size))
        ka = float(R.ref_abs_max(k.ravel(), k.size))
        va = float(R.ref_abs_max(v.ravel(), v.size))
        q8 = np.empty(q.shape, np.int8); R.ref_quantize(q.ravel(), q.size, qa, q8.ravel())
        k8 = np.empty(k.shape, np.int8); R.ref_quantize(k.ravel(), k.size, ka, k8.ravel())
        v8 = np.empty(v.shape, np.int8); R.ref_quantize(v.ravel(), v.size, va, v8.ravel())
        s32 = np.empty((B, H, S, S), np.int32)
        R.ref_qk_int32(q8.ravel(), k8.ravel(), B * H, S, D, s32.ravel())
        o, s_max = oracle.ref_fp32_attention(q, k, v, mask, batched=True)
        oa = float(R.ref_abs_max(o.ravel(), o.size))
        o8 = oracle.q128(q8, k8, v8, mask, (qa, ka, va, oa))
        probe = np.clip(np.rint(o * (127.0 / oa)), -127, 127).astype(np.int8)
        dev = float(R.ref_mean_rel_deviation(probe.ravel(), o.ravel(), o.size, oa))
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, q=q, k=k, v=v, mask=mask, ref_q8=q8, ref_k8=k8, ref_v8=v8,
                            ref_amax=np.array([qa, ka, va, oa], np.float32), ref_s_max=np.float32(s_max),
                            ref_s_int32=s32, ref_o_fp32=o, probe_o8=probe, ref_dev_pct=np.float64(dev),
                            oracle_o8=o8)
        print(f"{name}: B{B} H{H} S{S} D{D} amax=({qa:.4f},{ka:.4f},{va:.4f},{oa:.4f}) s_max={s_max:.4f} "
              f"ref_dev={dev:.4f}% -> {os.path.getsize(path)} bytes")


def make_cross(oracle, R):
    """96 query rows against 192 keys, the reference test's value distributions, random 20 % key mask."""
    B, H, Sq, Sk, D = 1, 2, 96, 192, 64
    rng = np.random.Generator(np.random.Philox(key=424242))
    mask = (rng.random((B, Sk)) < 0.2).astype(np.int8)
    q = (rng.random((B, H, Sq, D), dtype=np.float32) - np.float32(0.5)).astype(np.float32)
    k = (rng.random((B, H, Sk, D), dtype=np.float32) - np.float32(0.5)).astype(np.float32)
    v = np.abs(rng.random((B, H, Sk, D), dtype=np.float32) - np.float32(0.5)).astype(np.float32)
    qa = float(R.ref_abs_max(q.ravel(), q.size))
    ka = float(R.ref_abs_max(k.ravel(), k.size))
    va = float(R.ref_abs_max(v.ravel(), v.size))
    q8 = np.empty(q.shape, np.int8); R.ref_quantize(q.ravel(), q.size, qa, q8.ravel())
    k8 = np.empty(k.shape, np.int8); R.ref_quantize(k.ravel(), k.size, ka, k8.ravel())
    v8 = np.empty(v.shape, np.int8); R.ref_quantize(v.ravel(), v.size, va, v8.ravel())
    s32 = np.empty((B, H, Sq, Sk), np.int32)
    R.ref_qk_int32_cross(q8.ravel(), k8.ravel(), B * H, Sq, Sk, D, s32.ravel())
    o = oracle.ref_fp32_attention_cross(q, k, v, mask)
    oa = float(R.ref_abs_max(o.ravel(), o.size))
    o8 = oracle.q128(q8, k8, v8, mask, (qa, ka, va, oa))
    o8u = oracle.q128(q8, k8, v8, mask, (qa, ka, va, oa), p_levels=255)
    path = os.path.join(HERE, "cross_b1h2q96k192d64.npz")
    np.savez_compressed(path, q=q, k=k, v=v, mask=mask, ref_q8=q8, ref_k8=k8, ref_v8=v8,
                        ref_amax=np.array([qa, ka, va, oa], np.float32), ref_s_int32=s32, ref_o_fp32=o,
                        oracle_o8=o8, oracle_o8_uint8p=o8u)
    print(f"cross: B{B} H{H} Sq{Sq} Sk{Sk} D{D} amax=({qa:.4f},{ka:.4f},{va:.4f},{oa:.4f}) -> {os.path.getsize(path)} bytes")


if __name__ == "__main__":
    main()
