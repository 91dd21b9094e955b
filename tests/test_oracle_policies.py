"""CPU tests of the oracle for the whole-row P scaling policies: the C++ restatement (oracle_policy_x) against a
numpy transcription of the formulas of the reference's accuracy study (fmha_i8_quant_deviation.py:38-43,57-121),
and the ordering of the three policies the study reports (README.md:192-198: per-row better than static better
than the worst case)."""
import numpy as np
import pytest


def _study_numpy(q8, k8, v8, amax5, which):
    """One head, no mask, float32 throughout, in the study's own order of operations."""
    qa, ka, va, oa, s_max = (np.float32(x) for x in amax5)
    D = q8.shape[1]
    i32_s = q8.astype(np.int32) @ k8.astype(np.int32).T
    f_s = (i32_s.astype(np.float32) * (qa / np.float32(127)) * (ka / np.float32(127))) / np.float32(np.sqrt(D))      # :57-58
    f_p = np.zeros_like(f_s)
    for r in range(f_s.shape[0]):                                                       # :63-68
        e = np.exp(f_s[r] - f_s[r].max())
        f_p[r] = e / e.sum(dtype=np.float32)
    if which == "row":
        p_amax = f_p.max(axis=1, keepdims=True)                                         # :108-112
    elif which == "static":
        p_amax = np.float32(s_max)                                                      # :86
    else:
        p_amax = np.float32(1.0)                                                        # :61
    p8 = np.clip(np.round(f_p * (np.float32(127) / p_amax)), 0, 127).astype(np.int32)   # :38-43
    f_o = (p8 @ v8.astype(np.int32)).astype(np.float32) * (p_amax / np.float32(127)) * (va / np.float32(127))   # :72,:98,:118
    return f_o, np.clip(np.round(f_o * (np.float32(127) / oa)), -127, 127).astype(np.int8)


@pytest.mark.parametrize("which,code", [("row", 1), ("static", 2), ("worst", 3)])
def test_policy_oracle_follows_the_study(oracle, wl, which, code):
    w = wl.Workload("t", 1, 1, 256, 64)
    q, k, v, m = wl.make_fp32_np(w, seed=31)
    q8, qa = wl.quantize_np(q)
    k8, ka = wl.quantize_np(k)
    v8, va = wl.quantize_np(v)
    o, p_abs_max = oracle.fp32_attention(q, k, v, m)
    amax5 = (qa, ka, va, float(np.abs(o).max()), float(p_abs_max))
    _, want = _study_numpy(q8[0, 0], k8[0, 0], v8[0, 0], amax5, which)
    got = oracle.policy(q8, k8, v8, m, amax5, code)[0, 0]
    d = np.abs(got.astype(np.int32) - want.astype(np.int32))
    # the two differ only in exp()/summation rounding (and the score scale order), visible at rounding ties
    assert d.max() <= 1 and (d == 0).mean() > 0.995, (int(d.max()), float((d == 0).mean()))


def test_policies_rank_as_in_the_study(oracle, wl):
    """Summed absolute error against the fp32 output (fmha_i8_quant_error_seqlen.py): per-row < static < worst case."""
    w = wl.Workload("t", 1, 2, 512, 64)
    q, k, v, m = wl.make_fp32_np(w, seed=32)
    q8, qa = wl.quantize_np(q)
    k8, ka = wl.quantize_np(k)
    v8, va = wl.quantize_np(v)
    o, p_abs_max = oracle.fp32_attention(q, k, v, m)
    oa = float(np.abs(o).max())
    amax5 = (qa, ka, va, oa, float(p_abs_max))
    err = {}
    for name, code in (("row", 1), ("static", 2), ("worst", 3)):
        o8 = oracle.policy(q8, k8, v8, m, amax5, code).astype(np.float32) * (oa / 127.0)
        err[name] = float(np.abs(o8 - o).sum())
    assert err["row"] < err["static"] < err["worst"], err


def test_policy_oracle_masks_and_row_sampling(oracle, wl):
    w = wl.Workload("t", 2, 2, 192, 64, valid_choices=(64, 128))
    q, k, v, m = wl.make_fp32_np(w, seed=33)
    q8, qa = wl.quantize_np(q)
    k8, ka = wl.quantize_np(k)
    v8, va = wl.quantize_np(v)
    o, p_abs_max = oracle.fp32_attention(q, k, v, m)
    amax5 = (qa, ka, va, float(np.abs(o).max()), float(p_abs_max))
    full = oracle.policy(q8, k8, v8, m, amax5, 1)
    rows = np.array([0, 5, 191, 192, 400, 767], np.int64)
    part = oracle.policy(q8, k8, v8, m, amax5, 1, rows=rows)
    assert np.array_equal(part, full.reshape(-1, 64)[rows])
    assert oracle.mean_rel_deviation(full, o, amax5[3]) < 20.0
