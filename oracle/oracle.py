"""ctypes doors onto the CPU oracle (liboracle.so) and, when built, the reference's own code
(oracle/_ref/*.so).  TEST INFRASTRUCTURE ONLY -- the product package never imports this module.

Tiers (reference citations are file:line in jundaf2/INT8-Flash-Attention-FMHA-Quantization):
  fp32_attention   tier A, test_fmha_i8.cpp:142-159 (inc/cpuGEMM.hpp:8-31, inc/cpuSoftmax.hpp:11-51)
  qk_int32         tier B, the same GEMM on int8 -> int32
  q128             tier C, the device kernel's arithmetic, inc/fmha_i8.cuh:71-72,183-253,298-332
  quantize/abs_max inc/utils.hpp:23-39 ; mean_rel_deviation inc/utils.hpp:59-89
"""
import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
_c = ctypes
_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_i8p = np.ctypeslib.ndpointer(np.int8, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")


def reference_checkout():
    """Directory of a checkout of the reference project, or None.  Taken from the environment variable
    FMHA_REFERENCE_DIR, else from a directory named `reference` beside this repository."""
    cands = [os.environ.get("FMHA_REFERENCE_DIR"), os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")]
    for c in cands:
        if c and os.path.exists(os.path.join(c, "inc", "cpuGEMM.hpp")):
            return c
    return None


def build(force=False):
    """Compile liboracle.so (and oracle/_ref when a reference checkout is present)."""
    lib = os.path.join(HERE, "liboracle.so")
    if force or not os.path.exists(lib) or os.path.getmtime(lib) < os.path.getmtime(os.path.join(HERE, "oracle.cpp")):
        subprocess.check_call(["make", "-s", "-C", HERE, os.path.join(HERE, "liboracle.so")])
    ref = reference_checkout()
    if ref:
        subprocess.call(["make", "-s", "-C", HERE, "ref", "REF=" + ref])
    return lib


_lib = None


def lib():
    global _lib
    if _lib is None:
        path = os.path.join(HERE, "liboracle.so")
        if not os.path.exists(path):
            build()
        L = ctypes.CDLL(path)
        L.oracle_abs_max.restype = _c.c_float
        L.oracle_abs_max.argtypes = [_f32p, _c.c_int64]
        L.oracle_quantize.argtypes = [_f32p, _c.c_int64, _c.c_float, _i8p]
        L.oracle_mean_rel_deviation.restype = _c.c_double
        L.oracle_mean_rel_deviation.argtypes = [_i8p, _f32p, _c.c_int64, _c.c_float]
        L.oracle_qk_int32.argtypes = [_i8p, _i8p, _c.c_int, _c.c_int, _c.c_int, _i32p, _c.c_int]
        L.oracle_fp32_attention.argtypes = [_f32p, _f32p, _f32p, _i8p, _c.c_int, _c.c_int, _c.c_int, _c.c_int,
                                            _f32p, _c.POINTER(_c.c_float), _c.c_int]
        L.oracle_q128.argtypes = [_i8p, _i8p, _i8p, _i8p, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _f32p,
                                  _c.c_void_p, _c.c_int64, _i8p, _c.c_int]
        L.oracle_fp32_attention_x.argtypes = [_f32p, _f32p, _f32p, _i8p, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_int,
                                              _f32p, _c.POINTER(_c.c_float), _c.c_int]
        L.oracle_q128_x.argtypes = [_i8p, _i8p, _i8p, _i8p, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _f32p,
                                    _c.c_int, _c.c_void_p, _c.c_int64, _i8p, _c.c_int]
        L.oracle_policy_x.argtypes = [_i8p, _i8p, _i8p, _i8p, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _f32p,
                                      _c.c_int, _c.c_void_p, _c.c_int64, _i8p, _c.c_int]
        L.oracle_refkernel_emulate.argtypes = [_i8p, _i8p, _i8p, _i8p, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _f32p,
                                               _c.c_int, _c.c_int, _i8p, _c.c_int]
        L.oracle_row_scale.restype = _c.c_float
        L.oracle_row_scale.argtypes = [_c.c_int]
        _lib = L
    return _lib


def n_threads_default():
    return max(1, len(os.sched_getaffinity(0)))


def abs_max(x):
    x = np.ascontiguousarray(x, np.float32).ravel()
    return float(lib().oracle_abs_max(x, x.size))


def quantize(x, amax):
    x = np.ascontiguousarray(x, np.float32)
    out = np.empty(x.shape, np.int8)
    lib().oracle_quantize(x.ravel(), x.size, amax, out.ravel())
    return out


def mean_rel_deviation(o8, o_ref, o_amax):
    o8 = np.ascontiguousarray(o8, np.int8).ravel()
    o_ref = np.ascontiguousarray(o_ref, np.float32).ravel()
    return float(lib().oracle_mean_rel_deviation(o8, o_ref, o8.size, o_amax))


def qk_int32(q8, k8, threads=None):
    B, H, S, D = q8.shape
    s = np.empty((B, H, S, S), np.int32)
    lib().oracle_qk_int32(np.ascontiguousarray(q8).ravel(), np.ascontiguousarray(k8).ravel(), B * H, S, D,
                          s.ravel(), threads or n_threads_default())
    return s


def fp32_attention(q, k, v, mask, threads=None):
    """Tier A.  q float32 [B,H,Sq,D]; k,v float32 [B,H,Sk,D] (Sq == Sk in the reference's tests);
    mask int8 [B,Sk] (1 = masked key).  Returns (o [B,H,Sq,D], max|p|)."""
    B, H, Sq, D = q.shape
    Sk = k.shape[2]
    assert k.shape == (B, H, Sk, D) and v.shape == (B, H, Sk, D) and mask.shape == (B, Sk)
    o = np.empty((B, H, Sq, D), np.float32)
    pmax = _c.c_float(0)
    lib().oracle_fp32_attention_x(np.ascontiguousarray(q, np.float32).ravel(), np.ascontiguousarray(k, np.float32).ravel(),
                                  np.ascontiguousarray(v, np.float32).ravel(), np.ascontiguousarray(mask, np.int8).ravel(),
                                  B, H, Sq, Sk, D, o.ravel(), _c.byref(pmax), threads or n_threads_default())
    return o, float(pmax.value)


def q128(q8, k8, v8, mask, amax4, rows=None, threads=None, p_levels=128):
    """Tier C.  q8 int8 [B,H,Sq,D]; k8,v8 int8 [B,H,Sk,D]; mask int8 [B,Sk] (non-zero = masked key),
    amax4 = (q_amax, k_amax, v_amax, o_amax).  p_levels 128 = the reference kernel's signed P, 255 = the
    unsigned variant.  rows: optional int64 array of flattened row ids (bh*Sq + i); returns int8
    [len(rows), D] then, else int8 [B,H,Sq,D]."""
    B, H, Sq, D = q8.shape
    Sk = k8.shape[2]
    assert k8.shape == (B, H, Sk, D) and v8.shape == (B, H, Sk, D) and mask.shape == (B, Sk)
    assert p_levels in (128, 255)
    a = np.asarray(amax4, np.float32)
    assert a.size == 4
    q8 = np.ascontiguousarray(q8, np.int8)
    k8 = np.ascontiguousarray(k8, np.int8)
    v8 = np.ascontiguousarray(v8, np.int8)
    mask = np.ascontiguousarray(mask, np.int8)
    if rows is None:
        out = np.empty((B, H, Sq, D), np.int8)
        lib().oracle_q128_x(q8.ravel(), k8.ravel(), v8.ravel(), mask.ravel(), B, H, Sq, Sk, D, a, p_levels, None, 0,
                            out.ravel(), threads or n_threads_default())
    else:
        rows = np.ascontiguousarray(rows, np.int64)
        out = np.empty((rows.size, D), np.int8)
        lib().oracle_q128_x(q8.ravel(), k8.ravel(), v8.ravel(), mask.ravel(), B, H, Sq, Sk, D, a, p_levels,
                            rows.ctypes.data_as(_c.c_void_p), rows.size, out.ravel(), threads or n_threads_default())
    return out


def row_scale(D):
    return float(lib().oracle_row_scale(D))


# ----------------------------------------------------------------------------------------------
# The reference's own code (oracle/_ref).  Present only where it was built from a checkout.
# ----------------------------------------------------------------------------------------------
def ref_cpu_available(native=False):
    return os.path.exists(os.path.join(HERE, "_ref", "libref_cpu_native.so" if native else "libref_cpu.so"))


POLICY_ROW, POLICY_STATIC, POLICY_WORST = 1, 2, 3


def policy(q8, k8, v8, mask, amax5, which, rows=None, threads=None):
    """The whole-row P scaling policies of the reference's accuracy study (fmha_i8_quant_deviation.py:57-121) with int8
    output: which = POLICY_ROW ("dynamic"), POLICY_STATIC (p_amax = amax5[4] = s_max) or POLICY_WORST (p_amax = 1).
    q8 int8 [B,H,Sq,D]; k8, v8 int8 [B,H,Sk,D]; mask int8 [B,Sk]; amax5 = (q, k, v, o, s_max).  rows as in q128()."""
    B, H, Sq, D = q8.shape
    Sk = k8.shape[2]
    a = np.asarray(amax5, np.float32)
    assert a.size == 5 and mask.shape == (B, Sk)
    args = [np.ascontiguousarray(x, np.int8) for x in (q8, k8, v8, mask)]
    if rows is None:
        out = np.empty((B, H, Sq, D), np.int8)
        lib().oracle_policy_x(*args, B, H, Sq, Sk, D, a, int(which), None, 0, out, threads or n_threads_default())
    else:
        rows = np.ascontiguousarray(rows, np.int64)
        out = np.empty((rows.size, D), np.int8)
        lib().oracle_policy_x(*args, B, H, Sq, Sk, D, a, int(which), rows.ctypes.data, rows.size, out, threads or n_threads_default())
    return out


def refkernel_emulate(q8, k8, v8, mask, amax4, mask_minus_1e6=True, shuffle_as_written=True, threads=None):
    """CPU emulation of the reference CUDA kernel as written (inc/fmha_i8.cuh:87-332, 128-key tiles): tier C's
    arithmetic plus the kernel's own treatment of masked keys (int(-1e6) before scaling) and its P relayout with
    the semantics __shfl_sync really has.  Either departure can be switched off.  int8 [B,H,S,D], S % 128 == 0."""
    B, H, S, D = q8.shape
    assert S % 128 == 0 and k8.shape == q8.shape and v8.shape == q8.shape and mask.shape == (B, S)
    a = np.asarray(amax4, np.float32)
    assert a.size == 4
    out = np.empty((B, H, S, D), np.int8)
    lib().oracle_refkernel_emulate(np.ascontiguousarray(q8, np.int8), np.ascontiguousarray(k8, np.int8),
                                   np.ascontiguousarray(v8, np.int8), np.ascontiguousarray(mask, np.int8), B, H, S, D, a,
                                   1 if mask_minus_1e6 else 0, 1 if shuffle_as_written else 0, out,
                                   threads or n_threads_default())
    return out


def ref_gpu_available():
    return os.path.exists(os.path.join(HERE, "_ref", "libref_gpu.so"))


_ref = {}


def ref_cpu(native=False):
    key = "native" if native else "plain"
    if key not in _ref:
        L = ctypes.CDLL(os.path.join(HERE, "_ref", "libref_cpu_native.so" if native else "libref_cpu.so"))
        L.ref_abs_max.restype = _c.c_float
        L.ref_abs_max.argtypes = [_f32p, _c.c_int]
        L.ref_quantize.argtypes = [_f32p, _c.c_int64, _c.c_float, _i8p]
        L.ref_qk_int32.argtypes = [_i8p, _i8p, _c.c_int, _c.c_int, _c.c_int, _i32p]
        L.ref_fp32_attention_batched.argtypes = [_f32p, _f32p, _f32p, _i32p, _c.c_int, _c.c_int, _c.c_int, _c.c_int,
                                                 _f32p, _f32p, _f32p, _c.POINTER(_c.c_float)]
        L.ref_fp32_attention_threaded.argtypes = [_f32p, _f32p, _f32p, _i32p, _c.c_int, _c.c_int, _c.c_int,
                                                  _c.c_int, _c.c_int, _f32p, _c.c_int]
        L.ref_mean_rel_deviation.restype = _c.c_double
        L.ref_mean_rel_deviation.argtypes = [_i8p, _f32p, _c.c_int, _c.c_float]
        L.ref_fp32_attention_cross.argtypes = [_f32p, _f32p, _f32p, _i32p, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_int,
                                               _f32p, _f32p, _f32p]
        L.ref_qk_int32_cross.argtypes = [_i8p, _i8p, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _i32p]
        _ref[key] = L
    return _ref[key]


def ref_fp32_attention(q, k, v, mask, batched=True, threads=None, native=False):
    """The reference CPU golden (unchanged templates).  Returns (o, s_max or None)."""
    B, H, S, D = q.shape
    L = ref_cpu(native)
    q = np.ascontiguousarray(q, np.float32).ravel()
    k = np.ascontiguousarray(k, np.float32).ravel()
    v = np.ascontiguousarray(v, np.float32).ravel()
    m = np.ascontiguousarray(mask).astype(np.int32).ravel()
    o = np.zeros(B * H * S * D, np.float32)
    if batched:
        s = np.zeros(B * H * S * S, np.float32)
        p = np.zeros(B * H * S * S, np.float32)
        smax = _c.c_float(0)
        L.ref_fp32_attention_batched(q, k, v, m, B, H, S, D, s, p, o, _c.byref(smax))
        return o.reshape(B, H, S, D), float(smax.value)
    L.ref_fp32_attention_threaded(q, k, v, m, H, S, D, 0, B * H, o, threads or n_threads_default())
    return o.reshape(B, H, S, D), None


def ref_fp32_attention_cross(q, k, v, mask):
    """The reference CPU templates called with Sq != Sk: q [B,H,Sq,D], k,v [B,H,Sk,D], mask [B,Sk]."""
    B, H, Sq, D = q.shape
    Sk = k.shape[2]
    L = ref_cpu(False)
    o = np.zeros(B * H * Sq * D, np.float32)
    s = np.zeros(B * H * Sq * Sk, np.float32)
    p = np.zeros(B * H * Sq * Sk, np.float32)
    L.ref_fp32_attention_cross(np.ascontiguousarray(q, np.float32).ravel(), np.ascontiguousarray(k, np.float32).ravel(),
                               np.ascontiguousarray(v, np.float32).ravel(), np.ascontiguousarray(mask).astype(np.int32).ravel(),
                               B, H, Sq, Sk, D, s, p, o)
    return o.reshape(B, H, Sq, D)


def ref_gpu():
    if "gpu" not in _ref:
        L = ctypes.CDLL(os.path.join(HERE, "_ref", "libref_gpu.so"))
        L.ref_gpu_shape_ok.argtypes = [_c.c_int, _c.c_int]
        L.ref_gpu_fmha.argtypes = [_c.c_void_p, _c.POINTER(_c.c_float), _c.POINTER(_c.c_int)] + [_c.c_void_p] * 5
        if hasattr(L, "wmma_layout_probe"):
            L.wmma_layout_probe.argtypes = [_c.c_void_p, _c.c_void_p]
        _ref["gpu"] = L
    return _ref["gpu"]
