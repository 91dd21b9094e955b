"""CPU tests of the boundary: the shared library loads, exports every declared symbol, and rejects
bad arguments on the host before touching a GPU."""
import ctypes
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "fmha_i8_c.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fmha_i8_sm100_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol(pkg):
    names = declared_functions()
    assert len(names) >= 11
    L = pkg.lib()
    for n in names:
        assert getattr(L, n) is not None
    assert set(names) == set(pkg.EXPORTS)


def test_cpp_symbol_is_exported(pkg):
    # the reference's C++ entry point gpuImpl::FMHAInferI8(CUstream_st*, FMHAParamI8, AttnDataDescriptor, ...)
    L = ctypes.CDLL(pkg.LIB_PATH)
    assert getattr(L, "_ZN7gpuImpl11FMHAInferI8EP11CUstream_st11FMHAParamI818AttnDataDescriptorPKvS5_S5_S5_Pvb")


def test_struct_layouts_match_reference(pkg):
    d = pkg.AttnDataDescriptor(2, 128, 3, 64).as_c()
    assert list(d) == [2, 128, 3, 64] and ctypes.sizeof(d) == 16     # batch, seq, head, dim
    p = pkg.FMHAParamI8(1, 2, 3, 4, 5).as_c()
    assert list(p) == [1, 2, 3, 4, 5] and ctypes.sizeof(p) == 20
    assert pkg.AttnDataDescriptor() == pkg.AttnDataDescriptor(1, 64, 4, 64)      # reference defaults
    assert pkg.FMHAParamI8() == pkg.FMHAParamI8(0.0, 0.0, 0.0, 1.0, 1.0)


def _call(pkg, desc, amax=(1, 1, 1, 1, 1), ptrs=(256, 512, 768, 1024, 1280), flags=1):
    L = pkg.lib()
    a = (ctypes.c_float * 5)(*amax)
    d = (ctypes.c_int * 4)(*desc)
    vp = [ctypes.c_void_p(p) if p else None for p in ptrs]
    return L.fmha_i8_sm100_infer(None, a, d, *vp, flags)


def test_host_side_rejections(pkg):
    good = (1, 128, 2, 64)
    assert _call(pkg, good, ptrs=(0, 512, 768, 1024, 1280)) == pkg.ERR_NULL_POINTER
    assert _call(pkg, good, flags=0) == pkg.ERR_NO_CUDA_CORE_PATH
    assert _call(pkg, (1, 100, 2, 64)) == pkg.ERR_BAD_SHAPE         # seq_len not a multiple of 64
    assert _call(pkg, (1, 128, 2, 96)) == pkg.ERR_BAD_SHAPE         # head_dim
    assert _call(pkg, (1, 65536, 2, 64)) == pkg.ERR_BAD_SHAPE       # beyond the maximum
    assert _call(pkg, (0, 128, 2, 64)) == pkg.ERR_BAD_SHAPE
    assert _call(pkg, good, ptrs=(264, 512, 768, 1024, 1280)) == pkg.ERR_MISALIGNED
    assert _call(pkg, good, ptrs=(256, 512, 768, 1026, 1280)) == pkg.ERR_MISALIGNED  # mask needs 4 bytes
    assert _call(pkg, good, amax=(0, 1, 1, 1, 1)) == pkg.ERR_BAD_AMAX
    assert _call(pkg, good, amax=(1, 1, float("nan"), 1, 1)) == pkg.ERR_BAD_AMAX
    assert pkg.lib().fmha_i8_sm100_last_status() == pkg.ERR_BAD_AMAX
    L = pkg.lib()
    a = (ctypes.c_float * 5)(1, 1, 1, 1, 1)
    d = (ctypes.c_int * 4)(*good)
    vp = [ctypes.c_void_p(p) for p in (256, 512, 768, 1024, 1280)]
    assert L.fmha_i8_sm100_infer_slice(None, a, d, *vp, 1, 2, 1) == pkg.ERR_BAD_SLICE
    assert L.fmha_i8_sm100_infer_slice(None, a, d, *vp, -1, 1, 1) == pkg.ERR_BAD_SLICE
    assert "seq_len" in pkg.status_string(pkg.ERR_BAD_SHAPE)
    # flags: bit 1 (unsigned P) is defined, anything above is not
    assert _call(pkg, good, flags=1 | 4) == pkg.ERR_BAD_FLAGS
    assert _call(pkg, good, flags=2) == pkg.ERR_NO_CUDA_CORE_PATH
    # query rows != keys: desc5 = {batch, seq_q, seq_k, head, dim}; seq_q free, seq_k a multiple of 64
    def cross(desc5, begin=0, count=2):
        return L.fmha_i8_sm100_infer_cross(None, a, (ctypes.c_int * 5)(*desc5), *vp, begin, count, 1)
    assert cross((1, 0, 128, 2, 64)) == pkg.ERR_BAD_SHAPE
    assert cross((1, 40000, 128, 2, 64)) == pkg.ERR_BAD_SHAPE
    assert cross((1, 7, 100, 2, 64)) == pkg.ERR_BAD_SHAPE
    assert cross((1, 7, 128, 2, 32)) == pkg.ERR_BAD_SHAPE
    assert cross((1, 7, 128, 2, 64), begin=1, count=2) == pkg.ERR_BAD_SLICE
    assert L.fmha_i8_sm100_infer_cross(None, a, None, *vp, 0, 2, 1) == pkg.ERR_NULL_POINTER
    assert L.fmha_i8_sm100_calibrate_o_amax(None, a, (ctypes.c_int * 5)(1, 7, 128, 2, 64), *vp[:4], None, 1) == pkg.ERR_NULL_POINTER
    assert pkg.lib().fmha_i8_sm100_version() >= 100


def test_python_mirror_raises(pkg):
    with pytest.raises(pkg.FmhaError) as e:
        pkg.FMHAInferI8(0, pkg.FMHAParamI8(1, 1, 1, 1, 1), pkg.AttnDataDescriptor(1, 100, 2, 64),
                        256, 512, 768, 1024, 1280, True)
    assert e.value.status == pkg.ERR_BAD_SHAPE
    st = pkg.FMHAInferI8(0, pkg.FMHAParamI8(1, 1, 1, 1, 1), pkg.AttnDataDescriptor(1, 128, 2, 64),
                         256, 512, 768, 1024, 1280, False, check=False)
    assert st == pkg.ERR_NO_CUDA_CORE_PATH


def test_workload_table_and_mask_polarity(wl):
    c = wl.CONFIGS
    assert (c["C2"].B, c["C2"].H, c["C2"].S, c["C2"].D) == (32, 12, 512, 64)
    assert (c["C3"].B, c["C3"].H, c["C3"].S, c["C3"].D) == (8, 32, 2048, 128)
    assert (c["C4"].B, c["C4"].H, c["C4"].S, c["C4"].D) == (1, 32, 16384, 128)
    assert (c["C5"].B, c["C5"].H, c["C5"].S, c["C5"].D) == (256, 16, 256, 64)
    assert c["C3"].ops == 4.0 * 8 * 32 * 2048 * 2048 * 128
    assert c["C3"].bytes == 268451840
    m = wl.mask_from_valid(np.array([64, 128]), 128)
    assert m.dtype == np.int8 and m[0, 63] == 0 and m[0, 64] == 1 and m[1].sum() == 0   # 1 = masked key
    v = wl.valid_lengths(c["C2"], 2023)
    assert v.shape == (32,) and set(v.tolist()) <= {256, 320, 384, 448, 512}
    assert np.array_equal(v, wl.valid_lengths(c["C2"], 2023))
    assert wl.valid_lengths(c["C4"], 1).tolist() == [15360]
