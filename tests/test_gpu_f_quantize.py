"""GPU parity of the device-side quantisation producer (abs_max + float_quant2_int8,
reference inc/utils.hpp:23-39) through the C ABI: bit-exact against the reference's own outputs
in tests/golden/ and against the CPU oracle on ragged sizes."""
import numpy as np
import pytest

from _util import GOLDEN

pytestmark = [pytest.mark.gpu, pytest.mark.timeout(300)]


def _run(pkg, torch, x, entry="fmha_i8_sm100_quantize_f32"):
    tx = torch.from_numpy(np.ascontiguousarray(x, np.float32)).cuda()
    to = torch.full((tx.numel() + 64,), 0x5A, dtype=torch.int8, device="cuda")     # canary tail
    ta = torch.zeros(1, dtype=torch.float32, device="cuda")
    pkg.quantize_f32(None, tx, to, ta, n=tx.numel(), entry=entry)
    torch.cuda.synchronize()
    host = to.cpu().numpy()
    assert np.all(host[tx.numel():] == 0x5A), "wrote past the end of the output"
    return host[:tx.numel()].reshape(x.shape), float(ta.item())


def test_quantize_golden_bit_exact(pkg):
    import torch
    torch.cuda.set_device(0)
    for path in GOLDEN:
        g = np.load(path)
        for name, i in (("q", 0), ("k", 1), ("v", 2)):
            got, amax = _run(pkg, torch, g[name])
            assert np.float32(amax) == g["ref_amax"][i], (path, name)
            assert np.array_equal(got, g["ref_" + name + "8"]), (path, name)


@pytest.mark.parametrize("n", [1, 15, 16, 17, 4097, 65536, 65537, 3 * 65536 + 5, 1 << 22])
def test_quantize_ragged_sizes(pkg, oracle, n):
    import torch
    torch.cuda.set_device(0)
    rng = np.random.default_rng(n)
    x = (rng.standard_normal(n) * rng.choice([0.01, 1.0, 300.0])).astype(np.float32)
    x[-1] = np.float32(np.abs(x).max() * 1.5)           # the maximum sits in the ragged tail
    got, amax = _run(pkg, torch, x)
    assert np.float32(amax) == np.float32(oracle.abs_max(x))
    assert np.array_equal(got, oracle.quantize(x, oracle.abs_max(x)))


def test_quantize_all_zero_and_rejections(pkg):
    import torch
    torch.cuda.set_device(0)
    got, amax = _run(pkg, torch, np.zeros(1000, np.float32))
    assert amax == 0.0 and not got.any()
    x = torch.zeros(64, dtype=torch.float32, device="cuda")
    o = torch.zeros(64, dtype=torch.int8, device="cuda")
    L = pkg.lib()
    import ctypes
    vp = ctypes.c_void_p
    assert L.fmha_i8_sm100_quantize_f32(None, None, 64, vp(o.data_ptr()), None) == pkg.ERR_NULL_POINTER
    assert L.fmha_i8_sm100_quantize_f32(None, vp(x.data_ptr()), 0, vp(o.data_ptr()), None) == pkg.ERR_BAD_SHAPE
    assert L.fmha_i8_sm100_quantize_f32(None, vp(x.data_ptr() + 4), 8, vp(o.data_ptr()), None) == pkg.ERR_MISALIGNED
