"""GPU tests of the two tensor-core stages in isolation (bit-exact integer results) and of the
CUDA-core cross-check kernel, all through the C ABI."""
import numpy as np
import pytest

from _util import GOLDEN, assert_parity

pytestmark = [pytest.mark.gpu, pytest.mark.timeout(300)]


@pytest.fixture(scope="module")
def torch_dev():
    import torch
    assert torch.cuda.is_available()
    torch.cuda.set_device(0)
    return torch


def _clean(pkg):
    st, words = pkg.device_status()
    assert st == pkg.OK, f"device status words {words}"


@pytest.mark.parametrize("B,H,S,D", [(1, 2, 64, 64), (1, 1, 128, 128), (2, 3, 192, 64), (1, 2, 320, 128), (1, 1, 512, 64)])
def test_qk_stage_bit_exact(pkg, oracle, torch_dev, B, H, S, D):
    torch = torch_dev
    rng = np.random.default_rng(S + D)
    q8 = rng.integers(-127, 128, (B, H, S, D)).astype(np.int8)
    k8 = rng.integers(-127, 128, (B, H, S, D)).astype(np.int8)
    want = oracle.qk_int32(q8, k8)
    tq, tk = torch.from_numpy(q8).cuda(), torch.from_numpy(k8).cuda()
    ts = torch.full((B * H, S, S), -7, dtype=torch.int32, device="cuda")
    pkg.debug_qk(None, pkg.AttnDataDescriptor(B, S, H, D), tq, tk, ts)
    _clean(pkg)
    assert np.array_equal(ts.cpu().numpy().reshape(B, H, S, S), want)


def test_qk_stage_golden(pkg, torch_dev):
    """S_int32 against the reference's cpuGEMM<int32_t,int32_t,int8_t,int32_t> output."""
    torch = torch_dev
    for path in GOLDEN:
        g = np.load(path)
        B, H, S, D = g["ref_q8"].shape
        tq, tk = torch.from_numpy(g["ref_q8"]).cuda(), torch.from_numpy(g["ref_k8"]).cuda()
        ts = torch.zeros((B * H, S, S), dtype=torch.int32, device="cuda")
        pkg.debug_qk(None, pkg.AttnDataDescriptor(B, S, H, D), tq, tk, ts)
        _clean(pkg)
        assert np.array_equal(ts.cpu().numpy().reshape(B, H, S, S), g["ref_s_int32"]), path


@pytest.mark.parametrize("variant", [0, 1])
@pytest.mark.parametrize("B,H,S,D", [(1, 1, 128, 128), (1, 2, 64, 64), (2, 2, 192, 64), (1, 2, 320, 128)])
def test_pv_stage_bit_exact(pkg, torch_dev, variant, B, H, S, D):
    torch = torch_dev
    rng = np.random.default_rng(S * 3 + D + variant)
    p8 = rng.integers(-128, 1, (B * H, S, S)).astype(np.int8)      # the forward pass's range: -128..0
    v8 = rng.integers(-127, 128, (B, H, S, D)).astype(np.int8)
    want = np.einsum("hij,hjd->hid", p8.astype(np.int64), v8.reshape(B * H, S, D).astype(np.int64)).astype(np.int32)
    tp, tv = torch.from_numpy(p8).cuda(), torch.from_numpy(v8).cuda()
    to = torch.full((B * H, S, D), -7, dtype=torch.int32, device="cuda")
    pkg.debug_pv(None, pkg.AttnDataDescriptor(B, S, H, D), tp, tv, to, variant)
    _clean(pkg)
    assert np.array_equal(to.cpu().numpy(), want)


def test_simt_kernel_matches_oracle_on_golden(pkg, oracle, torch_dev):
    torch = torch_dev
    for path in GOLDEN:
        g = np.load(path)
        B, H, S, D = g["ref_q8"].shape
        amax = [float(x) for x in g["ref_amax"]]
        t = [torch.from_numpy(g[n]).cuda() for n in ("ref_q8", "ref_k8", "ref_v8", "mask")]
        to = torch.zeros_like(t[0])
        pkg.debug_simt(None, pkg.FMHAParamI8(*amax, 1.0), pkg.AttnDataDescriptor(B, S, H, D), *t, to)
        _clean(pkg)
        mx, f1, f0 = assert_parity(to.cpu().numpy(), g["oracle_o8"], path)
        assert f0 > 0.99, (path, f0)   # same operation order: differences only from expf rounding
