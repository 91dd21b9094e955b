"""GPU parity tests at the limits of the accepted shapes: the longest sequence (32768 keys = 256 key tiles,
the size of the per-unit mask tables) and more (batch x head) slices than a grid dimension holds.  Rows are
sampled for the CPU oracle; the bar is the one of tests/_util.py."""
import numpy as np
import pytest

from _util import assert_parity, sample_rows

pytestmark = [pytest.mark.gpu, pytest.mark.timeout(900)]


def _device_case(torch, B, H, S, D, seed, valid=None):
    g = torch.Generator(device="cuda").manual_seed(seed)
    q8, k8, v8 = (torch.randint(-127, 128, (B, H, S, D), dtype=torch.int8, device="cuda", generator=g) for _ in range(3))
    mask = torch.zeros((B, S), dtype=torch.int8, device="cuda")
    if valid is not None:
        for b, L in enumerate(valid):
            mask[b, L:] = 1
    return q8, k8, v8, mask


def _check(pkg, oracle, torch, q8, k8, v8, mask, amax, rows, what, uint8_p=False):
    B, H, S, D = q8.shape
    o8 = torch.full_like(q8, 0x5A)
    pkg.FMHAInferI8(None, pkg.FMHAParamI8(*amax, 1.0), pkg.AttnDataDescriptor(B, S, H, D), q8, k8, v8, mask, o8, True, uint8_p=uint8_p)
    st, words = pkg.device_status()
    assert st == pkg.OK, words
    want = oracle.q128(q8.cpu().numpy(), k8.cpu().numpy(), v8.cpu().numpy(), mask.cpu().numpy(), amax, rows=rows,
                       p_levels=255 if uint8_p else 128)
    got = o8.view(-1, D)[torch.from_numpy(rows).cuda()].cpu().numpy()
    return assert_parity(got, want, what)


def test_longest_sequence(pkg, oracle):
    """S = 32768, the documented maximum, with the last 1000 keys padded: 256 key tiles per unit."""
    import torch
    torch.cuda.set_device(0)
    B, H, S, D = 1, 2, 32768, 64
    q8, k8, v8, mask = _device_case(torch, B, H, S, D, seed=1, valid=[S - 1000])
    # integer data of full range: scores are huge, softmax is peaked -- and the last tile is partly masked
    amax = [0.05, 0.05, 1.0, 0.6]
    rows = sample_rows(B, H, S, 24, valid=np.array([S - 1000]), seed=3)
    _check(pkg, oracle, torch, q8, k8, v8, mask, amax, rows, "S=32768")
    _check(pkg, oracle, torch, q8, k8, v8, mask, amax, rows, "S=32768 unsigned P", uint8_p=True)


def test_more_slices_than_a_grid_dimension(pkg, oracle):
    """B*H = 70000 > 65535 with S = 64 (one half-filled query tile per slice): the persistent grid walks
    70000 units; valid lengths alternate between 64 and 40 keys."""
    import torch
    torch.cuda.set_device(0)
    B, H, S, D = 7000, 10, 64, 64
    q8, k8, v8, mask = _device_case(torch, B, H, S, D, seed=2)
    mask[1::2, 40:] = 1
    amax = [0.3, 0.3, 1.0, 0.5]
    rng = np.random.default_rng(0)
    heads = np.concatenate([[0, 1, B * H - 1, B * H - 2, 65535, 65536], rng.integers(0, B * H, 200)])
    rows = np.unique(np.concatenate([heads * S + r for r in (0, 17, 63)])).astype(np.int64)
    _check(pkg, oracle, torch, q8, k8, v8, mask, amax, rows, "B*H=70000")


@pytest.mark.parametrize("D", [64, 128])
def test_many_units_per_cta_with_changing_shape_of_unit(pkg, oracle, D):
    """384 work units on 148 persistent CTAs, so every CTA walks several units, and consecutive units of a CTA
    differ in kind: S = 576 gives three query-tile pairs per head, the last with a single half-filled tile;
    one batch is fully masked (units with no live key tile), one has 100 valid keys (one live tile), the rest
    have random masks.  Every element against the CUDA-core cross-check, sampled rows against the CPU oracle."""
    import torch
    torch.cuda.set_device(0)
    B, H, S = 4, 32, 576
    q8, k8, v8, mask = _device_case(torch, B, H, S, D, seed=11 + D)
    g = torch.Generator(device="cuda").manual_seed(5)
    mask[:] = (torch.rand((B, S), device="cuda", generator=g) < 0.2).to(torch.int8)
    mask[1, :] = 1
    mask[2, :] = 0
    mask[2, 100:] = 1
    amax = [0.1, 0.1, 1.0, 0.6]
    for up in (False, True):
        o8 = torch.full_like(q8, 0x5A)
        pkg.FMHAInferI8(None, pkg.FMHAParamI8(*amax, 1.0), pkg.AttnDataDescriptor(B, S, H, D), q8, k8, v8, mask, o8, True, uint8_p=up)
        chk = torch.empty_like(q8)
        pkg.debug_simt_x(None, pkg.FMHAParamI8(*amax, 1.0), pkg.AttnDataDescriptorX(B, S, S, H, D), q8, k8, v8, mask, chk, uint8_p=up)
        st, words = pkg.device_status()
        assert st == pkg.OK, words
        assert_parity(o8.cpu().numpy(), chk.cpu().numpy(), f"D={D} uint8_p={up} vs CUDA-core kernel")
        assert bool((o8[1] == 0).all())
        rows = sample_rows(B, H, S, 6, seed=D)
        want = oracle.q128(q8.cpu().numpy(), k8.cpu().numpy(), v8.cpu().numpy(), mask.cpu().numpy(), amax, rows=rows,
                           p_levels=255 if up else 128)
        assert_parity(o8.view(-1, D)[torch.from_numpy(rows).cuda()].cpu().numpy(), want, f"D={D} uint8_p={up} vs oracle")
