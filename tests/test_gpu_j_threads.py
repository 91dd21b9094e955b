"""GPU test of the threading contract of the C ABI: the device-pointer entry points may be called
concurrently from several host threads on different streams (the reference is a stateless function; the
multi-GPU runner relies on this).  Four threads run different shapes at the same time; every result must
equal the one computed alone."""
import threading

import numpy as np
import pytest

pytestmark = [pytest.mark.gpu, pytest.mark.timeout(300)]


def test_concurrent_host_threads_on_different_streams(pkg):
    import torch
    torch.cuda.set_device(0)
    shapes = [(2, 4, 512, 128), (3, 2, 320, 64), (1, 8, 1024, 128), (4, 4, 192, 64)]
    cases = []
    for i, (B, H, S, D) in enumerate(shapes):
        g = torch.Generator(device="cuda").manual_seed(100 + i)
        q, k, v = (torch.randint(-127, 128, (B, H, S, D), dtype=torch.int8, device="cuda", generator=g) for _ in range(3))
        m = (torch.rand((B, S), device="cuda", generator=g) < 0.2).to(torch.int8)
        prm = pkg.FMHAParamI8(0.2, 0.2, 1.0, 0.7, 1.0)
        desc = pkg.AttnDataDescriptor(B, S, H, D)
        alone = torch.empty_like(q)
        pkg.FMHAInferI8(None, prm, desc, q, k, v, m, alone, True)
        cases.append((prm, desc, q, k, v, m, alone))
    st, words = pkg.device_status()
    assert st == pkg.OK, words

    errors = []

    def worker(idx):
        try:
            torch.cuda.set_device(0)
            prm, desc, q, k, v, m, alone = cases[idx]
            stream = torch.cuda.Stream()
            outs = [torch.zeros_like(q) for _ in range(4)]
            for rep in range(40):
                pkg.FMHAInferI8(stream, prm, desc, q, k, v, m, outs[rep % 4], True)
            stream.synchronize()
            for o in outs:
                if not torch.equal(o, alone):
                    errors.append(f"thread {idx}: result differs from the one computed alone")
                    break
        except Exception as exc:      # surfaced below; a thread must not die silently
            errors.append(f"thread {idx}: {exc!r}")

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(len(cases))]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    st, words = pkg.device_status()
    assert st == pkg.OK, words
    assert not errors, errors


def test_host_buffer_entry_point_from_two_threads(pkg):
    """fmha_i8_sm100_infer_host keeps one set of staging buffers per device behind a per-device lock: two host
    threads that call it for the same device at the same time are serialised on that device's lock (not on a
    process-wide one, which would also serialise threads that drive different GPUs), and both get the right
    answer."""
    import torch
    torch.cuda.set_device(0)
    cases = []
    for i, (B, H, S, D) in enumerate([(2, 4, 256, 64), (1, 6, 384, 128)]):
        g = torch.Generator().manual_seed(7 + i)
        q, k, v = (torch.randint(-127, 128, (B, H, S, D), dtype=torch.int8, generator=g).pin_memory() for _ in range(3))
        m = (torch.rand((B, S), generator=g) < 0.2).to(torch.int8).pin_memory()
        prm = pkg.FMHAParamI8(0.2, 0.2, 1.0, 0.7, 1.0)
        desc = pkg.AttnDataDescriptor(B, S, H, D)
        alone = torch.empty_like(q)
        pkg.FMHAInferI8(None, prm, desc, q.cuda(), k.cuda(), v.cuda(), m.cuda(), (dev_o := torch.empty_like(q, device="cuda")), True)
        torch.cuda.synchronize()
        cases.append((prm, desc, q, k, v, m, dev_o.cpu()))
    errors = []

    def worker(idx):
        try:
            torch.cuda.set_device(0)
            prm, desc, q, k, v, m, want = cases[idx]
            out = torch.empty_like(q).pin_memory()
            for rep in range(10):
                out.zero_()
                pkg.FMHAInferI8Host(prm, desc, q, k, v, m, out)
                if not torch.equal(out, want):
                    errors.append(f"thread {idx} rep {rep}: wrong result")
                    break
        except Exception as exc:
            errors.append(f"thread {idx}: {exc!r}")

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    st, words = pkg.device_status()
    assert st == pkg.OK, words
    assert not errors, errors
