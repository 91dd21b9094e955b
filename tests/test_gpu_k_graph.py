"""GPU test: the forward call only enqueues one kernel on the caller's stream (tensor maps travel by value
as kernel parameters, nothing is allocated or synchronised), so it can be recorded into a CUDA graph and
replayed.  The first call on a device (which looks up device attributes) is made before the capture."""
import numpy as np
import pytest

pytestmark = [pytest.mark.gpu, pytest.mark.timeout(300)]


def test_forward_is_capturable_in_a_cuda_graph(pkg):
    import torch
    torch.cuda.set_device(0)
    B, H, S, D = 2, 4, 512, 128
    g = torch.Generator(device="cuda").manual_seed(7)
    q, k, v = (torch.randint(-127, 128, (B, H, S, D), dtype=torch.int8, device="cuda", generator=g) for _ in range(3))
    m = torch.zeros((B, S), dtype=torch.int8, device="cuda")
    m[1, 300:] = 1
    prm, desc = pkg.FMHAParamI8(0.2, 0.2, 1.0, 0.7, 1.0), pkg.AttnDataDescriptor(B, S, H, D)
    eager = torch.empty_like(q)
    pkg.FMHAInferI8(None, prm, desc, q, k, v, m, eager, True)            # also the first call on this device
    eager_u = torch.empty_like(q)
    pkg.FMHAInferI8(None, prm, desc, q, k, v, m, eager_u, True, uint8_p=True)
    torch.cuda.synchronize()

    out_a, out_b = torch.zeros_like(q), torch.zeros_like(q)
    graph = torch.cuda.CUDAGraph()
    launches0 = pkg.launch_count()
    with torch.cuda.graph(graph):
        pkg.FMHAInferI8(None, prm, desc, q, k, v, m, out_a, True)
        pkg.FMHAInferI8(None, prm, desc, q, k, v, m, out_b, True, uint8_p=True)
    assert pkg.launch_count() - launches0 == 2
    for _ in range(3):
        out_a.zero_()
        out_b.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out_a, eager) and torch.equal(out_b, eager_u)
    # new input values in the same buffers are picked up by a replay (addresses are baked in, data is not)
    q.copy_(torch.randint(-127, 128, q.shape, dtype=torch.int8, device="cuda", generator=g))
    pkg.FMHAInferI8(None, prm, desc, q, k, v, m, eager, True)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out_a, eager)
    st, words = pkg.device_status()
    assert st == pkg.OK, words
