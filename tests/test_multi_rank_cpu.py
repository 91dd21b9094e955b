"""Host-side logic of the multi-GPU path on CPU: two gloo ranks partition one problem over the
flattened batch*head axis, each computes its slice (with the oracle standing in for the device),
and rank 0 reassembles the whole output; timings are reduced with max over ranks."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    import importlib

    import torch
    import torch.distributed as dist
    import __graft_entry__ as ge
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ge.load_package()
    part = importlib.import_module("int8_fmha_b200.partition")
    wl = importlib.import_module("int8_fmha_b200.workloads")
    oracle = ge.load_oracle()

    w = wl.Workload("t", 3, 3, 128, 64, valid_choices=(64, 128))     # 9 heads: an uneven split over 2 ranks
    q, k, v, mask = wl.make_fp32_np(w, seed=17)                      # same seed everywhere: same problem
    q8, qa = wl.quantize_np(q)
    k8, ka = wl.quantize_np(k)
    v8, va = wl.quantize_np(v)
    amax = (qa, ka, va, 1.0)
    begin, count = part.slice_bounds(w.B * w.H, rank, world)
    rows = (np.arange(begin * w.S, (begin + count) * w.S)).astype(np.int64)
    mine = oracle.q128(q8, k8, v8, mask, amax, rows=rows, threads=1)          # this rank's heads only
    gathered = [None] * world
    dist.all_gather_object(gathered, (begin, count, mine))
    slowest = part.max_over_ranks(1.0 + rank)                                 # rank 1 is "slower"
    if rank == 0:
        whole = oracle.q128(q8, k8, v8, mask, amax, threads=1).reshape(-1, w.D)
        parts = sorted(gathered, key=lambda t: t[0])
        assert [p[0] for p in parts] == [0, 5] and [p[1] for p in parts] == [5, 4]
        assert np.array_equal(np.concatenate([p[2] for p in parts]), whole)
        assert slowest == float(world)
        open(os.path.join(out_dir, "ok"), "w").write("ok")
    dist.barrier()
    dist.destroy_process_group()


def test_slice_bounds(pkg):
    import importlib
    part = importlib.import_module("int8_fmha_b200.partition")
    for total in (1, 2, 7, 32, 256, 384, 4096):
        for world in (1, 2, 4, 8):
            spans = [part.slice_bounds(total, r, world) for r in range(world)]
            assert spans[0][0] == 0 and sum(c for _, c in spans) == total
            for (b0, c0), (b1, _) in zip(spans, spans[1:]):
                assert b0 + c0 == b1
            assert max(c for _, c in spans) - min(c for _, c in spans) <= 1
    with pytest.raises(ValueError):
        part.slice_bounds(8, 2, 2)


@pytest.mark.timeout(300)
def test_two_gloo_ranks_reassemble_the_whole(tmp_path, pkg, oracle):
    import torch.multiprocessing as mp
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok").exists()
