"""Host-side logic of the multi-GPU path on CPU: gloo ranks partition one problem over the
flattened batch*head axis, each computes its slice (with the oracle standing in for the device),
and rank 0 reassembles the whole output; timings are reduced with max over ranks.  The failure
cases are made on the host: one rank raises in its compute step, or skips its launch; the job
reports a partial result (which heads are missing, which rank failed) and nothing hangs."""
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


def _worker_with_failure(rank, world, port, out_dir, mode):
    """Three ranks; rank 1 fails on the host (it raises inside its compute step, or it never launches).  The others
    learn of it through the report exchange, rank 0 assembles a result with a hole, nothing hangs."""
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

    w = wl.Workload("t", 2, 4, 128, 64, valid_choices=(64, 128))     # 8 heads over 3 ranks: 3 + 3 + 2
    q, k, v, mask = wl.make_fp32_np(w, seed=23)
    q8, qa = wl.quantize_np(q)
    k8, ka = wl.quantize_np(k)
    v8, va = wl.quantize_np(v)
    amax = (qa, ka, va, 1.0)
    begin, count = part.slice_bounds(w.B * w.H, rank, world)
    ok, detail, mine = True, "", None
    try:
        if rank == 1 and mode == "raises":
            raise RuntimeError("injected host-side failure")
        if rank == 1 and mode == "skips":
            ok, detail = False, "launch skipped"
        else:
            rows = (np.arange(begin * w.S, (begin + count) * w.S)).astype(np.int64)
            mine = torch.from_numpy(oracle.q128(q8, k8, v8, mask, amax, rows=rows, threads=1).reshape(count, w.S, w.D))
    except RuntimeError as exc:
        ok, detail = False, str(exc)
    whole, cov = part.assemble_on_rank0(mine, begin, count, ok, w.B * w.H, detail)
    assert cov["complete"] is False and cov["heads_done"] == 5 and cov["heads_missing"] == [(3, 3)]
    assert [r for r, _ in cov["ranks_failed"]] == [1]
    if rank == 0:
        want = oracle.q128(q8, k8, v8, mask, amax, threads=1).reshape(w.B * w.H, w.S, w.D)
        got = whole.numpy()
        assert np.array_equal(got[:3], want[:3]) and np.array_equal(got[6:], want[6:])
        assert not got[3:6].any()
        open(os.path.join(out_dir, "ok_" + mode), "w").write(cov["ranks_failed"][0][1])
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


@pytest.mark.timeout(300)
@pytest.mark.parametrize("mode", ["raises", "skips"])
def test_a_failed_rank_leaves_a_hole_not_a_hang(tmp_path, pkg, oracle, mode):
    import torch.multiprocessing as mp
    port = 31500 + (os.getpid() % 2000) + (7 if mode == "skips" else 0)
    mp.spawn(_worker_with_failure, args=(3, port, str(tmp_path), mode), nprocs=3, join=True)
    assert (tmp_path / ("ok_" + mode)).exists()


def test_coverage_report(pkg):
    import importlib
    part = importlib.import_module("int8_fmha_b200.partition")
    full = part.coverage([(0, 0, 4, True, ""), (1, 4, 4, True, "")], 8)
    assert full == {"complete": True, "heads_done": 8, "heads_missing": [], "ranks_failed": []}
    hole = part.coverage([(0, 0, 4, True, ""), (1, 4, 4, False, "x")], 8)
    assert hole["complete"] is False and hole["heads_missing"] == [(4, 4)] and hole["ranks_failed"] == [(1, "x")]
