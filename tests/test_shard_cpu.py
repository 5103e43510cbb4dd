"""Multi-GPU host logic on CPU: two `gloo` ranks shard the utterances the way bench.py does,
"decode" their own share, and the results are gathered by item index. No data-path collective
exists on this path (utterances are independent); the only reductions are the gather of the
token lists and the max over ranks of the step time."""
import importlib.util
import os
import socket

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_mod", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_shard_is_a_balanced_partition():
    shard = _bench().shard
    for n in (0, 1, 7, 16, 33, 256):
        for world in (1, 2, 3, 4, 8):
            parts = [shard(n, r, world) for r in range(world)]
            flat = [i for p in parts for i in p]
            assert flat == list(range(n))                              # complete, ordered, disjoint
            assert max(len(p) for p in parts) - min(len(p) for p in parts) <= 1


def _rank_main(rank, world, port, n_items, out_dir):
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    shard = _bench().shard
    mine = shard(n_items, rank, world)
    # stand-in for the per-utterance device decode: a deterministic function of the item id
    result = {i: [i * 3 + j for j in range(i % 5)] for i in mine}
    gathered = [None] * world
    dist.all_gather_object(gathered, result)
    t = torch.tensor([10.0 + rank], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)                           # step time = max over ranks
    if rank == 0:
        merged = {}
        for g in gathered:
            merged.update(g)
        ok = sorted(merged) == list(range(n_items)) and all(merged[i] == [i * 3 + j for j in range(i % 5)]
                                                            for i in merged) and t.item() == 10.0 + world - 1
        open(os.path.join(out_dir, "ok"), "w").write("1" if ok else "0")
    dist.destroy_process_group()


def test_two_rank_gloo_gather(tmp_path):
    mp = pytest.importorskip("torch.multiprocessing")
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    mp.spawn(_rank_main, args=(2, port, 33, str(tmp_path)), nprocs=2, join=True)
    assert open(tmp_path / "ok").read() == "1"


def test_length_bucketed_workload_is_seeded_sorted_and_per_rank():
    """The cfg2 workload: lengths are a seeded draw per rank, ascending (so consecutive batches hold similar
    lengths), inside the stated range and on whole 10 ms."""
    import argparse
    b = _bench()
    args = argparse.Namespace(items=256, min_seconds=5.0, max_seconds=120.0)
    a0, a0_again, a1 = b.item_seconds(args, 0), b.item_seconds(args, 0), b.item_seconds(args, 1)
    assert a0 == a0_again and a0 != a1 and len(a0) == 256
    assert a0 == sorted(a0) and 5.0 <= a0[0] and a0[-1] <= 120.0
    assert all(abs(v * 100 - round(v * 100)) < 1e-6 for v in a0)
    batches = [a0[i:i + 64] for i in range(0, 256, 64)]
    assert all(batches[i][-1] <= batches[i + 1][0] for i in range(3))
