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
