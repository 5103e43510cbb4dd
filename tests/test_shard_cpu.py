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


# ---------------------------------------------------------------- dispatcher (mynah-asr_b200/dispatch.py)
def _dispatch():
    spec = importlib.util.spec_from_file_location("dispatch_mod", os.path.join(ROOT, "mynah-asr_b200", "dispatch.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _lengths():
    """The seeded 256 lengths of the length-bucketed workload (bench.py: U[5, 120] s, seed 4000)."""
    import numpy as np
    rng = np.random.default_rng(4000)
    return [float(v) for v in np.sort(np.round(rng.uniform(5.0, 120.0, 256), 2))]


def test_lpt_assignment_is_a_partition_and_balanced():
    d = _dispatch()
    lens = _lengths()
    for world in (1, 2, 4, 8):
        parts = d.lpt_assign(lens, world, bucket=64)
        flat = sorted(i for p in parts for i in p)
        assert flat == list(range(256)) and len(parts) == world          # every item exactly once
        assert d.imbalance(lens, parts) <= 1.05, (world, d.imbalance(lens, parts))
        for p in parts:                                                  # a rank's batches: at most 64, longest first
            bs = d.rank_batches(p, lens, 64)
            assert all(len(b) <= 64 for b in bs) and [i for b in bs for i in b] == sorted(p, key=lambda i: (-lens[i], i))
    # a contiguous split of the sorted list (what a naive shard does) is far from balanced
    naive = [list(range(r * 32, (r + 1) * 32)) for r in range(8)]
    assert d.imbalance(lens, naive) > 1.5
    # degenerate inputs
    assert d.lpt_assign([], 4) == [[], [], [], []]
    assert sorted(i for p in d.lpt_assign([3.0, 1.0, 2.0], 8) for i in p) == [0, 1, 2]


def test_sticky_streams_and_gather():
    d = _dispatch()
    for S, world in ((512, 8), (512, 1), (10, 4), (3, 8)):
        parts = d.sticky_streams(S, world)
        assert [s for p in parts for s in p] == list(range(S))
        assert max(len(p) for p in parts) - min(len(p) for p in parts if p or True) <= -(-S // world)
    assert [len(p) for p in d.sticky_streams(512, 8)] == [64] * 8
    assert d.gather_by_index([{1: "b", 0: "a"}, {2: "c"}], 3) == ["a", "b", "c"]
    with pytest.raises(ValueError):
        d.gather_by_index([{0: "a"}, {0: "b"}], 2)                       # produced twice
    with pytest.raises(ValueError):
        d.gather_by_index([{0: "a"}], 2)                                 # never produced


def _dispatch_rank_main(rank, world, port, out_dir):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    d = _dispatch()
    lens = _lengths()
    parts = d.lpt_assign(lens, world, bucket=64)                         # same on every rank: computed from the lengths alone
    mine = parts[rank]
    result = {i: ([i, int(lens[i] * 100)], [rank]) for i in mine}        # stand-in for (tokens, frames) of item i
    gathered = [None] * world
    dist.all_gather_object(gathered, result)
    if rank == 0:
        merged = d.gather_by_index(gathered, len(lens))
        ok = all(merged[i][0] == [i, int(lens[i] * 100)] for i in range(len(lens)))
        ok = ok and {r for m in merged for r in m[1]} == set(range(world))
        open(os.path.join(out_dir, "ok"), "w").write("1" if ok else "0")
    dist.destroy_process_group()


def test_two_rank_gloo_dispatch_and_gather(tmp_path):
    mp = pytest.importorskip("torch.multiprocessing")
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    mp.spawn(_dispatch_rank_main, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert open(os.path.join(str(tmp_path), "ok")).read() == "1"
