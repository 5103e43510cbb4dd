"""Host-side dispatcher: which GPU transcribes which utterance, which GPU keeps which stream.

The reference serves from one CPU: its server's batch thread collects requests for a short window and hands
them to `mynah_asr_transcribe_batch_ts` in waves (server/main.c:111-170, src/mynah_asr.c:599-679), and every
stream object lives in the one process (server/main.c:11-13). With one process per GPU and a full weight
replica on each, the units of work stay independent — utterances offline, streams online — so dispatch is a
partition of indices, computed identically on every rank from the lengths alone, and the only thing that
crosses ranks is the gather of the token lists by item index. No collective is on the data path.

* offline: `lpt_assign` — items sorted by length, cut into buckets of neighbouring lengths, buckets handed
  longest-first to the least-loaded rank (LPT), so that all GPUs finish together; `rank_batches` — a rank's
  items, longest first, in batches of at most `batch` (the packed batch is padding-free, so a batch only needs
  similar lengths for the lock-step decoder, not for the encoder);
* online: `sticky_streams` — stream s stays on rank s // ceil(S / N) for its whole life, because its K/V, conv
  and decoder state live in that GPU's memory;
* `gather_by_index` — merge of the per-rank results into the order of the request.
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Sequence


def item_cost(frames: float) -> float:
    """Relative cost of one utterance of `frames` encoder frames: the linears grow with T, attention with T^2
    (about a fifth of the total at 750 frames for the 1024-wide, 8-head encoders)."""
    return frames * (1.0 + frames / 3000.0)


def lpt_assign(lengths: Sequence[float], n_ranks: int, bucket: int = 64, frames_per_unit: float = 12.5) -> List[List[int]]:
    """lengths[i] = duration of item i (seconds; frames_per_unit encoder frames per unit). Returns, per rank, the
    indices of its items. Buckets hold at most `bucket` items of neighbouring length and shrink to
    len(lengths) // (4 n_ranks) when that is smaller, so that there are enough of them to balance."""
    n = len(lengths)
    if n_ranks <= 1:
        return [sorted(range(n), key=lambda i: (-lengths[i], i))]
    order = sorted(range(n), key=lambda i: (-lengths[i], i))
    size = max(1, min(bucket, n // (4 * n_ranks) if n >= 4 * n_ranks else 1))
    buckets = [order[i:i + size] for i in range(0, n, size)]
    cost = [sum(item_cost(lengths[i] * frames_per_unit) for i in b) for b in buckets]
    load = [0.0] * n_ranks
    out: List[List[int]] = [[] for _ in range(n_ranks)]
    for b in sorted(range(len(buckets)), key=lambda j: (-cost[j], j)):
        r = min(range(n_ranks), key=lambda k: (load[k], k))
        out[r].extend(buckets[b])
        load[r] += cost[b]
    return out


def imbalance(lengths: Sequence[float], parts: Iterable[Sequence[int]], frames_per_unit: float = 12.5) -> float:
    """max over ranks of the modelled load / mean load (1.0 = perfectly even)."""
    loads = [sum(item_cost(lengths[i] * frames_per_unit) for i in p) for p in parts]
    mean = sum(loads) / max(len(loads), 1)
    return max(loads) / mean if mean > 0 else 1.0


def rank_batches(items: Sequence[int], lengths: Sequence[float], batch: int = 64) -> List[List[int]]:
    """A rank's items, longest first, cut into batches of at most `batch`."""
    order = sorted(items, key=lambda i: (-lengths[i], i))
    return [order[i:i + batch] for i in range(0, len(order), batch)]


def sticky_streams(n_streams: int, n_ranks: int) -> List[List[int]]:
    """Stream s lives on one rank from open to close (its caches are in that GPU's memory): contiguous blocks of
    ceil(S / N) streams per rank."""
    per = -(-n_streams // max(n_ranks, 1))
    return [list(range(r * per, min((r + 1) * per, n_streams))) for r in range(n_ranks)]


def gather_by_index(per_rank: Iterable[Dict[int, object]], n_items: int) -> list:
    """per_rank: one {item index: result} per rank. Returns the results in request order; raises if an item is
    missing or was produced twice."""
    out: list = [None] * n_items
    seen = [False] * n_items
    for part in per_rank:
        for i, v in part.items():
            if i < 0 or i >= n_items or seen[i]:
                raise ValueError(f"item {i} gathered twice or out of range")
            out[i], seen[i] = v, True
    missing = [i for i, s in enumerate(seen) if not s]
    if missing:
        raise ValueError(f"items never produced: {missing[:8]}{'...' if len(missing) > 8 else ''}")
    return out
