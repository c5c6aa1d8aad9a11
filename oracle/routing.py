"""numpy restatement of the routing half of MoEFeedForward.gate_and_sort
(polkadot21/fastmoe, src/fastmoe/models/tiny_model.py:94-153) and of
prepare_grouped_metadata (src/fastmoe/kernels/ops.py:200-271).

TEST INFRASTRUCTURE — see oracle/__init__.py.

The reference sorts with torch.argsort without stable=True (tiny_model.py:112),
so the row order inside an expert segment is implementation-defined there. The
canonical order used here (and produced by the CUDA builder) is the stable one:
by expert id, then by flat routed position t*K+k. Counts and offsets do not
depend on that choice.
"""

from __future__ import annotations

import numpy as np


def topk_softmax(logits: np.ndarray, K: int):
    """torch.topk(logits, K) + softmax over the K selected values in fp32 (tiny_model.py:97-100).

    Returns (idx int64 [T, K], weights float32 [T, K]); values descend along K and
    equal values keep the lower expert id first. The caller rounds the weights to
    the activation dtype (`.type_as(x)`).
    """
    logits = np.asarray(logits, dtype=np.float32)
    # stable sort of the negated values: descending, ties by lower index
    order = np.argsort(-logits, axis=-1, kind="stable")[:, :K]
    vals = np.take_along_axis(logits, order, axis=-1)
    m = vals.max(axis=-1, keepdims=True)
    e = np.exp(vals - m, dtype=np.float32)
    w = e / e.sum(axis=-1, keepdims=True, dtype=np.float32)
    return order.astype(np.int64), w.astype(np.float32)


def build_index(topk_idx: np.ndarray, topk_w: np.ndarray, E: int, world: int = 1):
    """The index/offset builder (tiny_model.py:105-153) in canonical (stable) order.

    Returns a dict with
      reverse_map  int64 [N]  token of each sorted slot            (:121-125)
      sorted_w     [N]        gate weight of each sorted slot      (:128)
      counts       int64 [E]  torch.bincount(minlength=E)          (:138)
      offsets      int64 [E]  exclusive prefix sum of counts
      expert_counts_by_rank int64 [world, E/world]                 (:144-152)
      rank_counts  int64 [world]                                   (:150,153)
      slot_of      int32 [N]  sorted position of routed slot t*K+k (inverse of the sort)
    """
    T, K = topk_idx.shape
    flat = np.asarray(topk_idx, dtype=np.int64).reshape(-1)
    sort = np.argsort(flat, kind="stable")
    src = np.repeat(np.arange(T, dtype=np.int64), K)
    counts = np.bincount(flat, minlength=E).astype(np.int64)
    offsets = np.concatenate([[0], np.cumsum(counts)[:-1]]).astype(np.int64)
    slot_of = np.empty(T * K, dtype=np.int32)
    slot_of[sort] = np.arange(T * K, dtype=np.int32)
    by_rank = counts.reshape(world, E // world)
    return {
        "reverse_map": src[sort],
        "sorted_w": np.asarray(topk_w).reshape(-1)[sort],
        "counts": counts,
        "offsets": offsets,
        "expert_counts_by_rank": by_rank,
        "rank_counts": by_rank.sum(axis=1).astype(np.int64),
        "slot_of": slot_of,
    }


def prepare_metadata(sizes):
    """chunk_sizes int32, expert_offsets int64, max_rows, num_experts (ops.py:233-271)."""
    sizes = [int(s) for s in sizes]
    chunk_sizes = np.array(sizes, dtype=np.int32)
    offsets = np.concatenate([[0], np.cumsum(chunk_sizes, dtype=np.int64)[:-1]]).astype(np.int64)
    if len(sizes) == 0:
        offsets = np.zeros(0, np.int64)
    return chunk_sizes, offsets, (max(sizes) if sizes else 0), len(sizes)
