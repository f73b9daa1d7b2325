"""Batch sharding of the encoder path over the GPUs of one box: independent replicas, no collective on the data path.

Sequences of an encoder batch are independent (there is no cross-sequence operator between the input blob and the last
LayerNorm), so a batch is split by sequence: every rank owns a private copy of the packed weights and runs its shard
through the same kernels.  The host scatters inputs and gathers outputs; nothing crosses NVLink.

Two plans:
  * `contiguous_shards`  equal-length batches: rank r takes rows [r*B/G, (r+1)*B/G) (remainder spread over the first
    ranks), the layout the reference's multi-instance recipe uses (one `Instance` per `NetworkConfig.device_id`,
    include/tnn/core/common.h NetworkConfig; source/tnn/device/cuda/cuda_context.cc:47-52 binds the device once).
  * `balanced_shards`    ragged batches: sequences sorted by effective FLOPs (longest first) and dealt to the rank
    with the least accumulated work, so that the slowest shard — which sets the step time — is as short as possible.
"""
import numpy as np

from . import model_synth


def contiguous_shards(batch, world):
    """Row-index arrays, one per rank; sizes differ by at most one."""
    if world < 1:
        raise ValueError("world must be >= 1")
    base, rem = divmod(int(batch), world)
    out, start = [], 0
    for r in range(world):
        n = base + (1 if r < rem else 0)
        out.append(np.arange(start, start + n, dtype=np.int64))
        start += n
    return out


def sequence_cost(length, hidden, ffn=None, with_ffn=True):
    """Effective FLOPs of one encoder layer for a sequence of `length` valid tokens (padding earns nothing)."""
    return model_synth.layer_flops(int(length), hidden, ffn, with_ffn)


def balanced_shards(lengths, world, hidden, ffn=None, with_ffn=True, max_per_rank=None):
    """Longest-processing-time-first assignment of sequences to ranks by effective FLOPs.

    Returns row-index arrays (each sorted ascending so a shard keeps the caller's order).  `max_per_rank` bounds the
    number of sequences of a shard (a fixed-shape Instance cannot take more than the batch it was built for); by
    default ceil(B / world)."""
    lengths = np.asarray(lengths).astype(np.int64)
    batch = int(lengths.shape[0])
    if world < 1:
        raise ValueError("world must be >= 1")
    cap = -(-batch // world) if max_per_rank is None else int(max_per_rank)
    if cap * world < batch:
        raise ValueError("max_per_rank * world is smaller than the batch")
    cost = np.array([sequence_cost(n, hidden, ffn, with_ffn) for n in lengths], dtype=np.float64)
    order = np.argsort(-cost, kind="stable")
    load = np.zeros(world)
    rows = [[] for _ in range(world)]
    for i in order:
        open_ranks = [r for r in range(world) if len(rows[r]) < cap]
        r = min(open_ranks, key=lambda q: (load[q], q))
        rows[r].append(int(i))
        load[r] += cost[i]
    return [np.array(sorted(r), dtype=np.int64) for r in rows]


def shard_loads(shards, lengths, hidden, ffn=None, with_ffn=True):
    lengths = np.asarray(lengths)
    return [float(sum(sequence_cost(lengths[i], hidden, ffn, with_ffn) for i in s)) for s in shards]


def scatter(array, shards):
    """Per-rank slices (copies) of a batch-major host array."""
    return [np.ascontiguousarray(array[s]) for s in shards]


def gather(parts, shards, batch):
    """Inverse of `scatter`: reassembles per-rank outputs into the caller's row order."""
    first = next(p for p in parts if p.shape[0] > 0)
    out = np.empty((batch,) + first.shape[1:], dtype=first.dtype)
    seen = np.zeros(batch, dtype=bool)
    for p, s in zip(parts, shards):
        if p.shape[0] != len(s):
            raise ValueError("a shard's output has %d rows, its plan %d" % (p.shape[0], len(s)))
        out[s] = p
        seen[s] = True
    if not seen.all():
        raise ValueError("shards do not cover the batch")
    return out
