"""Data-parallel sharding of the encoder workload: one process per GPU, whole sequences per rank.

The encoder layer couples tokens only inside one sequence (attention is per batch entry,
reference Attention/Attention.cu:53 indexes blockIdx.y = batch entry; Linear and LayerNorm are
per token), so sequences are independent units: ranks take contiguous blocks of sequences and
no data-path collective is needed.  The only communication is the timing protocol (barrier,
max over ranks) and an optional gather of results for checking.

Everything here is host logic over torch.distributed; it runs on `gloo` (CPU) and `nccl`.
"""
from __future__ import annotations

from dataclasses import dataclass


def shard_range(n_units: int, world: int, rank: int) -> tuple[int, int]:
    """[start, stop) of the units rank owns: contiguous blocks, the first n_units % world
    ranks one unit longer.  Covers 0..n_units exactly once over all ranks."""
    if world <= 0 or not (0 <= rank < world) or n_units < 0:
        raise ValueError(f"bad shard request: n_units={n_units} world={world} rank={rank}")
    base, extra = divmod(n_units, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_rows(n_sequences: int, seq_len: int, world: int, rank: int) -> tuple[int, int]:
    """Token-row range [start, stop) of the rank's sequences in a [n_sequences * seq_len, h]
    activation matrix."""
    a, b = shard_range(n_sequences, world, rank)
    return a * seq_len, b * seq_len


@dataclass
class Job:
    """Rank / world of this process and the torch.distributed plumbing of the timing protocol."""
    rank: int = 0
    world: int = 1
    device: object = None  # torch.device of the tensors used for the collectives

    def barrier(self) -> None:
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()

    def max_over_ranks(self, value: float) -> float:
        """The slowest rank's time: the figure a multi-GPU measurement reports."""
        if self.world == 1:
            return float(value)
        import torch
        import torch.distributed as dist
        t = torch.tensor([value], dtype=torch.float64, device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def sum_over_ranks(self, value: float) -> float:
        if self.world == 1:
            return float(value)
        import torch
        import torch.distributed as dist
        t = torch.tensor([value], dtype=torch.float64, device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(t.item())

    def throughput(self, units_this_rank: int, seconds_this_rank: float) -> float:
        """Whole-job units per second: all ranks' units over the slowest rank's time."""
        total = self.sum_over_ranks(float(units_this_rank))
        return total / self.max_over_ranks(seconds_this_rank)

    def gather_rows(self, local, n_sequences: int, seq_len: int):
        """All ranks' result rows in sequence order on every rank (checking aid, not part of
        the timed path).  `local` is this rank's [rows, h] tensor."""
        if self.world == 1:
            return local
        import torch
        import torch.distributed as dist
        sizes = [shard_rows(n_sequences, seq_len, self.world, r) for r in range(self.world)]
        most = max(b - a for a, b in sizes)
        # equal-sized pieces (uneven all_gather is not portable across backends): pad, then trim
        padded = torch.zeros((most,) + tuple(local.shape[1:]), dtype=local.dtype,
                             device=local.device)
        padded[:local.shape[0]] = local
        parts = [torch.empty_like(padded) for _ in range(self.world)]
        dist.all_gather(parts, padded)
        return torch.cat([p[:b - a] for p, (a, b) in zip(parts, sizes)], dim=0)


# ---- head-parallel mode: one long sequence over several GPUs --------------------------------
# The attention block is cut into work units (head, range of 128-query blocks).  With `world`
# ranks and `nhead` heads every head is cut into world / gcd(nhead, world) query ranges, so
# that the nhead * qsplit units divide evenly over the ranks (12 heads on 8 GPUs: 24 units of
# half a head each, 3 per rank) and every rank does the same amount of attention work.  A rank
# projects Q, K, V only for the heads its units touch (rows of the fused weight), attends over
# its units and multiplies by those heads' columns of the output projection, which yields a
# partial [seq, hidden] sum; ONE all-reduce per layer adds the partial sums (the reference has no
# multi-GPU code; this is the tensor-parallel form of Attention/Attention.h:58-142 for a batch
# that cannot be sharded).  LayerNorm and the FFN run replicated.

QUERY_BLOCK = 128  # rows of one attention work item on the GPU


def head_parallel_plan(nhead: int, world: int, seq: int) -> tuple[int, int, int]:
    """(qsplit, units_per_rank, blocks_per_unit): every head is cut into `qsplit` ranges of
    `blocks_per_unit` query blocks; rank r owns units [r * units_per_rank, (r + 1) * ...)."""
    import math
    if nhead <= 0 or world <= 0 or seq <= 0:
        raise ValueError("bad head-parallel request")
    qsplit = world // math.gcd(nhead, world)
    nblocks = -(-seq // QUERY_BLOCK)
    if nblocks % qsplit:
        raise ValueError(f"{nblocks} query blocks of a {seq}-token sequence do not split into "
                         f"{qsplit} equal ranges for {nhead} heads on {world} ranks")
    return qsplit, nhead * qsplit // world, nblocks // qsplit


def units_of_rank(nhead: int, world: int, rank: int, seq: int) -> list[tuple[int, int]]:
    """The rank's work units as (head, first query block), in global unit order (unit u = head
    u // qsplit, query range u % qsplit)."""
    qsplit, per_rank, bpu = head_parallel_plan(nhead, world, seq)
    if not (0 <= rank < world):
        raise ValueError("rank out of range")
    return [(u // qsplit, (u % qsplit) * bpu) for u in range(rank * per_rank, (rank + 1) * per_rank)]


def head_slice(nhead: int, world: int, rank: int) -> tuple[int, int]:
    """[first, last) head of the rank when heads are dealt out whole: contiguous blocks, as
    shard_range."""
    return shard_range(nhead, world, rank)


def head_rows(w: dict, nhead: int, heads) -> dict:
    """The slice of one layer's attention weights that belongs to `heads` (numpy in, numpy out):
    wqkv rows of those heads (kept in Q | K | V order), the matching bias entries, wo columns."""
    import numpy as np
    hidden, vdim = w["wo"].shape
    kdim = (w["wqkv"].shape[0] - vdim) // 2
    if kdim % nhead or vdim % nhead:
        raise ValueError("kdim and vdim must be multiples of nhead")
    dqk, dv = kdim // nhead, vdim // nhead
    heads = list(heads)
    qk = np.concatenate([np.arange(h * dqk, (h + 1) * dqk) for h in heads]) if heads else np.zeros(0, int)
    vv = np.concatenate([np.arange(h * dv, (h + 1) * dv) for h in heads]) if heads else np.zeros(0, int)
    rows = np.concatenate([qk, kdim + qk, 2 * kdim + vv]).astype(np.int64)
    return {"wqkv": np.ascontiguousarray(w["wqkv"][rows]),
            "bqkv": np.ascontiguousarray(w["bqkv"][rows]),
            "wo": np.ascontiguousarray(w["wo"][:, vv.astype(np.int64)]),
            "nhead_local": len(heads), "dh_qk": dqk, "dh_v": dv}


def head_shard_weights(w: dict, nhead: int, world: int, rank: int) -> dict:
    """Whole heads per rank: the rank's slice of the attention weights.  The output bias is kept
    on rank 0 only (it must be added once)."""
    import numpy as np
    h0, h1 = head_slice(nhead, world, rank)
    out = head_rows(w, nhead, range(h0, h1))
    out["bo"] = w["bo"] if rank == 0 else np.zeros_like(w["bo"])
    return out
