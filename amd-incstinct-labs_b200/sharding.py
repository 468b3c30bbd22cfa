"""Multi-GPU host logic: one process per GPU, work sharded with no data-path
collective, except long-context decode, whose KV sequence is split across ranks
and whose partial results (O, lse) are all-gathered once and merged locally.

The reference is single-GPU (cdna3-prims/runtime/design.md:18-22); the merge is its
split-KV merge (cdna3-prims/include/cdna3/detail/fa_decode_kernel.hpp:75-92) applied
across GPUs instead of across the waves of one block.
"""
from __future__ import annotations


def shard_range(n_units: int, rank: int, world: int):
    """Contiguous, balanced [start, stop) of `n_units` independent units (segments,
    (batch, head) pairs, sequences) for `rank`; the first n_units % world ranks get one more."""
    if not (0 <= rank < world):
        raise ValueError("rank out of range")
    base, extra = divmod(n_units, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def kv_shard(n_keys: int, rank: int, world: int, align: int = 128):
    """(key_offset, length) of rank's contiguous chunk of a KV sequence of n_keys keys,
    chunk boundaries on multiples of `align` keys (the decode kernel's tile); trailing
    ranks may get a short or empty chunk."""
    if not (0 <= rank < world):
        raise ValueError("rank out of range")
    per = -(-n_keys // world)
    per = -(-per // align) * align
    start = min(rank * per, n_keys)
    return start, min(per, n_keys - start)


def packed_partial_elems(rows: int, D: int) -> int:
    """Floats in one rank's packed partial: O [rows, D] followed by lse [rows]."""
    return rows * (D + 1)


class LongContextDecoder:
    """Decode over a KV sequence sharded across the ranks of `group`.

    Every rank holds all queries and its own contiguous KV shard.  step() runs the
    split-KV kernel on the shard, writing normalised O (fp32) and lse into one packed
    buffer, all-gathers the packed buffers (NCCL over NVLink; ~1 MB per rank at batch 64,
    32 heads, D 128) into local memory, and merges them with the lse combine kernel.
    Remote data is only ever read after the collective has placed it in this GPU's memory.
    """

    def __init__(self, pkg, dist, batch: int, n_q_heads: int, D: int, dtype, device, group=None):
        import torch
        self.pkg, self.dist, self.group = pkg, dist, group
        self.world = dist.get_world_size(group) if dist is not None and dist.is_initialized() else 1
        self.rows, self.D = batch * n_q_heads, D
        n = packed_partial_elems(self.rows, D)
        self.part = torch.empty(n, dtype=torch.float32, device=device)
        self.gathered = torch.empty((self.world, n), dtype=torch.float32, device=device)
        self.o_view = self.part[: self.rows * D].view(batch, n_q_heads, D)
        self.lse_view = self.part[self.rows * D:].view(batch, n_q_heads)
        self.out = torch.empty((batch, n_q_heads, D), dtype=dtype, device=device)
        self.workspace = None

    def step(self, q, K_shard, V_shard, n_keys=None):
        pkg = self.pkg
        if self.workspace is None:
            self.workspace = pkg.decode_workspace(q, K_shard, n_keys)
        if self.world == 1:
            return pkg.decode(q, K_shard, V_shard, N=n_keys, out=self.out, workspace=self.workspace)
        pkg.decode_partial(q, K_shard, V_shard, N=n_keys, workspace=self.workspace, out=self.o_view, lse=self.lse_view)
        self.dist.all_gather_into_tensor(self.gathered.view(-1), self.part, group=self.group)
        return pkg.merge_lse_packed(self.gathered, self.rows, self.D, self.out)
