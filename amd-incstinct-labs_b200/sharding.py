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


def exchange_layout(rows: int, D: int, world: int):
    """Layout of one rank's receive buffer for the peer exchange, in 4-byte words:
    (slot_words, flag_offset_words, total_words).  Slots: [2 parities][world][rows*(D+1)]
    floats; the `world` int flag words follow on the next 256-byte boundary."""
    n = packed_partial_elems(rows, D)
    slot_words = 2 * world * n
    flag_off = -(-slot_words // 64) * 64
    return slot_words, flag_off, flag_off + 64 * (-(-world // 64))


class LongContextDecoder:
    """Decode over a KV sequence sharded across the ranks of `group`.

    Every rank holds all queries and its own contiguous KV shard.  step() runs the
    split-KV kernel on the shard and exchanges the normalised (O fp32, lse) partials
    (~1 MB per rank at batch 64, 32 heads, D 128), then merges them locally by lse.

    exchange = "peer": the combine kernel stores its partial straight into every rank's
      receive buffer over NVLink (peer-mapped symmetric memory) and raises a per-rank
      step flag; the merge kernel waits (bounded) for all flags.  Two launches, no
      collective call, no stream hand-over.
    exchange = "nccl": decode_partial -> all_gather_into_tensor -> merge.
    exchange = "auto": "peer" when the symmetric-memory rendezvous works, else "nccl".
    Remote memory is only ever written, never read: each GPU merges from its own memory.
    """

    def __init__(self, pkg, dist, batch: int, n_q_heads: int, D: int, dtype, device, group=None, exchange: str = "auto"):
        import torch
        self.pkg, self.dist, self.group = pkg, dist, group
        self.world = dist.get_world_size(group) if dist is not None and dist.is_initialized() else 1
        self.rows, self.D = batch * n_q_heads, D
        n = packed_partial_elems(self.rows, D)
        self.out = torch.empty((batch, n_q_heads, D), dtype=dtype, device=device)
        self.workspace = None
        self.seq = 0
        self.exchange = "none" if self.world == 1 else exchange
        if self.exchange in ("auto", "peer"):
            try:
                self._setup_peer(torch, device)
                self.exchange = "peer"
            except Exception:
                if self.exchange == "peer":
                    raise
                self.exchange = "nccl"
            if exchange == "auto":
                # all ranks must take the same path: agree on the weakest
                ok = torch.tensor([1 if self.exchange == "peer" else 0], device=device)
                dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
                self.exchange = "peer" if int(ok.item()) == 1 else "nccl"
        if self.exchange == "nccl":
            self.part = torch.empty(n, dtype=torch.float32, device=device)
            self.gathered = torch.empty((self.world, n), dtype=torch.float32, device=device)
            self.o_view = self.part[: self.rows * D].view(batch, n_q_heads, D)
            self.lse_view = self.part[self.rows * D:].view(batch, n_q_heads)

    def _setup_peer(self, torch, device):
        import torch.distributed._symmetric_memory as symm
        dist = self.dist
        group = self.group if self.group is not None else dist.group.WORLD
        rank = dist.get_rank(group)
        if self.world > self.pkg.MAX_PEERS:
            raise ValueError("too many ranks for the peer exchange")
        _, flag_off, total = exchange_layout(self.rows, self.D, self.world)
        self.recv = symm.empty(total, dtype=torch.float32, device=device)
        self.recv.zero_()
        handle = symm.rendezvous(self.recv, group)
        ptrs = [int(p) for p in handle.buffer_ptrs]
        if len(ptrs) != self.world or any(p == 0 for p in ptrs):
            raise RuntimeError("symmetric-memory rendezvous gave no peer pointers")
        self._handle = handle
        self.counter = torch.zeros(1, dtype=torch.int32, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self.px = self.pkg.peer_exchange(rank, self.world, ptrs, [p + 4 * flag_off for p in ptrs], self.counter.data_ptr())
        torch.cuda.synchronize(device)
        dist.barrier(group=self.group)                   # every buffer is zero before anyone stores into it

    def step(self, q, K_shard, V_shard, n_keys=None):
        pkg = self.pkg
        if self.workspace is None:
            self.workspace = pkg.decode_workspace(q, K_shard, n_keys)
        if self.world == 1:
            return pkg.decode(q, K_shard, V_shard, N=n_keys, out=self.out, workspace=self.workspace)
        if self.exchange == "peer":
            self.seq += 1
            pkg.decode_push(q, K_shard, V_shard, self.px, self.seq, N=n_keys, workspace=self.workspace)
            return pkg.merge_lse_wait(self.px, self.seq, self.rows, self.D, self.out, self.status)
        pkg.decode_partial(q, K_shard, V_shard, N=n_keys, workspace=self.workspace, out=self.o_view, lse=self.lse_view)
        self.dist.all_gather_into_tensor(self.gathered.view(-1), self.part, group=self.group)
        return pkg.merge_lse_packed(self.gathered, self.rows, self.D, self.out)

    def check(self):
        """Raise if a bounded wait of the peer exchange ever ran out (reads one word back)."""
        if self.exchange == "peer" and int(self.status.item()) != 0:
            raise RuntimeError("peer exchange: a wait for another rank's partial ran out")
