"""Host-side multi-GPU logic on CPU: partition arithmetic, and the long-context decode
protocol (shard -> (O, lse) partial -> one all-gather of packed buffers -> lse merge) run
as two gloo ranks, with the oracle standing in for the device kernels.  No GPU."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def sharding(b200p):
    import importlib
    return importlib.import_module(b200p.__name__ + ".sharding")


def test_shard_range_covers_everything_once(sharding):
    for n in (0, 1, 7, 256, 512, 1000):
        for world in (1, 2, 3, 4, 8):
            spans = [sharding.shard_range(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sharding.shard_range(10, 4, 4)


def test_kv_shard_is_tile_aligned_and_complete(sharding):
    for n in (1, 100, 128, 8192, 131072, 131073, 5000):
        for world in (1, 2, 4, 8):
            parts = [sharding.kv_shard(n, r, world) for r in range(world)]
            assert sum(l for _, l in parts) == n
            pos = 0
            for off, length in parts:
                assert off == pos or length == 0
                assert off % 128 == 0 or length == 0
                pos += length
    assert sharding.kv_shard(131072, 3, 8) == (3 * 16384, 16384)
    assert sharding.packed_partial_elems(64 * 32, 128) * 4 == 1056768       # bytes per rank at BASELINE config 4


def _rank_main(rank, world, port, tmp):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    import torch
    import oracle as orc
    import __graft_entry__ as ge
    sharding = __import__("importlib").import_module(ge.load_package().__name__ + ".sharding")
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        D, N, nqh, nkvh, batch = 64, 1000, 8, 2, 3
        rng = np.random.default_rng(99)                     # every rank draws the same full problem
        q = rng.standard_normal((batch, nqh, D)).astype(np.float32)
        K = rng.standard_normal((batch, nkvh, N, D)).astype(np.float32)
        V = rng.standard_normal((batch, nkvh, N, D)).astype(np.float32)
        off, length = sharding.kv_shard(N, rank, world)
        rows = batch * nqh
        part = np.zeros(sharding.packed_partial_elems(rows, D), np.float32)
        if length > 0:
            Ks, Vs = K[:, :, off:off + length].copy(), V[:, :, off:off + length].copy()
            o = orc.cpu_decode(q, Ks, Vs, D, length, nqh, nkvh, batch=batch)
            grp = nqh // nkvh
            s = np.einsum("bhd,bhnd->bhn", q.astype(np.float64), np.repeat(Ks, grp, axis=1).astype(np.float64)) / np.sqrt(D)
            lse = np.log(np.exp(s - s.max(-1, keepdims=True)).sum(-1)) + s.max(-1)
            part[:rows * D] = o.ravel(); part[rows * D:] = lse.ravel().astype(np.float32)
        else:
            part[rows * D:] = -np.inf
        gathered = torch.zeros(world, part.size)
        dist.all_gather_into_tensor(gathered.view(-1), torch.from_numpy(part))
        g = gathered.numpy()
        merged, _ = orc.merge_lse(g[:, :rows * D].reshape(world, rows, D).copy(), g[:, rows * D:].copy())
        ref = orc.cpu_decode(q, K, V, D, N, nqh, nkvh, batch=batch).reshape(rows, D)
        err = float(np.abs(merged - ref).max())
        with open(os.path.join(tmp, f"rank{rank}.txt"), "w") as f:
            f.write(repr(err))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_long_context_protocol_on_gloo_ranks(world, tmp_path):
    import torch.multiprocessing as mp
    port = 29500 + os.getpid() % 2000 + world
    mp.spawn(_rank_main, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        err = float(open(tmp_path / f"rank{r}.txt").read())
        assert err < 1e-5, (r, err)


def test_exchange_layout(sharding):
    """Receive buffer of the peer exchange: two parities of `world` packed partials, then
    the flag words on a 256-byte boundary."""
    for rows, D, world in [(2048, 128, 8), (24, 64, 3), (1, 128, 2)]:
        slot_words, flag_off, total = sharding.exchange_layout(rows, D, world)
        assert slot_words == 2 * world * rows * (D + 1)
        assert flag_off >= slot_words and flag_off % 64 == 0 and flag_off - slot_words < 64
        assert total >= flag_off + world and total % 64 == 0
