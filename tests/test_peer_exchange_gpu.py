"""The fused (O, lse) exchange of sharded decode, on ONE GPU: the ranks run one after the
other in stream order, their receive buffers all local, so every flag a merge waits for
was already raised by a finished kernel.  (The concurrent form needs one GPU per rank and
is exercised by the multi-GPU bench.)  Also the bounded wait: a flag nothing raises makes
the merge give up with a status word, and the context stays usable."""
import importlib

import numpy as np
import pytest

import oracle as orc

pytestmark = pytest.mark.gpu


def dev16(torch, f32):
    return torch.from_numpy(np.ascontiguousarray(f32)).cuda().bfloat16()


def make_ranks(b200p, torch, world, rows, D):
    sharding = importlib.import_module(b200p.__name__ + ".sharding")
    _, flag_off, total = sharding.exchange_layout(rows, D, world)
    bufs = [torch.zeros(total, dtype=torch.float32, device="cuda") for _ in range(world)]
    counters = [torch.zeros(1, dtype=torch.int32, device="cuda") for _ in range(world)]
    slots = [b.data_ptr() for b in bufs]
    flags = [b.data_ptr() + 4 * flag_off for b in bufs]
    pxs = [b200p.peer_exchange(r, world, slots, flags, counters[r].data_ptr()) for r in range(world)]
    return bufs, counters, pxs, flag_off


@pytest.mark.parametrize("world,D", [(2, 128), (4, 128), (8, 128), (3, 64)])
def test_push_then_merge_equals_whole(b200p, torch_cuda, world, D):
    torch = torch_cuda
    rng = np.random.default_rng(31 + world)
    N, nqh, nkvh, batch = 128 * 3 * world, 8, 2, 3
    q = dev16(torch, rng.standard_normal((batch, nqh, D)).astype(np.float32))
    K = dev16(torch, rng.standard_normal((batch, nkvh, N, D)).astype(np.float32))
    V = dev16(torch, rng.standard_normal((batch, nkvh, N, D)).astype(np.float32))
    rows = batch * nqh
    bufs, counters, pxs, flag_off = make_ranks(b200p, torch, world, rows, D)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    per = N // world
    ref = orc.cpu_decode(q.float().cpu().numpy(), K.float().cpu().numpy(), V.float().cpu().numpy(), D, N, nqh, nkvh,
                         batch=batch, threads=8)
    whole = b200p.decode(q, K, V)
    for seq in (1, 2, 3):                                   # both parities, counters reused
        for r in range(world):
            b200p.decode_push(q, K, V, pxs[r], seq, N=per, key_offset=r * per)
        for r in range(world):
            out = torch.empty((batch, nqh, D), dtype=torch.bfloat16, device="cuda")
            b200p.merge_lse_wait(pxs[r], seq, rows, D, out, status, wait_ns=200_000_000)
            assert np.abs(out.float().cpu().numpy() - ref).max() < 2e-2
            assert (out.float() - whole.float()).abs().max().item() < 1e-2
        assert int(status.item()) == 0
        for r in range(world):
            assert int(counters[r].item()) == 0
            f = bufs[r][flag_off: flag_off + world].view(torch.int32)
            assert f.tolist() == [seq] * world


def test_push_matches_decode_partial(b200p, torch_cuda):
    """The pushed slot holds exactly what decode_partial returns for the same shard."""
    torch = torch_cuda
    rng = np.random.default_rng(5)
    D, N, nqh, nkvh, batch, world = 128, 1024, 8, 2, 2, 2
    q = dev16(torch, rng.standard_normal((batch, nqh, D)).astype(np.float32))
    K = dev16(torch, rng.standard_normal((batch, nkvh, N, D)).astype(np.float32))
    V = dev16(torch, rng.standard_normal((batch, nkvh, N, D)).astype(np.float32))
    rows = batch * nqh
    n = rows * (D + 1)
    bufs, _, pxs, _ = make_ranks(b200p, torch, world, rows, D)
    per = N // world
    b200p.decode_push(q, K, V, pxs[1], 1, N=per, key_offset=per)           # rank 1, odd step -> slot [1][1]
    o, lse = b200p.decode_partial(q, K, V, N=per, key_offset=per)
    for g in range(world):
        slot = bufs[g][(1 * world + 1) * n: (1 * world + 2) * n]
        assert torch.equal(slot[: rows * D].view(batch, nqh, D), o)
        assert torch.equal(slot[rows * D:].view(batch, nqh), lse)
        assert float(bufs[g][: (1 * world + 1) * n].abs().sum()) == 0.0       # nothing else touched


def test_wait_runs_out_and_reports(b200p, torch_cuda):
    """Rank 1 never pushes: rank 0's merge gives up after the stated limit, sets the status
    word and returns; later launches on the same context work."""
    torch = torch_cuda
    D, nqh, batch, world = 128, 8, 2, 2
    rows = batch * nqh
    _, _, pxs, _ = make_ranks(b200p, torch, world, rows, D)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = torch.empty((batch, nqh, D), dtype=torch.bfloat16, device="cuda")
    b200p.merge_lse_wait(pxs[0], 1, rows, D, out, status, wait_ns=20_000_000)     # 20 ms
    torch.cuda.synchronize()
    assert int(status.item()) == 1
    x = torch.arange(64 * 4, dtype=torch.float32, device="cuda")
    assert b200p.segreduce(x, "sum").cpu().tolist() == [float(sum(range(64 * i, 64 * i + 64))) for i in range(4)]


def test_argument_errors(b200p, torch_cuda):
    torch = torch_cuda
    D, nqh, batch, world = 128, 8, 1, 2
    rows = batch * nqh
    _, _, pxs, _ = make_ranks(b200p, torch, world, rows, D)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = torch.empty((batch, nqh, D), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(b200p.B200PError):
        b200p.merge_lse_wait(pxs[0], 0, rows, D, out, status)                    # seq starts at 1
    with pytest.raises(ValueError):
        b200p.peer_exchange(0, 17, [1] * 17, [1] * 17, 1)
    bad = b200p.peer_exchange(0, 2, [out.data_ptr(), 0], [out.data_ptr(), out.data_ptr()], status.data_ptr())
    with pytest.raises(b200p.B200PError):
        b200p.merge_lse_wait(bad, 1, rows, D, out, status)
