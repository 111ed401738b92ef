"""The multi-GPU path on CPU: world_size-2 gloo ranks shard a batch exactly as bench.py's ranks
do (ccglib_b200.sharding), each computes its slice with the CPU oracle from its byte offsets into
the whole-batch arrays, and the gathered result must equal the unsharded oracle result."""
import os
import socket

import numpy as np
import pytest

import oracle_util as ou
from ccglib_b200 import sharding


def test_shares_cover_the_batch_exactly():
    for batch in (1, 2, 7, 64, 4096):
        for world in (1, 2, 3, 4, 8):
            shares = sharding.batch_shares(batch, world)
            assert sum(shares) == batch and max(shares) - min(shares) <= 1
            cursor = 0
            for r in range(world):
                first, count = sharding.batch_slice(batch, world, r)
                assert first == cursor and count == shares[r]
                cursor += count
    assert sharding.batch_shares(64, 8) == [8] * 8
    with pytest.raises(ValueError):
        sharding.batch_slice(4, 2, 2)


def test_item_bytes_match_the_layouts():
    assert sharding.item_bytes(8192, 8192, 8192, 16, 32) == (2 * 8192 * 8192 * 2,) * 2 + (
        2 * 8192 * 8192 * 4,)
    # 1-bit rows are whole 32-bit words
    assert sharding.item_bytes(4, 6, 70, 1, 32) == (2 * 4 * 12, 2 * 6 * 12, 2 * 4 * 6 * 4)
    # tiled layout is padded to whole tiles
    a, b, c = sharding.item_bytes(300, 200, 100, 16, 32, tiled=True, dims=(128, 256, 64))
    assert a == 2 * 384 * 128 * 2 and b == 2 * 256 * 128 * 2 and c == 2 * 300 * 200 * 4


def test_c_abi_share_equals_the_python_helper():
    """ccglib_b200_batch_share (what a C or C++ caller uses) against ccglib_b200.sharding."""
    from ccglib_b200 import capi

    cases = [(64, 8192, 8192, 8192, capi.FLOAT16, capi.FLOAT32, capi.OPT, 16, 32),
             (7, 300, 200, 100, capi.FLOAT16, capi.FLOAT16, capi.OPT, 16, 16),
             (5, 40, 72, 70, capi.INT1, capi.INT32, capi.BASIC, 1, 32),
             (32, 4096, 4096, 16384, capi.FLOAT8E4M3, capi.FLOAT32, capi.BASIC, 8, 32)]
    for batch, m, n, k, tin, tout, variant, in_bits, out_bits in cases:
        dims = capi.gemm_dims(tin, tout, variant)
        for world in (1, 2, 3, 8):
            for rank in range(world):
                want = sharding.byte_offsets(batch, world, rank, m, n, k, in_bits, out_bits,
                                             tiled=variant == capi.OPT, dims=dims)
                assert capi.batch_share(batch, m, n, k, tin, tout, variant, world, rank) == want
    with pytest.raises(capi.Error):
        capi.batch_share(4, 8, 8, 8, capi.FLOAT16, capi.FLOAT32, capi.BASIC, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, batch, M, N, K, out):
    import torch
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(77)  # every rank regenerates the same whole-batch inputs
    a = ou.random_storage(rng, (batch, 2, M, K), ou.F16, "uniform")
    b = ou.random_storage(rng, (batch, 2, N, K), ou.F16, "uniform")
    off = sharding.byte_offsets(batch, world, rank, M, N, K, 16, 32)
    a_mine = a.reshape(-1).view(np.uint8)[off["a"]:off["a"] + off["a_bytes"]].view(np.float16)
    b_mine = b.reshape(-1).view(np.uint8)[off["b"]:off["b"] + off["b_bytes"]].view(np.float16)
    a_mine = a_mine.reshape(off["count"], 2, M, K)
    b_mine = b_mine.reshape(off["count"], 2, N, K)
    c_mine = np.stack([ou.port_gemm(ou.F16, ou.F32, a_mine[i], b_mine[i], None, M, N, K)
                       for i in range(off["count"])]) if off["count"] else np.zeros((0, 2, M, N),
                                                                                    np.float32)
    # out-of-band gather of C (not part of the timed path): pad to the largest share
    cap = max(sharding.batch_shares(batch, world))
    padded = torch.zeros((cap, 2, M, N), dtype=torch.float32)
    padded[:off["count"]] = torch.from_numpy(c_mine)
    gathered = [torch.zeros_like(padded) for _ in range(world)]
    dist.all_gather(gathered, padded)
    # the timing reduction bench.py does: max over ranks
    t = torch.tensor([float(rank + 1)])
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        parts = [gathered[r][:sharding.batch_shares(batch, world)[r]].numpy() for r in range(world)]
        np.save(out, np.concatenate(parts))
        assert float(t) == world
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("batch", [5, 4])
def test_two_gloo_ranks_reproduce_the_unsharded_result(tmp_path, batch):
    import torch.multiprocessing as mp

    world, M, N, K = 2, 24, 40, 32
    out = str(tmp_path / "c.npy")
    mp.spawn(_rank_main, args=(world, _free_port(), batch, M, N, K, out), nprocs=world, join=True)
    rng = np.random.default_rng(77)
    a = ou.random_storage(rng, (batch, 2, M, K), ou.F16, "uniform")
    b = ou.random_storage(rng, (batch, 2, N, K), ou.F16, "uniform")
    want = np.stack([ou.port_gemm(ou.F16, ou.F32, a[i], b[i], None, M, N, K)
                     for i in range(batch)])
    assert np.array_equal(np.load(out), want)
