"""Batch sharding of the complex GEMM over the GPUs of one node.

Batch items are independent GEMMs and the batch is the outermost axis of every layout (basic,
tiled, packed and C), so rank r's share is a contiguous slice of A, B and C: no data-path
collective, no peer access.  The reference has no multi-GPU support; this is the only
distribution logic of the library and it is pure host arithmetic.
"""
from __future__ import annotations


def batch_shares(batch: int, world: int) -> list[int]:
    """Items per rank: as even as possible, the first `batch % world` ranks take one more."""
    if batch < 0 or world < 1:
        raise ValueError("batch must be >= 0 and world >= 1")
    base, extra = divmod(batch, world)
    return [base + (1 if r < extra else 0) for r in range(world)]


def batch_slice(batch: int, world: int, rank: int) -> tuple[int, int]:
    """(first item, number of items) of `rank`."""
    if not 0 <= rank < world:
        raise ValueError("rank out of range")
    shares = batch_shares(batch, world)
    return sum(shares[:rank]), shares[rank]


def _ceil(a: int, b: int) -> int:
    return -(-a // b)


def item_bytes(m: int, n: int, k: int, in_bits: int, out_bits: int, tiled: bool = False,
               dims: tuple[int, int, int] = (128, 256, 64)) -> tuple[int, int, int]:
    """Bytes of one batch item of A, B and C (tiled = the zero-padded opt layout with
    dims = (m_blk, n_blk, k_c))."""
    if tiled:
        m_blk, n_blk, k_c = dims
        kp = _ceil(k, k_c) * k_c
        a = 2 * _ceil(m, m_blk) * m_blk * kp * in_bits // 8
        b = 2 * _ceil(n, n_blk) * n_blk * kp * in_bits // 8
    else:
        row = _ceil(k * in_bits, 32) * 4 if in_bits == 1 else k * in_bits // 8
        a = 2 * m * row
        b = 2 * n * row
    return a, b, 2 * m * n * out_bits // 8


def byte_offsets(batch: int, world: int, rank: int, m: int, n: int, k: int, in_bits: int,
                 out_bits: int, tiled: bool = False,
                 dims: tuple[int, int, int] = (128, 256, 64)) -> dict:
    """Where rank's share starts in whole-batch A, B and C arrays, and how many items it has."""
    first, count = batch_slice(batch, world, rank)
    a, b, c = item_bytes(m, n, k, in_bits, out_bits, tiled, dims)
    return {"first": first, "count": count, "a": first * a, "b": first * b, "c": first * c,
            "a_bytes": count * a, "b_bytes": count * b, "c_bytes": count * c}
