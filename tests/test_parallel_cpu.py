"""Column-parallel sharding on CPU ranks (gloo, world size 2 and 4): shard slicing, the
all-gather layout and rank-count validation.  The shard compute is injected (the CPU
oracle), so only the host-side logic of bittorch_b200.parallel is under test here."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, tmpdir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import oracle
        from bittorch_b200.parallel import ColumnParallelTernaryLinear, column_range, shard_packed_columns

        g = torch.Generator().manual_seed(0)            # identical on every rank
        k, n, m = 100, 48 * world, 5
        w = torch.randn(n, k, generator=g)
        bias = torch.randn(n, generator=g)
        x = torch.randn(m, k, generator=g)
        codes, scale = oracle.ternarize(w.numpy(), 0.05)
        packed = torch.from_numpy(oracle.pack_transposed(codes))
        scale_t = torch.from_numpy(scale)

        wp, sc, b = shard_packed_columns(packed, scale_t, bias, rank, world)
        n0, n1 = column_range(n, rank, world)
        assert wp.is_contiguous() and wp.shape == ((k + 3) // 4, n1 - n0)
        assert np.array_equal(oracle.unpack_transposed(wp.numpy(), k), codes[n0:n1])

        def local(x2d):
            q, sx = oracle.act_quant(x2d.numpy())
            return torch.from_numpy(oracle.packed_forward_i8(q, sx, wp.numpy(), k, sc.numpy(), b.numpy()))

        layer = ColumnParallelTernaryLinear.from_full(k, packed, scale_t, bias, local_linear=local)
        assert layer.rank == rank and layer.world_size == world
        y = layer(x.reshape(1, m, k))
        q, sx = oracle.act_quant(x.numpy())
        y_ref = oracle.packed_forward_i8(q, sx, packed.numpy(), k, scale, bias.numpy())
        assert y.shape == (1, m, n)
        assert np.array_equal(y.reshape(m, n).numpy(), y_ref)

        with pytest.raises(ValueError, match="not divisible"):
            column_range(n + 1, rank, world)
        with pytest.raises(ValueError, match="shard has shape"):
            ColumnParallelTernaryLinear(k, n, packed, scale_t, bias, local_linear=local)
        open(os.path.join(tmpdir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_column_parallel_gather(world, tmp_path, oracle):
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all(os.path.exists(tmp_path / f"ok{r}") for r in range(world))


def test_single_process_is_identity_sharding():
    from bittorch_b200.parallel import column_range, shard_packed_columns

    assert column_range(64, 0, 1) == (0, 64)
    with pytest.raises(ValueError):
        column_range(64, 2, 2)
    p = torch.arange(24, dtype=torch.uint8).reshape(3, 8)
    wp, sc, b = shard_packed_columns(p, torch.arange(8.0), None, 1, 2)
    assert torch.equal(wp, p[:, 4:]) and torch.equal(sc, torch.arange(4.0, 8.0)) and b is None
