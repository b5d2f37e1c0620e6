"""The N>1 host path on CPU: two gloo ranks shard a GEMM by rows, compute their shards with the
CPU oracle, complete C with one in-place all-gather, and every rank must hold the full result."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_bounds():
    sys.path.insert(0, ROOT)
    from cantors_gift_b200.sharding import equal_shard, padded_rows, shard_bounds
    for total, world in [(4096, 8), (10, 3), (2, 4), (0, 2), (7, 7)]:
        spans = [shard_bounds(total, world, r) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == total
        assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
        sizes = [hi - lo for lo, hi in spans]
        assert max(sizes) - min(sizes) <= 1 and sizes == sorted(sizes, reverse=True)
        per, padded = padded_rows(total, world)
        assert padded >= total and padded - total < world and per * world == padded
        eq = [equal_shard(total, world, r) for r in range(world)]
        assert eq[-1][1] == total and all(hi - lo <= per for lo, hi in eq)
    with pytest.raises(ValueError):
        shard_bounds(4, 2, 2)


def _worker(rank, world, port, out_queue):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    from cantors_gift_b200.sharding import padded_rows
    from oracle import oracle as O
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        M, N, K = 50, 24, 40            # M not a multiple of world: padded shards
        rng = np.random.default_rng(2)  # same data on every rank
        A = rng.standard_normal((M, K), dtype=np.float32)
        B = rng.standard_normal((K, N), dtype=np.float32)
        bias = rng.standard_normal(N, dtype=np.float32)
        per, padded = padded_rows(M, world)
        Apad = np.zeros((padded, K), dtype=np.float32)
        Apad[:M] = A
        C = torch.zeros(padded, N)
        d = O.make_gemm_desc(per, N, K, O.F32, O.F32, epilogue="bias_gelu_tanh")
        shard = O.gemm(d, np.ascontiguousarray(Apad[rank * per:(rank + 1) * per]), B, bias=bias).reshape(per, N)
        C[rank * per:(rank + 1) * per] = torch.from_numpy(shard)
        # in-place all-gather: every rank's slot of the full buffer is its send buffer
        dist.all_gather_into_tensor(C.view(-1), C[rank * per:(rank + 1) * per].reshape(-1).clone())
        full = O.gemm(O.make_gemm_desc(M, N, K, O.F32, O.F32, epilogue="bias_gelu_tanh"), A, B, bias=bias).reshape(M, N)
        ok = np.array_equal(C[:M].numpy().view(np.uint32), full.view(np.uint32))
        t = torch.tensor([1.0 if ok else 0.0])
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        out_queue.put((rank, bool(t.item() == 1.0)))
    finally:
        dist.destroy_process_group()


def test_two_rank_row_sharded_gemm_allgather():
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(results) == [(0, True), (1, True)]
