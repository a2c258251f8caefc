"""CPU (gloo, world_size 2): host-side tensor-parallel logic -- shard planning, handle exchange, and the claim
that sharding preserves int8 codes and per-block integer accumulators (checked with the oracle)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from nve_b200.bench_random import SHAPES, ModelShape
from nve_b200.tp import exchange_handles, plan_shards


def test_shard_plan_covers_every_projection_once():
    for name, world in (("8b", 1), ("8b", 2), ("8b", 4), ("8b", 8), ("70b", 8), ("1b", 4)):
        shape = SHAPES[name]
        dims = {"q": (shape.num_heads * shape.head_dim, shape.hidden), "k": (shape.num_kv_heads * shape.head_dim, shape.hidden),
                "o": (shape.hidden, shape.num_heads * shape.head_dim), "gate": (shape.ffn, shape.hidden),
                "down": (shape.hidden, shape.ffn)}
        for proj, (N, K) in dims.items():
            cover = np.zeros((N // 8, K // 32), np.int32)
            for r in range(world):
                row0, rows, col0, cols, full_k = plan_shards(shape, r, world).slices[proj]
                assert full_k == K and cols % 32 == 0 and col0 % 32 == 0 and rows % 8 == 0
                cover[row0 // 8:(row0 + rows) // 8, col0 // 32:(col0 + cols) // 32] += 1
            assert np.all(cover == 1)
    with pytest.raises(ValueError):
        plan_shards(SHAPES["8b"], 0, 3)
    with pytest.raises(ValueError):
        plan_shards(ModelShape(4096, 14336, 32, 8, 128, 32), 0, 16)


def test_row_parallel_split_preserves_codes_and_accumulators(orc):
    """o_proj / down_proj split over K: local activation groups coincide with the global ones, so the int8 codes,
    scales and I[n, b] of every shard equal the unsharded ones, and the rank-ordered f32 sum stays in tolerance."""
    N, K, world = 64, 1024, 4
    W = orc.fill_normal(N * K, 3, 1, scale=0.02).reshape(N, K)
    nib, sc = orc.extract_for_gpu(orc.quantize_q4(W))
    x16 = orc.to_act16(orc.fill_normal(K, 3, 2))
    xq, xs = orc.quantize_q8(x16)
    I = orc.w4a8_idot(xq, nib)
    y_full = orc.w4a8_matvec_f64(xq, xs, nib, sc)
    ks = K // world
    total = np.zeros(N, np.float32)
    for r in range(world):
        xq_r, xs_r = orc.quantize_q8(x16[r * ks:(r + 1) * ks])
        assert np.array_equal(xq_r, xq[r * ks:(r + 1) * ks]) and np.array_equal(xs_r, xs[r * ks // 32:(r + 1) * ks // 32])
        nib_r = np.ascontiguousarray(nib[:, r * ks // 2:(r + 1) * ks // 2])
        sc_r = np.ascontiguousarray(sc[:, r * ks // 32:(r + 1) * ks // 32])
        assert np.array_equal(orc.w4a8_idot(xq_r, nib_r), I[:, r * ks // 32:(r + 1) * ks // 32])
        part = orc.w4a8_matvec_b200(xq_r, xs_r, nib_r, sc_r)
        total = part if r == 0 else (total + part).astype(np.float32)  # the kernel adds ranks in ascending order
    assert np.max(np.abs(total - y_full)) / np.sqrt(np.mean(y_full**2)) < 1e-5


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        handle = bytes([rank + 1]) * 64
        allh = exchange_handles(handle, world)
        ok = len(allh) == 64 * world and all(allh[64 * r:64 * (r + 1)] == bytes([r + 1]) * 64 for r in range(world))
        # max-over-ranks timing reduction used by the benchmark
        t = torch.tensor([float(rank + 1)], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        q.put((rank, ok and t.item() == float(world)))
    finally:
        dist.destroy_process_group()


def test_handle_exchange_gloo_world2():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(r for r, _ in res) == [0, 1] and all(ok for _, ok in res)
