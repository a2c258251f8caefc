"""GPU (needs >= 2 devices): tensor-parallel decode with the all-reduce fused into the row-parallel GEMVs.

Two ranks run as child processes, one per GPU; handles travel over a gloo group.  Checked: every rank ends with
a bit-identical hidden state, it matches the single-GPU run within tolerance (only the cross-rank f32 sum order
differs), and no bounded device-side wait expired."""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, q, dims):
    import torch
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from nve_b200 import cuda_kernels as ck
        from nve_b200.bench_random import ModelShape, build_state
        from nve_b200.gpu_layer import gpu_layer_forward_decode
        from nve_b200.tp import TpContext, build_tp_state, tp_layer_forward

        shape = ModelShape(*dims)
        ctx_len, seed = 16, 123
        state, imp, plan = build_tp_state(shape, seed, ctx_len, rank, world, fill_kv=False)
        tp = TpContext(rank, world, max_rows=shape.hidden)
        dist.barrier()
        # Layer by layer on the SAME input (the tensor-parallel trajectory): the two paths differ only in the order of
        # the cross-rank f32 sums, and q/k/v are column-parallel, so the K/V caches stay bit-identical; a free-running
        # comparison would mostly measure how a one-ulp difference is amplified by later int8 code flips.
        full = imp_full = None
        if rank == 0:
            full, imp_full = build_state(shape, seed, ctx_len, fill_kv=False)
        h = ck.fill_normal(shape.hidden, seed, 42, dtype=torch.float16).view(1, -1)
        worst = 0.0
        for pos in range(3):
            state.set_position(pos)
            for li in range(shape.num_layers):
                h_tp = tp_layer_forward(h, li, state, state.d_pos.data_ptr(), state.d_seqlen.data_ptr(),
                                        state.routing.use_w4a8(imp[li]))
                if rank == 0:
                    h_s = gpu_layer_forward_decode(h, li, full, pos, False, imp_full[li])
                    a, b = h_tp.double().view(-1), h_s.double().view(-1)
                    worst = max(worst, float((a - b).abs().max() / b.pow(2).mean().sqrt()))
                h = h_tp
            torch.cuda.synchronize()
        err = tp.error()
        result = {"rank": rank, "err": err, "h": h.view(torch.int16).cpu().numpy()}
        if rank == 0:
            result["worst_layer_err"] = worst
            result["routes"] = [state.routing.use_w4a8(v) for v in imp]
            # same inputs, column-parallel q/k/v: rank 0's KV heads hold the rows the single-GPU cache holds
            kv_same = all(torch.equal(full.kv_cache.k[li][:plan.local_kv_heads], state.kv_cache.k[li]) for li in
                          range(shape.num_layers))
            result["kv_same"] = bool(kv_same)
        dist.barrier()
        tp.destroy()
        q.put(result)
    finally:
        dist.destroy_process_group()


# The second shape is Llama-3.2-1B's: its two row-parallel projections have different K shards (o_proj 1024,
# down_proj 4096), hence different tile counts -- the all-reduce launches must still number their epochs in step.
@pytest.mark.parametrize("dims", [(512, 1024, 8, 2, 64, 4), (2048, 8192, 32, 8, 64, 2)])
def test_tp2_matches_single_gpu_and_ranks_agree(dims):
    import torch
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q, dims)) for r in range(2)]
    for p in procs:
        p.start()
    res = {}
    for _ in procs:
        r = q.get(timeout=300)
        res[r["rank"]] = r
    for p in procs:
        p.join(timeout=60)
    assert res[0]["err"] == 0 and res[1]["err"] == 0
    assert np.array_equal(res[0]["h"], res[1]["h"])  # replicated state is bit-identical on every rank
    assert any(res[0]["routes"]) and not all(res[0]["routes"])  # both precisions exercised
    tp = res[0]["h"].view(np.float16).astype(np.float64).reshape(-1)
    assert np.all(np.isfinite(tp))
    assert res[0]["kv_same"]
    assert res[0]["worst_layer_err"] < 1e-2  # max|tp - single| / RMS(single), worst layer, same inputs
