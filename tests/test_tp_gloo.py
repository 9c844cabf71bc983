"""Column-parallel sharding + all-gather, and row-parallel sharding + all-reduce, over CPU ranks (gloo, world size 2 and 4). The local
compute is the CPU oracle's baseline restatement, so what is under test is the host logic: who owns
which rows, the gather, and the layout of the reassembled [m, N]."""

from __future__ import annotations

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, q):
    import sys
    from pathlib import Path

    sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
    from llm_inference_engine_b200 import tp
    from oracle import muse_proj_oracle as oracle

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.set_num_threads(1)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        layers = {"qkv_gate": (512, 256), "o": (256, 256), "router": (64, 256)}
        full = oracle.target_weights(seed=3, layers=layers)
        cp = tp.ColumnParallelProjection(oracle.cpu_prepare, oracle.cpu_kernel_fn)
        state = cp.prepare(full)
        ok = True
        for layer in layers:
            assert state[layer].shape[0] == layers[layer][0] // world
            a, b = tp.shard_bounds(layers[layer][0], world, rank)
            ok &= torch.equal(state[layer], full[layer][a:b])
            for m in (1, 3, 16):
                data = oracle.target_input(m, layer, 50 + m, layers=layers)
                got = cp.kernel_fn(data, state)
                want = oracle.cpu_kernel_fn(data, oracle.cpu_prepare(full))
                ok &= got.shape == want.shape and got.dtype == want.dtype
                ok &= torch.allclose(got.float(), want.float(), rtol=1e-2, atol=1e-3)
                part = cp.kernel_fn_local(data, state)
                ok &= torch.allclose(part.float(), want[:, a:b].float(), rtol=1e-2, atol=1e-3)
        try:
            cp.kernel_fn({"x": data["x"], "config": dict(data["config"], n=8)}, state)
            ok = False
        except ValueError:
            pass
        # row-parallel: K columns sharded, partial products summed over the group
        rp = tp.RowParallelProjection(oracle.cpu_prepare, oracle.cpu_kernel_fn)
        bf16 = {k: v for k, v in full.items() if k != "router"}
        rstate = rp.prepare(bf16)
        for layer in bf16:
            a, b = tp.shard_bounds(layers[layer][1], world, rank)
            ok &= torch.equal(rstate[layer], bf16[layer][:, a:b]) and rstate[layer].is_contiguous()
            for m in (1, 5):
                data = oracle.target_input(m, layer, 80 + m, layers=layers)
                got = rp.kernel_fn({"x": rp.local_x(data["x"]), "config": data["config"]}, rstate)
                want = oracle.fp32_reference(data, bf16)
                ok &= tuple(got.shape) == tuple(want.shape) and got.dtype == torch.bfloat16
                ok &= torch.allclose(got.float(), want, rtol=2e-2, atol=2e-2)     # BF16 partials, summed in BF16
        try:
            rp.kernel_fn({"x": rp.local_x(data["x"]), "config": dict(data["config"], k=8)}, rstate)
            ok = False
        except ValueError:
            pass
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_column_parallel_over_gloo(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(results) == [(r, True) for r in range(world)]
