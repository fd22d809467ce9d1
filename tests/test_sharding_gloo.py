"""Column (N) sharding of the layer over ranks, exercised with world_size 2 on CPU (gloo): every rank generates only its
own shard, the shards tile the full tensors, and per-rank results of the path's arithmetic (taken from the CPU oracle
here; the GPU kernels are checked against the same oracle elsewhere) concatenate to the unsharded result with no
collective on the data path."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HID, INTER, M = 256, 512, 8  # a small layer with the benchmark's structure


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from flashnn_b200 import workloads as W
        from oracle import quant_oracle as O
        full = W.ffn_layer(M, 0, 1, HID, INTER)
        mine = W.ffn_layer(M, rank, world, HID, INTER)
        n_gu, n_dn = 2 * INTER // world, HID // world
        ok = torch.equal(mine["w_gu"], full["w_gu"][rank * n_gu:(rank + 1) * n_gu])
        ok &= torch.equal(mine["w_dn"], full["w_dn"][rank * n_dn:(rank + 1) * n_dn])
        ok &= torch.equal(mine["col_gu"], full["col_gu"][rank * n_gu:(rank + 1) * n_gu])
        ok &= torch.equal(mine["x"], full["x"]) and torch.equal(mine["h"], full["h"])  # activations are replicated
        q, s = O.dynamic_quantize(mine["x"])  # recomputed on every rank
        y = O.gemm_a8w8(q, mine["w_gu"], s.float(), mine["col_gu"], torch.bfloat16)
        # gather only to compare with the unsharded result (not part of the data path)
        parts = [torch.empty_like(y) for _ in range(world)]
        dist.all_gather(parts, y)
        if rank == 0:
            ref = O.gemm_a8w8(q, full["w_gu"], s.float(), full["col_gu"], torch.bfloat16)
            ok &= torch.equal(torch.cat(parts, dim=1).view(torch.int16), ref.view(torch.int16))
        flag = torch.tensor([1 if ok else 0])
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if rank == 0:
            out.put(int(flag.item()))
    finally:
        dist.destroy_process_group()


def test_two_rank_column_sharding():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=240)
        assert p.exitcode == 0
    assert out.get(timeout=10) == 1


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_shards_tile_the_full_layer(world):
    from flashnn_b200 import workloads as W
    full = W.ffn_layer(2, 0, 1, 64, 2048)  # 4096 gate/up rows: several 1024-row generator blocks, shard edges inside blocks
    rows = torch.cat([W.ffn_layer(2, r, world, 64, 2048)["w_gu"] for r in range(world)])
    assert torch.equal(rows, full["w_gu"])
    cols = torch.cat([W.ffn_layer(2, r, world, 64, 2048)["col_dn"] for r in range(world)])
    assert torch.equal(cols, full["col_dn"])
