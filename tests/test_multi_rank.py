"""World-size-2 checks of the batch-sharding harness on CPU (gloo): each rank runs its
shard of a graph (through the CPU oracle, since there is no GPU here), outputs are
gathered / filter gradients all-reduced, and the result must equal the unsharded run."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, case, out_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from fusilli_b200 import sharding as sh
    from fusilli_b200 import workloads as wl
    from fusilli_b200.graph import DataType
    from oracle import fusilli_oracle as orc

    rng = np.random.default_rng(7)  # same stream on every rank: the full problem
    if case == "matmul":
        B, M, N, K = 5, 24, 16, 32  # 5 matrices over 2 ranks: uneven shards
        a = rng.normal(0, 0.5, (B, M, K)).astype(np.float32)
        b = rng.normal(0, 0.5, (B, K, N)).astype(np.float32)
        bias = rng.normal(0, 0.5, (N,)).astype(np.float32)
        lo, hi = sh.shard_range(B, rank, world)
        g, ins, out = wl.matmul_bias(hi - lo, M, N, K, DataType.Float)
        res = orc.execute(g, {ins["a"]: a[lo:hi].ravel(), ins["b"]: b[lo:hi].ravel(), ins["bias"]: bias})[out]
        local = torch.from_numpy(res.reshape(hi - lo, M, N))
        full = sh.all_gather_leading(local, B)
        gf, insf, outf = wl.matmul_bias(B, M, N, K, DataType.Float)
        want = orc.execute(gf, {insf["a"]: a.ravel(), insf["b"]: b.ravel(), insf["bias"]: bias})[outf].reshape(B, M, N)
        ok = np.array_equal(full.numpy(), want)
    elif case == "wgrad":
        n, c, h, w, k = 6, 8, 6, 6, 16
        dy = rng.normal(0, 0.1, (n, h, w, k)).astype(np.float32)
        x = rng.normal(0, 0.5, (n, h, w, c)).astype(np.float32)
        lo, hi = sh.shard_range(n, rank, world)
        g, ins, dw_t = wl.conv_wgrad(hi - lo, c, h, w, k, 3, 3, 1, DataType.Float)
        part = orc.execute(g, {ins["dy"]: dy[lo:hi].ravel(), ins["x"]: x[lo:hi].ravel()})[dw_t]
        total = sh.all_reduce_wgrad(torch.from_numpy(part), torch.float32).numpy()
        gf, insf, dwf = wl.conv_wgrad(n, c, h, w, k, 3, 3, 1, DataType.Float)
        want = orc.execute(gf, {insf["dy"]: dy.ravel(), insf["x"]: x.ravel()})[dwf]
        ok = np.allclose(total, want, rtol=1e-5, atol=1e-6)
    else:  # timing reduction used by the bench: max over ranks
        ok = sh.max_over_ranks(float(rank + 1)) == float(world)
    with open(os.path.join(out_dir, f"{case}_{rank}.ok"), "w") as f:
        f.write("1" if ok else "0")
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("case", ["matmul", "wgrad", "max"])
def test_two_rank_sharding_matches_unsharded(case, tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), case, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert (tmp_path / f"{case}_{r}.ok").read_text() == "1", f"{case}: rank {r} disagrees"


def test_shard_ranges_cover_everything():
    from fusilli_b200 import sharding as sh
    for total in (1, 7, 8, 256, 32768):
        for world in (1, 2, 3, 4, 8):
            spans = [sh.shard_range(total, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            sizes = [e - b for b, e in spans]
            assert max(sizes) - min(sizes) <= 1
