"""CPU tests (gloo, world_size 2) of the tensor-parallel host logic: sharding packed codes by rows and
by columns with the carry halo, checked through the numpy oracle, and the all-reduce of partial products."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, q):
    try:
        _worker_body(rank, world, port, q)
    except Exception as e:          # report instead of leaving the parent to time out
        q.put((rank, False, repr(e)))
        raise


def _worker_body(rank, world, port, q):
    for p in (os.path.join(ROOT, "let-it-slide_b200"), os.path.join(ROOT, "oracle")):
        sys.path.insert(0, p)
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import rptc_oracle as o
    from rptc_b200 import CODE_HASH, LAYOUT_TILED, Format
    from rptc_b200.linear import RPTCLinear
    from rptc_b200.tp import shard_cols, shard_rows
    rng = np.random.default_rng(0)                       # same full layer on every rank
    m, n = 128, 1024
    words = rng.integers(0, 2**32, (m, n // 16), dtype=np.uint64).astype(np.uint32)
    lut = rng.standard_normal(512).astype(np.float16)
    x = rng.standard_normal(n).astype(np.float16)
    full = o.decode(words, lut, n, code=o.CODE_B, S=8)
    y_full = o.matvec_exact(full, x[None])[0]
    codes = torch.from_numpy(o.from_rowmajor(words, o.LAYOUT_TILED).view(np.int32))
    lin = RPTCLinear(n, m, Format(CODE_HASH, 2, 16, 8, LAYOUT_TILED), codes, torch.from_numpy(lut))
    # row-parallel (split the input columns): decode the shard with its halo, multiply, all-reduce
    sc = shard_cols(lin, rank, world)
    w_sc = o.decode(sc.codes.numpy().view(np.uint32), lut, n // world, code=o.CODE_B, S=8, layout=o.LAYOUT_TILED,
                    carry_in=None if sc.carry_in is None else sc.carry_in.numpy().view(np.uint32))
    nl = n // world
    ok_decode = np.array_equal(w_sc.view(np.uint16), full[:, rank * nl:(rank + 1) * nl].view(np.uint16))
    part = torch.from_numpy(o.matvec_exact(w_sc, x[None, rank * nl:(rank + 1) * nl])[0])
    dist.all_reduce(part)
    ok_sum = np.allclose(part.numpy(), y_full, rtol=1e-9, atol=1e-9)
    # column-parallel (split the output rows): a plain slice, gathered
    sr = shard_rows(lin, rank, world)
    w_sr = o.decode(sr.codes.numpy().view(np.uint32), lut, n, code=o.CODE_B, S=8, layout=o.LAYOUT_TILED)
    ml = m // world
    ok_rows = np.array_equal(w_sr.view(np.uint16), full[rank * ml:(rank + 1) * ml].view(np.uint16))
    gathered = [torch.zeros(ml, dtype=torch.float64) for _ in range(world)]
    dist.all_gather(gathered, torch.from_numpy(o.matvec_exact(w_sr, x[None])[0]))
    ok_gather = np.allclose(torch.cat(gathered).numpy(), y_full)
    q.put((rank, ok_decode, ok_sum, ok_rows, ok_gather))
    dist.destroy_process_group()


def test_sharding_and_allreduce_world2():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for r in res:
        assert all(r[1:]), r
