"""Two-rank CPU test (gloo) of the data-parallel logic around the attention step: ownership of
the global batch, and the identity the multi-GPU path relies on - summing the per-rank
parameter gradients equals the gradient of the whole batch, while outputs and input gradients
need no exchange.  The arithmetic here is the CPU restatement; the GPU path replaces gloo's
all-reduce by NCCL on the gradient bucket."""
import os
import socket

import numpy as np
import pytest

import cases
from boat_b200 import shard


def test_batch_ranges_partition_the_batch():
    for gb, world in ((8, 2), (7, 3), (4, 8), (32, 8), (1, 1)):
        ranges = [shard.batch_range(gb, world, r) for r in range(world)]
        assert ranges[0][0] == 0 and ranges[-1][1] == gb
        assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
        assert max(e - b for b, e in ranges) - min(e - b for b, e in ranges) <= 1
        assert shard.unit_range(gb, 4, world, 0) == (0, ranges[0][1] * 4)
    assert shard.element_offset(8, 16, 32, 2, 1) == 4 * 16 * 32
    with pytest.raises(ValueError):
        shard.batch_range(8, 2, 2)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, q):
    import torch
    import torch.distributed as dist
    from oracle import oracle
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        case = cases.Case("dp", 4, 24, 32, 4, causal=True, bias_std=0.1)
        inp = case.inputs()
        b0, b1 = shard.batch_range(case.B, world, rank)
        x, g = inp["q"][b0:b1], inp["dout"][b0:b1]
        res = oracle.port_step(x, x, x, inp["w"], inp["b"], g, case.nh, True)
        bucket = np.concatenate([w.ravel() for w in res["dw"]] + [b.ravel() for b in res["db"]]).astype(np.float32)
        t = torch.from_numpy(bucket.copy())
        dist.all_reduce(t)                                   # the one collective of the step
        full = oracle.port_step(inp["q"], inp["q"], inp["q"], inp["w"], inp["b"], inp["dout"], case.nh, True)
        want = np.concatenate([w.ravel() for w in full["dw"]] + [b.ravel() for b in full["db"]])
        err = float(np.abs(t.numpy() - want).max() / np.abs(want).max())
        local_ok = (np.array_equal(res["out"], full["out"][b0:b1]) and np.array_equal(res["dq"], full["dq"][b0:b1])
                    and np.array_equal(res["dk"], full["dk"][b0:b1]) and np.array_equal(res["dv"], full["dv"][b0:b1]))
        q.put((rank, err, local_ok))
    finally:
        dist.destroy_process_group()


def test_gradient_sum_over_two_ranks_equals_full_batch_gradient():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err, local_ok in results:
        assert err <= 1e-5, (rank, err)       # same sum, different association of the additions
        assert local_ok, rank                  # outputs and input gradients of a slice need no exchange


# ---- one fixed problem split at head granularity ------------------------------------------------------

def test_head_unit_ranges_and_their_rows():
    # config 4 of the benchmark: B=4, 16 heads, S=8192 over 8 ranks = 8 units = half a sequence each
    ranges = [shard.head_unit_range(4, 16, 8, r) for r in range(8)]
    assert ranges == [(8 * r, 8 * r + 8) for r in range(8)]
    assert [shard.unit_rows(u, 8192, 16) for u in ranges] == [(4096 * r, 4096 * r + 4096) for r in range(8)]
    # uneven: 3 batch entries of 4 heads over 5 ranks
    ranges = [shard.head_unit_range(3, 4, 5, r) for r in range(5)]
    assert ranges[0][0] == 0 and ranges[-1][1] == 12 and all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
    with pytest.raises(ValueError):
        shard.unit_rows((0, 1), 10, 4)          # heads do not divide the sequence: units straddle token rows


def unit_range_step(x_rows, g_rows, w, b, nh, S, causal):
    """The layer's step on the token rows of a contiguous unit range, composed from the restatement's
    attention core and plain row-wise projections (what boat_attention_forward_units + backward do)."""
    from oracle import oracle
    R, H = x_rows.shape
    hs = H // nh
    units = R * nh // S
    f64 = np.float64
    proj = [(x_rows.astype(f64) @ w[i].astype(f64) + b[i]).astype(np.float32) for i in range(3)]
    dctx = (g_rows.astype(f64) @ w[3].astype(f64).T).astype(np.float32)
    core = oracle.port_core(*(p.reshape(units, S, hs) for p in proj), dctx.reshape(units, S, hs), causal, 1.0 / np.sqrt(hs))
    ctx = core["o"].reshape(R, H)
    out = (ctx.astype(f64) @ w[3].astype(f64) + b[3]).astype(np.float32)
    dproj = [core[k].reshape(R, H).astype(f64) for k in ("dq", "dk", "dv")]
    dx = [(dproj[i] @ w[i].astype(f64).T).astype(np.float32) for i in range(3)]
    dw = [x_rows.astype(f64).T @ dproj[i] for i in range(3)] + [ctx.astype(f64).T @ g_rows.astype(f64)]
    db = [dproj[i].sum(0) for i in range(3)] + [g_rows.astype(f64).sum(0)]
    return dict(out=out, dx=dx, bucket=np.concatenate([m.ravel() for m in dw] + [v.ravel() for v in db]))


def _unit_worker(rank, world, port, q):
    import torch
    import torch.distributed as dist
    from oracle import oracle
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # 3 batch entries x 4 heads = 12 units over 2 ranks: rank 0 owns batch entry 0 and half of entry 1
        case = cases.Case("strong", 3, 24, 32, 4, causal=True, bias_std=0.1)
        inp = case.inputs()
        u = shard.head_unit_range(case.B, case.nh, world, rank)
        r0, r1 = shard.unit_rows(u, case.S, case.nh)
        x = inp["q"].reshape(-1, case.H)[r0:r1]
        g = inp["dout"].reshape(-1, case.H)[r0:r1]
        mine = unit_range_step(x, g, inp["w"], inp["b"], case.nh, case.S, True)
        t = torch.from_numpy(mine["bucket"].copy())
        dist.all_reduce(t)                                   # the one collective: the gradient bucket
        full = oracle.port_step(inp["q"], inp["q"], inp["q"], inp["w"], inp["b"], inp["dout"], case.nh, True)
        want = np.concatenate([w.ravel() for w in full["dw"]] + [b.ravel() for b in full["db"]])
        err_bucket = float(np.abs(t.numpy() - want).max() / np.abs(want).max())
        flat = lambda a: a.reshape(-1, case.H)[r0:r1]
        err_rows = max(cases.rel_err(mine["out"], flat(full["out"])), cases.rel_err(mine["dx"][0], flat(full["dq"])),
                       cases.rel_err(mine["dx"][1], flat(full["dk"])), cases.rel_err(mine["dx"][2], flat(full["dv"])))
        q.put((rank, u, err_bucket, err_rows))
    finally:
        dist.destroy_process_group()


def test_unit_ranges_of_one_problem_over_two_ranks_equal_the_full_step():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_unit_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(r[1] for r in results) == [(0, 6), (6, 12)]
    for rank, u, err_bucket, err_rows in results:
        assert err_bucket <= 1e-5, (rank, err_bucket)     # the summed per-range gradients are the full gradients
        assert err_rows <= 1e-5, (rank, err_rows)         # outputs and input gradients of the owned rows need no exchange
