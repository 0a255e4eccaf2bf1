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
