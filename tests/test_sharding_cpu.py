"""The multi-GPU host logic on CPU: world_size-2 gloo ranks shard a step, and the gathered shards equal the
unsharded tensors; the oracle run on the shards equals the oracle on the whole batch (the path has no
exchange step, so sharding by batch or by GVA group must not change any value)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, mode, ret):
    import sys
    from pathlib import Path
    repo = Path(__file__).resolve().parent.parent
    for p in (str(repo / "flash-linear-attention-npu_b200"), str(repo)):
        if p not in sys.path:
            sys.path.insert(0, p)
    import oracle
    from fla_b200 import sharding
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    try:
        inp = oracle.make_gdn_inputs(3, 40, 2, 4, K=16, V=8, seed=5, dtype=torch.float32, with_grad=False)
        full = oracle.gdn_reference_fwd_bwd(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], initial_state=inp["h0"])
        if mode == "batch":
            sh = sharding.shard_batch({n: inp[n] for n in ("q", "k", "v", "g", "beta", "h0")}, world, rank)
            part = oracle.gdn_reference_fwd_bwd(sh["q"], sh["k"], sh["v"], sh["g"], sh["beta"], initial_state=sh["h0"])
            o = sharding.gather_along(part["o"], 0)
            ht = sharding.gather_along(part["ht"], 0)
        else:
            q, k, v, g, b, h0 = sharding.shard_heads(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], inp["h0"],
                                                     world, rank)
            part = oracle.gdn_reference_fwd_bwd(q, k, v, g, b, initial_state=h0)
            o = sharding.gather_along(part["o"].contiguous(), 2)
            ht = sharding.gather_along(part["ht"].contiguous(), 1)
        ok = torch.allclose(o, full["o"], atol=1e-6) and torch.allclose(ht, full["ht"], atol=1e-6)
        slow = sharding.max_over_ranks(float(rank + 1), torch.device("cpu"))
        ret[rank] = bool(ok) and slow == float(world)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["batch", "heads"])
def test_two_rank_sharding_matches_single_rank(mode):
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        procs = [ctx.Process(target=_worker, args=(r, world, port, mode, ret)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(120)
            assert p.exitcode == 0
        assert all(ret.get(r) for r in range(world)), dict(ret)


def test_shard_range_keeps_groups_whole():
    from fla_b200.sharding import shard_range
    assert [shard_range(32, 8, r, granule=2) for r in range(8)] == [(4 * r, 4 * r + 4) for r in range(8)]
    assert [shard_range(10, 4, r) for r in range(4)] == [(0, 3), (3, 6), (6, 8), (8, 10)]
    with pytest.raises(ValueError):
        shard_range(9, 2, 0, granule=2)
