"""Two GPUs: a GDN forward+backward sharded by GVA group across ranks equals the single-GPU result bit for
bit (no exchange step on the path).  Skipped when fewer than two GPUs are visible."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    import sys
    from pathlib import Path
    import torch.distributed as dist
    repo = Path(__file__).resolve().parent.parent
    for p in (str(repo / "flash-linear-attention-npu_b200"), str(repo)):
        if p not in sys.path:
            sys.path.insert(0, p)
    import oracle
    from fla_b200 import sharding
    from fla_b200.ops import chunk_gated_delta_rule_fwd_bwd
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        inp = oracle.make_gdn_inputs(2, 192, 4, 8, seed=17)
        d = {n: t.cuda() for n, t in inp.items()}
        q, k, v, g, b, h0 = sharding.shard_heads(d["q"], d["k"], d["v"], d["g"], d["beta"], d["h0"], world, rank)
        vb, ve = sharding.shard_range(8, world, rank, granule=2)
        o, ht, grads = chunk_gated_delta_rule_fwd_bwd(q.contiguous(), k.contiguous(), v.contiguous(), g.contiguous(),
                                                      b.contiguous(), d["do"][:, :, vb:ve].contiguous(),
                                                      initial_state=h0.contiguous(), dht=d["dht"][:, vb:ve].contiguous())
        o_all = sharding.gather_along(o, 2)
        dq_all = sharding.gather_along(grads[0], 2)
        dg_all = sharding.gather_along(grads[3], 2)
        if rank == 0:
            o1, ht1, g1 = chunk_gated_delta_rule_fwd_bwd(d["q"], d["k"], d["v"], d["g"], d["beta"], d["do"],
                                                         initial_state=d["h0"], dht=d["dht"])
            ret["ok"] = bool(torch.equal(o_all, o1) and torch.equal(dq_all, g1[0]) and torch.equal(dg_all, g1[3]))
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sharded_by_gva_group_equals_single_gpu():
    import torch.multiprocessing as mp
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        procs = [ctx.Process(target=_worker, args=(r, world, port, ret)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(300)
        hung = [p for p in procs if p.is_alive()]
        for p in hung:                      # a worker that is still running after the limit is stopped, not left behind
            p.terminate()
            p.join(30)
        assert not hung, f"{len(hung)} worker(s) did not finish"
        assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
        assert ret.get("ok") is True
