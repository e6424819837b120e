"""Batch sharding on real GPUs (NCCL, one process per GPU): every rank runs the module on its own
samples, `allreduce_box_gradients` sums the packed (4, C, F) gradient with one collective, and the
result is compared with a full-batch run and with the oracle.  Needs at least two GPUs (skipped
otherwise); the CPU counterpart with gloo ranks is tests/test_distributed_gloo.py."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import PKG_DIR, ROOT, max_rel

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _module(bc, wl, dev):
    C, F = wl.stored[0].shape
    m = bc.BoxConv2d(C, F, wl.max_h, wl.max_w, reparametrization_factor=8).to(dev)
    with torch.no_grad():
        for p, v in zip((m.x_min, m.x_max, m.y_min, m.y_max), wl.stored):
            p.copy_(torch.from_numpy(v))
    return m.train()


def _worker(rank, world, port, out_dir):
    for p in (ROOT, PKG_DIR):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import box_convolution as bc
        from workloads import make_workload

        wl = make_workload("cfg2", batch=8, planes=6)
        per = wl.x.shape[0] // world
        sl = slice(rank * per, (rank + 1) * per)
        m = _module(bc, wl, dev)
        x = torch.from_numpy(wl.x[sl]).to(dev).requires_grad_()
        out = m(x)
        out.backward(torch.from_numpy(wl.grad_output[sl]).to(dev))
        packed, copied = bc.packed_box_gradient(m)
        assert not copied and packed.shape == (4,) + tuple(m.x_min.shape)      # one buffer, one collective
        local = packed.clone()
        work = bc.allreduce_box_gradients(m, async_op=True)
        work.wait()
        torch.cuda.synchronize()
        np.savez(os.path.join(out_dir, "rank%d.npz" % rank), out=out.detach().cpu().numpy(),
                 gin=x.grad.cpu().numpy(), local=local.cpu().numpy(),
                 gps=np.stack([p.grad.cpu().numpy() for p in (m.x_min, m.x_max, m.y_min, m.y_max)]))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least two GPUs")
def test_nccl_shards_reduce_to_the_full_batch(tmp_path):
    import box_convolution as bc
    from oracle import oracle
    from workloads import make_workload

    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    ranks = [dict(np.load(os.path.join(str(tmp_path), "rank%d.npz" % r))) for r in range(world)]

    wl = make_workload("cfg2", batch=8, planes=6)
    m = _module(bc, wl, torch.device("cuda", 0))
    x = torch.from_numpy(wl.x).cuda().requires_grad_()
    out = m(x)
    out.backward(torch.from_numpy(wl.grad_output).cuda())
    full_gps = np.stack([p.grad.cpu().numpy() for p in (m.x_min, m.x_max, m.y_min, m.y_max)])

    per = wl.x.shape[0] // world
    for r, d in enumerate(ranks):
        sl = slice(r * per, (r + 1) * per)
        assert np.array_equal(d["out"], out.detach().cpu().numpy()[sl]), r      # shards are slices, bit for bit
        assert np.array_equal(d["gin"], x.grad.cpu().numpy()[sl]), r
        # every rank holds the same reduced gradient: the sum of the local ones
        assert np.array_equal(d["gps"], ranks[0]["gps"]), r
    want = np.sum([d["local"].astype(np.float64) for d in ranks], axis=0)
    assert max_rel(ranks[0]["gps"], want) < 1e-6
    assert max_rel(ranks[0]["gps"], full_gps) < 1e-5
    _, _, ref_gps = oracle.boxconv2d_forward_backward(wl.x, wl.stored, wl.grad_output, wl.rep_h, wl.rep_w, True, True)
    for k in range(4):
        assert max_rel(ranks[0]["gps"][k], ref_gps[k]) < 1e-3, k
