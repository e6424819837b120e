"""Batch-sharded bookkeeping on CPU ranks (gloo, world size 2): every rank computes the parameter
gradients of its own samples (with the oracle standing in for the CUDA kernels), the packed
(4, C, F) buffers are summed with ONE all-reduce by `allreduce_box_gradients`, and the result must
equal the full-batch gradient.  Outputs and grad-input of a shard are slices of the full result."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import PKG_DIR, ROOT, max_rel


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


class _Params(torch.nn.Module):
    """Carries the four parameters of a BoxConv2d without needing a GPU."""

    def __init__(self, C, F):
        super().__init__()
        for n in ("x_min", "x_max", "y_min", "y_max"):
            setattr(self, n, torch.nn.Parameter(torch.zeros(C, F)))


def _worker(rank, world, port, packed_layout, out_dir):
    for p in (ROOT, PKG_DIR):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from box_convolution.distributed import allreduce_box_gradients, packed_box_gradient
        from oracle import oracle
        from workloads import make_workload

        wl = make_workload("cfg1", batch=4, planes=3)
        N, C, F, h, w = wl.shape
        per = N // world
        sl = slice(rank * per, (rank + 1) * per)
        out, gin, gps = oracle.boxconv2d_forward_backward(
            wl.x[sl], wl.stored, wl.grad_output[sl], wl.rep_h, wl.rep_w, True, True)

        m = _Params(C, F)
        if packed_layout:      # what the CUDA backward produces: four views of one buffer
            buf = torch.from_numpy(np.stack(gps)).clone()
            for i, p in enumerate((m.x_min, m.x_max, m.y_min, m.y_max)):
                p.grad = buf[i]
            packed, copied = packed_box_gradient(m)
            assert not copied and packed.data_ptr() == buf.data_ptr() and packed.shape == (4, C, F)
        else:                  # independent gradient tensors: the helper must stack and copy back
            for g, p in zip(gps, (m.x_min, m.x_max, m.y_min, m.y_max)):
                p.grad = torch.from_numpy(g).clone()
            assert packed_box_gradient(m)[1]
        allreduce_box_gradients(m)
        np.savez(os.path.join(out_dir, "rank%d.npz" % rank), out=out, gin=gin,
                 gps=np.stack([p.grad.numpy() for p in (m.x_min, m.x_max, m.y_min, m.y_max)]))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("packed_layout", [True, False])
def test_two_rank_shards_reduce_to_the_full_batch(tmp_path, packed_layout):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), packed_layout, str(tmp_path)), nprocs=world, join=True)

    from oracle import oracle
    from workloads import make_workload
    wl = make_workload("cfg1", batch=4, planes=3)
    ref_out, ref_gin, ref_gps = oracle.boxconv2d_forward_backward(
        wl.x, wl.stored, wl.grad_output, wl.rep_h, wl.rep_w, True, True)
    ranks = [np.load(os.path.join(tmp_path, "rank%d.npz" % r)) for r in range(world)]
    # both ranks hold the same reduced gradient, equal to the full-batch one
    assert np.array_equal(ranks[0]["gps"], ranks[1]["gps"])
    for k in range(4):
        assert max_rel(ranks[0]["gps"][k], ref_gps[k]) < 1e-5, k
    # per-sample results are independent of the sharding
    assert np.array_equal(np.concatenate([r["out"] for r in ranks]), ref_out)
    assert np.array_equal(np.concatenate([r["gin"] for r in ranks]), ref_gin)
