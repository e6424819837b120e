"""bc_boxconv2d_backward_static(): the backward pass for callers that can neither pass scratch
memory nor allocate it (a plugin called inside another component's stream capture, a process
whose device memory is fully assigned at start-up).  It must give what bc_boxconv2d_backward()
gives with a caller-provided workspace, also when the built-in scratch array still holds the
previous call's data.  Collected last (file name) so that a failure here cannot hide the other
tests under `pytest -x`."""
import ctypes

import numpy as np
import pytest
import torch

from conftest import max_rel
from workloads import make_workload

pytestmark = pytest.mark.gpu


def _backward(lib, static, x, go, stored, rep_h, rep_w, need_mask=31):
    N, C, h, w = x.shape
    F = stored[0].shape[1]
    gin = torch.full_like(x, float("nan"))
    gp = torch.full((4, C, F), float("nan"), device=x.device)
    stream = torch.cuda.current_stream().cuda_stream
    common = [x.data_ptr(), *[p.data_ptr() for p in stored], go.data_ptr(), rep_h, rep_w,
              N, C, F, h, w, 1, 1, need_mask, gin.data_ptr(), gp.data_ptr()]
    if static:
        status = lib.bc_boxconv2d_backward_static(*common, stream)
    else:
        nbytes = lib.bc_boxconv2d_backward_workspace(N, C, F, h, w, need_mask)
        ws = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=x.device)
        status = lib.bc_boxconv2d_backward(*common, ws.data_ptr(), ws.numel(), stream)
    torch.cuda.synchronize()
    return status, gin.cpu().numpy(), gp.cpu().numpy()


def test_static_scratch_backward_matches_workspace_backward_twice_in_a_row():
    from box_convolution import _cabi
    lib = _cabi.lib
    # two different problems back to back: the second call finds the first call's data in the array
    for cfg, batch, planes in (("cfg2", 3, 8), ("cfg1", 2, 5)):
        wl = make_workload(cfg, batch=batch, planes=planes)
        x = torch.from_numpy(wl.x).cuda()
        go = torch.from_numpy(wl.grad_output).cuda()
        stored = [torch.from_numpy(p).cuda() for p in wl.stored]
        st_ref, gin_ref, gp_ref = _backward(lib, False, x, go, stored, wl.rep_h, wl.rep_w)
        assert st_ref == 0
        for repeat in range(2):
            st, gin, gp = _backward(lib, True, x, go, stored, wl.rep_h, wl.rep_w)
            assert st == 0, (cfg, repeat, lib.bc_status_string(st))
            assert max_rel(gin, gin_ref) < 1e-4, (cfg, repeat)
            for k in range(4):
                assert max_rel(gp[k], gp_ref[k]) < 1e-3, (cfg, repeat, k)


def test_static_scratch_backward_takes_no_device_memory_and_serves_need_mask_subsets():
    """The property the entry point exists for: once the set-up call has been made, device memory in use
    is the same before and after the calls, and gradient subsets behave as with a workspace."""
    from box_convolution import _cabi
    lib = _cabi.lib
    wl = make_workload("cfg1", batch=2, planes=3)
    x = torch.from_numpy(wl.x).cuda()
    go = torch.from_numpy(wl.grad_output).cuda()
    stored = [torch.from_numpy(p).cuda() for p in wl.stored]
    N, C, h, w = x.shape
    F = stored[0].shape[1]
    masks = (31, 1, 30, 10)
    refs = {mask: _backward(lib, False, x, go, stored, wl.rep_h, wl.rep_w, mask) for mask in masks}
    outs = {mask: (torch.full_like(x, float("nan")), torch.full((4, C, F), float("nan"), device="cuda")) for mask in masks}
    stream = torch.cuda.current_stream().cuda_stream
    # The documented set-up step: the first call on a device (here the empty one) looks up the array's
    # address, and that is also the moment at which the CUDA driver, which loads modules lazily, places
    # the library's 4 MiB array on the device.  Nothing is allocated from then on.
    assert lib.bc_boxconv2d_backward_static(None, None, None, None, None, None, 8.0, 8.0,
                                            0, C, F, h, w, 1, 1, 1, None, None, stream) == 0
    torch.cuda.synchronize()
    # nothing between the two readings but the calls themselves (no tensor operations, which could
    # make PyTorch's own allocator ask the driver for memory)
    free_before, _ = torch.cuda.mem_get_info()
    allocated_before = torch.cuda.memory_allocated()
    statuses = {}
    for mask in masks:
        gin, gp = outs[mask]
        statuses[mask] = lib.bc_boxconv2d_backward_static(
            x.data_ptr(), *[p.data_ptr() for p in stored], go.data_ptr(), wl.rep_h, wl.rep_w,
            N, C, F, h, w, 1, 1, mask, gin.data_ptr(), gp.data_ptr(), stream)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert torch.cuda.memory_allocated() == allocated_before
    assert free_after == free_before
    for mask in masks:
        assert statuses[mask] == 0, (mask, lib.bc_status_string(statuses[mask]))
        gin, gp = (t.cpu().numpy() for t in outs[mask])
        _, gin_ref, gp_ref = refs[mask]
        if mask & 1:
            assert max_rel(gin, gin_ref) < 1e-4, mask
        else:
            assert np.isnan(gin).all(), mask                    # not asked for: untouched
        for k in range(4):
            if mask & (2 << k):
                assert max_rel(gp[k], gp_ref[k]) < 1e-3, (mask, k)
            else:
                assert np.isnan(gp[k]).all(), (mask, k)


def test_static_scratch_backward_empty_call_is_the_cheap_first_call():
    from box_convolution import _cabi
    lib = _cabi.lib
    stream = torch.cuda.current_stream().cuda_stream
    # N = 0, grad-input only: nothing to launch, no pointer is looked at, only the address look-up happens
    st = lib.bc_boxconv2d_backward_static(None, None, None, None, None, None, 8.0, 8.0,
                                          0, 4, 4, 64, 128, 1, 1, 1, None, None, stream)
    assert st == 0


def test_static_scratch_backward_refuses_what_does_not_fit():
    from box_convolution import _cabi
    lib = _cabi.lib
    # a 256x512 plane does not fit in shared memory: the general path needs integral images of all
    # N*C*F grad_output planes, far more than the built-in array
    N, C, F, h, w = 2, 4, 4, 256, 512
    assert lib.bc_boxconv2d_backward_workspace(N, C, F, h, w, 31) > (4 << 20)
    x = torch.zeros(N, C, h, w, device="cuda")
    go = torch.zeros(N, C * F, h, w, device="cuda")
    stored = [torch.zeros(C, F, device="cuda") for _ in range(4)]
    st, _, gp = _backward(lib, True, x, go, stored, 8.0 * h, 8.0 * w)
    assert st == -3                                  # BC_ERR_WORKSPACE, nothing launched
    assert b"scratch" in lib.bc_last_cuda_error()
    assert np.isnan(gp).all()                        # outputs untouched
