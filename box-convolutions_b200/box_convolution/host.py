"""Training step of a BoxConv2d block on batches that live in host memory.

``HostPipeline`` hands pinned host tensors to ``bc_boxconv2d_host_step``: the library cuts the
batch into chunks and overlaps, on three CUDA streams, the host-to-device copies of chunk i+1,
the kernels of chunk i and the device-to-host copies of chunk i-1.

``step`` runs one batch and returns when its results are in the host tensors.  ``submit`` /
``wait`` keep up to ``depth`` batches in flight, each on its own device workspace, so that the
input copies of the next batch run while the results of the current one are still on their way
back: the PCIe link then stays busy in both directions from one batch to the next.  Batches in
flight need distinct result tensors; a batch's tensors must not be touched until its ``wait``
returns."""
import torch

from ._cabi import check, lib


class HostPipeline:
    def __init__(self, module, batch, h, w, chunks=8, group=None, depth=2):
        self.module = module
        self.group = group
        self.shape = (batch, module.in_planes, module.num_filters, h, w)
        self.chunks = max(1, min(chunks, batch))
        self.depth = max(1, int(depth))
        dev = module.x_min.device
        with torch.cuda.device(dev):
            nbytes = lib.bc_boxconv2d_host_step_workspace(*self.shape, self.chunks)
            self.workspaces = [torch.empty(nbytes, dtype=torch.uint8, device=dev) for _ in range(self.depth)]
            self.copy_in, self.compute, self.copy_out = (torch.cuda.Stream(dev) for _ in range(3))
            # per workspace: kernels have consumed its inputs / its results have left for the host
            self._computed = [torch.cuda.Event() for _ in range(self.depth)]
            self._drained = [torch.cuda.Event() for _ in range(self.depth)]
        self._used = [False] * self.depth
        self._busy = [False] * self.depth
        self._next = 0

    @staticmethod
    def _check_host(t, shape, name):
        if t.is_cuda or t.dtype != torch.float32 or not t.is_contiguous() or tuple(t.shape) != tuple(shape):
            raise RuntimeError("HostPipeline: %s must be a contiguous float32 host tensor of shape %s" % (name, tuple(shape)))

    def submit(self, x_host, grad_output_host, out_host, grad_input_host, grad_params_host):
        """Enqueues one batch and returns a ticket for ``wait``.  Raises if ``depth`` batches are
        already in flight."""
        m = self.module
        N, C, F, h, w = self.shape
        self._check_host(x_host, (N, C, h, w), "x_host")
        self._check_host(grad_output_host, (N, C * F, h, w), "grad_output_host")
        self._check_host(out_host, (N, C * F, h, w), "out_host")
        self._check_host(grad_input_host, (N, C, h, w), "grad_input_host")
        self._check_host(grad_params_host, (4, C, F), "grad_params_host")
        slot = self._next
        if self._busy[slot]:
            raise RuntimeError("HostPipeline: %d batches are already in flight; wait() for the oldest first" % self.depth)
        dev = m.x_min.device
        with torch.cuda.device(dev):
            cur = torch.cuda.current_stream()
            for s in (self.copy_in, self.compute, self.copy_out):
                s.wait_stream(cur)
            if self._used[slot]:
                # the batch that used this workspace last: its inputs may be overwritten once its
                # kernels are done, its results once they have been copied out
                self.copy_in.wait_event(self._computed[slot])
                self.compute.wait_event(self._drained[slot])
            check(lib.bc_boxconv2d_host_step(
                x_host.data_ptr(), grad_output_host.data_ptr(), out_host.data_ptr(),
                grad_input_host.data_ptr(), grad_params_host.data_ptr(),
                m.x_min.data_ptr(), m.x_max.data_ptr(), m.y_min.data_ptr(), m.y_max.data_ptr(),
                float(m.reparametrization_h), float(m.reparametrization_w),
                float(m.max_input_h), float(m.max_input_w), N, C, F, h, w,
                int(bool(m.normalize)), int(bool(m.exact)), int(bool(m.training)), self.chunks,
                self.workspaces[slot].data_ptr(), self.workspaces[slot].numel(),
                self.copy_in.cuda_stream, self.compute.cuda_stream, self.copy_out.cuda_stream),
                "bc_boxconv2d_host_step")
            self._computed[slot].record(self.compute)
            self._drained[slot].record(self.copy_out)
        self._used[slot] = self._busy[slot] = True
        self._next = (slot + 1) % self.depth
        return (slot, grad_params_host)

    def wait(self, ticket):
        """Returns when the results of the batch behind `ticket` are in its host tensors."""
        slot, grad_params_host = ticket
        if not self._busy[slot]:
            return
        self._drained[slot].synchronize()
        self._busy[slot] = False
        if torch.distributed.is_available() and torch.distributed.is_initialized() \
                and torch.distributed.get_world_size(self.group) > 1:
            # the reduced gradient of a sharded batch: small enough to reduce from the host copy
            dev = self.module.x_min.device
            g = grad_params_host.to(dev, non_blocking=False)
            torch.distributed.all_reduce(g, group=self.group)
            grad_params_host.copy_(g)

    def step(self, x_host, grad_output_host, out_host, grad_input_host, grad_params_host):
        self.wait(self.submit(x_host, grad_output_host, out_host, grad_input_host, grad_params_host))
