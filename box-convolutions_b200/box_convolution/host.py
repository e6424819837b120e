"""Training step of a BoxConv2d block on batches that live in host memory.

``HostPipeline.step`` hands pinned host tensors to ``bc_boxconv2d_host_step``: the library cuts
the batch into chunks and overlaps, on three CUDA streams, the host-to-device copies of chunk
i+1, the kernels of chunk i and the device-to-host copies of chunk i-1.  Results are complete
when ``step`` returns."""
import torch

from ._cabi import check, lib


class HostPipeline:
    def __init__(self, module, batch, h, w, chunks=8, group=None):
        self.module = module
        self.group = group
        self.shape = (batch, module.in_planes, module.num_filters, h, w)
        self.chunks = max(1, min(chunks, batch))
        dev = module.x_min.device
        with torch.cuda.device(dev):
            nbytes = lib.bc_boxconv2d_host_step_workspace(*self.shape, self.chunks)
            self.workspace = torch.empty(nbytes, dtype=torch.uint8, device=dev)
            self.copy_in, self.compute, self.copy_out = (torch.cuda.Stream(dev) for _ in range(3))

    @staticmethod
    def _check_host(t, shape, name):
        if t.is_cuda or t.dtype != torch.float32 or not t.is_contiguous() or tuple(t.shape) != tuple(shape):
            raise RuntimeError("HostPipeline: %s must be a contiguous float32 host tensor of shape %s" % (name, tuple(shape)))

    def step(self, x_host, grad_output_host, out_host, grad_input_host, grad_params_host):
        m = self.module
        N, C, F, h, w = self.shape
        self._check_host(x_host, (N, C, h, w), "x_host")
        self._check_host(grad_output_host, (N, C * F, h, w), "grad_output_host")
        self._check_host(out_host, (N, C * F, h, w), "out_host")
        self._check_host(grad_input_host, (N, C, h, w), "grad_input_host")
        self._check_host(grad_params_host, (4, C, F), "grad_params_host")
        dev = m.x_min.device
        with torch.cuda.device(dev):
            cur = torch.cuda.current_stream()
            for s in (self.copy_in, self.compute, self.copy_out):
                s.wait_stream(cur)
            check(lib.bc_boxconv2d_host_step(
                x_host.data_ptr(), grad_output_host.data_ptr(), out_host.data_ptr(),
                grad_input_host.data_ptr(), grad_params_host.data_ptr(),
                m.x_min.data_ptr(), m.x_max.data_ptr(), m.y_min.data_ptr(), m.y_max.data_ptr(),
                float(m.reparametrization_h), float(m.reparametrization_w),
                float(m.max_input_h), float(m.max_input_w), N, C, F, h, w,
                int(bool(m.normalize)), int(bool(m.exact)), int(bool(m.training)), self.chunks,
                self.workspace.data_ptr(), self.workspace.numel(),
                self.copy_in.cuda_stream, self.compute.cuda_stream, self.copy_out.cuda_stream),
                "bc_boxconv2d_host_step")
            self.copy_out.synchronize()
            if torch.distributed.is_available() and torch.distributed.is_initialized() \
                    and torch.distributed.get_world_size(self.group) > 1:
                # the reduced gradient of a sharded batch: small enough to reduce from the host copy
                g = grad_params_host.to(dev, non_blocking=False)
                torch.distributed.all_reduce(g, group=self.group)
                grad_params_host.copy_(g)
