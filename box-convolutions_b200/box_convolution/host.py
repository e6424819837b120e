"""Training step of a BoxConv2d block on batches that live in host memory.

``HostPipeline.step`` splits the batch into chunks and overlaps, on three CUDA streams, the
host-to-device copies of chunk i+1, the forward/backward of chunk i and the device-to-host
copies of chunk i-1.  Host tensors should be pinned; results are complete when it returns."""
import torch

from .distributed import packed_box_gradient


class HostPipeline:
    def __init__(self, module, batch, h, w, chunks=4, group=None):
        self.module = module
        self.group = group
        dev = module.x_min.device
        C, F = module.in_planes, module.num_filters
        chunks = max(1, min(chunks, batch))
        bounds = [round(i * batch / chunks) for i in range(chunks + 1)]
        self.slices = [slice(a, b) for a, b in zip(bounds[:-1], bounds[1:]) if b > a]
        self.x_dev = [torch.empty((s.stop - s.start, C, h, w), device=dev).requires_grad_() for s in self.slices]
        self.go_dev = [torch.empty((s.stop - s.start, C * F, h, w), device=dev) for s in self.slices]
        self.copy_in, self.compute, self.copy_out = (torch.cuda.Stream(dev) for _ in range(3))

    def step(self, x_host, grad_output_host, out_host, grad_input_host, grad_params_host):
        m = self.module
        params = (m.x_min, m.x_max, m.y_min, m.y_max)
        for p in params:
            p.grad = None
        cur = torch.cuda.current_stream()
        for s in (self.copy_in, self.compute, self.copy_out):
            s.wait_stream(cur)
        alive = []
        for i, sl in enumerate(self.slices):
            ready, done = torch.cuda.Event(), torch.cuda.Event()
            with torch.cuda.stream(self.copy_in):
                self.x_dev[i].grad = None
                self.x_dev[i].data.copy_(x_host[sl], non_blocking=True)
                self.go_dev[i].copy_(grad_output_host[sl], non_blocking=True)
                ready.record()
            with torch.cuda.stream(self.compute):
                self.compute.wait_event(ready)
                out = m(self.x_dev[i])
                out.backward(self.go_dev[i])
                done.record()
            with torch.cuda.stream(self.copy_out):
                self.copy_out.wait_event(done)
                out_host[sl].copy_(out.detach(), non_blocking=True)
                grad_input_host[sl].copy_(self.x_dev[i].grad, non_blocking=True)
            alive.append(out)
        with torch.cuda.stream(self.compute):
            if self.group is not None or (torch.distributed.is_available() and torch.distributed.is_initialized()
                                          and torch.distributed.get_world_size() > 1):
                from .distributed import allreduce_box_gradients
                allreduce_box_gradients(m, self.group)
            packed, _ = packed_box_gradient(m)
            grad_params_host.copy_(packed, non_blocking=True)
        self.copy_in.synchronize()
        self.compute.synchronize()
        self.copy_out.synchronize()
        del alive
