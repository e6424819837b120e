"""Batch-sharded training: every rank runs the box block on its own samples with replicated
parameters; the only exchange is the sum of the parameter gradients (the reference's example
trainer gets the same effect from single-process ``nn.DataParallel``,
``examples/Cityscapes/train.py:125``)."""
import torch
import torch.distributed as dist


def packed_box_gradient(module):
    """The four parameter gradients as one (4, C, F) tensor.  The backward pass writes them into
    one buffer, so normally this is a view of that buffer (no copy); otherwise they are stacked
    and the second return value is True (the caller must copy the result back)."""
    grads = [module.x_min.grad, module.x_max.grad, module.y_min.grad, module.y_max.grad]
    if any(g is None for g in grads):
        raise RuntimeError("allreduce_box_gradients: run backward first")
    g0 = grads[0]
    n = g0.numel()
    same = all(g.is_contiguous() and g.untyped_storage().data_ptr() == g0.untyped_storage().data_ptr()
               and g.storage_offset() == g0.storage_offset() + i * n for i, g in enumerate(grads))
    if same and g0.untyped_storage().nbytes() >= (g0.storage_offset() + 4 * n) * g0.element_size():
        C, F = g0.shape
        return torch.as_strided(g0, (4, C, F), (C * F, F, 1)), False
    return torch.stack(grads), True


def allreduce_box_gradients(module, group=None, async_op=False):
    """Sums the parameter gradients of ``module`` over the ranks of ``group`` with ONE collective
    on the packed (4, C, F) buffer.  With ``async_op`` returns the work handle."""
    packed, copied = packed_box_gradient(module)
    work = dist.all_reduce(packed, op=dist.ReduceOp.SUM, group=group, async_op=async_op and not copied)
    if copied:
        for p, g in zip((module.x_min, module.x_max, module.y_min, module.y_max), packed):
            p.grad.copy_(g)
    return work
