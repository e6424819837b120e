"""The reference's example networks running UNMODIFIED on this package.

Their source files are loaded from a checkout of the reference at test time (never copied):
`examples/Cityscapes/models/ENet.py`, `examples/Cityscapes/models/ERFNet.py` and
`examples/mnist.py` all do `from box_convolution import BoxConv2d`, which resolves to this
package.  Skipped on machines without the checkout (its path: BOXCONV_REFERENCE, or a folder
`reference` beside the repository).

What is checked: the models construct, a synthetic 512 x 1024 frame (the reference's own runtime
scenario uses `torch.rand` frames too, `examples/Cityscapes/convnet-runtime-benchmark.py:25-27`)
goes forward and backward through every BoxConv2d of the network with finite results and finite,
non-trivial box gradients; the inference preparation of the runtime script (`exact = False` on every
BoxConv2d, BatchNorm and Dropout removed, `eval()`: lines 38-53 there) works and the prepared network
gives the same output twice (to rounding: the convolutions around the box blocks are cuDNN's).
"""
import importlib.util
import os
import sys

import pytest
import torch

from oracle import build_ref

pytestmark = pytest.mark.gpu

REFERENCE = build_ref.reference_root()
needs_reference = pytest.mark.skipif(REFERENCE is None, reason="no checkout of the reference on this machine")


def load_source(relative_path, name):
    path = os.path.join(REFERENCE, relative_path)
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def box_modules(model):
    import box_convolution as bc
    return [m for m in model.modules() if isinstance(m, bc.BoxConv2d)]


def prepare_for_inference(model):
    """What convnet-runtime-benchmark.py:38-53 does to a model before timing it."""
    def strip(module):
        for child_name, child in module.named_children():
            child_type = str(type(child))
            if "BatchNorm" in child_type or "Dropout" in child_type:
                module.__setattr__(child_name, torch.nn.Sequential())
            else:
                strip(child)

    for m in box_modules(model):
        m.exact = False
    strip(model)
    return model.eval()


def train_step_is_finite(model, frame):
    model.train()
    out = model(frame)
    assert torch.isfinite(out).all()
    out.float().mean().backward()
    boxes = box_modules(model)
    assert boxes
    for m in boxes:
        for p in (m.x_min, m.x_max, m.y_min, m.y_max):
            assert p.grad is not None and torch.isfinite(p.grad).all()
    assert any(float(m.x_min.grad.abs().max()) > 0 for m in boxes)
    return out


@needs_reference
@pytest.mark.parametrize("source,cls,n_boxes", [
    ("examples/Cityscapes/models/ENet.py", "BoxENet", 12),
    ("examples/Cityscapes/models/ERFNet.py", "BoxERFNet", 5),
])
def test_cityscapes_models_run_on_this_package(source, cls, n_boxes):
    assert torch.cuda.is_available()
    torch.manual_seed(0)
    mod = load_source(source, "reference_" + cls)
    model = getattr(mod, cls)(18).cuda()
    assert len(box_modules(model)) == n_boxes
    frame = torch.rand(1, 3, 512, 1024, device="cuda")
    out = train_step_is_finite(model, frame)
    assert out.shape == (1, 19, 512, 1024)
    model.zero_grad(set_to_none=True)
    prepare_for_inference(model)
    with torch.no_grad():
        a = model(frame)
        b = model(frame)
    # (cuDNN may pick non-deterministic convolution algorithms: close, not necessarily bit-equal)
    assert torch.isfinite(a).all() and torch.isfinite(b).all()
    assert float((a - b).abs().max()) <= 1e-3 * float(a.abs().max())
    assert all(not m.exact and not m.training for m in box_modules(model))


@needs_reference
def test_mnist_example_net_runs_on_this_package(tmp_path, monkeypatch):
    monkeypatch.chdir(tmp_path)             # the example opens a video file in the working directory
    mod = load_source("examples/mnist.py", "reference_mnist_example")
    torch.manual_seed(0)
    model = mod.Net().cuda()                # BoxConv2d(1, 40, 28, 28): 40 filters per plane
    digits = torch.rand(16, 1, 28, 28, device="cuda")
    model.train()
    out = model(digits)
    assert out.shape == (16, 10) and torch.isfinite(out).all()
    torch.nn.functional.nll_loss(out, torch.arange(16, device="cuda") % 10).backward()
    for p in (model.conv1.x_min, model.conv1.x_max, model.conv1.y_min, model.conv1.y_max):
        assert torch.isfinite(p.grad).all() and float(p.grad.abs().max()) > 0
