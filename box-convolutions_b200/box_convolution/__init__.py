"""Box convolutions on B200: the reference's Python surface (``from box_convolution import
BoxConv2d``) on top of hand-written sm_100a kernels.  CUDA only."""
from .module import BoxConv2d
from .function import BoxConvolutionFunction, reparametrize
from .ext import integral_image, box_convolution_forward, box_convolution_backward, clip_parameters
from .distributed import allreduce_box_gradients, packed_box_gradient
from .host import HostPipeline
from .inference import fused_box_block, fold_batchnorm, GraphedForward

__all__ = ["fused_box_block", "fold_batchnorm", "GraphedForward", "BoxConv2d", "BoxConvolutionFunction", "reparametrize", "integral_image",
           "box_convolution_forward", "box_convolution_backward", "clip_parameters",
           "allreduce_box_gradients", "packed_box_gradient", "HostPipeline"]
