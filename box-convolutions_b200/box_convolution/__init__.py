"""Box convolutions on B200: the reference's Python surface (``from box_convolution import
BoxConv2d``) on top of hand-written sm_100a kernels.  CUDA only."""
from .module import BoxConv2d
from .function import BoxConvolutionFunction, reparametrize
from .ext import integral_image, box_convolution_forward, box_convolution_backward, clip_parameters

__all__ = ["BoxConv2d", "BoxConvolutionFunction", "reparametrize", "integral_image",
           "box_convolution_forward", "box_convolution_backward", "clip_parameters"]
