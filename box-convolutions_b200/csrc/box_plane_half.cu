// Whole-plane kernels (box_plane_kernels.cuh) for float16 and bfloat16 tensors: the reference
// instantiates its kernels for at::Half (src/box_convolution_cuda_forward.cu:224,
// src/box_convolution_cuda_backward.cu:176,431).  Input, grad_output, output and grad_input are
// stored narrow; the integral images, all arithmetic and the parameter gradients are float.
#include "box_plane_kernels.cuh"

namespace bc {

int launch_forward_plane_narrow(const void *x, int io_kind, const BoxParams &bp, void *out, int N, int C, int F, int h,
                                int w, bool normalize, bool exact, cudaStream_t s)
{
    if (io_kind == BC_IO_F16)
        return launch_forward_plane_t<__half>(static_cast<const __half *>(x), bp, nullptr, static_cast<__half *>(out), N, C,
                                              F, h, w, normalize, exact, s);
    if (io_kind == BC_IO_BF16)
        return launch_forward_plane_t<__nv_bfloat16>(static_cast<const __nv_bfloat16 *>(x), bp, nullptr,
                                                     static_cast<__nv_bfloat16 *>(out), N, C, F, h, w, normalize, exact, s);
    return BC_ERR_UNSUPPORTED;
}

int launch_backward_plane_narrow(const void *x, const void *grad_output, int io_kind, const BoxParams &bp, float rep_h,
                                 float rep_w, int N, int C, int F, int h, int w, bool normalize, bool exact,
                                 int need_mask, void *grad_input, float *grad_params, float *partials, cudaStream_t s)
{
    if (io_kind == BC_IO_F16)
        return launch_backward_plane_t<__half>(static_cast<const __half *>(x), static_cast<const __half *>(grad_output), bp,
                                               rep_h, rep_w, N, C, F, h, w, normalize, exact, need_mask,
                                               static_cast<__half *>(grad_input), grad_params, partials, s);
    if (io_kind == BC_IO_BF16)
        return launch_backward_plane_t<__nv_bfloat16>(static_cast<const __nv_bfloat16 *>(x),
                                                      static_cast<const __nv_bfloat16 *>(grad_output), bp, rep_h, rep_w, N,
                                                      C, F, h, w, normalize, exact, need_mask,
                                                      static_cast<__nv_bfloat16 *>(grad_input), grad_params, partials, s);
    return BC_ERR_UNSUPPORTED;
}

int read_wait_timeouts_narrow(int *count) { return read_wait_timeouts_here(count); }

}  // namespace bc
