// Whole-plane kernels (box_plane_kernels.cuh) for float tensors, and the functions of the plane path
// that do not depend on the tensors' storage type.
#include "box_plane_kernels.cuh"

namespace bc {

bool plane_path_fits_forward(int F, int h, int w) { return plane_fits_forward(F, h, w); }
bool plane_path_fits_backward(int F, int h, int w) { return plane_fits_backward(F, h, w); }

int launch_forward_plane(const float *x, const BoxParams &bp, float *out, int N, int C, int F, int h,
                         int w, bool normalize, bool exact, cudaStream_t s)
{
    return launch_forward_plane_t<float>(x, bp, nullptr, out, N, C, F, h, w, normalize, exact, s);
}

int launch_forward_plane_fused(const float *x, const BoxParams &bp, const Fusion &fu, float *out, int N, int C,
                               int F, int h, int w, bool normalize, bool exact, cudaStream_t s)
{
    return launch_forward_plane_t<float>(x, bp, &fu, out, N, C, F, h, w, normalize, exact, s);
}

int launch_backward_plane(const float *x, const float *grad_output, const BoxParams &bp, float rep_h,
                          float rep_w, int N, int C, int F, int h, int w, bool normalize, bool exact,
                          int need_mask, float *grad_input, float *grad_params, float *partials,
                          cudaStream_t s)
{
    return launch_backward_plane_t<float>(x, grad_output, bp, rep_h, rep_w, N, C, F, h, w, normalize, exact, need_mask,
                                          grad_input, grad_params, partials, s);
}

// Number of bounded waits that expired on the current device since the library was loaded
// (synchronises).  Nonzero means an asynchronous copy never signalled completion.
int read_wait_timeouts(int *count)
{
    int here = 0, narrow = 0;
    int st = read_wait_timeouts_here(&here);
    if (st != BC_OK) return st;
    st = read_wait_timeouts_narrow(&narrow);
    if (st != BC_OK) return st;
    *count = here + narrow;
    return BC_OK;
}

}  // namespace bc
