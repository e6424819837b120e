// Shared declarations of the library's translation units.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "../../include/boxconv_b200.h"
#include "bc_taps.cuh"

namespace bc {

// The four parameter arrays plus the fp32 factors that turn stored values into pixels
// (1 for the entry points that already receive pixels).
struct BoxParams {
    const float *x_min, *x_max, *y_min, *y_max;
    float mul_h, mul_w;
};

struct Box {
    float xmin, xmax, ymin, ymax;
};

__device__ __forceinline__ Box load_box(const BoxParams &p, int k)
{
    Box b;
    b.xmin = __ldg(p.x_min + k) * p.mul_h;
    b.xmax = __ldg(p.x_max + k) * p.mul_h;
    b.ymin = __ldg(p.y_min + k) * p.mul_w;
    b.ymax = __ldg(p.y_max + k) * p.mul_w;
    return b;
}

// Records a CUDA launch error for bc_last_cuda_error() and maps it to a status code.
int check_launch(const char *what);

// Kernel ids reported by the profiling aid (bc_profile_get / bc_kernel_name).
enum KernelId {
    KID_INTEGRAL = 1, KID_FORWARD_GLOBAL, KID_BACKWARD_GLOBAL, KID_FINISH_PARAM_GRADS, KID_CLIP,
    KID_FORWARD_PLANE, KID_BACKWARD_PLANE, KID_SUM_CHUNKS, KID_COUNT
};

// Put around a kernel launch: counts it and, while profiling is enabled, records a CUDA event on
// the stream before and after it.
struct LaunchScope {
    LaunchScope(int kernel_id, cudaStream_t stream);
    ~LaunchScope();
    cudaStream_t stream;
    int slot;
};

// ---- launchers (one per translation unit) --------------------------------------------------
int launch_integral_image(const float *in, float *out, int64_t planes, int h, int w, cudaStream_t s);

int launch_forward_global(const float *integ, const BoxParams &bp, float *out, int N, int C, int F,
                          int h, int w, bool normalize, bool exact, cudaStream_t s);

// Backward from integral(grad_output) held in global memory.  Exactly one of x / x_integ is
// non-null: the input plane values are read from x, or rebuilt from the input's integral image.
size_t backward_partials_bytes(int N, int C, int F, int h, int w);
int launch_backward_global(const float *x, const float *x_integ, const float *go_integ,
                           const BoxParams &bp, float rep_h, float rep_w, int N, int C, int F,
                           int h, int w, bool normalize, bool exact, int need_mask,
                           float *grad_input, float *grad_params, float *partials, cudaStream_t s);

int launch_finish_param_grads(const float *partials, const BoxParams &bp, int count, int per_box,
                              bool normalize, bool exact, float rep_h, float rep_w, int need_mask,
                              float *grad_params, cudaStream_t s);

// Shared-memory-resident path for small planes (box_plane_smem.cu).
bool plane_path_fits_forward(int F, int h, int w);
bool plane_path_fits_backward(int F, int h, int w);
int launch_forward_plane(const float *x, const BoxParams &bp, float *out, int N, int C, int F, int h,
                         int w, bool normalize, bool exact, cudaStream_t s);
// partials: C*F*N*5 floats
int launch_backward_plane(const float *x, const float *grad_output, const BoxParams &bp, float rep_h,
                          float rep_w, int N, int C, int F, int h, int w, bool normalize, bool exact,
                          int need_mask, float *grad_input, float *grad_params, float *partials,
                          cudaStream_t s);

int read_wait_timeouts(int *count);

int launch_clip(float *x_min, float *x_max, float *y_min, float *y_max, int count, double rep_h,
                double rep_w, double max_h, double max_w, bool exact, cudaStream_t s);

}  // namespace bc
