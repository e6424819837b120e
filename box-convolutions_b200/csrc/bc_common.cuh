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
template <typename T>
struct BoxParamsT {
    const T *x_min, *x_max, *y_min, *y_max;
    T mul_h, mul_w;
};
using BoxParams = BoxParamsT<float>;

template <typename T>
struct BoxT {
    T xmin, xmax, ymin, ymax;
};
using Box = BoxT<float>;

template <typename T>
__device__ __forceinline__ BoxT<T> load_box(const BoxParamsT<T> &p, int k)
{
    BoxT<T> b;
    b.xmin = __ldg(p.x_min + k) * p.mul_h;
    b.xmax = __ldg(p.x_max + k) * p.mul_h;
    b.ymin = __ldg(p.y_min + k) * p.mul_w;
    b.ymax = __ldg(p.y_max + k) * p.mul_w;
    return b;
}

// What the fused inference forward does around the gather (all optional): ReLU on the input as
// it is read, then per output channel k = c*F + f:  out = act(scale[k] * box(x) + shift[k] + residual).
struct Fusion {
    int input_relu;
    const float *scale, *shift;     // (C*F) each, or null for 1 / 0
    const float *residual;          // (N, C*F, h, w) or null; may be the output buffer itself
    int output_relu;
};

// Records a CUDA launch error for bc_last_cuda_error() and maps it to a status code.
int check_launch(const char *what);
// For a runtime call that returned `e` != cudaSuccess: records it (whatever cudaGetLastError says:
// cudaErrorNotReady, for one, is not sticky) and returns BC_ERR_CUDA.
int cuda_failed(cudaError_t e, const char *what);

// Kernel ids reported by the profiling aid (bc_profile_get / bc_kernel_name).
enum KernelId {
    KID_INTEGRAL = 1, KID_FORWARD_GLOBAL, KID_BACKWARD_GLOBAL, KID_FINISH_PARAM_GRADS, KID_CLIP,
    KID_FORWARD_PLANE, KID_BACKWARD_PLANE, KID_SUM_CHUNKS, KID_BACKWARD_BAND, KID_INTEGRAL_BANDS, KID_FORWARD_BAND, KID_COUNT
};

// Put around a kernel launch: counts it and, while profiling is enabled, records a CUDA event on
// the stream before and after it.
struct LaunchScope {
    LaunchScope(int kernel_id, cudaStream_t stream);
    ~LaunchScope();
    cudaStream_t stream;
    cudaEvent_t after;      // null unless this launch is being timed
};

// ---- programmatic dependent launch ---------------------------------------------------------
// launch_overlapped() lets the GPU schedule a kernel's CTAs while the kernel in front of it in the
// stream is still running; such a kernel must call grid_dependency_wait() before it touches
// anything a predecessor in the stream may still be writing or reading (the wait returns when the
// kernel in front has completed and flushed, which in turn had waited for the one before it).
// What overlaps is launch latency and the instructions before the wait.
// grid_dependency_release() in the kernel in front allows the scheduling to begin before it exits.
#if defined(__CUDACC__)
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dependency_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <class... KArgs, class... Args>
inline cudaError_t launch_overlapped(void (*kernel)(KArgs...), unsigned grid, unsigned block, size_t smem,
                                     cudaStream_t stream, Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(block);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
#endif

// ---- launchers (one per translation unit) --------------------------------------------------
// (the general kernels exist for float and double; everything else is float only)
template <typename T>
int launch_integral_image(const T *in, T *out, int64_t planes, int h, int w, cudaStream_t s);
template <> int launch_integral_image<float>(const float *, float *, int64_t, int, int, cudaStream_t);
template <> int launch_integral_image<double>(const double *, double *, int64_t, int, int, cudaStream_t);

template <typename T>
int launch_forward_global(const T *integ, const BoxParamsT<T> &bp, T *out, int N, int C, int F,
                          int h, int w, bool normalize, bool exact, cudaStream_t s);

// Backward from integral(grad_output) held in global memory.  Exactly one of x / x_integ is
// non-null: the input plane values are read from x, or rebuilt from the input's integral image.
size_t backward_partials_bytes(int N, int C, int F, int h, int w, size_t elem_size = sizeof(float));
template <typename T>
int launch_backward_global(const T *x, const T *x_integ, const T *go_integ, const BoxParamsT<T> &bp,
                           T rep_h, T rep_w, int N, int C, int F, int h, int w, bool normalize,
                           bool exact, int need_mask, T *grad_input, T *grad_params, T *partials,
                           cudaStream_t s);

template <typename T>
int launch_clip(T *x_min, T *x_max, T *y_min, T *y_max, int count, double rep_h, double rep_w,
                double max_h, double max_w, bool exact, cudaStream_t s, T *packed = nullptr);

template <typename T>
int launch_finish_param_grads(const T *partials, const BoxParamsT<T> &bp, int count, int per_box,
                              bool normalize, bool exact, T rep_h, T rep_w, int need_mask,
                              T *grad_params, cudaStream_t s);

// float integral image with an optional ReLU on the values read
// lpad/rpad > 0 write rows as [lpad zeros | I[a][0..w] | rpad copies of I[a][w]] (pitch lpad + w + 1 + rpad)
int launch_integral_image_f32(const float *in, float *out, int64_t planes, int h, int w, bool relu_in,
                              cudaStream_t s, int lpad = 0, int rpad = 0);
// forward with the Fusion steps; a null `fu` is the plain forward
int launch_forward_global_fused(const float *integ, const BoxParams &bp, const Fusion &fu, float *out, int N,
                                int C, int F, int h, int w, bool normalize, bool exact, cudaStream_t s);
int launch_forward_plane_fused(const float *x, const BoxParams &bp, const Fusion &fu, float *out, int N, int C,
                               int F, int h, int w, bool normalize, bool exact, cudaStream_t s);

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
int read_wait_timeouts_narrow(int *count);

// The same whole-plane kernels on float16 / bfloat16 tensors (box_plane_half.cu); io_kind is
// BC_IO_F16 or BC_IO_BF16, the parameters, partial sums and parameter gradients are float.
int launch_forward_plane_narrow(const void *x, int io_kind, const BoxParams &bp, void *out, int N, int C, int F, int h,
                                int w, bool normalize, bool exact, cudaStream_t s);
int launch_backward_plane_narrow(const void *x, const void *grad_output, int io_kind, const BoxParams &bp, float rep_h,
                                 float rep_w, int N, int C, int F, int h, int w, bool normalize, bool exact,
                                 int need_mask, void *grad_input, float *grad_params, float *partials, cudaStream_t s);

// Column-band kernels for planes that do not fit in shared memory whole (box_band_smem.cu): they
// gather from integral images in global memory in the padded row layout
// (launch_integral_image_f32 with band_lpad() / band_rpad(w)), staged band by band.
int band_lpad();
int band_rpad(int w);
size_t band_integral_floats(int64_t planes, int h, int w);
bool band_path_fits_forward(int h, int w);
bool band_path_fits_backward(int F, int h, int w);
size_t band_partials_bytes(int N, int C, int F, int w);
// null `fu` = plain forward
int launch_forward_band(const float *integ_padded, const BoxParams &bp, const Fusion *fu, float *out, int N, int C,
                        int F, int h, int w, bool normalize, bool exact, cudaStream_t s);
int launch_backward_band(const float *x, const float *go_integ_padded, const BoxParams &bp, float rep_h, float rep_w,
                         int N, int C, int F, int h, int w, bool normalize, bool exact, int need_mask,
                         float *grad_input, float *grad_params, float *partials, cudaStream_t s);

}  // namespace bc
