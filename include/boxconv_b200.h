/*
 * boxconv_b200 -- C ABI of the Blackwell (sm_100a) box-convolution hot path.
 *
 * Every entry point takes plain device pointers and sizes, enqueues its kernels on the CUDA
 * stream it is given and returns without synchronising.  The library never allocates, frees
 * or copies behind the caller's back: outputs and scratch memory are supplied by the caller
 * (query the scratch size first).  Return value: BC_OK (0) or a negative BC_ERR_* code;
 * bc_status_string() gives a short text for it.  There is no CPU implementation behind any of
 * these calls.
 *
 * Conventions (those of the reference project): fp32 everywhere; the "x" axis is rows/height,
 * "y" is columns/width; box parameters come as four arrays of C*F floats (x_min, x_max, y_min,
 * y_max) indexed k = c*F + f, in actual pixels unless stated; an integral image of an h x w
 * plane has (h+1) x (w+1) entries with a zero first row and column.  Tensors are dense and
 * row-major: input (N,C,h,w), output / grad_output (N,C,F,h,w) == (N,C*F,h,w).
 *
 * Each declaration names the reference interface it stands in for (path in the reference
 * project : lines).
 */
#ifndef BOXCONV_B200_H
#define BOXCONV_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Same type as cudaStream_t; spelled out so that the header needs no CUDA include. */
typedef struct CUstream_st *bc_stream_t;

enum {
    BC_OK = 0,
    BC_ERR_NULL_POINTER = -1,   /* a required pointer is NULL */
    BC_ERR_BAD_SHAPE = -2,      /* a size is negative, zero where it may not be, or too large */
    BC_ERR_WORKSPACE = -3,      /* scratch memory missing or too small */
    BC_ERR_CUDA = -4,           /* the CUDA runtime reported an error at launch */
    BC_ERR_UNSUPPORTED = -5     /* the combination of arguments is not implemented */
};

/* need_mask bits of the backward entry points */
enum {
    BC_NEED_INPUT = 1,
    BC_NEED_X_MIN = 2,
    BC_NEED_X_MAX = 4,
    BC_NEED_Y_MIN = 8,
    BC_NEED_Y_MAX = 16,
    BC_NEED_ALL = 31
};

int bc_version(void);
const char *bc_status_string(int status);
/* Text of the last CUDA error seen by this thread inside the library ("" if none). */
const char *bc_last_cuda_error(void);

/* Zero-padded inclusive 2-D prefix sum of `planes` planes of h x w: in (planes,h,w) ->
 * out (planes,h+1,w+1).  Replaces integral_image(): src/integral_image_interface.cpp:8-27,
 * src/integral_image_cuda.cu:67-118 (two column scans and two cuBLAS transposes there; one
 * pass here). */
int bc_integral_image(const float *in, float *out, int64_t planes, int h, int w, bc_stream_t stream);

/* Box gather from a ready integral image: input_integrated (N,C,h+1,w+1) -> output
 * (N,C,F,h,w).  Replaces box_convolution_forward(): src/box_convolution_interface.cpp:13-139
 * with src/box_convolution_cuda_forward.cu:207-251 and the split/area helpers
 * src/box_convolution_cuda_misc.cu:16-72,238-301. */
int bc_box_convolution_forward(const float *input_integrated, const float *x_min,
                               const float *x_max, const float *y_min, const float *y_max,
                               float *output, int N, int C, int F, int h, int w, int normalize,
                               int exact, bc_stream_t stream);

/* Scratch bytes bc_box_convolution_backward() needs for these sizes. */
size_t bc_box_convolution_backward_workspace(int N, int C, int F, int h, int w, int need_mask);

/* Gradients w.r.t. the input and the four box parameters.  Replaces
 * box_convolution_backward(): src/box_convolution_interface.cpp:141-395 with
 * src/box_convolution_cuda_backward.cu:173-190,420-473 and the ATen reductions at
 * interface.cpp:274,343-391.
 *   input_integrated (N,C,h+1,w+1); grad_output (N,C,F,h,w);
 *   output: the forward result.  Accepted for signature compatibility and never read (the
 *           term the reference takes from it is recomputed); may be NULL.
 *   grad_input  (N,C,h,w), written iff need_mask & BC_NEED_INPUT;
 *   grad_params (4,C,F) in the order x_min, x_max, y_min, y_max (src/box_convolution.h:3),
 *               in reparametrized units (already multiplied by reparametrization_h / _w);
 *               rows whose need bit is clear are left untouched.
 * The workspace must be 256-byte aligned. */
int bc_box_convolution_backward(const float *input_integrated, const float *x_min,
                                const float *x_max, const float *y_min, const float *y_max,
                                const float *grad_output, const float *output,
                                float reparametrization_h, float reparametrization_w, int N,
                                int C, int F, int h, int w, int normalize, int exact,
                                int need_mask, float *grad_input, float *grad_params,
                                void *workspace, size_t workspace_bytes, bc_stream_t stream);

/* In-place projection of the stored (reparametrized) parameters, `count` = C*F values per
 * array.  Replaces clip_parameters(): src/box_convolution_interface.cpp:397-415 with
 * src/box_convolution_cuda_misc.cu:190-236 (two launches there, one here). */
int bc_clip_parameters(float *x_min, float *x_max, float *y_min, float *y_max, int count,
                       double reparametrization_h, double reparametrization_w,
                       double max_input_h, double max_input_w, int exact, bc_stream_t stream);

/* The same projection, which in addition leaves a packed (4, count) copy of the clipped values
 * (x_min, x_max, y_min, y_max) in packed_out: the snapshot of its parameters that a training
 * forward pass keeps for the backward pass (the reference's autograd Function makes fresh
 * pixel-unit copies, box_convolution/box_convolution_function.py:36-42,51), taken by the launch
 * that clips instead of by a copy kernel of its own. */
int bc_clip_parameters_packed(float *x_min, float *x_max, float *y_min, float *y_max, int count,
                              double reparametrization_h, double reparametrization_w,
                              double max_input_h, double max_input_w, int exact, float *packed_out,
                              bc_stream_t stream);

/* ---- float64 forms of the four functions above ----------------------------------------
 * The reference dispatches its operator over floating types (AT_DISPATCH_FLOATING_TYPES_AND_HALF,
 * src/box_convolution_interface.cpp:51,201; src/integral_image_interface.cpp:8-27) and its own
 * tests check gradients in float64 (test/test_boxconv.py).  Same arguments and behaviour as the
 * float entry points, every array (workspace contents included) in double. */
int bc_integral_image_f64(const double *in, double *out, int64_t planes, int h, int w, bc_stream_t stream);
int bc_box_convolution_forward_f64(const double *input_integrated, const double *x_min,
                                   const double *x_max, const double *y_min, const double *y_max,
                                   double *output, int N, int C, int F, int h, int w, int normalize,
                                   int exact, bc_stream_t stream);
size_t bc_box_convolution_backward_workspace_f64(int N, int C, int F, int h, int w, int need_mask);
int bc_box_convolution_backward_f64(const double *input_integrated, const double *x_min,
                                    const double *x_max, const double *y_min, const double *y_max,
                                    const double *grad_output, const double *output,
                                    double reparametrization_h, double reparametrization_w, int N,
                                    int C, int F, int h, int w, int normalize, int exact,
                                    int need_mask, double *grad_input, double *grad_params,
                                    void *workspace, size_t workspace_bytes, bc_stream_t stream);
int bc_clip_parameters_f64(double *x_min, double *x_max, double *y_min, double *y_max, int count,
                           double reparametrization_h, double reparametrization_w,
                           double max_input_h, double max_input_w, int exact, bc_stream_t stream);

/* ---- the module step, fused ------------------------------------------------------------
 * What BoxConvolutionFunction.forward / .backward do as a chain of extension calls
 * (box_convolution/box_convolution_function.py:32-65), taken from the input itself: the
 * parameters are the STORED ones and are multiplied by reparametrization_h / _w in fp32 as
 * reparametrize() does (function.py:17-27); integral images live in shared memory when a
 * plane fits there and in the workspace otherwise. */
size_t bc_boxconv2d_forward_workspace(int N, int C, int F, int h, int w);
int bc_boxconv2d_forward(const float *input, const float *x_min, const float *x_max,
                         const float *y_min, const float *y_max, float reparametrization_h,
                         float reparametrization_w, float *output, int N, int C, int F, int h,
                         int w, int normalize, int exact, void *workspace,
                         size_t workspace_bytes, bc_stream_t stream);

/* Inference forward of a whole box block tail in one pass: what BottleneckBoxConv does around the
 * box convolution once the network is in eval mode (examples/Cityscapes/models/ENet.py:282-304,
 * examples/Cityscapes/models/ERFNet.py:117-137 of the reference: ReLU, BoxConv2d, BatchNorm2d,
 * residual add, ReLU as separate PyTorch operators, each a full read and write of its tensor):
 *   out[n, k] = act( out_scale[k] * box(act_in(input))[n, k] + out_shift[k] + residual[n, k] ),
 *   k = c*F + f.
 *   input_relu   nonzero: ReLU on the input as it is read;
 *   out_scale, out_shift  (C*F) each, the folded BatchNorm of the output channels; NULL = 1 / 0;
 *   residual     (N, C*F, h, w) or NULL; may be the output buffer itself (in-place skip connection);
 *   output_relu  nonzero: ReLU on the result.
 * No gradients.  Workspace as bc_boxconv2d_forward_workspace(). */
int bc_boxconv2d_forward_fused(const float *input, const float *x_min, const float *x_max,
                               const float *y_min, const float *y_max, float reparametrization_h,
                               float reparametrization_w, float *output, int N, int C, int F, int h,
                               int w, int normalize, int exact, int input_relu, const float *out_scale,
                               const float *out_shift, const float *residual, int output_relu,
                               void *workspace, size_t workspace_bytes, bc_stream_t stream);

size_t bc_boxconv2d_backward_workspace(int N, int C, int F, int h, int w, int need_mask);
int bc_boxconv2d_backward(const float *input, const float *x_min, const float *x_max,
                          const float *y_min, const float *y_max, const float *grad_output,
                          float reparametrization_h, float reparametrization_w, int N, int C,
                          int F, int h, int w, int normalize, int exact, int need_mask,
                          float *grad_input, float *grad_params, void *workspace,
                          size_t workspace_bytes, bc_stream_t stream);

/* ---- a whole training step on a batch in host memory -------------------------------------
 * What a caller of the reference does around the module when its data sit in host memory
 * (copy in, BoxConv2d.forward with its parameter clip, backward, copy out:
 * box_convolution/box_convolution_module.py:216-222, box_convolution_function.py:32-65), as one
 * call on HOST buffers: x (N,C,h,w) and grad_output (N,C*F,h,w) in, output, grad_input and the
 * packed (4,C,F) parameter gradient out.  The batch is processed in `chunks` pieces whose copies
 * and kernels overlap on the three streams given; host buffers should be pinned.  The four
 * parameter arrays are device memory in stored units and are clipped in place when clip != 0.
 * The call only enqueues work: results are complete once `copy_out` has been synchronised, and
 * that must happen before the next call that uses the same workspace.  The workspace (device
 * memory, 256-byte aligned, size from the query) holds the device copies of all tensors. */
size_t bc_boxconv2d_host_step_workspace(int N, int C, int F, int h, int w, int chunks);
int bc_boxconv2d_host_step(const float *x_host, const float *grad_output_host, float *out_host,
                           float *grad_input_host, float *grad_params_host, float *x_min, float *x_max,
                           float *y_min, float *y_max, float reparametrization_h,
                           float reparametrization_w, double max_input_h, double max_input_w, int N,
                           int C, int F, int h, int w, int normalize, int exact, int clip, int chunks,
                           void *workspace, size_t workspace_bytes, bc_stream_t copy_in,
                           bc_stream_t compute, bc_stream_t copy_out);

/* ---- float16 / bfloat16 tensors ---------------------------------------------------------
 * The reference instantiates every kernel of the operator for at::Half
 * (AT_DISPATCH_FLOATING_TYPES_AND_HALF: src/box_convolution_cuda_forward.cu:224,
 * src/box_convolution_cuda_backward.cu:176,431, src/integral_image_cuda.cu:79).  These are
 * bc_boxconv2d_forward() / bc_boxconv2d_backward() for tensors stored in a 16-bit type: input,
 * grad_output, output and grad_input are arrays of 16-bit values of kind io_kind, read and written
 * as they are (no widened copies in global memory); the box parameters, the scratch memory and
 * grad_params are float, and so are the integral images and all arithmetic on chip (a 16-bit
 * integral image, which the reference's dispatch produces, loses the low bits of every box sum).
 * Served for planes that the shared-memory kernels hold: bc_boxconv2d_narrow_supported() tells;
 * other shapes return BC_ERR_UNSUPPORTED and the caller converts to float.  Scratch size as for the
 * float functions. */
enum { BC_IO_F16 = 1, BC_IO_BF16 = 2 };
int bc_boxconv2d_narrow_supported(int F, int h, int w);
int bc_boxconv2d_forward_narrow(const void *input, int io_kind, const float *x_min, const float *x_max,
                                const float *y_min, const float *y_max, float reparametrization_h,
                                float reparametrization_w, void *output, int N, int C, int F, int h,
                                int w, int normalize, int exact, bc_stream_t stream);
int bc_boxconv2d_backward_narrow(const void *input, int io_kind, const float *x_min, const float *x_max,
                                 const float *y_min, const float *y_max, const void *grad_output,
                                 float reparametrization_h, float reparametrization_w, int N, int C,
                                 int F, int h, int w, int normalize, int exact, int need_mask,
                                 void *grad_input, float *grad_params, void *workspace,
                                 size_t workspace_bytes, bc_stream_t stream);

/* ---- backward pass without caller-supplied scratch memory --------------------------------
 * This entry point has no counterpart in the reference (which allocates its temporaries with
 * at::empty on every call).  It is bc_boxconv2d_backward() for hosts that have no way to hand
 * over a workspace at the moment the gradient is needed and must not allocate one either: a
 * plugin invoked inside somebody else's stream capture (cudaMalloc is not allowed while a stream
 * is capturing), a serving process whose device memory was carved up completely at start-up, or
 * a callback running where the CUDA allocator may not be re-entered.  The scratch memory is a
 * fixed array of BC_STATIC_SCRATCH_BYTES that is part of the library image: every GPU that loads
 * the library holds it until the process exits.
 *
 *  - Problems whose scratch need (bc_boxconv2d_backward_workspace()) exceeds the array are
 *    refused with BC_ERR_WORKSPACE; nothing is launched.  Planes that fit in shared memory need
 *    20 bytes per (sample, plane, filter), so the array covers N*C*F up to about 200 000; larger
 *    planes need a full set of integral images and fit only when tiny.
 *  - The first call on each device looks up the array's device address (with that device
 *    current); make that first call outside any stream capture.  A call with N = 0 and
 *    need_mask = BC_NEED_INPUT launches nothing and needs no valid pointers, but does that look-up:
 *    the cheap way to make the first call.  No call allocates or frees; with the CUDA driver's lazy
 *    module loading the first call is also when the array itself is placed on the device (device
 *    memory in use grows by its size once, then stays).  The address is kept for
 *    the life of the process: after cudaDeviceReset() this entry point must not be used any more.
 *  - All calls on a device share the one array and it keeps what the previous call left.  Nothing
 *    in it has to start at zero: every word a call reads was written earlier by that same call.
 *    Two calls that overlap on the GPU (different streams, or graphs replayed concurrently) race
 *    on it and corrupt each other's parameter gradients: serialise them. */
#define BC_STATIC_SCRATCH_BYTES (4u << 20)
int bc_boxconv2d_backward_static(const float *input, const float *x_min, const float *x_max,
                                 const float *y_min, const float *y_max, const float *grad_output,
                                 float reparametrization_h, float reparametrization_w, int N, int C,
                                 int F, int h, int w, int normalize, int exact, int need_mask,
                                 float *grad_input, float *grad_params, bc_stream_t stream);

/* ---- measurement aids (no counterpart in the reference) ---------------------------------
 * bc_launch_count(): kernels launched by this library since it was loaded.
 * bc_profile_*: while enabled, every kernel launch is bracketed by a pair of CUDA events on the
 * launching stream, so that a benchmark can read per-kernel device times of a normal run.
 * Events are host-side objects created by bc_profile_start() on the device that is current at that
 * call, so one process profiles one device (launches on streams of another device fail to record);
 * recording must not be enabled while a stream is being captured into a CUDA graph.  After a device synchronisation,
 * bc_profile_get(i, ...) returns kernel id and milliseconds of record i;
 * bc_kernel_name(id) names the kernel. */
uint64_t bc_launch_count(void);
/* Kernels that stage planes with asynchronous bulk copies wait for them with a time limit
 * (about a second); *count receives how many such waits have expired on the current device since
 * the library was loaded.  Synchronises the device.  Anything but 0 means results are invalid. */
int bc_wait_timeouts(int *count);
int bc_profile_start(int capacity);
int bc_profile_stop(void);
int bc_profile_count(void);
int bc_profile_get(int index, int *kernel_id, float *milliseconds);
const char *bc_kernel_name(int kernel_id);

#ifdef __cplusplus
}
#endif
#endif /* BOXCONV_B200_H */
