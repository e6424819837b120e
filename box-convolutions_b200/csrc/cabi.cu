// The extern "C" surface declared in include/boxconv_b200.h: argument checks, workspace
// carving and dispatch to the kernels.  No allocation, no synchronisation.
#include <stdio.h>
#include <atomic>
#include <mutex>
#include <vector>
#include <string.h>

#include "bc_common.cuh"

namespace bc {

static thread_local char g_last_error[256] = "";

int check_launch(const char *what)
{
    const cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) return BC_OK;
    snprintf(g_last_error, sizeof(g_last_error), "%s: %s", what, cudaGetErrorString(e));
    return BC_ERR_CUDA;
}

int cuda_failed(cudaError_t e, const char *what)
{
    cudaGetLastError();     // clear the sticky copy, if the error left one
    snprintf(g_last_error, sizeof(g_last_error), "%s: %s", what, cudaGetErrorString(e));
    return BC_ERR_CUDA;
}

// ---- launch counter and per-kernel event timing
static std::atomic<uint64_t> g_launches{0};
static std::mutex g_prof_mutex;
static std::atomic<bool> g_prof_on{false};
static int g_prof_used = 0;
struct ProfRecord { int kid; cudaEvent_t a, b; };
static std::vector<ProfRecord> g_prof;

LaunchScope::LaunchScope(int kernel_id, cudaStream_t s) : stream(s), after(nullptr)
{
    g_launches.fetch_add(1, std::memory_order_relaxed);
    if (!g_prof_on.load(std::memory_order_acquire)) return;
    cudaEvent_t before;
    {
        // the record table may be grown by bc_profile_start() on another thread: take the two
        // events out under the lock and never touch the table again from this scope
        std::lock_guard<std::mutex> lock(g_prof_mutex);
        if (!g_prof_on.load(std::memory_order_relaxed) || g_prof_used >= (int)g_prof.size()) return;
        ProfRecord &r = g_prof[g_prof_used++];
        r.kid = kernel_id;
        before = r.a;
        after = r.b;
    }
    cudaEventRecord(before, stream);
}

LaunchScope::~LaunchScope()
{
    if (after) cudaEventRecord(after, stream);
}

static inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

static inline bool sizes_ok(int N, int C, int F, int h, int w)
{
    return N >= 0 && C >= 0 && F >= 0 && h >= 0 && w >= 0 && h < (1 << 24) && w < (1 << 24);
}

static inline bool any_empty(int N, int C, int F, int h, int w)
{
    return N == 0 || C == 0 || F == 0 || h == 0 || w == 0;
}

static inline size_t integral_bytes(int64_t planes, int h, int w)
{
    return align_up((size_t)planes * (size_t)(h + 1) * (size_t)(w + 1) * sizeof(float), 256);
}



// ---- the four extension functions, for float and double ------------------------------------
template <typename T>
static size_t integral_bytes_t(int64_t planes, int h, int w)
{
    return align_up((size_t)planes * (size_t)(h + 1) * (size_t)(w + 1) * sizeof(T), 256);
}

template <typename T>
static int integral_image_entry(const T *in, T *out, int64_t planes, int h, int w, cudaStream_t stream)
{
    if (planes < 0 || h < 0 || w < 0 || h >= (1 << 24) || w >= (1 << 24)) return BC_ERR_BAD_SHAPE;
    if (planes == 0) return BC_OK;
    if (!out || (!in && h > 0 && w > 0)) return BC_ERR_NULL_POINTER;
    return launch_integral_image<T>(in, out, planes, h, w, stream);
}

template <typename T>
static int forward_entry(const T *input_integrated, const T *x_min, const T *x_max, const T *y_min,
                         const T *y_max, T *output, int N, int C, int F, int h, int w, int normalize,
                         int exact, cudaStream_t stream)
{
    if (!sizes_ok(N, C, F, h, w)) return BC_ERR_BAD_SHAPE;
    if (any_empty(N, C, F, h, w)) return BC_OK;
    if (!input_integrated || !x_min || !x_max || !y_min || !y_max || !output) return BC_ERR_NULL_POINTER;
    const BoxParamsT<T> bp{x_min, x_max, y_min, y_max, T(1), T(1)};
    return launch_forward_global<T>(input_integrated, bp, output, N, C, F, h, w, normalize != 0, exact != 0, stream);
}

template <typename T>
static size_t backward_workspace_entry(int N, int C, int F, int h, int w, int need_mask)
{
    if (!sizes_ok(N, C, F, h, w) || any_empty(N, C, F, h, w) || !(need_mask & BC_NEED_ALL)) return 0;
    return integral_bytes_t<T>((int64_t)N * C * F, h, w) +
           align_up(backward_partials_bytes(N, C, F, h, w, sizeof(T)), 256);
}

template <typename T>
static int backward_entry(const T *input_integrated, const T *x_min, const T *x_max, const T *y_min,
                          const T *y_max, const T *grad_output, T reparametrization_h,
                          T reparametrization_w, int N, int C, int F, int h, int w, int normalize,
                          int exact, int need_mask, T *grad_input, T *grad_params, void *workspace,
                          size_t workspace_bytes, cudaStream_t stream)
{
    if (!sizes_ok(N, C, F, h, w)) return BC_ERR_BAD_SHAPE;
    need_mask &= BC_NEED_ALL;
    if (!need_mask) return BC_OK;
    const bool need_params = (need_mask & ~BC_NEED_INPUT) != 0;
    if (any_empty(N, C, F, h, w)) {
        // nothing to gather; parameter gradients of an empty batch are zero
        if (need_params && C > 0 && F > 0) {
            if (!grad_params) return BC_ERR_NULL_POINTER;
            for (int j = 0; j < 4; ++j)
                if (need_mask & (BC_NEED_X_MIN << j))
                    if (cudaError_t e = cudaMemsetAsync(grad_params + (size_t)j * C * F, 0, sizeof(T) * C * F, stream))
                        return cuda_failed(e, "memset");
        }
        return BC_OK;
    }
    if (!input_integrated || !x_min || !x_max || !y_min || !y_max || !grad_output) return BC_ERR_NULL_POINTER;
    if ((need_mask & BC_NEED_INPUT) && !grad_input) return BC_ERR_NULL_POINTER;
    if (need_params && !grad_params) return BC_ERR_NULL_POINTER;
    const size_t ib = integral_bytes_t<T>((int64_t)N * C * F, h, w);
    if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255) ||
        workspace_bytes < backward_workspace_entry<T>(N, C, F, h, w, need_mask))
        return BC_ERR_WORKSPACE;
    T *go_integ = static_cast<T *>(workspace);
    T *partials = reinterpret_cast<T *>(static_cast<char *>(workspace) + ib);

    int st = launch_integral_image<T>(grad_output, go_integ, (int64_t)N * C * F, h, w, stream);
    if (st != BC_OK) return st;
    const BoxParamsT<T> bp{x_min, x_max, y_min, y_max, T(1), T(1)};
    return launch_backward_global<T>(nullptr, input_integrated, go_integ, bp, reparametrization_h,
                                     reparametrization_w, N, C, F, h, w, normalize != 0, exact != 0,
                                     need_mask, grad_input, grad_params, partials, stream);
}

template <typename T>
static int clip_entry(T *x_min, T *x_max, T *y_min, T *y_max, int count, double reparametrization_h,
                      double reparametrization_w, double max_input_h, double max_input_w, int exact,
                      cudaStream_t stream, T *packed = nullptr)
{
    if (count < 0) return BC_ERR_BAD_SHAPE;
    if (count == 0) return BC_OK;
    if (!x_min || !x_max || !y_min || !y_max) return BC_ERR_NULL_POINTER;
    if (reparametrization_h == 0.0 || reparametrization_w == 0.0) return BC_ERR_BAD_SHAPE;
    return launch_clip<T>(x_min, x_max, y_min, y_max, count, reparametrization_h, reparametrization_w,
                          max_input_h, max_input_w, exact != 0, stream, packed);
}

}  // namespace bc

using namespace bc;

extern "C" {

int bc_version(void) { return 100; }

const char *bc_status_string(int status)
{
    switch (status) {
        case BC_OK: return "ok";
        case BC_ERR_NULL_POINTER: return "a required pointer is NULL";
        case BC_ERR_BAD_SHAPE: return "invalid or too large size";
        case BC_ERR_WORKSPACE: return "workspace missing, misaligned or too small";
        case BC_ERR_CUDA: return "CUDA error at kernel launch";
        case BC_ERR_UNSUPPORTED: return "unsupported combination of arguments";
        default: return "unknown status";
    }
}

const char *bc_last_cuda_error(void) { return g_last_error; }

int bc_integral_image(const float *in, float *out, int64_t planes, int h, int w, bc_stream_t stream)
{
    return integral_image_entry<float>(in, out, planes, h, w, stream);
}

int bc_integral_image_f64(const double *in, double *out, int64_t planes, int h, int w, bc_stream_t stream)
{
    return integral_image_entry<double>(in, out, planes, h, w, stream);
}

int bc_box_convolution_forward(const float *input_integrated, const float *x_min,
                               const float *x_max, const float *y_min, const float *y_max,
                               float *output, int N, int C, int F, int h, int w, int normalize,
                               int exact, bc_stream_t stream)
{
    return forward_entry<float>(input_integrated, x_min, x_max, y_min, y_max, output, N, C, F, h, w,
                                normalize, exact, stream);
}

int bc_box_convolution_forward_f64(const double *input_integrated, const double *x_min,
                                   const double *x_max, const double *y_min, const double *y_max,
                                   double *output, int N, int C, int F, int h, int w, int normalize,
                                   int exact, bc_stream_t stream)
{
    return forward_entry<double>(input_integrated, x_min, x_max, y_min, y_max, output, N, C, F, h, w,
                                 normalize, exact, stream);
}

size_t bc_box_convolution_backward_workspace(int N, int C, int F, int h, int w, int need_mask)
{
    return backward_workspace_entry<float>(N, C, F, h, w, need_mask);
}

size_t bc_box_convolution_backward_workspace_f64(int N, int C, int F, int h, int w, int need_mask)
{
    return backward_workspace_entry<double>(N, C, F, h, w, need_mask);
}

int bc_box_convolution_backward(const float *input_integrated, const float *x_min,
                                const float *x_max, const float *y_min, const float *y_max,
                                const float *grad_output, const float *output,
                                float reparametrization_h, float reparametrization_w, int N,
                                int C, int F, int h, int w, int normalize, int exact,
                                int need_mask, float *grad_input, float *grad_params,
                                void *workspace, size_t workspace_bytes, bc_stream_t stream)
{
    (void)output;
    return backward_entry<float>(input_integrated, x_min, x_max, y_min, y_max, grad_output,
                                 reparametrization_h, reparametrization_w, N, C, F, h, w, normalize,
                                 exact, need_mask, grad_input, grad_params, workspace, workspace_bytes,
                                 stream);
}

int bc_box_convolution_backward_f64(const double *input_integrated, const double *x_min,
                                    const double *x_max, const double *y_min, const double *y_max,
                                    const double *grad_output, const double *output,
                                    double reparametrization_h, double reparametrization_w, int N,
                                    int C, int F, int h, int w, int normalize, int exact,
                                    int need_mask, double *grad_input, double *grad_params,
                                    void *workspace, size_t workspace_bytes, bc_stream_t stream)
{
    (void)output;
    return backward_entry<double>(input_integrated, x_min, x_max, y_min, y_max, grad_output,
                                  reparametrization_h, reparametrization_w, N, C, F, h, w, normalize,
                                  exact, need_mask, grad_input, grad_params, workspace, workspace_bytes,
                                  stream);
}

int bc_clip_parameters(float *x_min, float *x_max, float *y_min, float *y_max, int count,
                       double reparametrization_h, double reparametrization_w,
                       double max_input_h, double max_input_w, int exact, bc_stream_t stream)
{
    return clip_entry<float>(x_min, x_max, y_min, y_max, count, reparametrization_h, reparametrization_w,
                             max_input_h, max_input_w, exact, stream);
}

int bc_clip_parameters_packed(float *x_min, float *x_max, float *y_min, float *y_max, int count,
                              double reparametrization_h, double reparametrization_w,
                              double max_input_h, double max_input_w, int exact, float *packed_out,
                              bc_stream_t stream)
{
    if (count > 0 && !packed_out) return BC_ERR_NULL_POINTER;
    return clip_entry<float>(x_min, x_max, y_min, y_max, count, reparametrization_h, reparametrization_w,
                             max_input_h, max_input_w, exact, stream, packed_out);
}

int bc_clip_parameters_f64(double *x_min, double *x_max, double *y_min, double *y_max, int count,
                           double reparametrization_h, double reparametrization_w,
                           double max_input_h, double max_input_w, int exact, bc_stream_t stream)
{
    return clip_entry<double>(x_min, x_max, y_min, y_max, count, reparametrization_h, reparametrization_w,
                              max_input_h, max_input_w, exact, stream);
}

size_t bc_boxconv2d_forward_workspace(int N, int C, int F, int h, int w)
{
    if (!sizes_ok(N, C, F, h, w) || any_empty(N, C, F, h, w)) return 0;
    if (plane_path_fits_forward(F, h, w)) return 0;
    if (band_path_fits_forward(h, w)) return align_up(band_integral_floats((int64_t)N * C, h, w) * sizeof(float), 256);
    return integral_bytes((int64_t)N * C, h, w);
}

// Forward of planes that do not fit in shared memory: integral images to the workspace (padded rows
// for the column-band kernel where a band fits, plain rows for the general kernel otherwise).
static int forward_from_workspace(const float *input, const BoxParams &bp, const Fusion *fu, float *output, int N,
                                  int C, int F, int h, int w, bool normalize, bool exact, float *integ,
                                  cudaStream_t stream)
{
    const bool relu_in = fu && fu->input_relu;
    if (band_path_fits_forward(h, w)) {
        int st = launch_integral_image_f32(input, integ, (int64_t)N * C, h, w, relu_in, stream, band_lpad(), band_rpad(w));
        if (st != BC_OK) return st;
        return launch_forward_band(integ, bp, fu, output, N, C, F, h, w, normalize, exact, stream);
    }
    int st = launch_integral_image_f32(input, integ, (int64_t)N * C, h, w, relu_in, stream);
    if (st != BC_OK) return st;
    if (fu) return launch_forward_global_fused(integ, bp, *fu, output, N, C, F, h, w, normalize, exact, stream);
    return launch_forward_global<float>(integ, bp, output, N, C, F, h, w, normalize, exact, stream);
}

int bc_boxconv2d_forward(const float *input, const float *x_min, const float *x_max,
                         const float *y_min, const float *y_max, float reparametrization_h,
                         float reparametrization_w, float *output, int N, int C, int F, int h,
                         int w, int normalize, int exact, void *workspace,
                         size_t workspace_bytes, bc_stream_t stream)
{
    if (!sizes_ok(N, C, F, h, w)) return BC_ERR_BAD_SHAPE;
    if (any_empty(N, C, F, h, w)) return BC_OK;
    if (!input || !x_min || !x_max || !y_min || !y_max || !output) return BC_ERR_NULL_POINTER;
    const BoxParams bp{x_min, x_max, y_min, y_max, reparametrization_h, reparametrization_w};
    if (plane_path_fits_forward(F, h, w))
        return launch_forward_plane(input, bp, output, N, C, F, h, w, normalize != 0, exact != 0, stream);
    if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255) ||
        workspace_bytes < bc_boxconv2d_forward_workspace(N, C, F, h, w))
        return BC_ERR_WORKSPACE;
    return forward_from_workspace(input, bp, nullptr, output, N, C, F, h, w, normalize != 0, exact != 0,
                                  static_cast<float *>(workspace), stream);
}

int bc_boxconv2d_forward_fused(const float *input, const float *x_min, const float *x_max,
                               const float *y_min, const float *y_max, float reparametrization_h,
                               float reparametrization_w, float *output, int N, int C, int F, int h,
                               int w, int normalize, int exact, int input_relu, const float *out_scale,
                               const float *out_shift, const float *residual, int output_relu,
                               void *workspace, size_t workspace_bytes, bc_stream_t stream)
{
    if (!sizes_ok(N, C, F, h, w)) return BC_ERR_BAD_SHAPE;
    if (any_empty(N, C, F, h, w)) return BC_OK;
    if (!input || !x_min || !x_max || !y_min || !y_max || !output) return BC_ERR_NULL_POINTER;
    const BoxParams bp{x_min, x_max, y_min, y_max, reparametrization_h, reparametrization_w};
    const Fusion fu{input_relu != 0, out_scale, out_shift, residual, output_relu != 0};
    if (plane_path_fits_forward(F, h, w))
        return launch_forward_plane_fused(input, bp, fu, output, N, C, F, h, w, normalize != 0, exact != 0, stream);
    if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255) ||
        workspace_bytes < bc_boxconv2d_forward_workspace(N, C, F, h, w))
        return BC_ERR_WORKSPACE;
    float *integ = static_cast<float *>(workspace);
    return forward_from_workspace(input, bp, &fu, output, N, C, F, h, w, normalize != 0, exact != 0, integ, stream);
}

size_t bc_boxconv2d_backward_workspace(int N, int C, int F, int h, int w, int need_mask)
{
    if (!sizes_ok(N, C, F, h, w) || any_empty(N, C, F, h, w) || !(need_mask & BC_NEED_ALL)) return 0;
    if (plane_path_fits_backward(F, h, w))
        return align_up((size_t)C * F * N * kNumSums * sizeof(float), 256);
    if (band_path_fits_backward(F, h, w))
        return align_up(band_integral_floats((int64_t)N * C * F, h, w) * sizeof(float), 256) +
               align_up(band_partials_bytes(N, C, F, w), 256);
    return integral_bytes((int64_t)N * C * F, h, w) + align_up(backward_partials_bytes(N, C, F, h, w), 256);
}

int bc_boxconv2d_backward(const float *input, const float *x_min, const float *x_max,
                          const float *y_min, const float *y_max, const float *grad_output,
                          float reparametrization_h, float reparametrization_w, int N, int C,
                          int F, int h, int w, int normalize, int exact, int need_mask,
                          float *grad_input, float *grad_params, void *workspace,
                          size_t workspace_bytes, bc_stream_t stream)
{
    if (!sizes_ok(N, C, F, h, w)) return BC_ERR_BAD_SHAPE;
    need_mask &= BC_NEED_ALL;
    if (!need_mask) return BC_OK;
    const bool need_params = (need_mask & ~BC_NEED_INPUT) != 0;
    if (any_empty(N, C, F, h, w)) {
        if (need_params && C > 0 && F > 0) {
            if (!grad_params) return BC_ERR_NULL_POINTER;
            for (int j = 0; j < 4; ++j)
                if (need_mask & (BC_NEED_X_MIN << j))
                    if (cudaError_t e = cudaMemsetAsync(grad_params + (size_t)j * C * F, 0, sizeof(float) * C * F, stream))
                        return cuda_failed(e, "memset");
        }
        return BC_OK;
    }
    if (!input || !x_min || !x_max || !y_min || !y_max || !grad_output) return BC_ERR_NULL_POINTER;
    if ((need_mask & BC_NEED_INPUT) && !grad_input) return BC_ERR_NULL_POINTER;
    if (need_params && !grad_params) return BC_ERR_NULL_POINTER;
    const BoxParams bp{x_min, x_max, y_min, y_max, reparametrization_h, reparametrization_w};
    const bool band = band_path_fits_backward(F, h, w);
    const size_t ib = band ? align_up(band_integral_floats((int64_t)N * C * F, h, w) * sizeof(float), 256)
                           : integral_bytes((int64_t)N * C * F, h, w);
    if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255) ||
        workspace_bytes < bc_boxconv2d_backward_workspace(N, C, F, h, w, need_mask))
        return BC_ERR_WORKSPACE;
    if (plane_path_fits_backward(F, h, w))
        return launch_backward_plane(input, grad_output, bp, reparametrization_h, reparametrization_w, N, C,
                                     F, h, w, normalize != 0, exact != 0, need_mask, grad_input,
                                     grad_params, static_cast<float *>(workspace), stream);
    float *go_integ = static_cast<float *>(workspace);
    float *partials = reinterpret_cast<float *>(static_cast<char *>(workspace) + ib);
    if (band) {
        int st = launch_integral_image_f32(grad_output, go_integ, (int64_t)N * C * F, h, w, false, stream, band_lpad(),
                                           band_rpad(w));
        if (st != BC_OK) return st;
        return launch_backward_band(input, go_integ, bp, reparametrization_h, reparametrization_w, N, C, F, h, w,
                                    normalize != 0, exact != 0, need_mask, grad_input, grad_params, partials, stream);
    }
    int st = launch_integral_image<float>(grad_output, go_integ, (int64_t)N * C * F, h, w, stream);
    if (st != BC_OK) return st;
    return launch_backward_global<float>(input, nullptr, go_integ, bp, reparametrization_h,
                                  reparametrization_w, N, C, F, h, w, normalize != 0, exact != 0,
                                  need_mask, grad_input, grad_params, partials, stream);
}

// ---- float16 / bfloat16 tensors on the shared-memory kernels
int bc_boxconv2d_narrow_supported(int F, int h, int w)
{
    return (F > 0 && h > 0 && w > 0 && plane_path_fits_forward(F, h, w) && plane_path_fits_backward(F, h, w)) ? 1 : 0;
}

int bc_boxconv2d_forward_narrow(const void *input, int io_kind, const float *x_min, const float *x_max,
                                const float *y_min, const float *y_max, float reparametrization_h,
                                float reparametrization_w, void *output, int N, int C, int F, int h,
                                int w, int normalize, int exact, bc_stream_t stream)
{
    if (!sizes_ok(N, C, F, h, w)) return BC_ERR_BAD_SHAPE;
    if (io_kind != BC_IO_F16 && io_kind != BC_IO_BF16) return BC_ERR_UNSUPPORTED;
    if (any_empty(N, C, F, h, w)) return BC_OK;
    if (!input || !x_min || !x_max || !y_min || !y_max || !output) return BC_ERR_NULL_POINTER;
    if (!plane_path_fits_forward(F, h, w)) return BC_ERR_UNSUPPORTED;
    const BoxParams bp{x_min, x_max, y_min, y_max, reparametrization_h, reparametrization_w};
    return launch_forward_plane_narrow(input, io_kind, bp, output, N, C, F, h, w, normalize != 0, exact != 0, stream);
}

int bc_boxconv2d_backward_narrow(const void *input, int io_kind, const float *x_min, const float *x_max,
                                 const float *y_min, const float *y_max, const void *grad_output,
                                 float reparametrization_h, float reparametrization_w, int N, int C,
                                 int F, int h, int w, int normalize, int exact, int need_mask,
                                 void *grad_input, float *grad_params, void *workspace,
                                 size_t workspace_bytes, bc_stream_t stream)
{
    if (!sizes_ok(N, C, F, h, w)) return BC_ERR_BAD_SHAPE;
    if (io_kind != BC_IO_F16 && io_kind != BC_IO_BF16) return BC_ERR_UNSUPPORTED;
    need_mask &= BC_NEED_ALL;
    if (!need_mask) return BC_OK;
    const bool need_params = (need_mask & ~BC_NEED_INPUT) != 0;
    if (any_empty(N, C, F, h, w)) {
        if (need_params && C > 0 && F > 0) {
            if (!grad_params) return BC_ERR_NULL_POINTER;
            for (int j = 0; j < 4; ++j)
                if (need_mask & (BC_NEED_X_MIN << j))
                    if (cudaError_t e = cudaMemsetAsync(grad_params + (size_t)j * C * F, 0, sizeof(float) * C * F, stream))
                        return cuda_failed(e, "memset");
        }
        return BC_OK;
    }
    if (!input || !x_min || !x_max || !y_min || !y_max || !grad_output) return BC_ERR_NULL_POINTER;
    if ((need_mask & BC_NEED_INPUT) && !grad_input) return BC_ERR_NULL_POINTER;
    if (need_params && !grad_params) return BC_ERR_NULL_POINTER;
    if (!plane_path_fits_backward(F, h, w)) return BC_ERR_UNSUPPORTED;
    if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255) ||
        workspace_bytes < bc_boxconv2d_backward_workspace(N, C, F, h, w, need_mask))
        return BC_ERR_WORKSPACE;
    const BoxParams bp{x_min, x_max, y_min, y_max, reparametrization_h, reparametrization_w};
    return launch_backward_plane_narrow(input, grad_output, io_kind, bp, reparametrization_h, reparametrization_w, N, C,
                                        F, h, w, normalize != 0, exact != 0, need_mask, grad_input, grad_params,
                                        static_cast<float *>(workspace), stream);
}

// ---- backward pass on the library's own scratch array (see the header for who needs this)
static __device__ __align__(256) unsigned char g_static_scratch[BC_STATIC_SCRATCH_BYTES];

// In host code `g_static_scratch` is only a handle for the runtime; the address kernels can use
// comes from cudaGetSymbolAddress, once per device, with that device current.
static void *static_scratch_address(int *status)
{
    static std::mutex mutex;
    static void *address[64] = {nullptr};
    int device = -1;
    if (cudaError_t e = cudaGetDevice(&device)) {
        *status = cuda_failed(e, "bc_boxconv2d_backward_static: cudaGetDevice");
        return nullptr;
    }
    if (device < 0 || device >= 64) {
        *status = BC_ERR_UNSUPPORTED;
        return nullptr;
    }
    std::lock_guard<std::mutex> lock(mutex);
    if (!address[device]) {
        void *p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess || !p) {
            *status = cuda_failed(e, "bc_boxconv2d_backward_static: cudaGetSymbolAddress");
            return nullptr;
        }
        address[device] = p;
    }
    *status = BC_OK;
    return address[device];
}

int bc_boxconv2d_backward_static(const float *input, const float *x_min, const float *x_max,
                                 const float *y_min, const float *y_max, const float *grad_output,
                                 float reparametrization_h, float reparametrization_w, int N, int C,
                                 int F, int h, int w, int normalize, int exact, int need_mask,
                                 float *grad_input, float *grad_params, bc_stream_t stream)
{
    if (!sizes_ok(N, C, F, h, w)) return BC_ERR_BAD_SHAPE;
    const size_t need = bc_boxconv2d_backward_workspace(N, C, F, h, w, need_mask);
    if (need > BC_STATIC_SCRATCH_BYTES) {
        snprintf(g_last_error, sizeof(g_last_error),
                 "bc_boxconv2d_backward_static: this problem needs %zu bytes of scratch, the built-in array has %u",
                 need, (unsigned)BC_STATIC_SCRATCH_BYTES);
        return BC_ERR_WORKSPACE;
    }
    int status = BC_OK;
    void *scratch = static_scratch_address(&status);
    if (!scratch) return status;
    return bc_boxconv2d_backward(input, x_min, x_max, y_min, y_max, grad_output, reparametrization_h,
                                 reparametrization_w, N, C, F, h, w, normalize, exact, need_mask,
                                 grad_input, grad_params, scratch, BC_STATIC_SCRATCH_BYTES, stream);
}

uint64_t bc_launch_count(void) { return g_launches.load(); }

int bc_wait_timeouts(int *count)
{
    if (!count) return BC_ERR_NULL_POINTER;
    return read_wait_timeouts(count);
}

int bc_profile_start(int capacity)
{
    if (capacity < 0) return BC_ERR_BAD_SHAPE;
    std::lock_guard<std::mutex> lock(g_prof_mutex);
    while ((int)g_prof.size() < capacity) {
        ProfRecord r{0, nullptr, nullptr};
        cudaError_t e = cudaEventCreate(&r.a);
        if (e == cudaSuccess) e = cudaEventCreate(&r.b);
        if (e != cudaSuccess) return cuda_failed(e, "bc_profile_start");
        g_prof.push_back(r);
    }
    g_prof_used = 0;
    g_prof_on.store(true, std::memory_order_release);
    return BC_OK;
}

int bc_profile_stop(void)
{
    std::lock_guard<std::mutex> lock(g_prof_mutex);
    g_prof_on.store(false, std::memory_order_release);
    return BC_OK;
}

int bc_profile_count(void)
{
    std::lock_guard<std::mutex> lock(g_prof_mutex);
    return g_prof_used;
}

int bc_profile_get(int index, int *kernel_id, float *milliseconds)
{
    std::lock_guard<std::mutex> lock(g_prof_mutex);
    if (index < 0 || index >= g_prof_used || !kernel_id || !milliseconds) return BC_ERR_BAD_SHAPE;
    *kernel_id = g_prof[index].kid;
    // (cudaErrorNotReady until the device has passed both events: synchronise first)
    if (cudaError_t e = cudaEventElapsedTime(milliseconds, g_prof[index].a, g_prof[index].b))
        return cuda_failed(e, "bc_profile_get");
    return BC_OK;
}

const char *bc_kernel_name(int kernel_id)
{
    switch (kernel_id) {
        case KID_INTEGRAL: return "integral_image_kernel";
        case KID_FORWARD_GLOBAL: return "forward_global_kernel";
        case KID_BACKWARD_GLOBAL: return "backward_global_kernel";
        case KID_FINISH_PARAM_GRADS: return "finish_param_grads_kernel";
        case KID_CLIP: return "clip_kernel";
        case KID_FORWARD_PLANE: return "forward_plane_kernel";
        case KID_BACKWARD_PLANE: return "backward_plane_kernel";
        case KID_SUM_CHUNKS: return "sum_chunk_grads_kernel";
        case KID_BACKWARD_BAND: return "backward_band_kernel";
        case KID_INTEGRAL_BANDS: return "integral_band_fixup_kernels";
        case KID_FORWARD_BAND: return "forward_band_kernel";
        default: return "unknown";
    }
}

}  // extern "C"
