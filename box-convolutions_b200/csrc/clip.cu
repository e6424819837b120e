// In-place projection of the stored box parameters (src/box_convolution.cpp:729-763,
// src/box_convolution_cuda_misc.cu:190-236): clamp both ends of every (min, max) pair to
// [-(max_size+1), max_size-1] pixels and widen pairs that have become narrower than the minimum
// size around their mean.  Arithmetic in double on the stored (reparametrized) values, like the
// reference.  One launch handles the x pair and the y pair.
#include "bc_common.cuh"

namespace bc {

namespace {

template <typename T>
__device__ __forceinline__ void clip_pair(T *pmin, T *pmax, double inv_rep, double min_size, double max_size)
{
    const double lo = -(max_size + 1) * inv_rep, hi = (max_size - 1) * inv_rep;
    double a = fmax(lo, fmin(hi, (double)*pmin));
    double b = fmax(lo, fmin(hi, (double)*pmax));
    if (a + (min_size - 0.9999) * inv_rep > b) {
        const T mean = (T)(0.5 * (a + b));   // rounded to the stored type, as the reference does
        a = mean - 0.5 * (min_size - 0.9999) * inv_rep;
        b = mean + 0.5 * (min_size - 0.9999) * inv_rep;
    }
    *pmin = (T)a;
    *pmax = (T)b;
}

// `packed` (may be null): a (4, count) copy of the clipped values in the order x_min, x_max, y_min,
// y_max, written by the same threads: the snapshot of the parameters that a forward pass keeps for
// its backward pass, without a launch of its own.
template <typename T>
__global__ void clip_kernel(T *x_min, T *x_max, T *y_min, T *y_max, int count,
                            double inv_rep_h, double inv_rep_w, double min_size, double max_h, double max_w,
                            T *packed)
{
    grid_dependency_release();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count) {
        clip_pair(x_min + i, x_max + i, inv_rep_h, min_size, max_h);
        if (packed) { packed[i] = x_min[i]; packed[count + i] = x_max[i]; }
    } else if (i < 2 * count) {
        const int j = i - count;
        clip_pair(y_min + j, y_max + j, inv_rep_w, min_size, max_w);
        if (packed) { packed[2 * count + j] = y_min[j]; packed[3 * count + j] = y_max[j]; }
    }
}

}  // namespace

template <typename T>
int launch_clip(T *x_min, T *x_max, T *y_min, T *y_max, int count, double rep_h,
                double rep_w, double max_h, double max_w, bool exact, cudaStream_t s, T *packed)
{
    if (count == 0) return BC_OK;
    // minimum sizes are single-precision constants in the reference (interface.cpp:405-406)
    const double min_size = (double)(exact ? 1.001f : 2.001f);
    const int threads = 128;
    const int blocks = (2 * count + threads - 1) / threads;
    LaunchScope scope(KID_CLIP, s);
    clip_kernel<T><<<blocks, threads, 0, s>>>(x_min, x_max, y_min, y_max, count, 1.0 / rep_h, 1.0 / rep_w,
                                           min_size, max_h, max_w, packed);
    return check_launch("clip_parameters");
}

template int launch_clip<float>(float *, float *, float *, float *, int, double, double, double, double, bool, cudaStream_t, float *);
template int launch_clip<double>(double *, double *, double *, double *, int, double, double, double, double, bool, cudaStream_t,
                                 double *);

}  // namespace bc
