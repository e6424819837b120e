// One training step of the box block on a batch that lives in (pinned) host memory.
//
// The batch is cut into chunks; three streams carry, for neighbouring chunks at the same time,
// the host-to-device copies of the inputs, the kernels (clip once, then forward and backward per
// chunk) and the device-to-host copies of the results, so that the PCIe link is busy in both
// directions while the GPU computes.  Parameter gradients are linear in the batch: each chunk
// leaves its own (4, C, F) gradient and a last small kernel adds them in a fixed order.
#include <mutex>
#include <vector>

#include "bc_common.cuh"

namespace bc {

namespace {

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct Layout {
    size_t x, go, out, gin, gp_chunks, gp_sum, scratch, total;
    size_t scratch_bytes;
};

Layout make_layout(int N, int C, int F, int h, int w, int chunks)
{
    Layout L{};
    const size_t E = (size_t)N * C * h * w * sizeof(float);
    const int nmax = (N + chunks - 1) / chunks;
    size_t off = 0;
    L.x = off;         off += align_up(E, 256);
    L.go = off;        off += align_up(E * F, 256);
    L.out = off;       off += align_up(E * F, 256);
    L.gin = off;       off += align_up(E, 256);
    L.gp_chunks = off; off += align_up((size_t)chunks * 4 * C * F * sizeof(float), 256);
    L.gp_sum = off;    off += align_up((size_t)4 * C * F * sizeof(float), 256);
    const size_t f = bc_boxconv2d_forward_workspace(nmax, C, F, h, w);
    const size_t b = bc_boxconv2d_backward_workspace(nmax, C, F, h, w, BC_NEED_ALL);
    L.scratch_bytes = align_up(f > b ? f : b, 256);
    L.scratch = off;   off += L.scratch_bytes;
    L.total = off;
    return L;
}

__global__ void sum_chunk_grads_kernel(const float *__restrict__ chunks, int n_chunks, int count, float *__restrict__ out)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    float s = 0.0f;
    for (int k = 0; k < n_chunks; ++k) s += chunks[(size_t)k * count + i];
    out[i] = s;
}

// Events used to order the three streams; host-side objects, created on first use per thread and
// per device (an event belongs to the device that was current when it was created, and the three
// streams of a call are streams of the current device).
constexpr int kMaxDevices = 64;
cudaEvent_t *events(int n, cudaError_t *err)
{
    static thread_local std::vector<cudaEvent_t> pools[kMaxDevices];
    int device = -1;
    *err = cudaGetDevice(&device);
    if (*err != cudaSuccess) return nullptr;
    if (device < 0 || device >= kMaxDevices) { *err = cudaErrorInvalidDevice; return nullptr; }
    std::vector<cudaEvent_t> &pool = pools[device];
    while ((int)pool.size() < n) {
        cudaEvent_t e;
        *err = cudaEventCreateWithFlags(&e, cudaEventDisableTiming);
        if (*err != cudaSuccess) return nullptr;
        pool.push_back(e);
    }
    return pool.data();
}

// First error of a chain of runtime calls, so that a failure is reported with its own code.
struct Chain {
    cudaError_t e = cudaSuccess;
    Chain &operator()(cudaError_t r) { if (e == cudaSuccess) e = r; return *this; }
    bool failed() const { return e != cudaSuccess; }
};

}  // namespace

}  // namespace bc

using namespace bc;

extern "C" {

size_t bc_boxconv2d_host_step_workspace(int N, int C, int F, int h, int w, int chunks)
{
    if (N <= 0 || C <= 0 || F <= 0 || h <= 0 || w <= 0 || chunks <= 0) return 0;
    if (chunks > N) chunks = N;
    return make_layout(N, C, F, h, w, chunks).total;
}

int bc_boxconv2d_host_step(const float *x_host, const float *grad_output_host, float *out_host,
                           float *grad_input_host, float *grad_params_host, float *x_min, float *x_max,
                           float *y_min, float *y_max, float reparametrization_h,
                           float reparametrization_w, double max_input_h, double max_input_w, int N,
                           int C, int F, int h, int w, int normalize, int exact, int clip, int chunks,
                           void *workspace, size_t workspace_bytes, bc_stream_t copy_in,
                           bc_stream_t compute, bc_stream_t copy_out)
{
    if (N <= 0 || C <= 0 || F <= 0 || h <= 0 || w <= 0 || chunks <= 0) return BC_ERR_BAD_SHAPE;
    if (!x_host || !grad_output_host || !out_host || !grad_input_host || !grad_params_host || !x_min ||
        !x_max || !y_min || !y_max)
        return BC_ERR_NULL_POINTER;
    if (chunks > N) chunks = N;
    const Layout L = make_layout(N, C, F, h, w, chunks);
    if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255) || workspace_bytes < L.total)
        return BC_ERR_WORKSPACE;
    char *ws = static_cast<char *>(workspace);
    float *x_dev = reinterpret_cast<float *>(ws + L.x), *go_dev = reinterpret_cast<float *>(ws + L.go);
    float *out_dev = reinterpret_cast<float *>(ws + L.out), *gin_dev = reinterpret_cast<float *>(ws + L.gin);
    float *gp_chunks = reinterpret_cast<float *>(ws + L.gp_chunks), *gp_sum = reinterpret_cast<float *>(ws + L.gp_sum);
    void *scratch = ws + L.scratch;

    cudaError_t ev_err = cudaSuccess;
    cudaEvent_t *ev = events(2 * chunks + 1, &ev_err);
    if (!ev) return cuda_failed(ev_err, "bc_boxconv2d_host_step: event pool");

    int st = BC_OK;
    if (clip) {
        st = bc_clip_parameters(x_min, x_max, y_min, y_max, C * F, reparametrization_h, reparametrization_w,
                                max_input_h, max_input_w, exact, compute);
        if (st != BC_OK) return st;
    }
    const size_t plane = (size_t)h * w;
    for (int k = 0; k < chunks; ++k) {
        const int n0 = (int)((int64_t)N * k / chunks), n1 = (int)((int64_t)N * (k + 1) / chunks);
        const int nk = n1 - n0;
        if (nk <= 0) continue;
        const size_t xo = (size_t)n0 * C * plane, oo = xo * F;
        const size_t xb = (size_t)nk * C * plane * sizeof(float), ob = xb * F;
        // inputs of chunk k
        Chain in;
        in(cudaMemcpyAsync(x_dev + xo, x_host + xo, xb, cudaMemcpyHostToDevice, copy_in));
        if (!in.failed()) in(cudaMemcpyAsync(go_dev + oo, grad_output_host + oo, ob, cudaMemcpyHostToDevice, copy_in));
        if (!in.failed()) in(cudaEventRecord(ev[2 * k], copy_in));
        if (!in.failed()) in(cudaStreamWaitEvent(compute, ev[2 * k], 0));
        if (in.failed()) return cuda_failed(in.e, "bc_boxconv2d_host_step: input copies");
        // kernels of chunk k (they share the scratch area: same stream, so in order)
        st = bc_boxconv2d_forward(x_dev + xo, x_min, x_max, y_min, y_max, reparametrization_h, reparametrization_w,
                                  out_dev + oo, nk, C, F, h, w, normalize, exact, scratch, L.scratch_bytes, compute);
        if (st != BC_OK) return st;
        st = bc_boxconv2d_backward(x_dev + xo, x_min, x_max, y_min, y_max, go_dev + oo, reparametrization_h,
                                   reparametrization_w, nk, C, F, h, w, normalize, exact, BC_NEED_ALL,
                                   gin_dev + xo, gp_chunks + (size_t)k * 4 * C * F, scratch, L.scratch_bytes, compute);
        if (st != BC_OK) return st;
        // results of chunk k
        Chain res;
        res(cudaEventRecord(ev[2 * k + 1], compute));
        if (!res.failed()) res(cudaStreamWaitEvent(copy_out, ev[2 * k + 1], 0));
        if (!res.failed()) res(cudaMemcpyAsync(out_host + oo, out_dev + oo, ob, cudaMemcpyDeviceToHost, copy_out));
        if (!res.failed()) res(cudaMemcpyAsync(grad_input_host + xo, gin_dev + xo, xb, cudaMemcpyDeviceToHost, copy_out));
        if (res.failed()) return cuda_failed(res.e, "bc_boxconv2d_host_step: result copies");
    }
    {
        const int count = 4 * C * F;
        LaunchScope scope(KID_SUM_CHUNKS, compute);
        sum_chunk_grads_kernel<<<(count + 127) / 128, 128, 0, compute>>>(gp_chunks, chunks, count, gp_sum);
    }
    st = check_launch("sum_chunk_grads");
    if (st != BC_OK) return st;
    Chain fin;
    fin(cudaEventRecord(ev[2 * chunks], compute));
    if (!fin.failed()) fin(cudaStreamWaitEvent(copy_out, ev[2 * chunks], 0));
    if (!fin.failed())
        fin(cudaMemcpyAsync(grad_params_host, gp_sum, (size_t)4 * C * F * sizeof(float), cudaMemcpyDeviceToHost, copy_out));
    if (fin.failed()) return cuda_failed(fin.e, "bc_boxconv2d_host_step: gradient copy");
    return BC_OK;
}

}  // extern "C"
