// gptb200_bias_grad_noalloc: the bias-gradient column sums (grad_b[n] += sum over rows of grad_y[m x n]) for
// callers that must not allocate device memory.
//
// Who that is: a host program that has handed the whole GPU to its own memory pool (a raw cudaMalloc from a
// plug-in would fail or fragment the pool), code that runs where the CUDA runtime forbids allocation (while a
// stream is being captured), and services with a fixed memory budget that is audited at start-up.
// The regular entry point (gptb200_linear_backward) keeps the partial row sums of this reduction in the
// context's scratch buffer, which it grows with cudaMalloc on demand; this one keeps them in a fixed array that
// is part of the library image, so a call never allocates, frees or touches a context.
//
// Cost and limits: the array below (1 MiB) is reserved on every GPU that loads the library, until the process
// exits.  n may be at most kMaxCols; larger requests are refused with GPTB200_ERR_TOO_LARGE.  All calls share the
// one array and it keeps the previous call's contents.  Nothing in it has to start at zero: stage 1 overwrites
// every partial sum that stage 2 reads.  Two calls that overlap on the GPU (different streams, or different host
// threads without ordering) race on the array -- order them on one stream or with events.
//
// The first call on each device looks up the array's device address (cudaGetSymbolAddress) and caches it.  That
// first call should be made before any stream capture begins.  The array used is the current device's copy:
// `cuda_stream` must be a stream of the device that is current when the call is made.
#include <mutex>

#include <cuda_runtime.h>

#include "../../include/gptb200.h"

namespace {

constexpr int kMaxCols = 8192;     // largest n accepted
constexpr int kMaxChunks = 32;     // row chunks reduced independently in stage 1
constexpr int kMaxDevices = 64;

// Partial column sums [chunk][n].  In host code this name is only a handle for the runtime, not an address a
// kernel can use: the device address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) float g_bias_partials[kMaxChunks * kMaxCols];

float *g_partials_addr[kMaxDevices] = {nullptr};
std::mutex g_setup_mutex;

// Stage 1: block (32, 8) sums 32 columns over one chunk of rows into partials[chunk][col].
__global__ void bias_grad_partial_static_kernel(float *__restrict__ partials, const float *__restrict__ gy, int m, int n, int rows_per_chunk)
{
    __shared__ float red[8][33];
    const int col = blockIdx.x * 32 + threadIdx.x;
    const int chunk = blockIdx.y;
    const long long r0 = 1LL * chunk * rows_per_chunk;
    const long long r1 = min(r0 + rows_per_chunk, static_cast<long long>(m));
    float s = 0.0f;
    if (col < n)
        for (long long r = r0 + threadIdx.y; r < r1; r += 8) s += gy[r * n + col];
    red[threadIdx.y][threadIdx.x] = s;
    __syncthreads();
    if (threadIdx.y == 0 && col < n) {
        float t = red[0][threadIdx.x];
#pragma unroll
        for (int i = 1; i < 8; ++i) t += red[i][threadIdx.x];
        partials[1LL * chunk * n + col] = t;
    }
}

// Stage 2: grad_b[col] += partials[0][col] + partials[1][col] + ... in that order.
__global__ void bias_grad_final_static_kernel(float *__restrict__ gb, const float *__restrict__ partials, int n, int chunks)
{
    const int col = blockIdx.x * blockDim.x + threadIdx.x;
    if (col >= n) return;
    float s = 0.0f;
    for (int c = 0; c < chunks; ++c) s += partials[1LL * c * n + col];
    gb[col] += s;
}

// Device address of the static array on the current device; looked up once per device.
int partials_for_current_device(float **out)
{
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return GPTB200_ERR_CUDA;
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (!g_partials_addr[dev]) {
        float *p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void **>(&p), g_bias_partials);
        if (e != cudaSuccess || !p) return GPTB200_ERR_CUDA;
        g_partials_addr[dev] = p;
    }
    *out = g_partials_addr[dev];
    return GPTB200_OK;
}

}  // namespace

extern "C" int gptb200_bias_grad_noalloc(float *grad_b, const float *grad_y, int m, int n, void *cuda_stream)
{
    if (m < 0 || n < 0) return GPTB200_ERR_INVALID_ARG;
    if (m == 0 || n == 0) return GPTB200_OK;
    if (!grad_b || !grad_y || 1LL * m * n > 0x7fffffffLL) return GPTB200_ERR_INVALID_ARG;
    if (n > kMaxCols) return GPTB200_ERR_TOO_LARGE;
    float *partials = nullptr;
    const int rc = partials_for_current_device(&partials);
    if (rc != GPTB200_OK) return rc;
    int chunks = (m + 255) / 256;
    if (chunks > kMaxChunks) chunks = kMaxChunks;
    const int rows_per_chunk = (m + chunks - 1) / chunks;
    chunks = (m + rows_per_chunk - 1) / rows_per_chunk;
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
    bias_grad_partial_static_kernel<<<dim3((n + 31) / 32, chunks), dim3(32, 8), 0, stream>>>(partials, grad_y, m, n, rows_per_chunk);
    if (cudaGetLastError() != cudaSuccess) return GPTB200_ERR_CUDA;
    bias_grad_final_static_kernel<<<(n + 127) / 128, 128, 0, stream>>>(grad_b, partials, n, chunks);
    return cudaGetLastError() == cudaSuccess ? GPTB200_OK : GPTB200_ERR_CUDA;
}
