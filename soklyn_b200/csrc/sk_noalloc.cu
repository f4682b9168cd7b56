// sk_column_sums_static: the batch column sums of a block's gradients (bias gradient and the
// two normalisation-parameter gradients) for callers that may not allocate device memory.
//
// Who that is: a host program whose device heap belongs to someone else. Examples are a
// serving process whose framework reserved all of HBM up front and treats any further
// cudaMalloc as an error, or a binding that is only handed raw device pointers and a stream
// and therefore cannot build an sk_ctx (creating a context allocates its workspace). For
// them the two-stage reduction keeps its partial sums in a fixed array that is part of this
// library's image instead of in a context workspace.
//
// Cost and limits: the array below occupies kStaticFloats * 4 bytes (3 MiB) on every GPU that
// loads the library, until the process exits. A call needs 3 * N floats per slab of rows and
// at least one slab, so N may not exceed kStaticFloats / 3 = 262144 columns; larger N is
// refused with SK_ERR_STATIC_LIMIT. All calls share the array: two calls that overlap on
// the GPU (different streams, or different host threads) race on it and must be serialised
// by the caller. Nothing in the array has to start at zero; every slab entry a call reads
// was written by the same call.
//
// The first call on each device looks the array's device address up (cudaGetSymbolAddress
// with that device current) and caches it; make that first call outside any stream capture.
// The cache is a plain per-device pointer: host threads that race on a device's first call all
// store the same value, which is harmless, but callers who want no data race at all should
// make the first call per device from one thread. No call here allocates or frees memory.
#include <cstdint>
#include <cuda_runtime.h>

#include "../../include/soklyn_b200.h"

namespace {

constexpr size_t kStaticFloats = 786432;   // 3 MiB
constexpr int kMaxDevices = 64;
constexpr int kThreads = 256;

static __device__ __align__(256) float g_static_scratch[kStaticFloats];

float *g_scratch_addr[kMaxDevices] = {nullptr};   // device address of g_static_scratch, per device

// Stage 1: block (bx, by) sums rows [by*rows_per_block, ...) of 32 adjacent columns of the
// three tensors into partial[by][which][col]. Same arithmetic as the context path.
__global__ void __launch_bounds__(kThreads)
static_colsum_partial(const float *__restrict__ d_prenorm, const float *__restrict__ d_norm_w,
                      const float *__restrict__ d_norm_b, float *__restrict__ partial, uint32_t M, uint32_t N,
                      uint32_t rows_per_block, uint32_t norm) {
    __shared__ float red[3][8][33];
    const uint32_t cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
    const uint32_t col = blockIdx.x * 32 + cx;
    const uint32_t r0 = blockIdx.y * rows_per_block;
    const uint32_t r1 = min(M, r0 + rows_per_block);
    float sb = 0.0f, sw = 0.0f, sn = 0.0f;
    if (col < N)
        for (uint32_t r = r0 + ry; r < r1; r += 8) {
            const size_t idx = (size_t)r * N + col;
            sb += d_prenorm[idx];
            if (norm > 0) sw += d_norm_w[idx];
            if (norm > 1) sn += d_norm_b[idx];
        }
    red[0][ry][cx] = sb;
    red[1][ry][cx] = sw;
    red[2][ry][cx] = sn;
    __syncthreads();
    if (ry < 3 && col < N) {
        float t = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) t += red[ry][i][cx];
        partial[((size_t)blockIdx.y * 3 + ry) * N + col] = t;
    }
}

// Stage 2: add the slabs in a fixed order.
__global__ void static_colsum_final(const float *__restrict__ partial, float *__restrict__ colsums, uint32_t N,
                                    uint32_t slabs) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= 3 * N) return;
    const uint32_t which = i / N, col = i % N;
    float t = 0.0f;
    for (uint32_t b = 0; b < slabs; ++b) t += partial[((size_t)b * 3 + which) * N + col];
    colsums[i] = t;
}

} // namespace

extern "C" int sk_column_sums_static(void *stream, const float *d_prenorm, const float *d_norm_w,
                                     const float *d_norm_b, float *colsums, uint32_t batch, uint32_t N,
                                     uint32_t norm) {
    if (!d_prenorm || !colsums) return SK_ERR_NULL_POINTER;
    if (norm > 3) return SK_ERR_INVALID_CONFIGURATION;
    if ((norm > 0 && !d_norm_w) || (norm > 1 && !d_norm_b)) return SK_ERR_NULL_POINTER;
    if (batch == 0) return SK_ERR_INVALID_BATCH_SIZE;
    if (N == 0) return SK_ERR_INVALID_CONFIGURATION;
    if ((size_t)3 * N > kStaticFloats) return SK_ERR_STATIC_LIMIT;   // not even one slab fits

    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return SK_ERR_DRIVER;
    if (!g_scratch_addr[dev]) {
        // once per device, with that device current: the symbol's name is only a host-side
        // handle, the kernels need its device address
        float *p = nullptr;
        if (cudaGetSymbolAddress((void **)&p, g_static_scratch) != cudaSuccess || !p) return SK_ERR_DRIVER;
        g_scratch_addr[dev] = p;
    }
    float *scratch = g_scratch_addr[dev];

    const uint32_t gx = (N + 31) / 32;
    uint32_t slabs = (4u * 148u + gx - 1) / gx;                         // enough blocks to cover the SMs
    const uint32_t fit = (uint32_t)(kStaticFloats / ((size_t)3 * N));   // slabs the array can hold (>= 1, checked above)
    if (slabs > fit) slabs = fit;                                       // wide N: fewer, taller slabs
    const uint32_t most = (batch + 7) / 8;
    if (slabs > most) slabs = most;
    if (slabs < 1) slabs = 1;
    const uint32_t rows_per_block = (batch + slabs - 1) / slabs;
    slabs = (batch + rows_per_block - 1) / rows_per_block;

    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    static_colsum_partial<<<dim3(gx, slabs), kThreads, 0, s>>>(d_prenorm, d_norm_w, d_norm_b, scratch, batch, N,
                                                                rows_per_block, norm);
    static_colsum_final<<<(3 * N + 255) / 256, 256, 0, s>>>(scratch, colsums, N, slabs);
    return cudaGetLastError() == cudaSuccess ? SK_OK : SK_ERR_DRIVER;
}
