// Pipelined gradient exchange of the data-parallel backward pass (one process per GPU, buffers of
// all ranks mapped into each other's address space). No counterpart in the reference, which is
// single-device; the order it must keep is the reference's: a hidden delta reads the next layer's
// weights AFTER their update (src/ffn.rs:141-163, src/io/device/ffn_device.rs:394-398).
//
// A weight matrix [K x N] is cut into `chunks` blocks of K/chunks rows; inside each block rank r owns
// K/(chunks*world) rows. Per block, in this order on every rank:
//   1. the dW GEMM writes the block's rows of the local, averaged 16-bit gradient and flag A[block][r]
//      is raised on every rank (signal_chunk_kernel);
//   2. exchange_chunk_kernel, on its own stream and on SMs the GEMMs leave free, waits for A[block][*],
//      pulls the rows this rank owns out of every rank's gradient buffer (peer loads over NVLink), adds
//      them in rank order, runs the optimiser step on the f32 master weights and moments, stores the new
//      16-bit rows into every rank's weight tensor (peer stores), and raises flag B[block][r] on every
//      rank once all its stores are out;
//   3. the dX GEMM of the layer below waits for B[block][*] before its TMA producer loads the block's rows.
// So reduce-scatter, optimiser and all-gather are one kernel, and they overlap the dW GEMM of the
// following blocks and the dX GEMM of the preceding ones. The kernel of the last block also sums the
// [3 x N] column sums of all ranks and steps bias and normalisation parameters (identically on every
// rank). Flags hold the step's epoch number and only grow; every wait is bounded and ends in an error
// code instead of a hang, and a kernel whose wait gave up leaves weights and moments untouched.
#pragma once

#include "sk_rowwise.cuh"

namespace sk {

constexpr int kMaxChunks = 8;
constexpr int kExchangeThreads = 512;
// Flag words of one layer in a rank's arena: [2][kMaxChunks][kMaxRanks] (A = gradients ready, B = rows landed).
constexpr int kFlagWordsPerLayer = 2 * kMaxChunks * kMaxRanks;
enum : int { kErrExchangeFlags = 6 };

__device__ __forceinline__ bool poll_flag_reached(const uint32_t *flag, uint32_t value) {
    const long long t0 = clock64();
    for (;;) {
        uint32_t v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
        if ((int32_t)(v - value) >= 0) return true;
        if (clock64() - t0 > 4000000000LL) return false;
        __nanosleep(100);
    }
}

__device__ __forceinline__ void store_flag_release(uint32_t *flag, uint32_t value) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(value) : "memory");
}

// Raise flag word `word` to `value` in every rank's flag array, after everything this GPU wrote before.
__global__ void signal_chunk_kernel(PeerPtrs flags, uint32_t world, uint32_t word, uint32_t value) {
    if (threadIdx.x < world) {
        __threadfence_system();
        store_flag_release(reinterpret_cast<uint32_t *>(flags.p[threadIdx.x]) + word, value);
    }
}

// Wait (bounded) until flags[chunk * stride + r] reached `value` for chunk < chunks, r < world.
__global__ void wait_words_kernel(const uint32_t *flags, uint32_t chunks, uint32_t stride, uint32_t world, uint32_t value,
                                  int *err) {
    for (uint32_t i = threadIdx.x; i < chunks * world; i += blockDim.x)
        if (!poll_flag_reached(flags + (i / world) * stride + i % world, value)) atomicCAS(err, 0, kErrExchangeFlags);
    __threadfence_system();
}

template <typename T> struct ExchangeArgs {
    PeerPtrs grad, w, flags, colsums;   // per rank: gradient buffer, weight tensor, flag words, column sums of the layer
    uint32_t world, rank, chunk, epoch;
    size_t off, len;                    // elements: this rank's rows of this block
    float *master, *dv, *dm;            // local f32 state, whole matrix
    Optim opt;
    Hyper hyp;                          // inv_m = 1: the staged gradients are already averaged
    uint32_t *done;                     // local counter, zero between launches
    int *err;
    uint32_t do_vector, N;              // last block: also the bias / normalisation-parameter step
    VectorParams<T> vp;
};

template <typename T, int W>
__global__ void __launch_bounds__(kExchangeThreads, 1) exchange_chunk_kernel(ExchangeArgs<T> a) {
    extern __shared__ uint8_t sm_exclusive[];   // requested only to keep the SM to this block
    __shared__ int ok_s;
    constexpr int V = 8;
    const uint32_t *my_flags = reinterpret_cast<const uint32_t *>(a.flags.p[a.rank]);
    if (threadIdx.x == 0) ok_s = 1;
    __syncthreads();
    if (threadIdx.x < W) {
        if (!poll_flag_reached(my_flags + (0 * kMaxChunks + a.chunk) * kMaxRanks + threadIdx.x, a.epoch)) {
            ok_s = 0;
            atomicCAS(a.err, 0, kErrExchangeFlags);
        }
        __threadfence_system();
    }
    __syncthreads();
    if (!ok_s) return;

    const size_t nvec = a.len / V, stride = (size_t)gridDim.x * blockDim.x;
    const T *src[W];
    T *dst[W];
#pragma unroll
    for (int s = 0; s < W; ++s) {
        src[s] = reinterpret_cast<const T *>(a.grad.p[s]) + a.off;
        dst[s] = reinterpret_cast<T *>(a.w.p[s]) + a.off;
    }
    float *master = a.master + a.off, *dv = a.dv + a.off, *dm = a.dm + a.off;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
        uint4 part[W];
#pragma unroll
        for (int s = 0; s < W; ++s) part[s] = __ldcg(reinterpret_cast<const uint4 *>(src[s] + i * V));
        const Pack<float, V> pp = load_pack<float, V>(master + i * V);
        const Pack<float, V> pv = load_pack<float, V>(dv + i * V);
        const Pack<float, V> pm = load_pack<float, V>(dm + i * V);
        float g[V], p[V], v[V], m[V];
#pragma unroll
        for (int j = 0; j < V; ++j) g[j] = 0.0f;
#pragma unroll
        for (int s = 0; s < W; ++s) {
            const Pack<T, V> &pk = *reinterpret_cast<const Pack<T, V> *>(&part[s]);
#pragma unroll
            for (int j = 0; j < V; ++j) g[j] += to_f32(pk.v[j]);
        }
        unpack<float, V>(pp, p);
        unpack<float, V>(pv, v);
        unpack<float, V>(pm, m);
#pragma unroll
        for (int j = 0; j < V; ++j) p[j] = optimiser_step_fast(p[j], v[j], m[j], g[j] * kLossScaleInv, a.opt, a.hyp, true);
        store_run<float, V>(dv + i * V, true, v);
        store_run<float, V>(dm + i * V, true, m);
        store_run<float, V>(master + i * V, true, p);
        Pack<T, V> out;
#pragma unroll
        for (int j = 0; j < V; ++j) out.v[j] = from_f32<T>(p[j]);
#pragma unroll
        for (int s = 0; s < W; ++s) *reinterpret_cast<uint4 *>(dst[s] + i * V) = *reinterpret_cast<const uint4 *>(&out);
    }

    if (a.do_vector) {   // column sums of all ranks, added in rank order, then the same step on every rank
        for (uint32_t col = blockIdx.x * blockDim.x + threadIdx.x; col < a.N; col += gridDim.x * blockDim.x) {
            float s3[3] = {0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int s = 0; s < W; ++s) {
                const float *cs = reinterpret_cast<const float *>(a.colsums.p[s]);
#pragma unroll
                for (int w = 0; w < 3; ++w) s3[w] += __ldcg(cs + (size_t)w * a.N + col);
            }
            vector_step<T>(a.vp, col, s3);
        }
    }

    // all stores of this block are out -> the last block to finish raises B[chunk][rank] everywhere
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        const uint32_t old = atomicAdd(a.done, 1u);
        if (old == gridDim.x - 1) {
            *a.done = 0;
            __threadfence_system();
            for (int s = 0; s < W; ++s)
                store_flag_release(reinterpret_cast<uint32_t *>(a.flags.p[s]) + (1 * kMaxChunks + a.chunk) * kMaxRanks + a.rank, a.epoch);
        }
    }
}

} // namespace sk
