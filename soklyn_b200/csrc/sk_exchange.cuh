// Pipelined gradient exchange of the data-parallel backward pass (one process per GPU, buffers of
// all ranks mapped into each other's address space). No counterpart in the reference, which is
// single-device; the order it must keep is the reference's: a hidden delta reads the next layer's
// weights AFTER their update (src/ffn.rs:141-163, src/io/device/ffn_device.rs:394-398).
//
// A weight matrix [K x N] is cut into `chunks` blocks of K/chunks rows; inside each block rank r owns
// K/(chunks*world) rows. Per block, on every rank:
//   1. the dW GEMM writes the block's rows of the local, averaged 16-bit gradient; flag A[block][r] is
//      raised on every other rank (signal_chunk_kernel);
//   2. reduce_rows_kernel (second stream, on the SMs the GEMMs leave free) waits for the other ranks'
//      A[block] flags, pulls the rows this rank owns out of every rank's gradient buffer (peer loads over
//      NVLink, many loads in flight per thread), adds them in rank order and writes the f32 sum locally
//      (the reduce-scatter);
//   3. the optimiser step of those rows runs on the main stream with every SM (it is bound by local HBM
//      traffic, 32 bytes per parameter, which a few SMs cannot move): f32 master weights, moments, and
//      the new 16-bit rows in the rank's own weight tensor;
//   4. spread_rows_kernel (second stream) stores the new 16-bit rows into every other rank's weight tensor
//      (peer stores) and raises flag B[block][r] there (the all-gather);
//   5. the dX GEMM of the layer below waits, in its TMA producer, for the other ranks' B flags of just the
//      blocks its tile needs.
// Steps of one GPU are ordered by stream order and events only; the only in-kernel waits are for flags
// that OTHER GPUs raise, every one bounded, ending in an error code instead of a hang, and a kernel whose
// wait gave up (or that finds the error word set) changes nothing and raises no flag. The last block's
// reduce kernel also adds the [3 x N] column sums of all ranks for the bias / normalisation-parameter step.
// Flags hold the step's epoch number and only grow.
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

// Raise flag word `word` to `value` in every OTHER rank's flag array, after everything this GPU wrote before.
__global__ void signal_chunk_kernel(PeerPtrs flags, uint32_t world, uint32_t self, uint32_t word, uint32_t value) {
    if (threadIdx.x < world && threadIdx.x != self) {
        __threadfence_system();
        store_flag_release(reinterpret_cast<uint32_t *>(flags.p[threadIdx.x]) + word, value);
    }
}

// Wait (bounded) until flags[chunk * stride + r] reached `value` for chunk < chunks and every rank r but `self`.
__global__ void wait_words_kernel(const uint32_t *flags, uint32_t chunks, uint32_t stride, uint32_t world, uint32_t self,
                                  uint32_t value, int *err) {
    for (uint32_t i = threadIdx.x; i < chunks * world; i += blockDim.x)
        if (i % world != self && !poll_flag_reached(flags + (i / world) * stride + i % world, value))
            atomicCAS(err, 0, kErrExchangeFlags);
    __threadfence_system();
}

struct ReduceArgs {
    PeerPtrs grad, flags, colsums;   // per rank: gradient buffer, flag words, column sums of the layer
    uint32_t world, rank, chunk, epoch;
    size_t off, len;                 // elements: this rank's rows of this block inside the [K x N] matrix
    float *sum;                      // local f32 [len]: the summed gradient of those rows
    int *err;
    uint32_t do_colsums, N;          // last block: also colsum_total[3 x N] = sum over ranks
    float *colsum_total;
};

// Reduce-scatter of one block: U 16-byte runs per thread and rank are in flight together (W * U = 16).
template <typename T, int W>
__global__ void __launch_bounds__(kExchangeThreads, 1) reduce_rows_kernel(ReduceArgs a) {
    extern __shared__ uint8_t sm_exclusive[];   // requested only to keep the SM to this block
    __shared__ int ok_s;
    constexpr int V = 8, U = 16 / W;
    const uint32_t *my_flags = reinterpret_cast<const uint32_t *>(a.flags.p[a.rank]);
    if (threadIdx.x == 0) ok_s = *reinterpret_cast<volatile int *>(a.err) == 0;
    __syncthreads();
    if (threadIdx.x < W && threadIdx.x != a.rank) {   // this rank's own gradient is ordered by an event
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
#pragma unroll
    for (int s = 0; s < W; ++s) src[s] = reinterpret_cast<const T *>(a.grad.p[s]) + a.off;
    for (size_t base = (size_t)blockIdx.x * blockDim.x + threadIdx.x; base < nvec; base += stride * U) {
        uint4 part[U][W];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const size_t i = base + (size_t)u * stride;
            if (i < nvec) {
#pragma unroll
                for (int s = 0; s < W; ++s) part[u][s] = __ldcg(reinterpret_cast<const uint4 *>(src[s] + i * V));
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const size_t i = base + (size_t)u * stride;
            if (i < nvec) {
                float g[V];
#pragma unroll
                for (int j = 0; j < V; ++j) g[j] = 0.0f;
#pragma unroll
                for (int s = 0; s < W; ++s) {
                    const Pack<T, V> &pk = *reinterpret_cast<const Pack<T, V> *>(&part[u][s]);
#pragma unroll
                    for (int j = 0; j < V; ++j) g[j] += to_f32(pk.v[j]);
                }
                store_run<float, V>(a.sum + i * V, true, g);
            }
        }
    }
    if (a.do_colsums) {
        for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < 3 * a.N; i += gridDim.x * blockDim.x) {
            float t = 0.0f;
#pragma unroll
            for (int s = 0; s < W; ++s) t += __ldcg(reinterpret_cast<const float *>(a.colsums.p[s]) + i);
            a.colsum_total[i] = t;
        }
    }
}

struct SpreadArgs {
    PeerPtrs w, flags;               // per rank: weight tensor, flag words of the layer
    uint32_t world, rank, chunk, epoch;
    size_t off, len;                 // elements: this rank's rows of this block
    uint32_t *done;                  // local counter, zero between launches
    const int *err;
};

// All-gather of one block: this rank's new 16-bit rows into every other rank's weight tensor, then B[block][rank].
template <typename T, int W>
__global__ void __launch_bounds__(kExchangeThreads, 1) spread_rows_kernel(SpreadArgs a) {
    extern __shared__ uint8_t sm_exclusive[];
    constexpr int V = 8, U = 8;
    if (*reinterpret_cast<const volatile int *>(a.err) != 0) return;   // an earlier wait gave up: publish nothing
    const size_t nvec = a.len / V, stride = (size_t)gridDim.x * blockDim.x;
    const T *mine = reinterpret_cast<const T *>(a.w.p[a.rank]) + a.off;
    for (size_t base = (size_t)blockIdx.x * blockDim.x + threadIdx.x; base < nvec; base += stride * U) {
        uint4 v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const size_t i = base + (size_t)u * stride;
            if (i < nvec) v[u] = __ldcg(reinterpret_cast<const uint4 *>(mine + i * V));
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const size_t i = base + (size_t)u * stride;
            if (i < nvec) {
#pragma unroll
                for (int s = 0; s < W; ++s)
                    if ((uint32_t)s != a.rank) *reinterpret_cast<uint4 *>(reinterpret_cast<T *>(a.w.p[s]) + a.off + i * V) = v[u];
            }
        }
    }
    // all stores of this block are out -> the last block to finish raises B[chunk][rank] on the other ranks
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        const uint32_t old = atomicAdd(a.done, 1u);
        if (old == gridDim.x - 1) {
            *a.done = 0;
            __threadfence_system();
            for (int s = 0; s < W; ++s)
                if ((uint32_t)s != a.rank)
                    store_flag_release(reinterpret_cast<uint32_t *>(a.flags.p[s]) + (1 * kMaxChunks + a.chunk) * kMaxRanks + a.rank, a.epoch);
        }
    }
}

} // namespace sk
