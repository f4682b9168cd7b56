// Gradient exchange of the data-parallel backward pass (one process per GPU, buffers of all ranks
// mapped into each other's address space). No counterpart in the reference, which is single-device;
// the order it must keep is the reference's: a hidden delta reads the next layer's weights AFTER their
// update (src/ffn.rs:141-163, src/io/device/ffn_device.rs:394-398).
//
// A weight matrix [K x N] is cut into `chunks` blocks of K/chunks rows; inside each block rank r owns
// K/(chunks*world) rows. Per block, on every rank and all on the context's stream:
//   1. the dW GEMM writes the block's rows of the local, averaged 16-bit gradient; flag A[block][r] is
//      raised on every other rank (signal_chunk_kernel);
//   2. exchange_update_kernel waits for the other ranks' A[block] flags and is then reduce-scatter +
//      optimiser + all-gather in one kernel over every SM: it obtains the sum of the rows this rank owns
//      (either by loading them from every rank's gradient buffer over NVLink and adding, or, when the arenas
//      are bound to an NVSwitch multicast object, by ONE multimem.ld_reduce per 16 bytes: the switch adds),
//      runs the optimiser step (f32 master weights, moments), and stores the new 16-bit rows into every
//      rank's weight tensor (peer stores, or ONE multimem.st the switch delivers everywhere); the last
//      thread block to finish raises flag B[block][r] on every other rank;
//   3. the dX GEMM of the layer below waits, in its TMA producer, for the other ranks' B flags of just the
//      blocks its tile needs.
// With multicast each GPU sends, per 67 M-parameter layer on 8 GPUs, 134 MB instead of 234 MB. The kernel of
// the last block also adds the [3 x N] column sums of all ranks and steps bias and normalisation parameters
// (identically on every rank). Work of one GPU is ordered by its stream; the only in-kernel waits are for
// flags that OTHER GPUs raise, every one bounded, ending in an error code instead of a hang, and a kernel
// whose wait gave up (or that finds the error word set) changes nothing and raises no flag. Flags hold the
// step's epoch number and only grow.
#pragma once

#include "sk_rowwise.cuh"

namespace sk {

constexpr int kMaxChunks = 8;
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

// ---- NVSwitch multicast (NVLS) forms of the two transfers -------------------------------------------
// With the arenas of all ranks bound to one multicast object, a load from the multicast address of the
// gradient buffer is reduced inside the switch (each GPU then receives only the sum of the rows it owns),
// and a store to the multicast address of the weight tensor lands in every GPU's copy (each GPU sends its
// rows once). Per 67 M-parameter layer on 8 GPUs that is 134 MB per NVLink direction instead of 234 MB.
// The switch adds the 16-bit partial gradients with f32 accumulation and returns the sum rounded to the
// 16-bit type (the plain form keeps the f32 sum): one more rounding of 2^-11 (f16) on the summed gradient.
template <typename T> __device__ __forceinline__ uint4 multimem_sum_16bit(const void *mc_addr);
template <> __device__ __forceinline__ uint4 multimem_sum_16bit<__half>(const void *mc_addr) {
    uint4 r;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(mc_addr) : "memory");
    return r;
}
template <> __device__ __forceinline__ uint4 multimem_sum_16bit<__nv_bfloat16>(const void *mc_addr) {
    uint4 r;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(mc_addr) : "memory");
    return r;
}
__device__ __forceinline__ void multimem_store_16B(void *mc_addr, const uint4 &v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
                 ::"l"(mc_addr), "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)),
                   "f"(__uint_as_float(v.w)) : "memory");
}

template <typename T> struct ExchangeArgs {
    PeerPtrs grad, w, flags, colsums;   // per rank: gradient buffer, weight tensor, flag words, column sums of the layer
    const void *mc_grad;                // multicast addresses of the gradient buffers / weight tensors, or nullptr
    void *mc_w;
    uint32_t world, rank, chunk, epoch;
    size_t off, len;                    // elements: this rank's rows of this block inside the [K x N] matrix
    float *master, *dv, *dm;            // local f32 state, whole matrix
    Optim opt;
    Hyper hyp;                          // inv_m = 1: the staged gradients are already averaged
    uint32_t *done;                     // local counter, zero between launches
    int *err;
    uint32_t do_vector, N;              // last block: also the bias / normalisation-parameter step
    VectorParams<T> vp;
};

template <typename T, int W, bool MC>
__global__ void __launch_bounds__(kRowThreads) exchange_update_kernel(ExchangeArgs<T> a) {
    __shared__ int ok_s;
    constexpr int V = 8;
    const uint32_t *my_flags = reinterpret_cast<const uint32_t *>(a.flags.p[a.rank]);
    if (threadIdx.x == 0) ok_s = *reinterpret_cast<volatile int *>(a.err) == 0;
    __syncthreads();
    if (threadIdx.x < W && threadIdx.x != a.rank) {   // this rank's own gradient precedes the kernel on its stream
        if (!poll_flag_reached(my_flags + (0 * kMaxChunks + a.chunk) * kMaxRanks + threadIdx.x, a.epoch)) {
            ok_s = 0;
            atomicCAS(a.err, 0, kErrExchangeFlags);
        }
        __threadfence_system();
    }
    __syncthreads();
    if (!ok_s) return;

    const size_t nvec = a.len / V, stride = (size_t)gridDim.x * blockDim.x;
    float *master = a.master + a.off, *dv = a.dv + a.off, *dm = a.dm + a.off;
    // U runs of 16 bytes per thread and pass: their remote loads (the long latency: NVLink, and the switch's
    // reduction with multicast) are all issued before the first is used; the local state of each run is then
    // loaded, stepped and stored in turn.
    constexpr int U = MC ? 4 : (W >= 8 ? 1 : 8 / W);
    for (size_t base = (size_t)blockIdx.x * blockDim.x + threadIdx.x; base < nvec; base += stride * U) {
        uint4 part[U][MC ? 1 : W];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const size_t i = base + (size_t)u * stride;
            if (i < nvec) {
                if (MC) {   // the switch adds the ranks' rows (f32 accumulation) and returns the sum in the 16-bit type
                    part[u][0] = multimem_sum_16bit<T>(reinterpret_cast<const T *>(a.mc_grad) + a.off + i * V);
                } else {
#pragma unroll
                    for (int s = 0; s < W; ++s)
                        part[u][MC ? 0 : s] = __ldcg(reinterpret_cast<const uint4 *>(reinterpret_cast<const T *>(a.grad.p[s]) + a.off + i * V));
                }
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const size_t i = base + (size_t)u * stride;
            if (i >= nvec) continue;
            float g[V];
#pragma unroll
            for (int j = 0; j < V; ++j) g[j] = 0.0f;
#pragma unroll
            for (int s = 0; s < (MC ? 1 : W); ++s) {
                const Pack<T, V> &pk = *reinterpret_cast<const Pack<T, V> *>(&part[u][s]);
#pragma unroll
                for (int j = 0; j < V; ++j) g[j] += to_f32(pk.v[j]);
            }
            float p[V], v[V], m[V];
            load_run<float, V>(master + i * V, true, p);
            load_run<float, V>(dv + i * V, true, v);
            load_run<float, V>(dm + i * V, true, m);
#pragma unroll
            for (int j = 0; j < V; ++j) p[j] = optimiser_step_fast(p[j], v[j], m[j], g[j] * kLossScaleInv, a.opt, a.hyp, true);
            store_run<float, V>(dv + i * V, true, v);
            store_run<float, V>(dm + i * V, true, m);
            store_run<float, V>(master + i * V, true, p);
            Pack<T, V> out;
#pragma unroll
            for (int j = 0; j < V; ++j) out.v[j] = from_f32<T>(p[j]);
            const uint4 o = *reinterpret_cast<const uint4 *>(&out);
            if (MC) {
                multimem_store_16B(reinterpret_cast<T *>(a.mc_w) + a.off + i * V, o);   // lands in every rank's copy
            } else {
#pragma unroll
                for (int s = 0; s < W; ++s) *reinterpret_cast<uint4 *>(reinterpret_cast<T *>(a.w.p[s]) + a.off + i * V) = o;
            }
        }
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
