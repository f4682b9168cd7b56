// FFMA-tiled GEMM for the f32 path and for 16-bit shapes the tensor-core kernel cannot
// take (leading dimensions that are not multiples of 16 bytes, tiny matrices).
//
//   C[m, n] = sum_k A(m, k) * B(k, n),   one fused-multiply-add chain per output in
//   increasing k (the summation order of the reference's dev_gemm, src/cuda/kernel/math.cu:8-50).
//
// A and B are read through (contiguous-direction, leading-dimension) pairs so that the
// three products of a DenseBlock run straight from the row-major tensors:
//   forward  Y = X.W        A k-contiguous (X[m*K+k]),   B n-contiguous (W[k*N+n])
//   dX       S = dY.W^T     A k-contiguous (dY[m*E+k]),  B k-contiguous (W[n*E+k])
//   dW       G = X^T.dY     A m-contiguous (X[k*K+m]),   B n-contiguous (dY[k*N+n])
// Tiles are staged in shared memory as [k][m] and [k][n] f32 panels with 128-bit
// coalesced global loads, register prefetch of the next panel, and a TM x TN register
// block per thread. The epilogue functor gets runs of TN consecutive columns.
#pragma once

#include "sk_epilogue.cuh"

namespace sk {

constexpr int kSimtThreads = 256;
constexpr int kSimtBK = 16;

// Load E contiguous elements starting at p (valid: how many of them exist) as f32.
template <typename T, int E>
__device__ __forceinline__ void load_guarded(const T *p, int valid, bool vec_ok, float (&out)[E]) {
    if (vec_ok && valid >= E) {
        load_run<T, E>(p, true, out);
    } else {
#pragma unroll
        for (int i = 0; i < E; ++i) out[i] = i < valid ? to_f32(p[i]) : 0.0f;
    }
}

// BK: depth of one panel. These small tiles are used when the problem has few tiles (small or thin matrices),
// where a block's time is one global-memory round trip per panel, not arithmetic: a deep panel (64 for the
// 32 x 32 tile: eight elements per thread and operand in flight) divides the number of round trips.
template <typename TA, typename TB, bool A_KCONTIG, bool B_NCONTIG, int BM, int BN, int TM, int TN, int BK, class Epi>
__global__ void __launch_bounds__(kSimtThreads)
gemm_simt_kernel(const TA *__restrict__ A, const TB *__restrict__ B, uint32_t M, uint32_t N, uint32_t K,
                 size_t lda, size_t ldb, bool a_vec, bool b_vec, Epi epi) {
    constexpr int EA = BM * BK / kSimtThreads; // elements of A per thread per panel
    constexpr int EB = BN * BK / kSimtThreads;
    static_assert((BM / TM) * (BN / TN) == kSimtThreads, "thread block must cover the tile");
    static_assert(EA >= 1 && EB >= 1 && BK % EA == 0 && BK % EB == 0, "panel split");
    constexpr int PAD = 1;   // odd row pitch: the column-wise stores of a K-contiguous operand spread over the banks
    __shared__ float As[BK][BM + PAD];
    __shared__ float Bs[BK][BN + PAD];

    const int t = threadIdx.x;
    const uint32_t m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int tx = t % (BN / TN), ty = t / (BN / TN);

    // per-thread source coordinates inside a panel
    int a_mn, a_k, b_mn, b_k;
    if (A_KCONTIG) { a_mn = t / (BK / EA); a_k = (t % (BK / EA)) * EA; }
    else           { a_k = t / (BM / EA); a_mn = (t % (BM / EA)) * EA; }
    if (B_NCONTIG) { b_k = t / (BN / EB); b_mn = (t % (BN / EB)) * EB; }
    else           { b_mn = t / (BK / EB); b_k = (t % (BK / EB)) * EB; }

    float ra[EA], rb[EB];
    auto fetch = [&](uint32_t k0) {
        if (A_KCONTIG) {
            const uint32_t m = m0 + a_mn, k = k0 + a_k;
            const int valid = m < M ? (int)K - (int)k : 0;
            load_guarded<TA, EA>(A + (size_t)m * lda + k, valid, a_vec, ra);
        } else {
            const uint32_t m = m0 + a_mn, k = k0 + a_k;
            const int valid = k < K ? (int)M - (int)m : 0;
            load_guarded<TA, EA>(A + (size_t)k * lda + m, valid, a_vec, ra);
        }
        if (B_NCONTIG) {
            const uint32_t n = n0 + b_mn, k = k0 + b_k;
            const int valid = k < K ? (int)N - (int)n : 0;
            load_guarded<TB, EB>(B + (size_t)k * ldb + n, valid, b_vec, rb);
        } else {
            const uint32_t n = n0 + b_mn, k = k0 + b_k;
            const int valid = n < N ? (int)K - (int)k : 0;
            load_guarded<TB, EB>(B + (size_t)n * ldb + k, valid, b_vec, rb);
        }
    };
    auto stage = [&]() {
        if (A_KCONTIG) {
#pragma unroll
            for (int i = 0; i < EA; ++i) As[a_k + i][a_mn] = ra[i];
        } else {
#pragma unroll
            for (int i = 0; i < EA; ++i) As[a_k][a_mn + i] = ra[i];
        }
        if (B_NCONTIG) {
#pragma unroll
            for (int i = 0; i < EB; ++i) Bs[b_k][b_mn + i] = rb[i];
        } else {
#pragma unroll
            for (int i = 0; i < EB; ++i) Bs[b_k + i][b_mn] = rb[i];
        }
    };

    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

    fetch(0);
    for (uint32_t k0 = 0; k0 < K; k0 += BK) {
        stage();
        __syncthreads();
        if (k0 + BK < K) fetch(k0 + BK);
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) b[j] = Bs[kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }

    const uint32_t col0 = n0 + tx * TN;
    if (col0 >= N) return;
    const uint32_t ncols = min((uint32_t)TN, N - col0);
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const uint32_t row = m0 + ty * TM + i;
        if (row < M) epi.template run<TN>(row, col0, acc[i], ncols);
    }
}

__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t v, float &lo, float &hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
// acc.lo = a.lo * b.lo + acc.lo, acc.hi = a.hi * b.hi + acc.hi, each rounded to nearest like fmaf
__device__ __forceinline__ void fma_f32x2(uint64_t &acc, uint64_t a, uint64_t b) {
    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc) : "l"(a), "l"(b));
}

// The same product for large problems: 128 x 128 x 16 tiles, two shared-memory buffers (the next
// panel is stored while the current one is still being read: one barrier per 16-deep step), 128-bit
// shared-memory reads, and an 8 x 8 register block per thread laid out as 2 x 2 groups of 4 x 4, 64
// apart, so that the 16 threads of a row read 256 contiguous bytes of the B panel (no bank conflicts)
// and the two rows of a warp read two broadcast addresses of the A panel. (A warp of 8 x 4 threads
// needs a third fewer shared-memory wavefronts and measured 1 % slower.) Two blocks per SM. The summation order per output is the same increasing-k chain of fused
// multiply-adds, so results equal the kernel above bit for bit. The epilogue functor gets runs of 4
// consecutive columns.
template <typename TA, typename TB, bool A_KCONTIG, bool B_NCONTIG, class Epi>
__global__ void __launch_bounds__(kSimtThreads, 2)
gemm_simt128_kernel(const TA *__restrict__ A, const TB *__restrict__ B, uint32_t M, uint32_t N, uint32_t K, size_t lda,
                    size_t ldb, bool a_vec, bool b_vec, Epi epi) {
    constexpr int BM = 128, BN = 128, BK = kSimtBK, E = BM * BK / kSimtThreads;   // 8 elements per thread per panel
    constexpr int LD = BM + 4;
    __shared__ __align__(16) float As[2][BK][LD];
    __shared__ __align__(16) float Bs[2][BK][LD];

    const int t = threadIdx.x;
    const uint32_t m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int tx = t & 15, ty = t >> 4;

    int a_mn, a_k, b_mn, b_k;
    if (A_KCONTIG) { a_mn = t / (BK / E); a_k = (t % (BK / E)) * E; }
    else           { a_k = t / (BM / E); a_mn = (t % (BM / E)) * E; }
    if (B_NCONTIG) { b_k = t / (BN / E); b_mn = (t % (BN / E)) * E; }
    else           { b_mn = t / (BK / E); b_k = (t % (BK / E)) * E; }

    float ra[E], rb[E];
    auto fetch = [&](uint32_t k0) {
        if (A_KCONTIG) {
            const uint32_t m = m0 + a_mn, k = k0 + a_k;
            load_guarded<TA, E>(A + (size_t)m * lda + k, m < M ? (int)K - (int)k : 0, a_vec, ra);
        } else {
            const uint32_t m = m0 + a_mn, k = k0 + a_k;
            load_guarded<TA, E>(A + (size_t)k * lda + m, k < K ? (int)M - (int)m : 0, a_vec, ra);
        }
        if (B_NCONTIG) {
            const uint32_t n = n0 + b_mn, k = k0 + b_k;
            load_guarded<TB, E>(B + (size_t)k * ldb + n, k < K ? (int)N - (int)n : 0, b_vec, rb);
        } else {
            const uint32_t n = n0 + b_mn, k = k0 + b_k;
            load_guarded<TB, E>(B + (size_t)n * ldb + k, n < N ? (int)K - (int)k : 0, b_vec, rb);
        }
    };
    auto stage = [&](int buf) {
        if (A_KCONTIG) {
#pragma unroll
            for (int i = 0; i < E; ++i) As[buf][a_k + i][a_mn] = ra[i];
        } else {
            *reinterpret_cast<float4 *>(&As[buf][a_k][a_mn]) = make_float4(ra[0], ra[1], ra[2], ra[3]);
            *reinterpret_cast<float4 *>(&As[buf][a_k][a_mn + 4]) = make_float4(ra[4], ra[5], ra[6], ra[7]);
        }
        if (B_NCONTIG) {
            *reinterpret_cast<float4 *>(&Bs[buf][b_k][b_mn]) = make_float4(rb[0], rb[1], rb[2], rb[3]);
            *reinterpret_cast<float4 *>(&Bs[buf][b_k][b_mn + 4]) = make_float4(rb[4], rb[5], rb[6], rb[7]);
        } else {
#pragma unroll
            for (int i = 0; i < E; ++i) Bs[buf][b_k + i][b_mn] = rb[i];
        }
    };

    // Accumulators as pairs of adjacent columns: one fma.rn.f32x2 (two round-to-nearest FMAs, the same
    // arithmetic per element as fmaf) per pair halves the instructions issued per flop, which leaves the
    // issue slots the shared-memory loads need.
    uint64_t acc2[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc2[i][j] = 0ull;   // two +0.0f

    fetch(0);
    stage(0);
    __syncthreads();
    int buf = 0;
    for (uint32_t k0 = 0; k0 < K; k0 += BK) {
        const bool more = k0 + BK < K;
        if (more) fetch(k0 + BK);
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            const float4 a0 = *reinterpret_cast<const float4 *>(&As[buf][kk][ty * 4]);
            const float4 a1 = *reinterpret_cast<const float4 *>(&As[buf][kk][64 + ty * 4]);
            const float4 b0 = *reinterpret_cast<const float4 *>(&Bs[buf][kk][tx * 4]);
            const float4 b1 = *reinterpret_cast<const float4 *>(&Bs[buf][kk][64 + tx * 4]);
            const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            const uint64_t b[4] = {pack_f32x2(b0.x, b0.y), pack_f32x2(b0.z, b0.w), pack_f32x2(b1.x, b1.y), pack_f32x2(b1.z, b1.w)};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const uint64_t aa = pack_f32x2(a[i], a[i]);
#pragma unroll
                for (int j = 0; j < 4; ++j) fma_f32x2(acc2[i][j], aa, b[j]);
            }
        }
        if (more) stage(buf ^ 1);
        __syncthreads();
        buf ^= 1;
    }
    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) unpack_f32x2(acc2[i][j], acc[i][2 * j], acc[i][2 * j + 1]);

#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint32_t row = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
        if (row >= M) continue;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t col0 = n0 + h * 64 + tx * 4;
            if (col0 >= N) continue;
            const float r[4] = {acc[i][h * 4], acc[i][h * 4 + 1], acc[i][h * 4 + 2], acc[i][h * 4 + 3]};
            epi.template run<4>(row, col0, r, min(4u, N - col0));
        }
    }
}

// Host-side launcher: picks the tile so that small problems still spread over the SMs.
template <typename TA, typename TB, bool A_KCONTIG, bool B_NCONTIG, class Epi>
cudaError_t launch_gemm_simt(cudaStream_t stream, int num_sms, const TA *A, size_t lda, const TB *B, size_t ldb,
                             uint32_t M, uint32_t N, uint32_t K, const Epi &epi) {
    auto aligned = [](const void *p, size_t ld, size_t es) {
        return (reinterpret_cast<uintptr_t>(p) % 16 == 0) && ((ld * es) % 16 == 0);
    };
    const bool a_vec = aligned(A, lda, sizeof(TA)), b_vec = aligned(B, ldb, sizeof(TB));
    auto ctas = [&](uint32_t bm, uint32_t bn) { return (size_t)((M + bm - 1) / bm) * ((N + bn - 1) / bn); };
    if (ctas(128, 128) >= (size_t)num_sms) {
        dim3 grid((N + 127) / 128, (M + 127) / 128);
        gemm_simt128_kernel<TA, TB, A_KCONTIG, B_NCONTIG, Epi>
            <<<grid, kSimtThreads, 0, stream>>>(A, B, M, N, K, lda, ldb, a_vec, b_vec, epi);
    } else if (ctas(64, 64) >= (size_t)num_sms) {
        dim3 grid((N + 63) / 64, (M + 63) / 64);
        gemm_simt_kernel<TA, TB, A_KCONTIG, B_NCONTIG, 64, 64, 4, 4, 32, Epi>
            <<<grid, kSimtThreads, 0, stream>>>(A, B, M, N, K, lda, ldb, a_vec, b_vec, epi);
    } else {
        dim3 grid((N + 31) / 32, (M + 31) / 32);
        gemm_simt_kernel<TA, TB, A_KCONTIG, B_NCONTIG, 32, 32, 2, 2, 64, Epi>
            <<<grid, kSimtThreads, 0, stream>>>(A, B, M, N, K, lda, ldb, a_vec, b_vec, epi);
    }
    return cudaGetLastError();
}

} // namespace sk
