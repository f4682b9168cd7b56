// Memory-bound kernels of the DenseBlock path: normalisation + activation + dropout,
// softmax + output-layer delta, column sums with the bias / norm-parameter step, casts
// and fills. Each streams its tensors once with 128-bit accesses and reduces with warp
// shuffles; the bound is HBM bandwidth.
#pragma once

#include "sk_epilogue.cuh"

namespace sk {

constexpr int kRowThreads = 256;

struct ActDrop {
    uint32_t act, use_dropout, seed, row_offset;
    float leaky, mask_coeff;
};

// activation + dropout on V values of one row (ffn/forward.cu:130-161), written to
// predrop / out / mask at idx.
template <typename T, int V>
__device__ __forceinline__ void act_drop_store(const ActDrop &ad, const float (&pre)[V], uint32_t row, uint32_t col0,
                                               size_t idx, T *predrop, T *out, T *mask, bool vec, uint32_t ncols) {
    float a[V], o[V], mk[V];
    const uint32_t grow = row + ad.row_offset;
    const float scale = 1.0f / (1.0f - ad.mask_coeff);
    activation_v<kFastMath<T>, V>(ad.act, pre, a, ad.leaky);
#pragma unroll
    for (int j = 0; j < V; ++j) {
        const bool keep = ad.use_dropout ? dropout_keep(col0 + j, grow, ad.seed, ad.mask_coeff) : true;
        mk[j] = keep ? scale : 0.0f;
        o[j] = ad.use_dropout ? (keep ? a[j] * scale : 0.0f) : a[j];
    }
    if (vec) {
        store_run<T, V>(predrop + idx, true, a);
        store_run<T, V>(out + idx, true, o);
        if (ad.use_dropout) store_run<T, V>(mask + idx, true, mk);
    } else {
        for (uint32_t j = 0; j < ncols; ++j) {
            predrop[idx + j] = from_f32<T>(a[j]);
            out[idx + j] = from_f32<T>(o[j]);
            if (ad.use_dropout) mask[idx + j] = from_f32<T>(mk[j]);
        }
    }
}

// RMSNorm (norm 1) / LayerNorm (norm 2) of one row per block, fused with activation and
// dropout: reads prenorm once from HBM (later passes over the row hit L2, or shared memory
// when `cached`), writes centered, preact, predrop, out, (mask) and rstd[row]. The output loop
// is kept rolled so that the activation code exists once (instruction-cache footprint).
// Reference: ffn/forward.cu:44-73 (RMS, products in T arithmetic), :74-126 (LayerNorm).
template <typename T>
__global__ void __launch_bounds__(kRowThreads)
norm_rows_kernel(const T *__restrict__ prenorm, const T *__restrict__ norm_w, const T *__restrict__ norm_b,
                 T *__restrict__ centered, T *__restrict__ preact, T *__restrict__ predrop, T *__restrict__ out,
                 T *__restrict__ mask, T *__restrict__ rstd_out, uint32_t N, uint32_t norm, ActDrop ad,
                 bool vec_ok, bool cached) {
    extern __shared__ __align__(16) float row_cache[];
    __shared__ float red[32];
    constexpr int V = 8;
    const uint32_t row = blockIdx.x;
    const size_t base = (size_t)row * N;
    const uint32_t nvec = vec_ok ? N / V : 0; // vec_ok implies N % 8 == 0

    // pass 1: sum (LayerNorm) or sum of squares (RMSNorm)
    float s = 0.0f;
    for (uint32_t c = threadIdx.x; c < nvec; c += blockDim.x) {
        float x[V];
        load_run<T, V>(prenorm + base + (size_t)c * V, true, x);
#pragma unroll
        for (int j = 0; j < V; ++j) {
            s += norm == 1 ? x[j] * x[j] : x[j];
            if (cached) row_cache[c * V + j] = x[j];
        }
    }
    if (!vec_ok)
        for (uint32_t c = threadIdx.x; c < N; c += blockDim.x) {
            const float x = to_f32(prenorm[base + c]);
            s += norm == 1 ? x * x : x;
            if (cached) row_cache[c] = x;
        }
    s = block_sum(s, red);
    float mean = 0.0f, var;
    if (norm == 1) {
        var = s / (float)N + 1e-6f;
    } else {
        mean = s / (float)N;
        float q = 0.0f;
        for (uint32_t c = threadIdx.x; c < N; c += blockDim.x) {
            const float d = (cached ? row_cache[c] : to_f32(prenorm[base + c])) - mean;
            q += d * d;
        }
        q = block_sum(q, red);
        var = q / (float)N + 1e-6f;
    }
    const float rstd = rsqrtf(var);
    const T rstd_t = from_f32<T>(rstd);
    if (threadIdx.x == 0) rstd_out[row] = rstd_t;

    // pass 2: outputs
    auto emit = [&](uint32_t col0, const float(&x)[V], bool vec, uint32_t ncols) {
        float cen[V], pre[V];
        if (norm == 1) {
#pragma unroll
            for (int j = 0; j < V; ++j) {
                cen[j] = x[j];
                const uint32_t c = col0 + j < N ? col0 + j : N - 1;
                pre[j] = to_f32(mul_t(mul_t(from_f32<T>(x[j]), rstd_t), norm_w[c]));
            }
        } else {
#pragma unroll
            for (int j = 0; j < V; ++j) {
                const uint32_t c = col0 + j < N ? col0 + j : N - 1;
                const float d = x[j] - mean;
                cen[j] = d;
                pre[j] = round_to<T>(d * rstd * to_f32(norm_w[c]) + to_f32(norm_b[c]));
            }
        }
        const size_t idx = base + col0;
        if (vec) {
            store_run<T, V>(centered + idx, true, cen);
            store_run<T, V>(preact + idx, true, pre);
        } else {
            for (uint32_t j = 0; j < ncols; ++j) {
                centered[idx + j] = from_f32<T>(cen[j]);
                preact[idx + j] = from_f32<T>(pre[j]);
            }
        }
        act_drop_store<T, V>(ad, pre, row, col0, idx, predrop, out, mask, vec, ncols);
    };
    if (vec_ok) {
#pragma unroll 1
        for (uint32_t c = threadIdx.x; c < nvec; c += blockDim.x) {
            float x[V];
            if (cached) {
#pragma unroll
                for (int j = 0; j < V; ++j) x[j] = row_cache[c * V + j];
            } else {
                load_run<T, V>(prenorm + base + (size_t)c * V, true, x);
            }
            emit(c * V, x, true, V);
        }
    } else {
        for (uint32_t c0 = threadIdx.x * V; c0 < N; c0 += blockDim.x * V) {
            float x[V];
            const uint32_t ncols = min((uint32_t)V, N - c0);
#pragma unroll
            for (int j = 0; j < V; ++j)
                x[j] = (uint32_t)j < ncols ? (cached ? row_cache[c0 + j] : to_f32(prenorm[base + c0 + j])) : 0.0f;
            emit(c0, x, false, ncols);
        }
    }
}

// BatchNorm (norm 3): statistics over the batch of each column, always from the batch
// (ffn/forward.cu:74-126 with n = m). One block owns 32 adjacent columns so that every
// access is a coalesced 32-wide row segment; 8 row lanes split the batch.
template <typename T>
__global__ void __launch_bounds__(kRowThreads)
norm_cols_kernel(const T *__restrict__ prenorm, const T *__restrict__ norm_w, const T *__restrict__ norm_b,
                 T *__restrict__ centered, T *__restrict__ preact, T *__restrict__ predrop, T *__restrict__ out,
                 T *__restrict__ mask, T *__restrict__ rstd_out, uint32_t M, uint32_t N, ActDrop ad) {
    __shared__ float red[8][33];
    const uint32_t cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
    const uint32_t col = blockIdx.x * 32 + cx;
    const bool live = col < N;
    auto reduce = [&](float v) {
        red[ry][cx] = v;
        __syncthreads();
        float t = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) t += red[i][cx];
        __syncthreads();
        return t;
    };
    float s = 0.0f;
    if (live) for (uint32_t r = ry; r < M; r += 8) s += to_f32(prenorm[(size_t)r * N + col]);
    const float mean = reduce(s) / (float)M;
    float q = 0.0f;
    if (live) for (uint32_t r = ry; r < M; r += 8) { const float d = to_f32(prenorm[(size_t)r * N + col]) - mean; q += d * d; }
    const float rstd = rsqrtf(reduce(q) / (float)M + 1e-6f);
    if (!live) return;
    if (ry == 0) rstd_out[col] = from_f32<T>(rstd);
    const float nw = to_f32(norm_w[col]), nb = to_f32(norm_b[col]);
    for (uint32_t r = ry; r < M; r += 8) {
        const size_t idx = (size_t)r * N + col;
        const float d = to_f32(prenorm[idx]) - mean;
        centered[idx] = from_f32<T>(d);
        float pre[1] = {round_to<T>(d * rstd * nw + nb)};
        preact[idx] = from_f32<T>(pre[0]);
        act_drop_store<T, 1>(ad, pre, r, col, idx, predrop, out, mask, false, 1);
    }
}

// BatchNorm with the batch split over several devices, in three phases around two sums over
// ranks (stats is f32 [2 x N]): phase 0 writes this shard's column sums of prenorm to stats[0];
// phase 1 takes the summed stats[0] and writes this shard's sums of (x - mean)^2 to stats[1];
// phase 2 takes both summed rows and does what norm_cols_kernel does after its reductions.
// m_stat is the whole batch. Same thread layout as norm_cols_kernel.
template <typename T>
__global__ void __launch_bounds__(kRowThreads)
norm_cols_phase_kernel(uint32_t phase, float *__restrict__ stats, uint32_t m_stat, const T *__restrict__ prenorm,
                       const T *__restrict__ norm_w, const T *__restrict__ norm_b, T *__restrict__ centered,
                       T *__restrict__ preact, T *__restrict__ predrop, T *__restrict__ out, T *__restrict__ mask,
                       T *__restrict__ rstd_out, uint32_t M, uint32_t N, ActDrop ad) {
    __shared__ float red[8][33];
    const uint32_t cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
    const uint32_t col = blockIdx.x * 32 + cx;
    const bool live = col < N;
    auto reduce = [&](float v) {
        red[ry][cx] = v;
        __syncthreads();
        float t = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) t += red[i][cx];
        __syncthreads();
        return t;
    };
    if (phase == 0) {
        float s = 0.0f;
        if (live) for (uint32_t r = ry; r < M; r += 8) s += to_f32(prenorm[(size_t)r * N + col]);
        s = reduce(s);
        if (live && ry == 0) stats[col] = s;
        return;
    }
    const float mean = live ? stats[col] / (float)m_stat : 0.0f;
    if (phase == 1) {
        float q = 0.0f;
        if (live) for (uint32_t r = ry; r < M; r += 8) { const float d = to_f32(prenorm[(size_t)r * N + col]) - mean; q += d * d; }
        q = reduce(q);
        if (live && ry == 0) stats[N + col] = q;
        return;
    }
    if (!live) return;
    const float rstd = rsqrtf(stats[N + col] / (float)m_stat + 1e-6f);
    if (ry == 0) rstd_out[col] = from_f32<T>(rstd);
    const float nw = to_f32(norm_w[col]), nb = to_f32(norm_b[col]);
    for (uint32_t r = ry; r < M; r += 8) {
        const size_t idx = (size_t)r * N + col;
        const float d = to_f32(prenorm[idx]) - mean;
        centered[idx] = from_f32<T>(d);
        float pre[1] = {round_to<T>(d * rstd * nw + nb)};
        preact[idx] = from_f32<T>(pre[0]);
        act_drop_store<T, 1>(ad, pre, r, col, idx, predrop, out, mask, false, 1);
    }
}

// Output-layer delta, one warp per row: optional in-place softmax of `out`
// (util.cu:95-173), then delta and the normalisation backward with loss scale 512
// (ffn/backward.cu:12-56). Also writes the 16-bit copy of d_prenorm when given.
template <typename T>
__global__ void __launch_bounds__(kRowThreads)
output_error_kernel(T *__restrict__ out, const T *__restrict__ preact, const T *__restrict__ target,
                    const float *__restrict__ norm_w, float *__restrict__ grad, float *__restrict__ d_prenorm,
                    float *__restrict__ d_norm_w, float *__restrict__ d_norm_b, T *__restrict__ d_prenorm_lp,
                    const T *__restrict__ rstd, const T *__restrict__ centered, const T *__restrict__ prenorm,
                    uint32_t M, uint32_t N, uint32_t err_mode, uint32_t norm, uint32_t act, float leaky) {
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= M) return;
    const size_t base = (size_t)row * N;
    const float inv_m = 1.0f / (float)M, inv_n = 1.0f / (float)N;
    float mx = 0.0f, total = 1.0f;
    if (act == 5) {
        mx = -INFINITY;
        for (uint32_t c = lane; c < N; c += 32) mx = fmaxf(mx, to_f32(out[base + c]));
        mx = warp_max(mx);
        float s = 0.0f;
        for (uint32_t c = lane; c < N; c += 32) s += expf(to_f32(out[base + c]) - mx);
        total = warp_sum(s);
    }
    const float rrow = (norm == 1 || norm == 2) ? to_f32(rstd[row]) : 0.0f;
    for (uint32_t c = lane; c < N; c += 32) {
        const size_t idx = base + c;
        float o = to_f32(out[idx]);
        if (act == 5) {
            const T sm = from_f32<T>(expf(o - mx) / total);
            out[idx] = sm;           // softmax lands in `out`, as in the reference
            o = to_f32(sm);
        } else {
            o = activation(act, o, leaky);
        }
        const float tg = to_f32(target[idx]);
        float delta = 0.0f;
        if (err_mode == 0) delta = activation_derivative(act, o - tg, o, to_f32(preact[idx]), leaky);
        else if ((err_mode == 1 && act == 5) || (err_mode == 2 && act == 1)) delta = o - tg;
        grad[idx] = delta;
        const float r = norm == 3 ? to_f32(rstd[c]) : rrow;
        const float pv = norm == 1 ? to_f32(prenorm[idx]) : 0.0f;
        const float cv = norm >= 2 ? to_f32(centered[idx]) : 0.0f;
        const NormGrad g = norm_gradients(norm, delta, pv, cv, r, norm_w[c], inv_n, inv_m);
        const float dp = g.d_prenorm * kLossScale;
        d_prenorm[idx] = dp;
        d_norm_w[idx] = g.d_norm_w;
        d_norm_b[idx] = g.d_norm_b;
        if (d_prenorm_lp) d_prenorm_lp[idx] = from_f32<T>(dp * kLpScale);
    }
}

// Output-layer delta without softmax: purely element-wise, 8 elements per thread with 128-bit
// accesses (ffn/backward.cu:12-56). Requires N % 8 == 0 and 16-byte aligned tensors. Three blocks per SM
// (80 registers): the kernel is bound by how many loads an SM keeps in flight.
template <typename T>
__global__ void __launch_bounds__(kRowThreads, 3)
output_error_elem_kernel(const T *__restrict__ out, const T *__restrict__ preact, const T *__restrict__ target,
                         const float *__restrict__ norm_w, float *__restrict__ grad, float *__restrict__ d_prenorm,
                         float *__restrict__ d_norm_w, float *__restrict__ d_norm_b, T *__restrict__ d_prenorm_lp,
                         const T *__restrict__ rstd, const T *__restrict__ centered, const T *__restrict__ prenorm,
                         uint32_t M, uint32_t N, uint32_t err_mode, uint32_t norm, uint32_t act, float leaky) {
    constexpr int V = 8;
    const uint32_t nvec = N / V;
    const size_t total = (size_t)M * nvec, stride = (size_t)gridDim.x * blockDim.x;
    const float inv_m = 1.0f / (float)M, inv_n = 1.0f / (float)N;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const uint32_t row = (uint32_t)(i / nvec), col0 = (uint32_t)(i % nvec) * V;
        const size_t idx = (size_t)row * N + col0;
        float o[V], pa[V], tg[V], xv[V], nw[V], rs[V], gr[V], dp[V], gw[V], gb[V];
        load_run<T, V>(out + idx, true, o);
        load_run<T, V>(target + idx, true, tg);
        if (err_mode == 0) load_run<T, V>(preact + idx, true, pa);
        if (norm == 1) load_run<T, V>(prenorm + idx, true, xv);
        else if (norm >= 2) load_run<T, V>(centered + idx, true, xv);
        if (norm) load_run<float, V>(norm_w + col0, true, nw);
        if (norm == 3) load_run<T, V>(rstd + col0, true, rs);
        const float rrow = (norm == 1 || norm == 2) ? to_f32(rstd[row]) : 0.0f;
#pragma unroll
        for (int j = 0; j < V; ++j) {
            const float a = activation(act, o[j], leaky);
            float delta = 0.0f;
            if (err_mode == 0) delta = activation_derivative(act, a - tg[j], a, pa[j], leaky);
            else if (err_mode == 2 && act == 1) delta = a - tg[j];
            gr[j] = delta;
            const NormGrad g = norm_gradients(norm, delta, norm ? xv[j] : 0.0f, norm ? xv[j] : 0.0f,
                                              norm == 3 ? rs[j] : rrow, norm ? nw[j] : 0.0f, inv_n, inv_m);
            dp[j] = g.d_prenorm * kLossScale;
            gw[j] = g.d_norm_w;
            gb[j] = g.d_norm_b;
        }
        store_run<float, V>(grad + idx, true, gr);
        store_run<float, V>(d_prenorm + idx, true, dp);
        store_run<float, V>(d_norm_w + idx, true, gw);
        store_run<float, V>(d_norm_b + idx, true, gb);
        if (d_prenorm_lp) {
            float lp[V];
#pragma unroll
            for (int j = 0; j < V; ++j) lp[j] = dp[j] * kLpScale;
            store_run<T, V>(d_prenorm_lp + idx, true, lp);
        }
    }
}

// Column sums over the batch of d_prenorm, d_norm_w, d_norm_b (the row-0 work of
// ffn/backward.cu:181-194). Stage 1: each block sums `rows_per_block` rows of 32 columns
// into partial[blockIdx.y][which][col]; stage 2 adds the partials in a fixed order.
__global__ void __launch_bounds__(kRowThreads)
colsum_partial_kernel(const float *__restrict__ d_prenorm, const float *__restrict__ d_norm_w,
                      const float *__restrict__ d_norm_b, float *__restrict__ partial, uint32_t M, uint32_t N,
                      uint32_t rows_per_block, uint32_t norm) {
    __shared__ float red[3][8][33];
    const uint32_t cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
    const uint32_t col = blockIdx.x * 32 + cx;
    const uint32_t r0 = blockIdx.y * rows_per_block, r1 = min(M, r0 + rows_per_block);
    float sb = 0.0f, sw = 0.0f, sn = 0.0f;
    if (col < N)
        for (uint32_t r = r0 + ry; r < r1; r += 8) {
            const size_t idx = (size_t)r * N + col;
            sb += d_prenorm[idx];
            if (norm > 0) sw += d_norm_w[idx];
            if (norm > 1) sn += d_norm_b[idx];
        }
    red[0][ry][cx] = sb; red[1][ry][cx] = sw; red[2][ry][cx] = sn;
    __syncthreads();
    if (ry < 3 && col < N) {
        float t = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) t += red[ry][i][cx];
        partial[((size_t)blockIdx.y * 3 + ry) * N + col] = t;
    }
}

// Folds `nin` partial slabs [3 x N] into gridDim.y slabs (slab y takes inputs y*per .. y*per+per-1), in a
// fixed order: used when the slabs come from the dX epilogue, one per 32 rows.
__global__ void colsum_fold_kernel(const float *__restrict__ in, float *__restrict__ out, uint32_t N, uint32_t nin,
                                   uint32_t per) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= 3 * N) return;
    const uint32_t b0 = blockIdx.y * per, b1 = min(nin, b0 + per);
    float t0 = 0.0f, t1 = 0.0f, t2 = 0.0f, t3 = 0.0f;
    uint32_t b = b0;
    for (; b + 4 <= b1; b += 4) {
        t0 += in[(size_t)b * 3 * N + i];
        t1 += in[(size_t)(b + 1) * 3 * N + i];
        t2 += in[(size_t)(b + 2) * 3 * N + i];
        t3 += in[(size_t)(b + 3) * 3 * N + i];
    }
    for (; b < b1; ++b) t0 += in[(size_t)b * 3 * N + i];
    out[(size_t)blockIdx.y * 3 * N + i] = (t0 + t1) + (t2 + t3);
}

// Stage 2 without update: colsums[which][col] = sum of partials (raw, still x512).
__global__ void colsum_final_kernel(const float *__restrict__ partial, float *__restrict__ colsums, uint32_t N,
                                    uint32_t nblocks) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= 3 * N) return;
    const uint32_t which = i / N, col = i % N;
    float t = 0.0f;
    for (uint32_t b = 0; b < nblocks; ++b) t += partial[((size_t)b * 3 + which) * N + col];
    colsums[i] = t;
}

// Bias and normalisation-parameter step of one column from its three sums (ffn/backward.cu:196-224).
template <typename T> struct VectorParams {
    T *b; float *master_b, *dv_b, *dm_b;
    T *nw; float *master_nw, *dv_nw, *dm_nw;
    T *nb; float *master_nb, *dv_nb, *dm_nb;
    uint32_t use_bias, norm;
    Optim lin, nrm;
    Hyper hyp;
};
template <typename T>
__device__ __forceinline__ void vector_step(const VectorParams<T> &P, uint32_t col, const float (&s)[3]) {
    auto step = [&](T *p, float *master, float *dv, float *dm, float sum, const Optim &o) {
        float v = dv[col], m = dm[col];
        const float np = optimiser_step(master[col], v, m, sum * kLossScaleInv, o, P.hyp, false);
        dv[col] = v; dm[col] = m; master[col] = np;
        if ((void *)p != (void *)master) p[col] = from_f32<T>(np);
    };
    if (P.use_bias) step(P.b, P.master_b, P.dv_b, P.dm_b, s[0], P.lin);
    if (P.norm > 0) {
        step(P.nw, P.master_nw, P.dv_nw, P.dm_nw, s[1], P.nrm);
        if (P.norm > 1) step(P.nb, P.master_nb, P.dv_nb, P.dm_nb, s[2], P.nrm);
    }
}

// `nblocks` partial slabs [3 x N] are summed first (1 slab for finished sums), then the step.
template <typename T>
__global__ void vector_update_kernel(const float *__restrict__ partial, uint32_t nblocks, uint32_t N, VectorParams<T> P,
                                     const int *abort_flag = nullptr) {
    const uint32_t col = blockIdx.x * blockDim.x + threadIdx.x;
    if (col >= N) return;
    if (abort_flag && *reinterpret_cast<const volatile int *>(abort_flag) != 0) return;   // the sums are not complete
    float s[3] = {0.0f, 0.0f, 0.0f};
    for (uint32_t k = 0; k < nblocks; ++k)
#pragma unroll
        for (int w = 0; w < 3; ++w) s[w] += partial[((size_t)k * 3 + w) * N + col];
    vector_step<T>(P, col, s);
}

// Small batches: column sums and the step in one launch. One block per 32 columns, its 8 row lanes
// walk all M rows (same layout and summation order as colsum_partial_kernel with one row block).
template <typename T>
__global__ void __launch_bounds__(kRowThreads)
colsum_update_kernel(const float *__restrict__ d_prenorm, const float *__restrict__ d_norm_w,
                     const float *__restrict__ d_norm_b, uint32_t M, uint32_t N, VectorParams<T> P) {
    __shared__ float red[3][8][33];
    const uint32_t cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
    const uint32_t col = blockIdx.x * 32 + cx;
    float sb = 0.0f, sw = 0.0f, sn = 0.0f;
    if (col < N)
        for (uint32_t r = ry; r < M; r += 8) {
            const size_t idx = (size_t)r * N + col;
            sb += d_prenorm[idx];
            if (P.norm > 0) sw += d_norm_w[idx];
            if (P.norm > 1) sn += d_norm_b[idx];
        }
    red[0][ry][cx] = sb; red[1][ry][cx] = sw; red[2][ry][cx] = sn;
    __syncthreads();
    if (ry == 0 && col < N) {
        float s[3] = {0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int w = 0; w < 3; ++w)
#pragma unroll
            for (int i = 0; i < 8; ++i) s[w] += red[w][i][cx];
        vector_step<T>(P, col, s);
    }
}

// Weight step from a finished f32 gradient (data-parallel path, after the sum over ranks).
template <typename T>
__global__ void __launch_bounds__(kRowThreads)
weight_update_kernel(const float *__restrict__ dw, T *w, float *master, float *dv, float *dm, size_t len,
                     Optim opt, Hyper hyp, bool vec_ok) {
    constexpr int V = 4;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    if (vec_ok) {
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < len / V; i += stride) {
            float g[V], p[V], v[V], m[V];
            load_run<float, V>(dw + i * V, true, g);
            load_run<float, V>(master + i * V, true, p);
            load_run<float, V>(dv + i * V, true, v);
            load_run<float, V>(dm + i * V, true, m);
#pragma unroll
            for (int j = 0; j < V; ++j) p[j] = optimiser_step(p[j], v[j], m[j], g[j] * kLossScaleInv, opt, hyp, true);
            store_run<float, V>(dv + i * V, true, v);
            store_run<float, V>(dm + i * V, true, m);
            store_run<float, V>(master + i * V, true, p);
            if ((void *)w != (void *)master) store_run<T, V>(w + i * V, true, p);
        }
    } else {
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < len; i += stride) {
            float v = dv[i], m = dm[i];
            const float p = optimiser_step(master[i], v, m, dw[i] * kLossScaleInv, opt, hyp, true);
            dv[i] = v; dm[i] = m; master[i] = p;
            if ((void *)w != (void *)master) w[i] = from_f32<T>(p);
        }
    }
}

// Weight step on a contiguous range of elements from a gradient stored as G (f32 or the
// 16-bit storage type), already averaged over the batch: g = grad * grad_scale (the remaining
// loss-scale factor). Used by the sharded data-parallel update, where each rank steps 1/W of
// every weight matrix. With `abort_flag` given, a non-zero word there (a bounded wait of an earlier
// kernel gave up, so `grad` is not complete) makes the kernel leave everything untouched.
template <typename T, typename G>
__global__ void __launch_bounds__(kRowThreads)
weight_update_range_kernel(const G *__restrict__ grad, float grad_scale, T *w, float *master, float *dv, float *dm,
                           size_t len, Optim opt, Hyper hyp, bool vec_ok, const int *abort_flag = nullptr) {
    constexpr int V = 8;
    if (abort_flag && *reinterpret_cast<const volatile int *>(abort_flag) != 0) return;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    if (vec_ok) {
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < len / V; i += stride) {
            float g[V], p[V], v[V], m[V];
            load_run<G, V>(grad + i * V, true, g);
            load_run<float, V>(master + i * V, true, p);
            load_run<float, V>(dv + i * V, true, v);
            load_run<float, V>(dm + i * V, true, m);
#pragma unroll
            for (int j = 0; j < V; ++j) p[j] = optimiser_step_fast(p[j], v[j], m[j], g[j] * grad_scale, opt, hyp, true);
            store_run<float, V>(dv + i * V, true, v);
            store_run<float, V>(dm + i * V, true, m);
            store_run<float, V>(master + i * V, true, p);
            if ((void *)w != (void *)master) store_run<T, V>(w + i * V, true, p);
        }
    } else {
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < len; i += stride) {
            float v = dv[i], m = dm[i];
            const float p = optimiser_step_fast(master[i], v, m, to_f32(grad[i]) * grad_scale, opt, hyp, true);
            dv[i] = v; dm[i] = m; master[i] = p;
            if ((void *)w != (void *)master) w[i] = from_f32<T>(p);
        }
    }
}

// ---- peer exchange (one process per GPU, buffers mapped into each other's address space) ----
struct PeerPtrs { void *p[kMaxRanks]; };

// Publish `value` in slot `slot` of every rank's flag array (release at system scope, so that
// everything this GPU wrote before, including peer stores of earlier kernels, is visible first).
__global__ void signal_peers_kernel(PeerPtrs flags, uint32_t world, uint32_t slot, uint32_t value) {
    if (threadIdx.x < world) {
        __threadfence_system();
        volatile uint32_t *f = reinterpret_cast<volatile uint32_t *>(flags.p[threadIdx.x]) + slot;
        *f = value;
        __threadfence_system();
    }
}

// Wait until every slot of the local flag array has reached `value`. The wait is bounded (about two
// seconds of SM clock); on expiry the error word is set and the kernel returns, so a rank that
// never signals costs an error status, not a hung GPU.
__global__ void wait_flags_kernel(const uint32_t *flags, uint32_t world, uint32_t value, int *err) {
    if (threadIdx.x >= world) return;
    const volatile uint32_t *f = flags + threadIdx.x;
    const long long t0 = clock64();
    while ((int32_t)(*f - value) < 0) {
        if (clock64() - t0 > 4000000000LL) { atomicCAS(err, 0, 5); break; }
        __nanosleep(200);
    }
    __threadfence_system();
}

// Owner side of the fused exchange, reduce-scatter + optimiser + all-gather in one kernel: pull the
// rows this rank owns out of every rank's gradient buffer (peer loads over NVLink, 512 contiguous
// bytes per warp), add them, run the optimiser step (f32 master, moments) and store the new 16-bit
// rows into every rank's weight tensor (peer stores). Loads and stores use opposite NVLink directions.
template <typename T>
__global__ void __launch_bounds__(kRowThreads)
reduce_update_broadcast_kernel(PeerPtrs grad_rows, uint32_t world, size_t shard_len, float *master, float *dv,
                               float *dm, PeerPtrs w_rows, Optim opt, Hyper hyp, const int *abort_flag) {
    constexpr int V = 8;
    // the flag wait that precedes this kernel gave up: the other ranks' gradients are not complete, change nothing
    if (abort_flag && *reinterpret_cast<const volatile int *>(abort_flag) != 0) return;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < shard_len / V; i += stride) {
        float g[V], p[V], v[V], m[V];
#pragma unroll
        for (int j = 0; j < V; ++j) g[j] = 0.0f;
        Pack<T, V> part[kMaxRanks];
#pragma unroll
        for (int s = 0; s < kMaxRanks; ++s)       // all loads in flight before the first use
            if ((uint32_t)s < world) part[s] = load_pack<T, V>(reinterpret_cast<const T *>(grad_rows.p[s]) + i * V);
#pragma unroll
        for (int s = 0; s < kMaxRanks; ++s)
            if ((uint32_t)s < world) {
#pragma unroll
                for (int j = 0; j < V; ++j) g[j] += to_f32(part[s].v[j]);
            }
        load_run<float, V>(master + i * V, true, p);
        load_run<float, V>(dv + i * V, true, v);
        load_run<float, V>(dm + i * V, true, m);
#pragma unroll
        for (int j = 0; j < V; ++j) p[j] = optimiser_step_fast(p[j], v[j], m[j], g[j] * kLossScaleInv, opt, hyp, true);
        store_run<float, V>(dv + i * V, true, v);
        store_run<float, V>(dm + i * V, true, m);
        store_run<float, V>(master + i * V, true, p);
        for (uint32_t s = 0; s < world; ++s) store_run<T, V>(reinterpret_cast<T *>(w_rows.p[s]) + i * V, true, p);
    }
}

// util.cuh:9-19 casts and math.cuh:69-73 fill, grid-stride.
template <typename S, typename D>
__global__ void cast_kernel(const S *__restrict__ src, D *__restrict__ dst, size_t len) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < len; i += stride) dst[i] = from_f32<D>(to_f32(src[i]));
}
template <typename T> __global__ void fill_kernel(T *dst, float v, size_t len) {
    const T tv = from_f32<T>(v);
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < len; i += stride) dst[i] = tv;
}

} // namespace sk
