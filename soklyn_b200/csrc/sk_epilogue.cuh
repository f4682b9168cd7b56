// Fused GEMM epilogues of the DenseBlock path. Each functor receives V consecutive
// columns of one output row with their f32 accumulators and does everything the
// reference does in the kernels that follow its GEMM (bias, activation, dropout;
// activation derivative, mask and normalisation backward; loss-scale removal and the
// optimiser step). The same functors serve the FFMA kernel and the tcgen05 kernel.
#pragma once

#include "sk_device.cuh"

namespace sk {

// ---- runs of V contiguous elements -----------------------------------------------------
// Packs wider than 16 bytes keep 16-byte alignment (two or more 128-bit accesses).
template <typename T, int V> struct alignas(sizeof(T) * V > 16 ? 16 : sizeof(T) * V) Pack { T v[V]; };

template <typename T, int V>
__device__ __forceinline__ void load_run(const T *p, bool vec, float (&out)[V]) {
    if (vec) {
        const Pack<T, V> pk = *reinterpret_cast<const Pack<T, V> *>(p);
#pragma unroll
        for (int i = 0; i < V; ++i) out[i] = to_f32(pk.v[i]);
    } else {
#pragma unroll
        for (int i = 0; i < V; ++i) out[i] = to_f32(p[i]);
    }
}

template <typename T, int V>
__device__ __forceinline__ void store_run(T *p, bool vec, const float (&in)[V]) {
    if (vec) {
        Pack<T, V> pk;
#pragma unroll
        for (int i = 0; i < V; ++i) pk.v[i] = from_f32<T>(in[i]);
        *reinterpret_cast<Pack<T, V> *>(p) = pk;
    } else {
#pragma unroll
        for (int i = 0; i < V; ++i) p[i] = from_f32<T>(in[i]);
    }
}

// ---- forward: Z = X.W + b, then (no normalisation) activation and dropout ------------------
// Reference: ffn/forward.cu:8-28 (bias), :130-161 (activation + dropout).
template <typename T> struct EpiForward {
    const T *bias;     // nullptr when the bias is not used (BatchNorm)
    T *z;              // prenorm (has_norm) or preact
    T *predrop, *out, *mask;
    uint32_t N;
    uint32_t has_norm, act, use_dropout, seed, row_offset;
    float leaky, mask_coeff;
    bool vec_ok;       // all pointers 16-byte aligned and N a multiple of 8

    __device__ __forceinline__ void one(uint32_t row, uint32_t col, float acc) const {
        const size_t idx = (size_t)row * N + col;
        float zv = acc;
        if (bias) zv += to_f32(bias[col]);
        const T zt = from_f32<T>(zv);
        z[idx] = zt;
        if (has_norm) return;
        const float a = activation(act, to_f32(zt), leaky);
        predrop[idx] = from_f32<T>(a);
        if (use_dropout) {
            const uint32_t grow = row + row_offset;
            if (dropout_keep(col, grow, seed, mask_coeff)) {
                const float scale = 1.0f / (1.0f - mask_coeff);
                mask[idx] = from_f32<T>(scale);
                out[idx] = from_f32<T>(a * scale);
            } else {
                mask[idx] = from_f32<T>(0.0f);
                out[idx] = from_f32<T>(0.0f);
            }
        } else {
            out[idx] = from_f32<T>(a);
        }
    }

    template <int V>
    __device__ __forceinline__ void run(uint32_t row, uint32_t col0, const float (&acc)[V], uint32_t ncols) const {
        if (!(vec_ok && ncols == V)) {
            for (uint32_t j = 0; j < ncols; ++j) one(row, col0 + j, acc[j]);
            return;
        }
        const size_t idx = (size_t)row * N + col0;
        float zv[V], a[V], o[V], mk[V];
        if (bias) {
            float b[V];
            load_run<T, V>(bias + col0, true, b);
#pragma unroll
            for (int j = 0; j < V; ++j) zv[j] = round_to<T>(acc[j] + b[j]);
        } else {
#pragma unroll
            for (int j = 0; j < V; ++j) zv[j] = round_to<T>(acc[j]);
        }
        store_run<T, V>(z + idx, true, zv);
        if (has_norm) return;
#pragma unroll
        for (int j = 0; j < V; ++j) a[j] = activation(act, zv[j], leaky);
        store_run<T, V>(predrop + idx, true, a);
        if (use_dropout) {
            const uint32_t grow = row + row_offset;
            const float scale = 1.0f / (1.0f - mask_coeff);
#pragma unroll
            for (int j = 0; j < V; ++j) {
                const bool keep = dropout_keep(col0 + j, grow, seed, mask_coeff);
                mk[j] = keep ? scale : 0.0f;
                o[j] = keep ? a[j] * scale : 0.0f;
            }
            store_run<T, V>(mask + idx, true, mk);
            store_run<T, V>(out + idx, true, o);
        } else {
            store_run<T, V>(out + idx, true, a);
        }
    }
};

// ---- hidden delta: S = dY_next . W_next^T, times act', times mask, normalisation backward ----
// Reference: ffn/backward.cu:59-102 and util.cu:175-215 (loss scale 1).
template <typename T> struct EpiHidden {
    const T *predrop, *preact, *mask, *prenorm, *centered, *rstd;
    const float *norm_w;   // f32 master copy of the normalisation weights
    float *grad, *d_prenorm, *d_norm_w, *d_norm_b;
    T *d_prenorm_lp;       // 16-bit copy for the next tensor-core GEMMs, or nullptr
    uint32_t N, norm, act;
    float leaky, inv_n, inv_m;
    bool vec_ok;

    __device__ __forceinline__ void one(uint32_t row, uint32_t col, float s) const {
        const size_t idx = (size_t)row * N + col;
        const float delta = to_f32(mask[idx]) *
                            activation_derivative(act, s, to_f32(predrop[idx]), to_f32(preact[idx]), leaky);
        grad[idx] = delta;
        const float r = norm ? to_f32(rstd[norm == 3 ? col : row]) : 0.0f;
        const float pv = norm == 1 ? to_f32(prenorm[idx]) : 0.0f;
        const float cv = norm >= 2 ? to_f32(centered[idx]) : 0.0f;
        const NormGrad g = norm_gradients(norm, delta, pv, cv, r, norm_w[col], inv_n, inv_m);
        d_prenorm[idx] = g.d_prenorm;
        d_norm_w[idx] = g.d_norm_w;
        d_norm_b[idx] = g.d_norm_b;
        if (d_prenorm_lp) d_prenorm_lp[idx] = from_f32<T>(g.d_prenorm);
    }

    template <int V>
    __device__ __forceinline__ void run(uint32_t row, uint32_t col0, const float (&acc)[V], uint32_t ncols) const {
        if (!(vec_ok && ncols == V)) {
            for (uint32_t j = 0; j < ncols; ++j) one(row, col0 + j, acc[j]);
            return;
        }
        const size_t idx = (size_t)row * N + col0;
        float pd[V], pa[V], mk[V], xv[V], nw[V], rs[V];
        float gr[V], dp[V], gw[V], gb[V];
        load_run<T, V>(predrop + idx, true, pd);
        load_run<T, V>(preact + idx, true, pa);
        load_run<T, V>(mask + idx, true, mk);
        if (norm == 1) load_run<T, V>(prenorm + idx, true, xv);
        else if (norm >= 2) load_run<T, V>(centered + idx, true, xv);
        if (norm) load_run<float, V>(norm_w + col0, true, nw);
        if (norm == 3) load_run<T, V>(rstd + col0, true, rs);
        const float rrow = (norm == 1 || norm == 2) ? to_f32(rstd[row]) : 0.0f;
#pragma unroll
        for (int j = 0; j < V; ++j) {
            const float delta = mk[j] * activation_derivative(act, acc[j], pd[j], pa[j], leaky);
            gr[j] = delta;
            const float r = norm == 3 ? rs[j] : rrow;
            const NormGrad g = norm_gradients(norm, delta, norm ? xv[j] : 0.0f, norm ? xv[j] : 0.0f, r,
                                              norm ? nw[j] : 0.0f, inv_n, inv_m);
            dp[j] = g.d_prenorm;
            gw[j] = g.d_norm_w;
            gb[j] = g.d_norm_b;
        }
        store_run<float, V>(grad + idx, true, gr);
        store_run<float, V>(d_prenorm + idx, true, dp);
        store_run<float, V>(d_norm_w + idx, true, gw);
        store_run<float, V>(d_norm_b + idx, true, gb);
        if (d_prenorm_lp) store_run<T, V>(d_prenorm_lp + idx, true, dp);
    }
};

// ---- weight gradient with the optimiser step fused in ------------------------------------------
// Reference: ffn/backward.cu:157-234 (dW part) with :105-154.
template <typename T> struct EpiWeightUpdate {
    T *w;
    float *master, *dv, *dm;   // master == (float*)w in f32 mode
    uint32_t N;
    Optim opt;
    Hyper hyp;
    bool vec_ok;

    template <int V>
    __device__ __forceinline__ void run(uint32_t row, uint32_t col0, const float (&acc)[V], uint32_t ncols) const {
        const size_t idx = (size_t)row * N + col0;
        const bool vec = vec_ok && ncols == V;
        float p[V], v[V], m[V];
        if (vec) {
            load_run<float, V>(master + idx, true, p);
            load_run<float, V>(dv + idx, true, v);
            load_run<float, V>(dm + idx, true, m);
        } else {
            for (uint32_t j = 0; j < V; ++j) {
                const bool ok = j < ncols;
                p[j] = ok ? master[idx + j] : 0.0f;
                v[j] = ok ? dv[idx + j] : 0.0f;
                m[j] = ok ? dm[idx + j] : 0.0f;
            }
        }
#pragma unroll
        for (int j = 0; j < V; ++j) p[j] = optimiser_step(p[j], v[j], m[j], acc[j] * kLossScaleInv, opt, hyp, true);
        if (vec) {
            store_run<float, V>(dv + idx, true, v);
            store_run<float, V>(dm + idx, true, m);
            store_run<float, V>(master + idx, true, p);
            if ((void *)w != (void *)master) store_run<T, V>(w + idx, true, p);
        } else {
            for (uint32_t j = 0; j < ncols; ++j) {
                dv[idx + j] = v[j];
                dm[idx + j] = m[j];
                master[idx + j] = p[j];
                if ((void *)w != (void *)master) w[idx + j] = from_f32<T>(p[j]);
            }
        }
    }
};

// ---- plain f32 store (raw batch sums for the data-parallel exchange) ------------------------------
struct EpiStoreF32 {
    float *c;
    uint32_t N;
    bool vec_ok;
    template <int V>
    __device__ __forceinline__ void run(uint32_t row, uint32_t col0, const float (&acc)[V], uint32_t ncols) const {
        const size_t idx = (size_t)row * N + col0;
        if (vec_ok && ncols == V) store_run<float, V>(c + idx, true, acc);
        else for (uint32_t j = 0; j < ncols; ++j) c[idx + j] = acc[j];
    }
};

} // namespace sk
