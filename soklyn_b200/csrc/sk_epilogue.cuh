// Fused GEMM epilogues of the DenseBlock path. Each functor receives V consecutive
// columns of one output row with their f32 accumulators and does everything the
// reference does in the kernels that follow its GEMM (bias, activation, dropout;
// activation derivative, mask and normalisation backward; loss-scale removal and the
// optimiser step). The same functors serve the FFMA kernel and the tcgen05 kernel.
//
// Two call forms:
//   run<V>(row, col0, acc, ncols)            everything at once (FFMA kernel, ragged edges)
//   cols(col0) / prefetch(...) / finish(...) for the tensor-core kernel, whose epilogue threads
//       keep one column group for several rows: cols() loads what depends on the columns only
//       (bias, normalisation weights) once, prefetch() issues the raw loads of the next row's
//       run before the current one is finished, finish() consumes them. These are used only
//       when every tensor allows 128-bit accesses (vec_ok) and the run has all 8 columns.
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

// Raw (unconverted) run of V elements, for loads issued ahead of their use.
template <typename T, int V> __device__ __forceinline__ Pack<T, V> load_pack(const T *p) {
    return *reinterpret_cast<const Pack<T, V> *>(p);
}
template <typename T, int V> __device__ __forceinline__ void unpack(const Pack<T, V> &pk, float (&out)[V]) {
#pragma unroll
    for (int i = 0; i < V; ++i) out[i] = to_f32(pk.v[i]);
}

struct NoPre {};
template <typename T> constexpr bool kFastMath = sizeof(T) == 2;   // 16-bit storage hides approximate math

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

    // vector path; b = bias of these columns (zeros when unused)
    template <int V>
    __device__ __forceinline__ void core(uint32_t row, uint32_t col0, const float (&acc)[V], const float (&b)[V]) const {
        const size_t idx = (size_t)row * N + col0;
        float zv[V], a[V], o[V], mk[V];
#pragma unroll
        for (int j = 0; j < V; ++j) zv[j] = round_to<T>(acc[j] + b[j]);
        store_run<T, V>(z + idx, true, zv);
        if (has_norm) return;
        activation_v<kFastMath<T>, V>(act, zv, a, leaky);
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

    template <int V>
    __device__ __forceinline__ void run(uint32_t row, uint32_t col0, const float (&acc)[V], uint32_t ncols) const {
        if (!(vec_ok && ncols == V)) {
            for (uint32_t j = 0; j < ncols; ++j) one(row, col0 + j, acc[j]);
            return;
        }
        float b[V];
        if (bias) load_run<T, V>(bias + col0, true, b);
        else {
#pragma unroll
            for (int j = 0; j < V; ++j) b[j] = 0.0f;
        }
        core<V>(row, col0, acc, b);
    }

    struct Cols { float b[8]; };
    using Pre = NoPre;
    __device__ __forceinline__ void cols(uint32_t col0, Cols &c) const {
        if (bias) load_run<T, 8>(bias + col0, true, c.b);
        else {
#pragma unroll
            for (int j = 0; j < 8; ++j) c.b[j] = 0.0f;
        }
    }
    __device__ __forceinline__ void prefetch(uint32_t, uint32_t, Pre &) const {}
    __device__ __forceinline__ void finish(uint32_t row, uint32_t col0, const float (&acc)[8], const Pre &, const Cols &c) const {
        core<8>(row, col0, acc, c.b);
    }
};

// ---- hidden delta: S = dY_next . W_next^T, times act', times mask, normalisation backward ----
// Reference: ffn/backward.cu:59-102 and util.cu:175-215 (loss scale 1).
// ACT / NORM >= 0 fix the activation and the normalisation at compile time (specialised kernels
// for the common pairs, with every mode switch folded away); -1 reads them from the fields.
template <typename T, int ACT = -1, int NORM = -1> struct EpiHidden {
    const T *predrop, *preact, *mask, *prenorm, *centered, *rstd;
    const float *norm_w;   // f32 master copy of the normalisation weights
    float *grad, *d_prenorm, *d_norm_w, *d_norm_b;
    T *d_prenorm_lp;       // 16-bit copy for the next tensor-core GEMMs, or nullptr
    uint32_t N, norm, act;
    float leaky, inv_n, inv_m;
    bool vec_ok;
    // Optional: column sums of d_prenorm, d_norm_w and d_norm_b per group of 32 rows, written as
    // partial[group][which][col] while the values are in registers, so that the weight-update call
    // that follows need not read the three tensors again. Only with vec_ok and on the tensor-core
    // kernel (every element then goes through finish()).
    float *colsum_partial;
    uint32_t colsum_groups;
    // Lean backward: with the column sums taken here nothing in the backward pass reads grad, the f32
    // d_prenorm, d_norm_w or d_norm_b again (the GEMMs read d_prenorm_lp), so their stores are skipped.
    // Only set together with colsum_partial.
    uint32_t lean;
    // Factor that brings the accumulators back to the scale of the reference's dY (the 16-bit copy of the
    // next layer's d_prenorm is stored scaled down by kLpScale): 1 in f32, 1 / kLpScale in 16-bit modes.
    float acc_scale;
    struct Acc { float dp[8], gw[8], gb[8]; };

    __device__ __forceinline__ uint32_t A() const { return ACT >= 0 ? (uint32_t)ACT : act; }
    __device__ __forceinline__ uint32_t Nm() const { return NORM >= 0 ? (uint32_t)NORM : norm; }

    __device__ __forceinline__ void one(uint32_t row, uint32_t col, float s) const {
        const size_t idx = (size_t)row * N + col;
        const float delta = to_f32(mask[idx]) *
                            activation_derivative(act, s * acc_scale, to_f32(predrop[idx]), to_f32(preact[idx]), leaky);
        grad[idx] = delta;
        const float r = norm ? to_f32(rstd[norm == 3 ? col : row]) : 0.0f;
        const float pv = norm == 1 ? to_f32(prenorm[idx]) : 0.0f;
        const float cv = norm >= 2 ? to_f32(centered[idx]) : 0.0f;
        const NormGrad g = norm_gradients(norm, delta, pv, cv, r, norm_w[col], inv_n, inv_m);
        d_prenorm[idx] = g.d_prenorm;
        d_norm_w[idx] = g.d_norm_w;
        d_norm_b[idx] = g.d_norm_b;
        if (d_prenorm_lp) d_prenorm_lp[idx] = from_f32<T>(g.d_prenorm * kLpScale);
    }

    // vector path on unpacked inputs of one run. nw: normalisation weights of the columns,
    // rs: rstd per column (BatchNorm) or the row's rstd in every slot (RMSNorm / LayerNorm).
    template <int V>
    __device__ __forceinline__ void core(uint32_t row, uint32_t col0, const float (&acc)[V], const float (&pd)[V],
                                         const float (&pa)[V], const float (&mk)[V], const float (&xv)[V],
                                         const float (&nw)[V], const float (&rs)[V], Acc *sums = nullptr) const {
        const size_t idx = (size_t)row * N + col0;
        float gr[V], dp[V], gw[V], gb[V];
#pragma unroll
        for (int j = 0; j < V; ++j) gr[j] = acc[j] * acc_scale;
        activation_derivative_v<kFastMath<T>, V>(A(), gr, pd, pa, leaky);
#pragma unroll
        for (int j = 0; j < V; ++j) gr[j] *= mk[j];
        if (Nm() == 0) {
#pragma unroll
            for (int j = 0; j < V; ++j) { dp[j] = gr[j]; gw[j] = 0.0f; gb[j] = 0.0f; }
        } else if (Nm() == 1) {
#pragma unroll
            for (int j = 0; j < V; ++j) {
                const float r = rs[j];
                gw[j] = gr[j] * xv[j] * r;
                gb[j] = 0.0f;
                dp[j] = nw[j] * r * (gr[j] - r * r * xv[j] * xv[j] * inv_n);
            }
        } else {
            const float inv = Nm() == 2 ? inv_n : inv_m;
#pragma unroll
            for (int j = 0; j < V; ++j) {
                const float r = rs[j];
                gb[j] = gr[j];
                gw[j] = gr[j] * xv[j] * r;
                dp[j] = nw[j] * r * (gr[j] - gr[j] * inv - r * r * xv[j] * xv[j] * gr[j] * inv);
            }
        }
        if (!lean) {
            store_run<float, V>(grad + idx, true, gr);
            store_run<float, V>(d_prenorm + idx, true, dp);
            store_run<float, V>(d_norm_w + idx, true, gw);
            store_run<float, V>(d_norm_b + idx, true, gb);
        }
        if (d_prenorm_lp) {
            float lp[V];
#pragma unroll
            for (int j = 0; j < V; ++j) lp[j] = dp[j] * kLpScale;
            store_run<T, V>(d_prenorm_lp + idx, true, lp);
        }
        if constexpr (V == 8) {
            if (sums && colsum_partial) {
#pragma unroll
                for (int j = 0; j < 8; ++j) { sums->dp[j] += dp[j]; sums->gw[j] += gw[j]; sums->gb[j] += gb[j]; }
            }
        }
    }

    template <int V>
    __device__ __forceinline__ void run(uint32_t row, uint32_t col0, const float (&acc)[V], uint32_t ncols) const {
        if (!(vec_ok && ncols == V)) {
            for (uint32_t j = 0; j < ncols; ++j) one(row, col0 + j, acc[j]);
            return;
        }
        const size_t idx = (size_t)row * N + col0;
        float pd[V], pa[V], mk[V], xv[V], nw[V], rs[V];
        load_run<T, V>(predrop + idx, true, pd);
        load_run<T, V>(preact + idx, true, pa);
        load_run<T, V>(mask + idx, true, mk);
        if (Nm() == 1) load_run<T, V>(prenorm + idx, true, xv);
        else if (Nm() >= 2) load_run<T, V>(centered + idx, true, xv);
        if (Nm()) load_run<float, V>(norm_w + col0, true, nw);
        if (Nm() == 3) load_run<T, V>(rstd + col0, true, rs);
        else if (Nm()) {
            const float r = to_f32(rstd[row]);
#pragma unroll
            for (int j = 0; j < V; ++j) rs[j] = r;
        }
        core<V>(row, col0, acc, pd, pa, mk, xv, nw, rs);
    }

    // the specialised kernels are small enough to be unrolled with two passes of loads in flight
    static constexpr bool kPingPong = ACT >= 0 && NORM >= 0;
    static constexpr int kGroup = kPingPong ? 2 : 1;
    struct Cols { float nw[8], rs[8]; };
    struct Pre { Pack<T, 8> pd, pa, mk, xv; T rrow; };
    static constexpr bool kHasAcc = ACT >= 0 && NORM >= 0;   // the generic functor has no registers to spare
    __device__ __forceinline__ void acc_init(Acc &a) const {
#pragma unroll
        for (int j = 0; j < 8; ++j) { a.dp[j] = 0.0f; a.gw[j] = 0.0f; a.gb[j] = 0.0f; }
    }
    // Called by all 32 lanes of the warp after the four passes of a chunk: lanes that hold the same
    // columns (equal lane % 4) add their rows up, lanes 0-3 store the sums of the 32-row group.
    __device__ __forceinline__ void acc_flush(Acc &a, uint32_t group, uint32_t col0, uint32_t lane, bool valid) const {
        if (!colsum_partial) return;
#pragma unroll
        for (int off = 4; off < 32; off <<= 1) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                a.dp[j] += __shfl_xor_sync(0xffffffffu, a.dp[j], off);
                if (Nm() >= 1) a.gw[j] += __shfl_xor_sync(0xffffffffu, a.gw[j], off);
                if (Nm() >= 2) a.gb[j] += __shfl_xor_sync(0xffffffffu, a.gb[j], off);
            }
        }
        if (valid && lane < 4 && group < colsum_groups) {
            float *base = colsum_partial + (size_t)group * 3 * N + col0;
            store_run<float, 8>(base, true, a.dp);
            store_run<float, 8>(base + N, true, a.gw);
            store_run<float, 8>(base + 2 * (size_t)N, true, a.gb);
        }
    }
    __device__ __forceinline__ void cols(uint32_t col0, Cols &c) const {
        if (Nm()) load_run<float, 8>(norm_w + col0, true, c.nw);
        if (Nm() == 3) load_run<T, 8>(rstd + col0, true, c.rs);
    }
    __device__ __forceinline__ void prefetch(uint32_t row, uint32_t col0, Pre &p) const {
        const size_t idx = (size_t)row * N + col0;
        p.pd = load_pack<T, 8>(predrop + idx);
        p.pa = load_pack<T, 8>(preact + idx);
        p.mk = load_pack<T, 8>(mask + idx);
        if (Nm() == 1) p.xv = load_pack<T, 8>(prenorm + idx);
        else if (Nm() >= 2) p.xv = load_pack<T, 8>(centered + idx);
        if (Nm() == 1 || Nm() == 2) p.rrow = rstd[row];
    }
    __device__ __forceinline__ void finish(uint32_t row, uint32_t col0, const float (&acc)[8], const Pre &p, const Cols &c) const {
        finish_impl(row, col0, acc, p, c, nullptr);
    }
    __device__ __forceinline__ void finish(uint32_t row, uint32_t col0, const float (&acc)[8], const Pre &p, const Cols &c,
                                           Acc &sums) const {
        finish_impl(row, col0, acc, p, c, &sums);
    }
    __device__ __forceinline__ void finish_impl(uint32_t row, uint32_t col0, const float (&acc)[8], const Pre &p, const Cols &c,
                                                Acc *sums) const {
        float pd[8], pa[8], mk[8], xv[8], rs[8];
        unpack<T, 8>(p.pd, pd);
        unpack<T, 8>(p.pa, pa);
        unpack<T, 8>(p.mk, mk);
        if (Nm()) unpack<T, 8>(p.xv, xv);
        if (Nm() == 3) {
#pragma unroll
            for (int j = 0; j < 8; ++j) rs[j] = c.rs[j];
        } else if (Nm()) {
            const float r = to_f32(p.rrow);
#pragma unroll
            for (int j = 0; j < 8; ++j) rs[j] = r;
        }
        core<8>(row, col0, acc, pd, pa, mk, xv, c.nw, rs, sums);
    }
};

// ---- weight gradient with the optimiser step fused in ------------------------------------------
// Reference: ffn/backward.cu:157-234 (dW part) with :105-154.
template <typename T, int KIND = -1, int REGU = -1> struct EpiWeightUpdate {
    T *w;
    float *master, *dv, *dm;   // master == (float*)w in f32 mode
    uint32_t N;
    float gscale;              // accumulator -> batch sum of the unscaled gradient: 1/512, over kLpScale when dY is the 16-bit copy
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
        for (int j = 0; j < V; ++j) p[j] = optimiser_step(p[j], v[j], m[j], acc[j] * gscale, opt, hyp, true);
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

    static constexpr bool kPingPong = KIND >= 0 && REGU >= 0;
    struct Cols {};
    struct Pre { Pack<float, 8> p, v, m; };
    __device__ __forceinline__ void cols(uint32_t, Cols &) const {}
    __device__ __forceinline__ void prefetch(uint32_t row, uint32_t col0, Pre &q) const {
        const size_t idx = (size_t)row * N + col0;
        q.p = load_pack<float, 8>(master + idx);
        q.v = load_pack<float, 8>(dv + idx);
        q.m = load_pack<float, 8>(dm + idx);
    }
    __device__ __forceinline__ void finish(uint32_t row, uint32_t col0, const float (&acc)[8], const Pre &q, const Cols &) const {
        const size_t idx = (size_t)row * N + col0;
        float p[8], v[8], m[8];
        unpack<float, 8>(q.p, p);
        unpack<float, 8>(q.v, v);
        unpack<float, 8>(q.m, m);
#pragma unroll
        for (int j = 0; j < 8; ++j) p[j] = optimiser_step_fast<KIND, REGU>(p[j], v[j], m[j], acc[j] * gscale, opt, hyp, true);
        store_run<float, 8>(dv + idx, true, v);
        store_run<float, 8>(dm + idx, true, m);
        store_run<float, 8>(master + idx, true, p);
        if ((void *)w != (void *)master) store_run<T, 8>(w + idx, true, p);
    }
};

// ---- plain f32 store (raw batch sums for the data-parallel exchange) ------------------------------
struct EpiStoreF32 {
    float *c;
    uint32_t N;
    float scale;   // 1, or 1 / kLpScale when dY is the 16-bit copy
    bool vec_ok;
    template <int V>
    __device__ __forceinline__ void run(uint32_t row, uint32_t col0, const float (&acc)[V], uint32_t ncols) const {
        const size_t idx = (size_t)row * N + col0;
        float v[V];
#pragma unroll
        for (int j = 0; j < V; ++j) v[j] = acc[j] * scale;
        if (vec_ok && ncols == V) store_run<float, V>(c + idx, true, v);
        else for (uint32_t j = 0; j < ncols; ++j) c[idx + j] = v[j];
    }

    struct Cols {};
    using Pre = NoPre;
    __device__ __forceinline__ void cols(uint32_t, Cols &) const {}
    __device__ __forceinline__ void prefetch(uint32_t, uint32_t, Pre &) const {}
    __device__ __forceinline__ void finish(uint32_t row, uint32_t col0, const float (&acc)[8], const Pre &, const Cols &) const {
        run<8>(row, col0, acc, 8);
    }
};

// ---- scaled store in the storage type (16-bit gradient payload of the data-parallel exchange) ----
template <typename T> struct EpiStoreScaled {
    T *c;
    uint32_t N;
    float scale;
    bool vec_ok;
    template <int V>
    __device__ __forceinline__ void run(uint32_t row, uint32_t col0, const float (&acc)[V], uint32_t ncols) const {
        const size_t idx = (size_t)row * N + col0;
        float v[V];
#pragma unroll
        for (int j = 0; j < V; ++j) v[j] = acc[j] * scale;
        if (vec_ok && ncols == V) store_run<T, V>(c + idx, true, v);
        else for (uint32_t j = 0; j < ncols; ++j) c[idx + j] = from_f32<T>(v[j]);
    }

    struct Cols {};
    using Pre = NoPre;
    __device__ __forceinline__ void cols(uint32_t, Cols &) const {}
    __device__ __forceinline__ void prefetch(uint32_t, uint32_t, Pre &) const {}
    __device__ __forceinline__ void finish(uint32_t row, uint32_t col0, const float (&acc)[8], const Pre &, const Cols &) const {
        run<8>(row, col0, acc, 8);
    }
};

constexpr int kMaxRanks = 8;   // ranks of one NVSwitch domain the fused exchange addresses

} // namespace sk
