/*
 * CPU restatement of Soklyn's DenseBlock / FeedForwardNetwork arithmetic, f32 only.
 *
 * TEST INFRASTRUCTURE, NOT PRODUCT: this file is the parity checker and the timed
 * CPU baseline. Nothing under soklyn_b200/ may call it; the shipped path is CUDA only.
 *
 * Each function names the reference source it follows (paths inside Felix1G/soklyn).
 * The reference has no CPU path and no numeric test vectors for this code, so the
 * restatement is pinned by running the reference's own CUDA kernels (built from the
 * reference tree into oracle/_ref, see ref_runner.cu) and by the vectors those kernels
 * produced, stored under tests/golden/.
 *
 * All matrices are row-major. "threads" is the reference block size (tile_dim^2, 256
 * for tile_dim 16); the strided partial sums + tree reduction of the reference are
 * reproduced so that the f32 rounding order of row/column statistics is the same.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define OK_MAX_THREADS 1024
#define OK_LOSS_SCALE 512.0f

/* src/util/core.rs:90-94 — per-step, per-layer dropout seed. */
uint32_t ok_scramble_seed(uint32_t step, uint32_t layer_id) {
    uint32_t h = step * 1103515245u + layer_id;
    h = (h ^ (h >> 16)) * 1103515245u;
    return h ^ (h >> 15);
}

/* src/cuda/kernel/math.cuh:45-53 — integer hash to a uniform in [0,1].
 * The 64-bit multiplier only contributes its low word once the state is
 * truncated to 32 bits. */
float ok_rand(uint32_t col, uint32_t row, uint32_t seed) {
    uint32_t s = (row * 1103515245u) ^ (col * 0x4C957F2Du) ^ seed;
    s ^= s >> 17;
    s = s * 1103515245u + 12345u;
    s ^= s >> 15;
    return (float)s / 4294967296.0f; /* float(0xFFFFFFFF) rounds to 2^32 */
}

/* src/cuda/kernel/util.cu:8-47 */
float ok_activation(uint32_t act, float x, float leaky) {
    switch (act) {
    case 1: return 1.0f / (1.0f + expf(-x));
    case 2: return fmaxf(0.0f, x);
    case 3: return x > 0.0f ? x : leaky * x;
    case 4: return tanhf(x);
    case 6: return x / (1.0f + expf(-x));
    case 7: {
        const float ex = expf(x);
        const float sp = x > 20.0f ? x : logf(1.0f + ex);
        const float es = expf(sp), esi = 1.0f / es;
        return x * ((es - esi) / (es + esi));
    }
    default: return x; /* 0 identity, 5 softmax (handled by ok_softmax) */
    }
}

/* src/cuda/kernel/util.cu:49-93 — delta times act'(.), using the stored
 * activation output (out_v) and the activation input (in_x). */
float ok_activation_derivative(uint32_t act, float delta, float out_v, float in_x, float leaky) {
    switch (act) {
    case 1: return delta * (out_v * (1.0f - out_v));
    case 2: return delta * (out_v > 0.0f ? 1.0f : 0.0f);
    case 3: return delta * (out_v > 0.0f ? 1.0f : leaky);
    case 4: return delta * (1.0f - out_v * out_v);
    case 6: {
        const float sg = 1.0f / (1.0f + expf(-in_x));
        return delta * (sg + out_v * (1.0f - sg));
    }
    case 7: {
        const float ex = expf(in_x);
        const float sp = in_x > 20.0f ? in_x : logf(1.0f + ex);
        const float es = expf(sp), esi = 1.0f / es;
        const float th = (es - esi) / (es + esi);
        const float sg = ex / (1.0f + ex);
        return delta * (th + in_x * sg * (1.0f - th * th));
    }
    default: return delta;
    }
}

/* Strided partial sums followed by the halving tree of
 * src/cuda/kernel/util.cuh:33-41 (blockDim.x = threads, a power of two). */
static float ok_tree_sum(float *part, uint32_t threads) {
    for (uint32_t s = threads >> 1; s > 0; s >>= 1)
        for (uint32_t t = 0; t < s; ++t) part[t] += part[t + s];
    return part[0];
}

/* src/cuda/kernel/ffn/forward.cu:8-28 with math.cu:8-50 — Z = X.W (+ b),
 * one fused-multiply-add chain per output in increasing k. */
void ok_forward_pass_0(float *z, const float *x, const float *w, const float *b,
                       uint32_t use_bias, uint32_t m, uint32_t n, uint32_t wc) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < (int64_t)m; ++r) {
        float *acc = (float *)calloc(wc, sizeof(float));
        const float *xr = x + (size_t)r * n;
        for (uint32_t k = 0; k < n; ++k) {
            const float a = xr[k];
            const float *wk = w + (size_t)k * wc;
            for (uint32_t c = 0; c < wc; ++c) acc[c] = fmaf(a, wk[c], acc[c]);
        }
        float *zr = z + (size_t)r * wc;
        for (uint32_t c = 0; c < wc; ++c) zr[c] = use_bias ? acc[c] + b[c] : acc[c];
        free(acc);
    }
}

/* src/cuda/kernel/ffn/forward.cu:31-127 — normalisation: 1 RMSNorm and 2 LayerNorm
 * reduce over the features of one row, 3 BatchNorm over the batch of one column.
 * Writes centered, preact and rstd (indexed by row, or by column for BatchNorm). */
void ok_forward_pass_1(float *preact, float *centered, const float *prenorm,
                       const float *norm_w, const float *norm_b, float *rstd_out,
                       uint32_t m, uint32_t wc, uint32_t norm, uint32_t threads) {
    if (threads == 0 || threads > OK_MAX_THREADS) threads = 256;
    const uint32_t groups = norm == 3 ? wc : m;
    const uint32_t len = norm == 3 ? m : wc;
#pragma omp parallel for schedule(static)
    for (int64_t g = 0; g < (int64_t)groups; ++g) {
        float part[OK_MAX_THREADS];
        const size_t base = norm == 3 ? (size_t)g : (size_t)g * wc;
        const size_t step = norm == 3 ? wc : 1;
        if (norm == 1) {
            for (uint32_t t = 0; t < threads; ++t) {
                float s = 0.0f;
                for (uint32_t i = t; i < len; i += threads) {
                    const float v = prenorm[base + i * step];
                    s += v * v;
                }
                part[t] = s;
            }
            const float var = ok_tree_sum(part, threads) / (float)len + 1e-6f;
            const float rstd = 1.0f / sqrtf(var);
            rstd_out[g] = rstd;
            for (uint32_t i = 0; i < len; ++i) {
                const size_t idx = base + i * step;
                centered[idx] = prenorm[idx];
                preact[idx] = prenorm[idx] * rstd * norm_w[i];
            }
        } else if (norm == 2 || norm == 3) {
            for (uint32_t t = 0; t < threads; ++t) {
                float s = 0.0f;
                for (uint32_t i = t; i < len; i += threads) s += prenorm[base + i * step];
                part[t] = s;
            }
            const float mean = ok_tree_sum(part, threads) / (float)len;
            for (uint32_t t = 0; t < threads; ++t) {
                float s = 0.0f;
                for (uint32_t i = t; i < len; i += threads) {
                    const float v = prenorm[base + i * step] - mean;
                    s += v * v;
                }
                part[t] = s;
            }
            const float var = ok_tree_sum(part, threads) / (float)len + 1e-6f;
            const float rstd = 1.0f / sqrtf(var);
            rstd_out[g] = rstd;
            for (uint32_t i = 0; i < len; ++i) {
                const size_t idx = base + i * step;
                const uint32_t col = norm == 2 ? i : (uint32_t)g;
                const float c = prenorm[idx] - mean;
                centered[idx] = c;
                preact[idx] = c * rstd * norm_w[col] + norm_b[col];
            }
        }
    }
}

/* src/cuda/kernel/ffn/forward.cu:130-161 — activation then inverted dropout.
 * row_offset is added to the row used by the hash so that a batch shard
 * reproduces the mask of the whole batch (0 for the single-device reference).
 * With use_dropout == 0 the mask is left untouched. */
void ok_forward_pass_2(float *out, float *predrop, const float *preact, float *mask,
                       uint32_t m, uint32_t n, uint32_t act, float leaky,
                       uint32_t use_dropout, float mask_coeff, uint32_t seed, uint32_t row_offset) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < (int64_t)m; ++r) {
        const uint32_t grow = (uint32_t)r + row_offset;
        for (uint32_t c = 0; c < n; ++c) {
            const size_t idx = (size_t)r * n + c;
            const float a = ok_activation(act, preact[idx], leaky);
            predrop[idx] = a;
            if (use_dropout) {
                if (ok_rand(c, grow, seed + grow * 7u) >= mask_coeff) {
                    const float scale = 1.0f / (1.0f - mask_coeff);
                    mask[idx] = scale;
                    out[idx] = a * scale;
                } else {
                    mask[idx] = 0.0f;
                    out[idx] = 0.0f;
                }
            } else {
                out[idx] = a;
            }
        }
    }
}

/* src/cuda/kernel/util.cu:95-173 — in-place row softmax. The partial sums are
 * strided over `threads` lanes, folded with the shuffle-down tree inside each
 * warp of 32 and then across warps, as the reference does. */
void ok_softmax(float *out, uint32_t m, uint32_t n, uint32_t threads) {
    if (threads == 0 || threads > OK_MAX_THREADS) threads = 256;
    const uint32_t warps = threads / 32;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < (int64_t)m; ++r) {
        float *row = out + (size_t)r * n;
        float mx = -INFINITY;
        for (uint32_t c = 0; c < n; ++c) mx = fmaxf(mx, row[c]);
        float part[OK_MAX_THREADS];
        for (uint32_t t = 0; t < threads; ++t) {
            float s = 0.0f;
            for (uint32_t c = t; c < n; c += threads) s += expf(row[c] - mx);
            part[t] = s;
        }
        float wsum[32];
        for (uint32_t w = 0; w < 32; ++w) wsum[w] = 0.0f;
        for (uint32_t w = 0; w < warps; ++w) {
            float *l = part + w * 32;
            for (uint32_t off = 16; off > 0; off >>= 1)
                for (uint32_t i = 0; i < off; ++i) l[i] += l[i + off];
            wsum[w] = l[0];
        }
        for (uint32_t off = 16; off > 0; off >>= 1)
            for (uint32_t i = 0; i < off; ++i) wsum[i] += wsum[i + off];
        const float total = wsum[0];
        for (uint32_t c = 0; c < n; ++c) row[c] = expf(row[c] - mx) / total;
    }
}

/* src/cuda/kernel/util.cu:175-215 — per-element normalisation backward. */
static inline void ok_norm_gradients(float *d_prenorm, float *dnw, float *dnb,
                                     const float *centered, const float *prenorm, float rstd,
                                     float delta, float n_w, float loss_scale, uint32_t norm,
                                     size_t idx, float inv_n, float inv_m) {
    float gw = 0.0f, gb = 0.0f, d = delta;
    if (norm == 1) {
        const float p = prenorm[idx];
        gw = delta * p * rstd;
        d = n_w * rstd * (delta - rstd * rstd * p * p * inv_n);
    } else if (norm == 2 || norm == 3) {
        const float c = centered[idx];
        const float inv = norm == 2 ? inv_n : inv_m;
        gb = delta;
        gw = delta * c * rstd;
        d = n_w * rstd * (delta - delta * inv - rstd * rstd * c * c * delta * inv);
    }
    d_prenorm[idx] = d * loss_scale;
    dnw[idx] = gw;
    dnb[idx] = gb;
}

/* src/cuda/kernel/ffn/backward.cu:12-56 — output-layer delta. err_mode 0 MSE,
 * 1 cross-entropy (needs act 5), 2 binary cross-entropy (needs act 1).
 * `out` already holds the softmax when act == 5. d_prenorm carries x512. */
void ok_output_error(const float *out, const float *preact, const float *target,
                     const float *master_norm_w, float *grad, float *d_prenorm,
                     float *dnw, float *dnb, const float *rstd, const float *centered,
                     const float *prenorm, uint32_t m, uint32_t n, uint32_t err_mode,
                     uint32_t norm, uint32_t act, float leaky) {
    const float inv_m = 1.0f / (float)m, inv_n = 1.0f / (float)n;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < (int64_t)m; ++r) {
        for (uint32_t c = 0; c < n; ++c) {
            const size_t idx = (size_t)r * n + c;
            const float o = ok_activation(act, out[idx], leaky);
            float delta = 0.0f;
            if (err_mode == 0)
                delta = ok_activation_derivative(act, o - target[idx], o, preact[idx], leaky);
            else if ((err_mode == 1 && act == 5) || (err_mode == 2 && act == 1))
                delta = o - target[idx];
            grad[idx] = delta;
            ok_norm_gradients(d_prenorm, dnw, dnb, centered, prenorm,
                              rstd[norm == 3 ? c : (uint32_t)r], delta, master_norm_w[c],
                              OK_LOSS_SCALE, norm, idx, inv_n, inv_m);
        }
    }
}

/* src/cuda/kernel/ffn/backward.cu:59-102 — hidden-layer delta:
 * S = dY_next . W_next^T (increasing k), times act', times mask, then the
 * normalisation backward with loss scale 1. inv_m uses m_stat (the whole batch
 * when rows are sharded; equal to m for the single-device reference). */
void ok_hidden_error(const float *next_d_prenorm, const float *w_next, const float *master_norm_w,
                     float *grad, float *d_prenorm, float *dnw, float *dnb,
                     const float *rstd, const float *centered, const float *prenorm,
                     const float *predrop, const float *preact, const float *mask,
                     uint32_t m, uint32_t n, uint32_t ec, uint32_t norm, uint32_t act,
                     float leaky, uint32_t m_stat) {
    const float inv_m = 1.0f / (float)m_stat, inv_n = 1.0f / (float)n;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < (int64_t)m; ++r) {
        const float *dy = next_d_prenorm + (size_t)r * ec;
        for (uint32_t c = 0; c < n; ++c) {
            const float *wr = w_next + (size_t)c * ec;
            float s = 0.0f;
            for (uint32_t k = 0; k < ec; ++k) s = fmaf(dy[k], wr[k], s);
            const size_t idx = (size_t)r * n + c;
            const float delta = mask[idx] * ok_activation_derivative(act, s, predrop[idx], preact[idx], leaky);
            grad[idx] = delta;
            ok_norm_gradients(d_prenorm, dnw, dnb, centered, prenorm,
                              rstd[norm == 3 ? c : (uint32_t)r], delta, master_norm_w[c],
                              1.0f, norm, idx, inv_n, inv_m);
        }
    }
}

/* Optimiser hyper-parameters of one parameter group (src/util/function.rs:76-116:
 * ordinal 0 = SGD{v_coeff -> beta1, nesterov}, 1 = Adam{m_coeff -> beta1,
 * v_coeff -> beta2, epsilon}), packed as src/io/device/ffn_device.rs:254-269 does. */
typedef struct {
    uint32_t kind;
    float beta1, beta2, epsilon;
    uint32_t nesterov;
} ok_optim;

/* src/cuda/kernel/ffn/backward.cu:105-154 — one parameter update.
 * acc is the batch sum already divided by the loss scale. */
static inline void ok_update_param(float *param, float *dv, float *dm, size_t idx, float acc,
                                   float inv_m, float lr, float clamp, const ok_optim *o,
                                   uint32_t step, uint32_t regu, float regu_coeff, int apply_regu) {
    float p = param[idx], v = dv[idx], mo = dm[idx];
    const float g = acc * inv_m;
    if (apply_regu) {
        const float sign = p > 0.0f ? 1.0f : (p < 0.0f ? -1.0f : 0.0f);
        if (regu == 1) p -= regu_coeff * sign;
        if (regu == 2) p -= 2.0f * regu_coeff * p;
    }
    if (o->kind == 0) {
        v = o->beta1 * v + g;
        float u = lr * (o->nesterov ? g + o->beta1 * v : v);
        u = fminf(fmaxf(u, -clamp), clamp);
        p -= u;
    } else if (o->kind == 1) {
        mo = o->beta1 * mo + (1.0f - o->beta1) * g;
        v = o->beta2 * v + (1.0f - o->beta2) * g * g;
        const float mc = mo / (1.0f - powf(o->beta1, (float)step));
        const float vc = v / (1.0f - powf(o->beta2, (float)step));
        float u = lr * (mc / (sqrtf(vc) + o->epsilon));
        u = fminf(fmaxf(u, -clamp), clamp);
        p -= u;
    }
    param[idx] = p;
    dv[idx] = v;
    dm[idx] = mo;
}

/* Batch sums only (no update): dW = X^T . dY in increasing batch order, and the
 * column sums of dY, dNorm_w, dNorm_b. Used by the data-parallel checks, where the
 * sums of all shards are added before one update. Any output may be NULL. */
void ok_grad_sums(const float *x, const float *d_prenorm, const float *dnw, const float *dnb,
                  float *dw, float *db, float *sum_nw, float *sum_nb,
                  uint32_t m, uint32_t n, uint32_t wr) {
    if (dw) {
#pragma omp parallel for schedule(static)
        for (int64_t r = 0; r < (int64_t)wr; ++r) {
            float *acc = dw + (size_t)r * n;
            for (uint32_t c = 0; c < n; ++c) acc[c] = 0.0f;
            for (uint32_t bi = 0; bi < m; ++bi) {
                const float a = x[(size_t)bi * wr + r];
                const float *dy = d_prenorm + (size_t)bi * n;
                for (uint32_t c = 0; c < n; ++c) acc[c] = fmaf(a, dy[c], acc[c]);
            }
        }
    }
    for (uint32_t c = 0; c < n; ++c) {
        float sb = 0.0f, sw = 0.0f, sn = 0.0f;
        for (uint32_t bi = 0; bi < m; ++bi) {
            const size_t i = (size_t)bi * n + c;
            sb += d_prenorm[i];
            if (dnw) sw += dnw[i];
            if (dnb) sn += dnb[i];
        }
        if (db) db[c] = sb;
        if (sum_nw) sum_nw[c] = sw;
        if (sum_nb) sum_nb[c] = sn;
    }
}

/* Apply the optimiser to precomputed batch sums (same arithmetic as the tail of
 * src/cuda/kernel/ffn/backward.cu:196-233). m_stat is the divisor (whole batch). */
void ok_apply_sums(float *w, float *b, float *dv_w, float *dv_b, float *dm_w, float *dm_b,
                   float *norm_w, float *norm_b, float *dv_nw, float *dv_nb, float *dm_nw, float *dm_nb,
                   const float *dw, const float *db, const float *sum_nw, const float *sum_nb,
                   uint32_t use_bias, uint32_t norm, uint32_t m_stat, uint32_t n, uint32_t wr,
                   float lr, float clamp, const ok_optim *lin, const ok_optim *nrm,
                   uint32_t regu, float regu_coeff, uint32_t step) {
    const float inv_m = 1.0f / (float)m_stat;
    const float inv_ls = 1.0f / OK_LOSS_SCALE;
    for (uint32_t c = 0; c < n; ++c) {
        if (use_bias)
            ok_update_param(b, dv_b, dm_b, c, db[c] * inv_ls, inv_m, lr, clamp, lin, step, regu, regu_coeff, 0);
        if (norm > 0) {
            ok_update_param(norm_w, dv_nw, dm_nw, c, sum_nw[c] * inv_ls, inv_m, lr, clamp, nrm, step, regu, regu_coeff, 0);
            if (norm > 1)
                ok_update_param(norm_b, dv_nb, dm_nb, c, sum_nb[c] * inv_ls, inv_m, lr, clamp, nrm, step, regu, regu_coeff, 0);
        }
    }
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < (int64_t)wr; ++r)
        for (uint32_t c = 0; c < n; ++c) {
            const size_t idx = (size_t)r * n + c;
            ok_update_param(w, dv_w, dm_w, idx, dw[idx] * inv_ls, inv_m, lr, clamp, lin, step, regu, regu_coeff, 1);
        }
}

/* src/cuda/kernel/ffn/backward.cu:157-234 — weight gradient, bias / norm-parameter
 * gradients and the in-place optimiser step of one layer. In f32 mode the reference
 * passes the parameters themselves as their "master" copy, as done here. */
void ok_backward_pass(const float *x, float *w, float *b, const float *d_prenorm,
                      float *dv_w, float *dv_b, float *dm_w, float *dm_b,
                      float *norm_w, float *norm_b, const float *dnw, const float *dnb,
                      float *dv_nw, float *dv_nb, float *dm_nw, float *dm_nb,
                      uint32_t use_bias, uint32_t norm, uint32_t m, uint32_t n, uint32_t wr,
                      float lr, float clamp, const ok_optim *lin, const ok_optim *nrm,
                      uint32_t regu, float regu_coeff, uint32_t step) {
    float *dw = (float *)malloc((size_t)wr * n * sizeof(float));
    float *cs = (float *)malloc((size_t)3 * n * sizeof(float));
    ok_grad_sums(x, d_prenorm, norm > 0 ? dnw : NULL, norm > 1 ? dnb : NULL,
                 dw, cs, cs + n, cs + 2 * (size_t)n, m, n, wr);
    ok_apply_sums(w, b, dv_w, dv_b, dm_w, dm_b, norm_w, norm_b, dv_nw, dv_nb, dm_nw, dm_nb,
                  dw, cs, cs + n, cs + 2 * (size_t)n, use_bias, norm, m, n, wr,
                  lr, clamp, lin, nrm, regu, regu_coeff, step);
    free(dw);
    free(cs);
}

/* Fill and the f32 <-> f16 casts of src/cuda/kernel/util.cuh:9-19 are exercised
 * through numpy in the tests (IEEE round-to-nearest-even on both sides). */
