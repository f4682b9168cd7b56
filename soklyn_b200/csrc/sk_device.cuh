// Device-side arithmetic shared by every kernel of the DenseBlock path: storage-type
// conversion, activations and their derivatives, the dropout hash, the per-element
// normalisation backward and the optimiser step. Formulas follow the reference
// (Felix1G/soklyn src/cuda/kernel/util.cu, math.cuh, ffn/backward.cu); the code is new.
#pragma once

#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

namespace sk {

constexpr float kLossScale = 512.0f;          // ffn/backward.cu:8
constexpr float kLossScaleInv = 1.0f / 512.0f;
// The 16-bit copy of d_prenorm that feeds the tensor-core GEMMs (d_prenorm_lp) holds d_prenorm * kLpScale,
// i.e. the delta at an effective loss scale of 32 instead of 512. The reference keeps d_prenorm in f32
// (src/mlp.rs:273-276), where the factor 512 costs nothing; in f16 it overflows (|delta| * 512 > 65504 from
// |delta| = 128 on, which the wide network reaches at its first step), and infinities in dY poison dW and
// every delta below. A power of two, so the copy loses no precision; the consumers multiply it back.
constexpr float kLpScale = 1.0f / 16.0f;
constexpr float kLpScaleInv = 16.0f;

// ---- storage types -------------------------------------------------------------------
__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Value after a round trip through the storage type (what a later kernel of the
// reference would read back from memory).
template <typename T> __device__ __forceinline__ float round_to(float v) { return to_f32(from_f32<T>(v)); }

// Product in the storage type's own arithmetic (the reference's RMSNorm multiplies in T).
__device__ __forceinline__ float mul_t(float a, float b) { return a * b; }
__device__ __forceinline__ __half mul_t(__half a, __half b) { return __hmul(a, b); }
__device__ __forceinline__ __nv_bfloat16 mul_t(__nv_bfloat16 a, __nv_bfloat16 b) { return __hmul(a, b); }

// ---- activations: util.cu:8-47 ---------------------------------------------------------
__device__ __forceinline__ float activation(uint32_t act, float x, float leaky) {
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
    default: return x;
    }
}

// delta * act'(.) from the stored activation output and input: util.cu:49-93
__device__ __forceinline__ float activation_derivative(uint32_t act, float delta, float out_v, float in_x, float leaky) {
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

// ---- the same on runs of V values, with the mode switch outside the element loop --------
// FAST selects the hardware approximations (ex2/lg2/rcp.approx, ~2^-21 relative) in place of
// the IEEE library routines. It is used only where results are stored in a 16-bit type,
// whose own rounding (2^-11 / 2^-8) is far coarser.
template <bool FAST> __device__ __forceinline__ float x_exp(float x) { return FAST ? __expf(x) : expf(x); }
template <bool FAST> __device__ __forceinline__ float x_log(float x) { return FAST ? __logf(x) : logf(x); }
template <bool FAST> __device__ __forceinline__ float x_div(float a, float b) { return FAST ? __fdividef(a, b) : a / b; }
template <bool FAST> __device__ __forceinline__ float x_tanh(float x) {
    if (!FAST) return tanhf(x);
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <bool FAST, int V>
__device__ __forceinline__ void activation_v(uint32_t act, const float (&x)[V], float (&y)[V], float leaky) {
    switch (act) {
    case 1:
#pragma unroll
        for (int j = 0; j < V; ++j) y[j] = x_div<FAST>(1.0f, 1.0f + x_exp<FAST>(-x[j]));
        break;
    case 2:
#pragma unroll
        for (int j = 0; j < V; ++j) y[j] = fmaxf(0.0f, x[j]);
        break;
    case 3:
#pragma unroll
        for (int j = 0; j < V; ++j) y[j] = x[j] > 0.0f ? x[j] : leaky * x[j];
        break;
    case 4:
#pragma unroll
        for (int j = 0; j < V; ++j) y[j] = x_tanh<FAST>(x[j]);
        break;
    case 6:
#pragma unroll
        for (int j = 0; j < V; ++j) y[j] = x_div<FAST>(x[j], 1.0f + x_exp<FAST>(-x[j]));
        break;
    case 7:
#pragma unroll
        for (int j = 0; j < V; ++j) {
            const float ex = x_exp<FAST>(x[j]);
            const float sp = x[j] > 20.0f ? x[j] : x_log<FAST>(1.0f + ex);
            const float es = x_exp<FAST>(sp), esi = x_div<FAST>(1.0f, es);
            y[j] = x[j] * x_div<FAST>(es - esi, es + esi);
        }
        break;
    default:
#pragma unroll
        for (int j = 0; j < V; ++j) y[j] = x[j];
        break;
    }
}

// d[j] <- d[j] * act'(.) from the stored activation output and input
template <bool FAST, int V>
__device__ __forceinline__ void activation_derivative_v(uint32_t act, float (&d)[V], const float (&out_v)[V],
                                                        const float (&in_x)[V], float leaky) {
    switch (act) {
    case 1:
#pragma unroll
        for (int j = 0; j < V; ++j) d[j] *= out_v[j] * (1.0f - out_v[j]);
        break;
    case 2:
#pragma unroll
        for (int j = 0; j < V; ++j) d[j] *= out_v[j] > 0.0f ? 1.0f : 0.0f;
        break;
    case 3:
#pragma unroll
        for (int j = 0; j < V; ++j) d[j] *= out_v[j] > 0.0f ? 1.0f : leaky;
        break;
    case 4:
#pragma unroll
        for (int j = 0; j < V; ++j) d[j] *= 1.0f - out_v[j] * out_v[j];
        break;
    case 6:
#pragma unroll
        for (int j = 0; j < V; ++j) {
            const float sg = x_div<FAST>(1.0f, 1.0f + x_exp<FAST>(-in_x[j]));
            d[j] *= sg + out_v[j] * (1.0f - sg);
        }
        break;
    case 7:
#pragma unroll
        for (int j = 0; j < V; ++j) {
            const float ex = x_exp<FAST>(in_x[j]);
            const float sp = in_x[j] > 20.0f ? in_x[j] : x_log<FAST>(1.0f + ex);
            const float es = x_exp<FAST>(sp), esi = x_div<FAST>(1.0f, es);
            const float th = x_div<FAST>(es - esi, es + esi);
            const float sg = x_div<FAST>(ex, 1.0f + ex);
            d[j] *= th + in_x[j] * sg * (1.0f - th * th);
        }
        break;
    default: break;
    }
}

// ---- dropout hash: math.cuh:45-53; the result must match bit for bit -----------------------
__device__ __forceinline__ float dropout_uniform(uint32_t col, uint32_t row, uint32_t seed) {
    uint32_t s = (row * 1103515245u) ^ (col * 0x4C957F2Du) ^ seed;
    s ^= s >> 17;
    s = s * 1103515245u + 12345u;
    s ^= s >> 15;
    return __uint2float_rn(s) * 2.3283064365386963e-10f; // exact division by 2^32
}

// keep decision of forward.cu:148-156 for global row `grow`
__device__ __forceinline__ bool dropout_keep(uint32_t col, uint32_t grow, uint32_t seed, float mask_coeff) {
    return dropout_uniform(col, grow, seed + grow * 7u) >= mask_coeff;
}

// ---- normalisation backward, element-wise: util.cu:175-215 -----------------------------
struct NormGrad { float d_prenorm, d_norm_w, d_norm_b; };

__device__ __forceinline__ NormGrad norm_gradients(uint32_t norm, float delta, float prenorm_v, float centered_v,
                                                   float rstd, float n_w, float inv_n, float inv_m) {
    NormGrad g{delta, 0.0f, 0.0f};
    if (norm == 1) {
        g.d_norm_w = delta * prenorm_v * rstd;
        g.d_prenorm = n_w * rstd * (delta - rstd * rstd * prenorm_v * prenorm_v * inv_n);
    } else if (norm == 2 || norm == 3) {
        const float inv = norm == 2 ? inv_n : inv_m;
        g.d_norm_b = delta;
        g.d_norm_w = delta * centered_v * rstd;
        g.d_prenorm = n_w * rstd * (delta - delta * inv - rstd * rstd * centered_v * centered_v * delta * inv);
    }
    return g;
}

// ---- optimiser: ffn/backward.cu:105-154 ---------------------------------------------------
struct Optim {
    uint32_t kind;       // 0 SGD, 1 Adam
    float beta1, beta2, epsilon;
    uint32_t nesterov;
    float bc1, bc2;      // 1 - beta^step, computed once on the host with powf
    float inv_bc1, inv_bc2;
};

struct Hyper {
    float lr, clamp, inv_m;
    uint32_t regu;
    float regu_coeff;
};

// One parameter step. `acc` is the batch sum divided by the loss scale. Returns the new
// master value; m/v are updated in place.
__device__ __forceinline__ float optimiser_step(float p, float &v, float &mo, float acc, const Optim &o,
                                                const Hyper &h, bool apply_regu) {
    const float g = acc * h.inv_m;
    if (apply_regu) {
        const float sign = p > 0.0f ? 1.0f : (p < 0.0f ? -1.0f : 0.0f);
        if (h.regu == 1) p -= h.regu_coeff * sign;
        if (h.regu == 2) p -= 2.0f * h.regu_coeff * p;
    }
    if (o.kind == 0) {
        v = o.beta1 * v + g;
        float u = h.lr * (o.nesterov ? g + o.beta1 * v : v);
        u = fminf(fmaxf(u, -h.clamp), h.clamp);
        p -= u;
    } else if (o.kind == 1) {
        mo = o.beta1 * mo + (1.0f - o.beta1) * g;
        v = o.beta2 * v + (1.0f - o.beta2) * g * g;
        const float mc = mo / o.bc1;
        const float vc = v / o.bc2;
        float u = h.lr * (mc / (sqrtf(vc) + o.epsilon));
        u = fminf(fmaxf(u, -h.clamp), h.clamp);
        p -= u;
    }
    return p;
}

__device__ __forceinline__ float sqrt_approx(float x) {
    float y;
    asm("sqrt.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// The same step with the two bias corrections as multiplications by host-side reciprocals and
// the final quotient through rcp/sqrt approximations (relative error ~1e-7 on the update).
// KIND / REGU >= 0 fix the optimiser and the regularisation at compile time (the kernels that
// are specialised for the common cases), -1 reads them from the arguments.
template <int KIND = -1, int REGU = -1>
__device__ __forceinline__ float optimiser_step_fast(float p, float &v, float &mo, float acc, const Optim &o,
                                                     const Hyper &h, bool apply_regu) {
    const float g = acc * h.inv_m;
    const uint32_t regu = REGU >= 0 ? (uint32_t)REGU : h.regu;
    const uint32_t kind = KIND >= 0 ? (uint32_t)KIND : o.kind;
    if (apply_regu && regu) {
        const float sign = p > 0.0f ? 1.0f : (p < 0.0f ? -1.0f : 0.0f);
        if (regu == 1) p -= h.regu_coeff * sign;
        if (regu == 2) p -= 2.0f * h.regu_coeff * p;
    }
    float u;
    if (kind == 0) {
        v = o.beta1 * v + g;
        u = h.lr * (o.nesterov ? g + o.beta1 * v : v);
    } else {
        mo = o.beta1 * mo + (1.0f - o.beta1) * g;
        v = o.beta2 * v + (1.0f - o.beta2) * g * g;
        u = h.lr * __fdividef(mo * o.inv_bc1, sqrt_approx(v * o.inv_bc2) + o.epsilon);
    }
    u = fminf(fmaxf(u, -h.clamp), h.clamp);
    return p - u;
}

// ---- warp / block reductions ------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// Sum over a block of up to 1024 threads; every thread gets the total. `red` holds 32 floats.
__device__ __forceinline__ float block_sum(float v, float *red) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads(); // protect `red` from the previous use
    if (lane == 0) red[wid] = v;
    __syncthreads();
    float t = lane < nw ? red[lane] : 0.0f;
    return warp_sum(t);
}

} // namespace sk
