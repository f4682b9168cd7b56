/*
 * Launcher for the REFERENCE's own CUDA kernels (Felix1G/soklyn src/cuda/nn_math.cu),
 * used to pin the CPU oracle and as the "reference" arm of the benchmark.
 *
 * TEST INFRASTRUCTURE, NOT PRODUCT. oracle/build_ref.py compiles the reference's
 * nn_math.cu, unmodified and where it lies in the reference tree, to compute_75 PTX
 * (the same target as the reference's build.rs:15-18) into oracle/_ref/nn_math.ptx.
 * Like the reference (src/io/device.rs:62-107) this file loads that PTX as a module
 * and looks the kernels up by name; it then restates the host glue of
 * src/io/device/ffn_device.rs: which kernel, which arguments, which grid / block /
 * shared memory, and the stream synchronisation after every launch. It takes the same
 * block descriptor as the product library so that one harness can drive both.
 */
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <string>
#include <vector>
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "../include/soklyn_b200.h"

namespace {
CUmodule g_module = nullptr;
std::map<std::string, CUfunction> g_funcs;
cudaStream_t g_stream = nullptr;
int g_sync = 1;       /* the reference synchronises after every launch */
uint32_t g_tile = 16; /* GpuContext tile_dim */
unsigned long long g_launches = 0;

struct Dim { uint32_t x, y; };

/* calculate_cfg2d, src/io/device.rs:211-221 */
inline Dim grid2d(uint32_t x, uint32_t y) { return Dim{(x + g_tile - 1) / g_tile, (y + g_tile - 1) / g_tile}; }
inline Dim block2d() { return Dim{g_tile, g_tile}; }

/* scramble_seed, src/util/core.rs:90-94 */
inline uint32_t scramble(uint32_t step, uint32_t id) {
    uint32_t h = step * 1103515245u + id;
    h = (h ^ (h >> 16)) * 1103515245u;
    return h ^ (h >> 15);
}

/* master_tensor, src/io/device.rs:262-272 */
inline const void *master(const float *m, const void *fallback) { return m ? (const void *)m : fallback; }

template <typename... A>
int launch(const char *name, Dim grid, Dim block, uint32_t smem, bool sync, A... a) {
    auto it = g_funcs.find(name);
    if (it == g_funcs.end()) {
        CUfunction f;
        if (!g_module || cuModuleGetFunction(&f, g_module, name) != CUDA_SUCCESS) {
            fprintf(stderr, "ref_runner: kernel %s not found\n", name);
            return SK_ERR_DRIVER;
        }
        it = g_funcs.emplace(name, f).first;
    }
    void *args[] = {(void *)&a...};
    CUresult r = cuLaunchKernel(it->second, grid.x, grid.y, 1, block.x, block.y, 1, smem, (CUstream)g_stream, args, nullptr);
    ++g_launches;
    if (r == CUDA_SUCCESS && sync && g_sync) r = cuStreamSynchronize((CUstream)g_stream);
    if (r != CUDA_SUCCESS) {
        const char *s = nullptr;
        cuGetErrorString(r, &s);
        fprintf(stderr, "ref_runner: %s: %s\n", name, s ? s : "?");
        return SK_ERR_DRIVER;
    }
    return SK_OK;
}

/* gpu_broadcast, src/io/device/util_device.rs:49-78 (no synchronisation after it) */
int fill_f32(float *dst, float v, size_t len) {
    const uint32_t t2 = g_tile * g_tile;
    return launch("broadcast_kernel_f32", Dim{(uint32_t)((len + t2 - 1) / t2), 1}, Dim{t2, 1}, 0, false, dst, v, (uint32_t)len);
}
} // namespace

extern "C" {

/* Load the PTX text at `ptx_path` (src/io/device.rs:62-71) into the current context. */
int ref_load(const char *ptx_path) {
    FILE *f = fopen(ptx_path, "rb");
    if (!f) return SK_ERR_DRIVER;
    std::vector<char> buf;
    char tmp[65536];
    size_t n;
    while ((n = fread(tmp, 1, sizeof tmp, f)) > 0) buf.insert(buf.end(), tmp, tmp + n);
    fclose(f);
    buf.push_back(0);
    cudaFree(0); /* make the runtime's primary context current */
    if (g_module) { cuModuleUnload(g_module); g_module = nullptr; g_funcs.clear(); }
    CUresult r = cuModuleLoadData(&g_module, buf.data());
    if (r != CUDA_SUCCESS) {
        const char *s = nullptr;
        cuGetErrorString(r, &s);
        fprintf(stderr, "ref_runner: cuModuleLoadData: %s\n", s ? s : "?");
        return SK_ERR_DRIVER;
    }
    return SK_OK;
}

int ref_configure(void *stream, uint32_t tile_dim, int sync_each_launch) {
    g_stream = reinterpret_cast<cudaStream_t>(stream);
    g_tile = tile_dim;
    g_sync = sync_each_launch;
    return SK_OK;
}
unsigned long long ref_launch_count(void) { return g_launches; }
int ref_sync(void) { return cudaStreamSynchronize(g_stream) == cudaSuccess ? SK_OK : SK_ERR_DRIVER; }

/* gpu_broadcast, src/io/device/util_device.rs:49-78, for Tensor::fill / zeroing. dtype as in sk_dense. */
int ref_fill(void *dst, uint32_t dtype, float value, size_t len) {
    if (len == 0) return SK_OK;
    const uint32_t t2 = g_tile * g_tile;
    const Dim grid{(uint32_t)((len + t2 - 1) / t2), 1}, block{t2, 1};
    if (dtype == SK_F32) return launch("broadcast_kernel_f32", grid, block, 0, false, dst, value, (uint32_t)len);
    if (dtype == SK_F16) return launch("broadcast_kernel_f16", grid, block, 0, false, dst, __float2half_rn(value), (uint32_t)len);
    return SK_ERR_UNSUPPORTED_CAST;
}

/* gpu_cast_t, src/io/device/util_device.rs:7-47 */
int ref_cast(const void *src, uint32_t src_dtype, void *dst, uint32_t dst_dtype, size_t len) {
    if (len == 0) return SK_OK;
    const uint32_t t2 = g_tile * g_tile;
    const Dim grid{(uint32_t)((len + t2 - 1) / t2), 1}, block{t2, 1};
    if (src_dtype == SK_F32 && dst_dtype == SK_F16) return launch("cast_f32_f16_t_kernel", grid, block, 0, false, src, dst, (uint32_t)len);
    if (src_dtype == SK_F16 && dst_dtype == SK_F32) return launch("cast_f16_f32_t_kernel", grid, block, 0, false, src, dst, (uint32_t)len);
    return SK_ERR_UNSUPPORTED_CAST;
}

/* src/io/device/ffn_device.rs:12-139 */
int ref_dense_forward(const sk_dense *L, const void *x, uint32_t /*x_rows*/, uint32_t batch,
                      uint32_t use_dropout, uint32_t step, uint32_t /*row_offset*/) {
    const bool h = L->dtype == SK_F16;
    if (h && g_tile != 16) return SK_ERR_HARDWARE_CONSTRAINT;
    const uint32_t seed = scramble(step, L->tensor_id);
    const uint32_t use_bias = L->norm != SK_NORM_BATCH;
    void *z = L->norm == SK_NORM_DISABLED ? L->preact : L->prenorm;
    const uint32_t t2 = g_tile * g_tile, es = h ? 2 : 4;
    int rc = launch(h ? "forward_pass_0_f16" : "forward_pass_0_f32", grid2d(L->N, batch), block2d(), 2 * t2 * es, true,
                    z, x, (const void *)L->w, (const void *)L->b, use_bias, batch, L->K, L->N, g_tile);
    if (rc) return rc;
    if (L->norm != SK_NORM_DISABLED) {
        const uint32_t gx = L->norm == SK_NORM_BATCH ? L->N : batch;
        rc = launch(h ? "forward_pass_1_f16" : "forward_pass_1_f32", Dim{gx, 1}, Dim{t2, 1}, t2 * 4, true,
                    L->preact, L->centered, (const void *)L->prenorm, (const void *)L->norm_w, (const void *)L->norm_b,
                    L->norm_rstd, batch, L->N, L->norm);
        if (rc) return rc;
    }
    return launch(h ? "forward_pass_2_f16" : "forward_pass_2_f32", grid2d(L->N, batch), block2d(), 0, true,
                  L->out, L->predrop, (const void *)L->preact, L->mask, batch, L->N, L->act, L->leaky_coeff,
                  use_dropout, L->mask_coeff, seed);
}

/* src/io/device/ffn_device.rs:141-231 */
int ref_output_error(const sk_dense *L, const void *target, uint32_t /*target_rows*/, uint32_t rows,
                     uint32_t loss, uint32_t act, float leaky) {
    const bool h = L->dtype == SK_F16;
    const size_t len = (size_t)L->max_batch * L->N;
    const uint32_t t2 = g_tile * g_tile;
    int rc;
    if ((rc = fill_f32(L->d_norm_w, 0.0f, len))) return rc;
    if ((rc = fill_f32(L->d_norm_b, 0.0f, len))) return rc;
    const uint32_t m = rows, n = L->N;
    if (act == SK_ACT_SOFTMAX) {
        rc = launch(h ? "softmax_kernel_f16" : "softmax_kernel_f32", Dim{m, 1}, Dim{t2, 1}, 0, true, L->out, m, n);
        if (rc) return rc;
    }
    return launch(h ? "compute_output_layer_error_f16" : "compute_output_layer_error_f32", grid2d(n, m), block2d(), 0, true,
                  (const void *)L->out, (const void *)L->preact, target, master(L->master_norm_w, L->norm_w),
                  L->grad, L->d_prenorm, L->d_norm_w, L->d_norm_b, (const void *)L->norm_rstd,
                  (const void *)L->centered, (const void *)L->prenorm, m, n, loss, L->norm, act, leaky);
}

/* src/io/device/ffn_device.rs:234-358 */
int ref_backward_update(const sk_dense *L, const void *x, uint32_t /*x_rows*/, uint32_t batch,
                        const sk_optim *lin, const sk_optim *nrm, float lr, float clamp, uint32_t step) {
    const bool h = L->dtype == SK_F16;
    const uint32_t use_bias = L->norm != SK_NORM_BATCH;
    return launch(h ? "backward_pass_f16" : "backward_pass_f32", grid2d(L->N, L->K), block2d(), 0, true,
                  x, L->w, L->b, master(L->master_w, L->w), master(L->master_b, L->b), L->d_prenorm,
                  L->dv_w, L->dv_b, L->dm_w, L->dm_b, L->norm_w, L->norm_b,
                  master(L->master_norm_w, L->norm_w), master(L->master_norm_b, L->norm_b),
                  L->d_norm_w, L->d_norm_b, L->dv_norm_w, L->dv_norm_b, L->dm_norm_w, L->dm_norm_b,
                  use_bias, L->norm, batch, L->N, L->K, lr, clamp, lin->kind, nrm->kind,
                  lin->beta1, lin->beta2, lin->epsilon, lin->nesterov,
                  nrm->beta1, nrm->beta2, nrm->epsilon, nrm->nesterov, L->regu, L->regu_coeff, step);
}

/* src/io/device/ffn_device.rs:360-436 (the trailing gpu_backward_pass is ref_backward_update) */
int ref_hidden_error(const sk_dense *cur, const sk_dense *next, uint32_t batch, uint32_t /*batch_stat*/) {
    const bool h = cur->dtype == SK_F16;
    if (h && g_tile != 16) return SK_ERR_HARDWARE_CONSTRAINT;
    const size_t len = (size_t)cur->max_batch * cur->N;
    const uint32_t t2 = g_tile * g_tile;
    int rc;
    if ((rc = fill_f32(cur->d_norm_w, 0.0f, len))) return rc;
    if ((rc = fill_f32(cur->d_norm_b, 0.0f, len))) return rc;
    const uint32_t n = cur->N, ec = next->N;
    return launch(h ? "compute_hidden_layer_error_f16" : "compute_hidden_layer_error_f32", grid2d(n, batch), block2d(),
                  h ? 2 * t2 * 2 : 0, true,
                  (const void *)next->d_prenorm, master(next->master_w, next->w), master(cur->master_norm_w, cur->norm_w),
                  cur->grad, cur->d_prenorm, cur->d_norm_w, cur->d_norm_b, (const void *)cur->norm_rstd,
                  (const void *)cur->centered, (const void *)cur->prenorm, (const void *)cur->predrop,
                  (const void *)cur->preact, (const void *)cur->mask, batch, n, ec, cur->norm, cur->act, cur->leaky_coeff);
}

} /* extern "C" */
