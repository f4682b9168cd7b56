// C ABI of the DenseBlock path: context, argument checks and kernel dispatch.
// The checks restate DenseBlock's own (Felix1G/soklyn src/mlp.rs:492-519, 548-580,
// 607-642, 674-736, 756-821) so that a binding can forward status codes unchanged.
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>
#include <type_traits>
#include <vector>

#include "../../include/soklyn_b200.h"
#include <map>
#include <tuple>

#include "sk_gemm_simt.cuh"
#include "sk_exchange.cuh"
#include "sk_gemm_tc.cuh"
#include "sk_rowwise.cuh"

struct sk_ctx {
    int device = 0;
    uint32_t tile_dim = 16;
    cudaStream_t stream = nullptr;
    bool own_stream = false;
    void *workspace = nullptr;
    size_t workspace_bytes = 0;
    int num_sms = 148;
    size_t smem_optin = 0;
    uint64_t launches = 0;
    char err[512] = {0};
    // tensor-core path
    int cc_major = 0;
    uint32_t gemm_engine = 0;              // 0 auto, 1 FFMA only
    int *tc_err = nullptr;                 // device word a tcgen05 kernel sets when a bounded wait gives up
    void *encode_tiled = nullptr;          // cuTensorMapEncodeTiled, resolved through the runtime
    std::map<std::tuple<const void *, uint64_t, uint64_t, uint64_t, uint32_t, uint32_t>, CUtensorMap> tmaps;
    uint64_t tc_launches = 0;
    uint32_t tc_group_n = 8;               // tile columns walked together (SK_TC_GROUP_N at context creation)
    uint32_t handover_min_rows = 0;        // column sums ride in the dX epilogue from this many rows on (SK_HANDOVER_MIN_ROWS at context creation)
    uint32_t reserve_sms = 0;              // SMs the tensor-core GEMMs leave free (for a concurrent exchange kernel)
    bool lean = false;                     // SK_OPTION_LEAN_BACKWARD
    // data-parallel backward
    uint32_t *dp_counters = nullptr;       // one completion counter per (layer, block), zero between launches
    // f32 GEMMs on the tensor cores (SK_OPTION_F32_TENSOR_CORES): device copies of the tensor maps of a launch
    bool f32_tensor = false;
    sk::TcSplitMaps *split_maps = nullptr; // ring of kSplitMapSlots entries
    uint32_t split_slot = 0;
    // Column sums handed from the dX epilogue to the weight update of the same layer. Only inside
    // sk_ffn_backward (nothing can touch the tensors or the workspace in between there).
    bool in_ffn_backward = false;
    bool colsum_handover = false;             // SK_OPTION_COLSUM_HANDOVER
    const void *fused_colsum_key = nullptr;   // d_prenorm of the layer whose partial sums sit in the workspace
    uint32_t fused_colsum_groups = 0, fused_colsum_batch = 0;
    // whole-step graphs (sk_step_begin / sk_step_end)
    struct StepGraph { cudaGraphExec_t exec = nullptr; bool warmed = false; };
    StepGraph step_graphs[SK_STEP_SLOTS];
    int step_open = -1;                    // slot between begin and end
    bool step_capturing = false;
    cudaStream_t record_stream = nullptr;  // the calls of a step are recorded on this stream (the legacy default stream
    cudaStream_t user_stream = nullptr;    // cannot be captured); `stream` points here meanwhile, user_stream keeps the caller's
    uint64_t step_stats[4] = {0, 0, 0, 0}; // instantiated, updated in place, launched, unrecorded steps
    // optional per-class event timing
    bool profiling = false;
    std::vector<cudaEvent_t> ev_pool;      // pairs: [2i] start, [2i+1] stop
    std::vector<uint32_t> ev_class;        // class of pair i
    size_t ev_used = 0;
};

namespace {
using namespace sk;

constexpr uint32_t kSplitMapSlots = 16;
constexpr uint32_t kDpMaxLayers = 64;
constexpr uint32_t kDpCounterWords = kDpMaxLayers * kMaxChunks;

int fail(sk_ctx *c, int code, const char *fmt, ...) {
    if (c) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(c->err, sizeof c->err, fmt, ap);
        va_end(ap);
    }
    return code;
}

int step_recording(sk_ctx *c) {
    return fail(c, SK_ERR_INVALID_CONFIGURATION, "not while a step graph is being recorded (sk_step_end or sk_step_abort first)");
}

int check_cuda(sk_ctx *c, cudaError_t e, const char *what) {
    if (e == cudaSuccess) return SK_OK;
    return fail(c, SK_ERR_DRIVER, "%s: %s", what, cudaGetErrorString(e));
}

// Brackets one launch with events when profiling is on.
struct ProfScope {
    sk_ctx *c;
    size_t slot = (size_t)-1;
    cudaStream_t st;
    ProfScope(sk_ctx *ctx, uint32_t cls, cudaStream_t on = nullptr) : c(ctx), st(on ? on : ctx->stream) {
        if (!c->profiling) return;
        if (c->ev_used * 2 + 2 > c->ev_pool.size()) {
            cudaEvent_t a, b;
            if (cudaEventCreate(&a) != cudaSuccess || cudaEventCreate(&b) != cudaSuccess) return;
            c->ev_pool.push_back(a); c->ev_pool.push_back(b); c->ev_class.push_back(cls);
        }
        slot = c->ev_used++;
        c->ev_class[slot] = cls;
        cudaEventRecord(c->ev_pool[2 * slot], st);
    }
    ~ProfScope() { if (slot != (size_t)-1) cudaEventRecord(c->ev_pool[2 * slot + 1], st); }
};

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// 2-D TMA descriptor over a row-major 16-bit matrix: `inner` contiguous elements per row, `outer`
// rows `ld` elements apart, fetched in boxes of 64 x box_outer with the 128-byte swizzle.
// The descriptor is returned by value: the cache may be cleared by the next lookup.
bool get_tmap(sk_ctx *c, const void *ptr, uint32_t dtype, uint64_t inner, uint64_t outer, uint64_t ld,
              uint32_t box_outer, CUtensorMap *out) {
    auto key = std::make_tuple(ptr, inner, outer, ld, box_outer, dtype);
    auto it = c->tmaps.find(key);
    if (it != c->tmaps.end()) { *out = it->second; return true; }
    if (c->tmaps.size() > 512) c->tmaps.clear();
    CUtensorMap m;
    const cuuint64_t gdim[2] = {inner, outer};
    const cuuint64_t gstride[1] = {ld * 2};
    const cuuint32_t box[2] = {64, box_outer};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = reinterpret_cast<EncodeTiledFn>(c->encode_tiled)(
        &m, dtype == SK_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
        const_cast<void *>(ptr), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return false;
    c->tmaps.emplace(key, m);
    *out = m;
    return true;
}

// SMs a tensor-core GEMM may occupy.
inline uint32_t tc_sms(const sk_ctx *c) {
    const uint32_t n = (uint32_t)c->num_sms;
    return c->reserve_sms < n ? n - c->reserve_sms : 1u;
}

// Can the tensor-core kernel take these operands? (16-byte aligned bases, row pitches that are
// multiples of 16 bytes, a Blackwell device, and the engine not forced to FFMA)
bool tc_eligible(const sk_ctx *c, uint32_t dtype, const void *a, size_t lda, const void *b, size_t ldb) {
    if (dtype == SK_F32 || c->gemm_engine == 1 || c->cc_major != 10 || !c->encode_tiled || !c->tc_err) return false;
    auto ok = [](const void *p, size_t ld) { return reinterpret_cast<uintptr_t>(p) % 16 == 0 && ld % 8 == 0; };
    return ok(a, lda) && ok(b, ldb);
}

// cudaFuncSetAttribute is per device: one bit per device ordinal and kernel instantiation.
template <typename T, bool A_MN, bool B_MN, int BN, class Epi>
cudaError_t launch_tc_bn(sk_ctx *c, const CUtensorMap &ta, const CUtensorMap &tb, uint32_t M, uint32_t N, uint32_t K,
                         const Epi &epi, const TcGate &gate, uint32_t group_n) {
    using S = TcShape<BN>;
    static uint64_t attr_set[4] = {0, 0, 0, 0};   // devices 0..255
    auto kernel = gemm_tc_kernel<A_MN, B_MN, BN, Epi>;
    const unsigned dev = (unsigned)c->device & 255u;
    if (!(attr_set[dev >> 6] >> (dev & 63) & 1ull)) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kSmemBytes);
        if (e != cudaSuccess) return e;
        attr_set[dev >> 6] |= 1ull << (dev & 63);
    }
    const uint32_t tiles = ((M + kTcBM - 1) / kTcBM) * ((N + BN - 1) / BN);
    const uint32_t sms = tc_sms(c);
    const uint32_t grid = tiles < sms ? tiles : sms;
    const uint32_t idesc = tc::make_instr_desc(std::is_same<T, __nv_bfloat16>::value ? 1u : 0u, A_MN, B_MN, kTcBM, BN);
    kernel<<<grid, kTcThreads, S::kSmemBytes, c->stream>>>(ta, tb, M, N, K, idesc, group_n, epi, gate, c->tc_err, nullptr);
    c->tc_launches++;
    return cudaGetLastError();
}

// C[M x N] = A.B on the tensor cores. A_MN / B_MN: operand contiguous along M / N (else along K).
template <typename T, bool A_MN, bool B_MN, class Epi>
cudaError_t launch_gemm_tc(sk_ctx *c, uint32_t dtype, const T *A, size_t lda, const T *B, size_t ldb, uint32_t M,
                           uint32_t N, uint32_t K, const Epi &epi, const TcGate &gate = TcGate{}) {
    const uint32_t sms = tc_sms(c);
    auto cost = [&](uint32_t bn) {
        const uint64_t tiles = (uint64_t)((M + kTcBM - 1) / kTcBM) * ((N + bn - 1) / bn);
        return ((tiles + sms - 1) / sms) * bn;
    };
    // A 128-wide tile re-reads the A panel twice as often per flop and measured about 0.8 of the
    // 256-wide tile's rate at equal occupancy, so it has to save more than a fifth of the waves.
    const bool wide = N > 128 && cost(256) * 4 <= cost(128) * 5;
    const uint32_t bn = wide ? 256 : 128;
    CUtensorMap ta, tb;
    const bool ok_a = A_MN ? get_tmap(c, A, dtype, M, K, lda, 64, &ta) : get_tmap(c, A, dtype, K, M, lda, kTcBM, &ta);
    const bool ok_b = B_MN ? get_tmap(c, B, dtype, N, K, ldb, 64, &tb) : get_tmap(c, B, dtype, K, N, ldb, bn, &tb);
    if (!ok_a || !ok_b) return cudaErrorInvalidValue;
    uint32_t group_n = c->tc_group_n;
    if (gate.flags) {   // a group of tile columns must not reach into a block of rows that arrives later
        const uint32_t per_chunk = gate.rows_per_chunk / bn;
        if (per_chunk >= 1 && per_chunk < group_n) group_n = per_chunk;
        if (per_chunk == 0) group_n = 1;
    }
    return wide ? launch_tc_bn<T, A_MN, B_MN, 256, Epi>(c, ta, tb, M, N, K, epi, gate, group_n)
                : launch_tc_bn<T, A_MN, B_MN, 128, Epi>(c, ta, tb, M, N, K, epi, gate, group_n);
}

// ---- f32 operands on the tensor cores: three bf16 parts per operand, six partial products --------------
// part[0] + part[1] + part[2] == x up to the last bit of f32 (each part holds the next 8 significant bits).
__global__ void __launch_bounds__(256) split_bf16x3_kernel(const float *__restrict__ src, __nv_bfloat16 *__restrict__ p0,
                                                            __nv_bfloat16 *__restrict__ p1, __nv_bfloat16 *__restrict__ p2,
                                                            size_t len) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < len; i += stride) {
        const float x = src[i];
        const __nv_bfloat16 a = __float2bfloat16_rn(x);
        const float r1 = x - __bfloat162float(a);
        const __nv_bfloat16 b = __float2bfloat16_rn(r1);
        const float r2 = r1 - __bfloat162float(b);
        p0[i] = a; p1[i] = b; p2[i] = __float2bfloat16_rn(r2);
    }
}

// Smallest shape worth the split passes, and what the split copies need of the workspace.
inline bool split_worthwhile(uint32_t M, uint32_t N, uint32_t K) { return (double)M * N * K >= (double)(1u << 28); }

template <bool A_MN, bool B_MN, class Epi>
cudaError_t launch_gemm_tc_split(sk_ctx *c, const float *A, size_t lda, const float *B, size_t ldb, uint32_t M, uint32_t N,
                                 uint32_t K, const Epi &epi, bool *taken) {
    *taken = false;
    if (!c->f32_tensor || c->cc_major != 10 || !c->encode_tiled || !c->tc_err || !c->split_maps) return cudaSuccess;
    if (!split_worthwhile(M, N, K) || lda % 8 || ldb % 8 || reinterpret_cast<uintptr_t>(A) % 16 || reinterpret_cast<uintptr_t>(B) % 16)
        return cudaSuccess;
    // elements of the row-major sources the GEMM touches
    const size_t len_a = (size_t)(A_MN ? K : M) * lda, len_b = (size_t)(B_MN ? K : N) * ldb;
    const size_t pad = 128;   // elements: keeps every part 256-byte aligned
    const size_t ea = (len_a + pad - 1) / pad * pad, eb = (len_b + pad - 1) / pad * pad;
    if ((3 * ea + 3 * eb) * sizeof(__nv_bfloat16) > c->workspace_bytes) return cudaSuccess;
    __nv_bfloat16 *base = (__nv_bfloat16 *)c->workspace;
    __nv_bfloat16 *pa[3] = {base, base + ea, base + 2 * ea}, *pb[3] = {base + 3 * ea, base + 3 * ea + eb, base + 3 * ea + 2 * eb};
    auto blocks = [&](size_t len) { size_t b = (len + 1023) / 1024; const size_t cap = (size_t)c->num_sms * 16; return (unsigned)(b > cap ? cap : b); };
    split_bf16x3_kernel<<<blocks(len_a), 256, 0, c->stream>>>(A, pa[0], pa[1], pa[2], len_a);
    split_bf16x3_kernel<<<blocks(len_b), 256, 0, c->stream>>>(B, pb[0], pb[1], pb[2], len_b);
    c->launches += 2;
    const uint32_t sms = tc_sms(c);
    constexpr uint32_t bn = 128;   // the split kernel's tile: four accumulator buffers of 128 columns
    TcSplitMaps maps;
    for (int i = 0; i < 3; ++i) {
        const bool ok_a = A_MN ? get_tmap(c, pa[i], SK_BF16, M, K, lda, 64, &maps.a[i]) : get_tmap(c, pa[i], SK_BF16, K, M, lda, kTcBM, &maps.a[i]);
        const bool ok_b = B_MN ? get_tmap(c, pb[i], SK_BF16, N, K, ldb, 64, &maps.b[i]) : get_tmap(c, pb[i], SK_BF16, K, N, ldb, bn, &maps.b[i]);
        if (!ok_a || !ok_b) return cudaErrorInvalidValue;
    }
    TcSplitMaps *dev = c->split_maps + (c->split_slot++ % kSplitMapSlots);
    cudaError_t e = cudaMemcpyAsync(dev, &maps, sizeof maps, cudaMemcpyHostToDevice, c->stream);
    if (e != cudaSuccess) return e;
    *taken = true;
    const uint32_t tiles = ((M + kTcBM - 1) / kTcBM) * ((N + bn - 1) / bn);
    const uint32_t grid = tiles < sms ? tiles : sms;
    const uint32_t idesc = tc::make_instr_desc(1u, A_MN, B_MN, kTcBM, bn);
    static uint64_t attr_set[4] = {0, 0, 0, 0};
    const unsigned d = (unsigned)c->device & 255u;
    auto kernel = gemm_tc_kernel<A_MN, B_MN, bn, Epi, true>;
    if (!(attr_set[d >> 6] >> (d & 63) & 1ull)) {
        if ((e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TcShape<bn>::kSmemBytes)) != cudaSuccess) return e;
        attr_set[d >> 6] |= 1ull << (d & 63);
    }
    kernel<<<grid, kTcThreads, TcShape<bn>::kSmemBytes, c->stream>>>(maps.a[0], maps.b[0], M, N, K, idesc, c->tc_group_n, epi, TcGate{}, c->tc_err, dev);
    c->tc_launches++;
    return cudaGetLastError();
}

// Engine choice for one product of the DenseBlock path.
template <typename TA, typename TB, bool A_KCONTIG, bool B_NCONTIG, class Epi>
cudaError_t run_gemm(sk_ctx *c, uint32_t dtype, const TA *A, size_t lda, const TB *B, size_t ldb, uint32_t M, uint32_t N,
                     uint32_t K, const Epi &epi, const TcGate &gate = TcGate{}) {
    if constexpr (std::is_same<TA, TB>::value && !std::is_same<TA, float>::value) {
        if (tc_eligible(c, dtype, A, lda, B, ldb))
            return launch_gemm_tc<TA, !A_KCONTIG, B_NCONTIG, Epi>(c, dtype, A, lda, B, ldb, M, N, K, epi, gate);
    }
    if (gate.flags) return cudaErrorNotSupported;   // only the tensor-core kernel can wait for rows in flight
    if constexpr (std::is_same<TA, float>::value && std::is_same<TB, float>::value) {
        bool taken = false;
        const cudaError_t e = launch_gemm_tc_split<!A_KCONTIG, B_NCONTIG, Epi>(c, A, lda, B, ldb, M, N, K, epi, &taken);
        if (taken || e != cudaSuccess) return e;
    }
    return launch_gemm_simt<TA, TB, A_KCONTIG, B_NCONTIG, Epi>(c->stream, c->num_sms, A, lda, B, ldb, M, N, K, epi);
}

inline bool aligned16(const void *p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; }
constexpr uint32_t kSmallBatchRows = 256;   // up to here column sums and the vector step share one launch
constexpr uint32_t kHandoverMinRows = 512;   // below this a separate column-sum pass costs as little as the heavier dX epilogue (measured: 0.4 % of a step gained at 512 rows, 1.4 % at 1024, none at 256)
constexpr uint32_t kColsumFold = 8;   // slabs the per-32-row column sums of the dX epilogue are folded into

Optim make_optim(const sk_optim *o, uint32_t step) {
    Optim r{};
    r.kind = o->kind; r.beta1 = o->beta1; r.beta2 = o->beta2; r.epsilon = o->epsilon; r.nesterov = o->nesterov;
    r.bc1 = 1.0f - powf(o->beta1, (float)step);
    r.bc2 = 1.0f - powf(o->beta2, (float)step);
    r.inv_bc1 = 1.0f / r.bc1;
    r.inv_bc2 = 1.0f / r.bc2;
    return r;
}

int check_layer(sk_ctx *c, const sk_dense *L, bool training) {
    if (!c || !L) return SK_ERR_NULL_POINTER;
    if (L->dtype > SK_BF16) return fail(c, SK_ERR_INVALID_CONFIGURATION, "unknown dtype %u", L->dtype);
    if (L->K == 0 || L->N == 0) return fail(c, SK_ERR_INVALID_CONFIGURATION, "Input or output size cannot be 0.");
    if (L->max_batch == 0) return fail(c, SK_ERR_INVALID_CONFIGURATION, "Batch size cannot be 0.");
    if (L->norm > 3 || L->act > 7 || L->regu > 2) return fail(c, SK_ERR_INVALID_CONFIGURATION, "ordinal out of range");
    if (L->dtype != SK_F32 && c->tile_dim != 16)
        return fail(c, SK_ERR_HARDWARE_CONSTRAINT, "16-bit precision requires a tile dimension of 16, found %u", c->tile_dim);
    if (!L->w || !L->b || !L->norm_w || !L->norm_b || !L->out || !L->predrop || !L->preact || !L->centered ||
        !L->prenorm || !L->norm_rstd || !L->mask)
        return fail(c, SK_ERR_NULL_POINTER, "forward tensor pointer is NULL");
    if (training) {
        if (!L->is_training) return fail(c, SK_ERR_TRAINING_MODE_REQUIRED, "block is in inference mode");
        if (!L->grad || !L->d_prenorm || !L->d_norm_w || !L->d_norm_b || !L->dv_w || !L->dv_b || !L->dm_w || !L->dm_b ||
            !L->dv_norm_w || !L->dv_norm_b || !L->dm_norm_w || !L->dm_norm_b)
            return fail(c, SK_ERR_NULL_POINTER, "training tensor pointer is NULL");
        if (L->dtype != SK_F32 && (!L->master_w || !L->master_b || !L->master_norm_w || !L->master_norm_b || !L->d_prenorm_lp))
            return fail(c, SK_ERR_NULL_POINTER, "16-bit training needs master copies and d_prenorm_lp");
    }
    return SK_OK;
}

// DenseBlock::check_input_dimension (src/mlp.rs:492-519) + the batch checks of forward/backward.
int check_batch(sk_ctx *c, const sk_dense *L, uint32_t x_rows, uint32_t batch) {
    if (x_rows < batch) return fail(c, SK_ERR_MISMATCHED_DIMENSIONS, "input rows vs explicit batch size: expected %u, found %u", batch, x_rows);
    if (x_rows > L->max_batch) return fail(c, SK_ERR_ALLOCATION_LIMIT, "input batches: received %u exceeds max %u", x_rows, L->max_batch);
    if (L->act == SK_ACT_SOFTMAX) return fail(c, SK_ERR_INVALID_CONFIGURATION, "Softmax activation can only be passed into the compute_loss function.");
    if (batch == 0) return fail(c, SK_ERR_INVALID_BATCH_SIZE, "Batch size must be more than zero.");
    if (L->norm == SK_NORM_BATCH && batch == 1) return fail(c, SK_ERR_INVALID_BATCH_SIZE, "BatchNorm needs a batch size of more than 1.");
    return SK_OK;
}

template <typename T> inline float *master_of(float *m, void *p) { return m ? m : reinterpret_cast<float *>(p); }

// all [rows x N] tensors of a block can be accessed with 128-bit runs
bool layer_vec_ok(const sk_dense *L) {
    const void *ps[] = {L->b, L->norm_w, L->norm_b, L->out, L->predrop, L->preact, L->centered, L->prenorm, L->norm_rstd,
                        L->mask, L->grad, L->d_prenorm, L->d_norm_w, L->d_norm_b, L->d_prenorm_lp, L->master_norm_w};
    for (const void *p : ps) if (p && !aligned16(p)) return false;
    return L->N % 8 == 0;
}

// ------------------------------------------------------------------------------------------
template <typename T>
int forward_impl(sk_ctx *c, const sk_dense *L, const void *x, uint32_t batch, uint32_t use_dropout, uint32_t step,
                 uint32_t row_offset, bool gemm_only = false) {
    const uint32_t seed = sk_scramble_seed(step, L->tensor_id);
    const bool has_norm = L->norm != SK_NORM_DISABLED;
    const bool vec = layer_vec_ok(L);
    EpiForward<T> epi{};
    epi.bias = L->norm != SK_NORM_BATCH ? (const T *)L->b : nullptr;
    epi.z = (T *)(has_norm ? L->prenorm : L->preact);
    epi.predrop = (T *)L->predrop; epi.out = (T *)L->out; epi.mask = (T *)L->mask;
    epi.N = L->N; epi.has_norm = has_norm; epi.act = L->act; epi.use_dropout = use_dropout; epi.seed = seed;
    epi.row_offset = row_offset; epi.leaky = L->leaky_coeff; epi.mask_coeff = L->mask_coeff; epi.vec_ok = vec;
    int rc;
    {
        ProfScope ps(c, SK_PROF_GEMM_FORWARD);
        rc = check_cuda(c, run_gemm<T, T, true, true>(c, L->dtype, (const T *)x, L->K, (const T *)L->w,
                                                               L->N, batch, L->N, L->K, epi), "forward gemm");
    }
    c->launches++;
    if (rc || !has_norm || gemm_only) return rc;
    ProfScope ps(c, SK_PROF_NORM);
    ActDrop ad{L->act, use_dropout, seed, row_offset, L->leaky_coeff, L->mask_coeff};
    if (L->norm == SK_NORM_BATCH) {
        norm_cols_kernel<T><<<(L->N + 31) / 32, kRowThreads, 0, c->stream>>>(
            (const T *)L->prenorm, (const T *)L->norm_w, (const T *)L->norm_b, (T *)L->centered, (T *)L->preact,
            (T *)L->predrop, (T *)L->out, (T *)L->mask, (T *)L->norm_rstd, batch, L->N, ad);
    } else {
        const size_t cache_bytes = (size_t)L->N * sizeof(float);
        const bool cached = cache_bytes <= c->smem_optin;
        // rows stream straight from global memory (the second pass hits L2): no shared memory,
        // so eight blocks fit an SM; the shared-memory row cache is kept for rows of odd length
        const bool use_cache = cached && !vec;
        norm_rows_kernel<T><<<batch, kRowThreads, use_cache ? cache_bytes : 0, c->stream>>>(
            (const T *)L->prenorm, (const T *)L->norm_w, (const T *)L->norm_b, (T *)L->centered, (T *)L->preact,
            (T *)L->predrop, (T *)L->out, (T *)L->mask, (T *)L->norm_rstd, L->N, L->norm, ad, vec, use_cache);
    }
    c->launches++;
    return check_cuda(c, cudaGetLastError(), "forward norm");
}

// BatchNorm forward in phases for a batch that is split over devices (see norm_cols_phase_kernel).
template <typename T>
int forward_batchnorm_impl(sk_ctx *c, const sk_dense *L, const void *x, uint32_t batch, uint32_t batch_stat, uint32_t phase,
                           float *stats, uint32_t use_dropout, uint32_t step, uint32_t row_offset) {
    if (phase == 0) {
        const int rc = forward_impl<T>(c, L, x, batch, use_dropout, step, row_offset, true);
        if (rc) return rc;
    }
    ProfScope ps(c, SK_PROF_NORM);
    ActDrop ad{L->act, use_dropout, sk_scramble_seed(step, L->tensor_id), row_offset, L->leaky_coeff, L->mask_coeff};
    norm_cols_phase_kernel<T><<<(L->N + 31) / 32, kRowThreads, 0, c->stream>>>(
        phase, stats, batch_stat, (const T *)L->prenorm, (const T *)L->norm_w, (const T *)L->norm_b, (T *)L->centered,
        (T *)L->preact, (T *)L->predrop, (T *)L->out, (T *)L->mask, (T *)L->norm_rstd, batch, L->N, ad);
    c->launches++;
    return check_cuda(c, cudaGetLastError(), "forward batch norm phase");
}

template <typename T>
int output_error_impl(sk_ctx *c, const sk_dense *L, const void *target, uint32_t rows, uint32_t loss, uint32_t act,
                      float leaky) {
    // rows below `rows` are fully overwritten; the reference zeroes d_norm_* first, which
    // only shows in the rows beyond.
    if (rows < L->max_batch) {
        const size_t off = (size_t)rows * L->N, bytes = (size_t)(L->max_batch - rows) * L->N * sizeof(float);
        cudaMemsetAsync(L->d_norm_w + off, 0, bytes, c->stream);
        cudaMemsetAsync(L->d_norm_b + off, 0, bytes, c->stream);
    }
    const uint32_t warps = kRowThreads / 32;
    ProfScope ps(c, SK_PROF_OUTPUT_ERROR);
    if (act != SK_ACT_SOFTMAX && layer_vec_ok(L) && aligned16(target)) {
        const size_t total = (size_t)rows * (L->N / 8);
        size_t blocks = (total + kRowThreads - 1) / kRowThreads;
        const size_t cap = (size_t)c->num_sms * 16;
        if (blocks > cap) blocks = cap;
        output_error_elem_kernel<T><<<(uint32_t)blocks, kRowThreads, 0, c->stream>>>(
            (const T *)L->out, (const T *)L->preact, (const T *)target, master_of<T>(L->master_norm_w, L->norm_w), L->grad,
            L->d_prenorm, L->d_norm_w, L->d_norm_b, L->dtype == SK_F32 ? nullptr : (T *)L->d_prenorm_lp,
            (const T *)L->norm_rstd, (const T *)L->centered, (const T *)L->prenorm, rows, L->N, loss, L->norm, act, leaky);
        c->launches++;
        return check_cuda(c, cudaGetLastError(), "output error");
    }
    output_error_kernel<T><<<(rows + warps - 1) / warps, kRowThreads, 0, c->stream>>>(
        (T *)L->out, (const T *)L->preact, (const T *)target, master_of<T>(L->master_norm_w, L->norm_w), L->grad,
        L->d_prenorm, L->d_norm_w, L->d_norm_b, L->dtype == SK_F32 ? nullptr : (T *)L->d_prenorm_lp,
        (const T *)L->norm_rstd, (const T *)L->centered, (const T *)L->prenorm, rows, L->N, loss, L->norm, act, leaky);
    c->launches++;
    return check_cuda(c, cudaGetLastError(), "output error");
}

template <typename T>
int hidden_error_impl(sk_ctx *c, const sk_dense *cur, const sk_dense *next, uint32_t batch, uint32_t batch_stat,
                      const TcGate &gate = TcGate{}) {
    const bool f32 = cur->dtype == SK_F32;
    EpiHidden<T> epi{};
    epi.predrop = (const T *)cur->predrop; epi.preact = (const T *)cur->preact; epi.mask = (const T *)cur->mask;
    epi.prenorm = (const T *)cur->prenorm; epi.centered = (const T *)cur->centered; epi.rstd = (const T *)cur->norm_rstd;
    epi.norm_w = master_of<T>(cur->master_norm_w, cur->norm_w);
    epi.grad = cur->grad; epi.d_prenorm = cur->d_prenorm; epi.d_norm_w = cur->d_norm_w; epi.d_norm_b = cur->d_norm_b;
    epi.d_prenorm_lp = f32 ? nullptr : (T *)cur->d_prenorm_lp;
    epi.N = cur->N; epi.norm = cur->norm; epi.act = cur->act; epi.leaky = cur->leaky_coeff;
    epi.inv_n = 1.0f / (float)cur->N; epi.inv_m = 1.0f / (float)batch_stat; epi.vec_ok = layer_vec_ok(cur);
    epi.acc_scale = f32 ? 1.0f : kLpScaleInv;
    const uint32_t ec = next->N;
    const T *dy = f32 ? (const T *)next->d_prenorm : (const T *)next->d_prenorm_lp;
    const T *wn = f32 ? (const T *)master_of<T>(next->master_w, next->w) : (const T *)next->w;
    // Column sums for the weight update that follows, taken in the epilogue when that update is
    // certain to be the next call, the tensor-core kernel runs and the partial sums fit.
    epi.colsum_partial = nullptr; epi.colsum_groups = 0;
    c->fused_colsum_key = nullptr;
    const bool specialised = !f32 && ((cur->act == SK_ACT_SILU && cur->norm == SK_NORM_RMS) ||
                                      (cur->act == SK_ACT_MISH && cur->norm == SK_NORM_LAYER));
    if ((c->in_ffn_backward || c->colsum_handover) && specialised && batch >= c->handover_min_rows && epi.vec_ok && tc_eligible(c, cur->dtype, dy, ec, wn, ec)) {
        const uint32_t groups = (batch + 31) / 32;
        const size_t need = ((size_t)groups + kColsumFold) * 3 * cur->N * sizeof(float);
        if (need <= c->workspace_bytes) {
            epi.colsum_partial = (float *)c->workspace; epi.colsum_groups = groups;
            c->fused_colsum_key = cur->d_prenorm; c->fused_colsum_groups = groups; c->fused_colsum_batch = batch;
        }
    }
    epi.lean = c->lean && epi.colsum_partial != nullptr;
    if (!epi.lean && batch < cur->max_batch) {   // the reference zeroes d_norm_* first, which only shows in the rows beyond
        const size_t off = (size_t)batch * cur->N, bytes = (size_t)(cur->max_batch - batch) * cur->N * sizeof(float);
        cudaMemsetAsync(cur->d_norm_w + off, 0, bytes, c->stream);
        cudaMemsetAsync(cur->d_norm_b + off, 0, bytes, c->stream);
    }
    ProfScope ps(c, SK_PROF_GEMM_DX);
    cudaError_t e;
    // kernels specialised for the activation / normalisation pairs of the wide and the classifier networks
    if (!f32 && cur->act == SK_ACT_SILU && cur->norm == SK_NORM_RMS) {
        EpiHidden<T, SK_ACT_SILU, SK_NORM_RMS> se;
        static_assert(sizeof(se) == sizeof(epi), "specialised functor has the same fields");
        memcpy(&se, &epi, sizeof se);
        e = run_gemm<T, T, true, false>(c, cur->dtype, dy, ec, wn, ec, batch, cur->N, ec, se, gate);
    } else if (!f32 && cur->act == SK_ACT_MISH && cur->norm == SK_NORM_LAYER) {
        EpiHidden<T, SK_ACT_MISH, SK_NORM_LAYER> se;
        memcpy(&se, &epi, sizeof se);
        e = run_gemm<T, T, true, false>(c, cur->dtype, dy, ec, wn, ec, batch, cur->N, ec, se, gate);
    } else {
        e = run_gemm<T, T, true, false>(c, cur->dtype, dy, ec, wn, ec, batch, cur->N, ec, epi, gate);
    }
    int rc = check_cuda(c, e, "hidden error gemm");
    if (rc) c->fused_colsum_key = nullptr;
    c->launches++;
    return rc;
}

// Column-sum stage 1 into the workspace; returns the number of partial slabs (0 on error).
uint32_t launch_colsum_partial(sk_ctx *c, const sk_dense *L, uint32_t batch, int *rc) {
    const uint32_t gx = (L->N + 31) / 32;
    uint32_t gy = (uint32_t)((4 * c->num_sms + gx - 1) / gx);
    gy = gy < 1 ? 1 : gy;
    const uint32_t max_gy = (batch + 7) / 8;
    if (gy > max_gy) gy = max_gy;
    const uint32_t rows_per_block = (batch + gy - 1) / gy;
    gy = (batch + rows_per_block - 1) / rows_per_block;
    const size_t need = (size_t)gy * 3 * L->N * sizeof(float);
    if (need > c->workspace_bytes) {
        *rc = fail(c, SK_ERR_WORKSPACE, "column sums need %zu bytes of workspace, context has %zu", need, c->workspace_bytes);
        return 0;
    }
    ProfScope ps(c, SK_PROF_COLSUM);
    colsum_partial_kernel<<<dim3(gx, gy), kRowThreads, 0, c->stream>>>(L->d_prenorm, L->d_norm_w, L->d_norm_b,
                                                                        (float *)c->workspace, batch, L->N, rows_per_block, L->norm);
    c->launches++;
    *rc = check_cuda(c, cudaGetLastError(), "column sums");
    return *rc ? 0 : gy;
}

// If the dX epilogue of this layer left per-32-row column sums in the workspace, folds them into
// kColsumFold slabs and returns those; otherwise runs the column-sum kernel over the three tensors.
const float *column_sum_slabs(sk_ctx *c, const sk_dense *L, uint32_t batch, uint32_t *nslabs, int *rc) {
    if (c->fused_colsum_key && c->fused_colsum_key == L->d_prenorm && c->fused_colsum_batch == batch) {
        const uint32_t groups = c->fused_colsum_groups, per = (groups + kColsumFold - 1) / kColsumFold;
        const uint32_t slabs = (groups + per - 1) / per;
        float *folded = (float *)c->workspace + (size_t)groups * 3 * L->N;
        c->fused_colsum_key = nullptr;
        ProfScope ps(c, SK_PROF_COLSUM);
        colsum_fold_kernel<<<dim3((3 * L->N + 255) / 256, slabs), 256, 0, c->stream>>>((const float *)c->workspace, folded,
                                                                                      L->N, groups, per);
        c->launches++;
        *rc = check_cuda(c, cudaGetLastError(), "column sums (fold)");
        *nslabs = slabs;
        return folded;
    }
    c->fused_colsum_key = nullptr;
    *nslabs = launch_colsum_partial(c, L, batch, rc);
    return (const float *)c->workspace;
}

template <typename T>
VectorParams<T> vector_params(const sk_dense *L, const Optim &lin, const Optim &nrm, const Hyper &hyp) {
    return VectorParams<T>{(T *)L->b, master_of<T>(L->master_b, L->b), L->dv_b, L->dm_b,
                           (T *)L->norm_w, master_of<T>(L->master_norm_w, L->norm_w), L->dv_norm_w, L->dm_norm_w,
                           (T *)L->norm_b, master_of<T>(L->master_norm_b, L->norm_b), L->dv_norm_b, L->dm_norm_b,
                           L->norm != SK_NORM_BATCH, L->norm, lin, nrm, hyp};
}

template <typename T>
int vector_update_launch(sk_ctx *c, const sk_dense *L, const float *partial, uint32_t nblocks, const Optim &lin,
                         const Optim &nrm, const Hyper &hyp, const int *abort_flag = nullptr) {
    ProfScope ps(c, SK_PROF_UPDATE);
    vector_update_kernel<T><<<(L->N + 127) / 128, 128, 0, c->stream>>>(partial, nblocks, L->N, vector_params<T>(L, lin, nrm, hyp),
                                                                         abort_flag);
    c->launches++;
    return check_cuda(c, cudaGetLastError(), "bias / norm parameter step");
}

// Column sums + bias / normalisation-parameter step of a block. Small batches take both in one
// launch; otherwise the sums come from the dX epilogue or the two-stage column-sum kernel.
template <typename T>
int column_sums_and_vector_update(sk_ctx *c, const sk_dense *L, uint32_t batch, const Optim &lin, const Optim &nrm,
                                  const Hyper &hyp) {
    const bool handed = c->fused_colsum_key && c->fused_colsum_key == L->d_prenorm && c->fused_colsum_batch == batch;
    if (!handed && batch <= kSmallBatchRows) {
        c->fused_colsum_key = nullptr;
        ProfScope ps(c, SK_PROF_UPDATE);
        colsum_update_kernel<T><<<(L->N + 31) / 32, kRowThreads, 0, c->stream>>>(L->d_prenorm, L->d_norm_w, L->d_norm_b, batch,
                                                                             L->N, vector_params<T>(L, lin, nrm, hyp));
        c->launches++;
        return check_cuda(c, cudaGetLastError(), "column sums + bias / norm parameter step");
    }
    int rc = SK_OK;
    uint32_t nslabs = 0;
    const float *slabs = column_sum_slabs(c, L, batch, &nslabs, &rc);
    if (rc) return rc;
    return vector_update_launch<T>(c, L, slabs, nslabs, lin, nrm, hyp);
}

template <typename T>
int backward_update_impl(sk_ctx *c, const sk_dense *L, const void *x, uint32_t batch, const sk_optim *lin_,
                         const sk_optim *nrm_, float lr, float clamp, uint32_t step) {
    const Optim lin = make_optim(lin_, step), nrm = make_optim(nrm_, step);
    const Hyper hyp{lr, clamp, 1.0f / (float)batch, L->regu, L->regu_coeff};
    int rc = SK_OK;
    if ((rc = column_sums_and_vector_update<T>(c, L, batch, lin, nrm, hyp))) return rc;
    const bool f32 = L->dtype == SK_F32;
    EpiWeightUpdate<T> epi{};
    epi.w = (T *)L->w; epi.master = master_of<T>(L->master_w, L->w); epi.dv = L->dv_w; epi.dm = L->dm_w;
    epi.N = L->N; epi.opt = lin; epi.hyp = hyp;
    epi.gscale = f32 ? kLossScaleInv : kLossScaleInv * kLpScaleInv;
    epi.vec_ok = L->N % 8 == 0 && aligned16(L->w) && aligned16(epi.master) && aligned16(L->dv_w) && aligned16(L->dm_w);
    ProfScope ps(c, SK_PROF_GEMM_DW);
    if (f32) {
        rc = check_cuda(c, run_gemm<T, float, false, true>(c, L->dtype, (const T *)x, L->K, L->d_prenorm,
                                                                    L->N, L->K, L->N, batch, epi), "weight gradient gemm");
    } else if (lin.kind == SK_OPT_ADAM && L->regu == SK_REGU_NONE) {   // specialised: Adam, no regularisation
        EpiWeightUpdate<T, SK_OPT_ADAM, SK_REGU_NONE> se;
        static_assert(sizeof(se) == sizeof(epi), "specialised functor has the same fields");
        memcpy(&se, &epi, sizeof se);
        rc = check_cuda(c, run_gemm<T, T, false, true>(c, L->dtype, (const T *)x, L->K, (const T *)L->d_prenorm_lp, L->N,
                                                        L->K, L->N, batch, se), "weight gradient gemm");
    } else {
        rc = check_cuda(c, run_gemm<T, T, false, true>(c, L->dtype, (const T *)x, L->K,
                                                                (const T *)L->d_prenorm_lp, L->N, L->K, L->N, batch, epi),
                        "weight gradient gemm");
    }
    c->launches++;
    return rc;
}

template <typename T>
int backward_grads_impl(sk_ctx *c, const sk_dense *L, const void *x, uint32_t batch, float *dw, float *colsums) {
    int rc = SK_OK;
    const uint32_t nblocks = launch_colsum_partial(c, L, batch, &rc);
    if (rc) return rc;
    colsum_final_kernel<<<(3 * L->N + 255) / 256, 256, 0, c->stream>>>((const float *)c->workspace, colsums, L->N, nblocks);
    c->launches++;
    if ((rc = check_cuda(c, cudaGetLastError(), "column sums (final)"))) return rc;
    EpiStoreF32 epi{dw, L->N, L->dtype == SK_F32 ? 1.0f : kLpScaleInv, L->N % 8 == 0 && aligned16(dw)};
    ProfScope ps(c, SK_PROF_GEMM_DW);
    if (L->dtype == SK_F32)
        rc = check_cuda(c, run_gemm<T, float, false, true>(c, L->dtype, (const T *)x, L->K, L->d_prenorm,
                                                                    L->N, L->K, L->N, batch, epi), "weight gradient gemm");
    else
        rc = check_cuda(c, run_gemm<T, T, false, true>(c, L->dtype, (const T *)x, L->K,
                                                                (const T *)L->d_prenorm_lp, L->N, L->K, L->N, batch, epi),
                        "weight gradient gemm");
    c->launches++;
    return rc;
}

// dW as the storage type, already divided by batch_stat (the loss scale stays in), plus the raw
// f32 column sums: the payload of the sharded data-parallel exchange.
template <typename T>
int backward_grads_lp_impl(sk_ctx *c, const sk_dense *L, const void *x, uint32_t batch, uint32_t batch_stat, void *g,
                           float *colsums) {
    int rc = SK_OK;
    uint32_t nblocks = 0;
    const float *slabs = column_sum_slabs(c, L, batch, &nblocks, &rc);
    if (rc) return rc;
    colsum_final_kernel<<<(3 * L->N + 255) / 256, 256, 0, c->stream>>>(slabs, colsums, L->N, nblocks);
    c->launches++;
    if ((rc = check_cuda(c, cudaGetLastError(), "column sums (final)"))) return rc;
    EpiStoreScaled<T> epi{(T *)g, L->N, (L->dtype == SK_F32 ? 1.0f : kLpScaleInv) / (float)batch_stat, L->N % 8 == 0 && aligned16(g)};
    ProfScope ps(c, SK_PROF_GEMM_DW);
    if (L->dtype == SK_F32)
        rc = check_cuda(c, run_gemm<T, float, false, true>(c, L->dtype, (const T *)x, L->K, L->d_prenorm,
                                                                    L->N, L->K, L->N, batch, epi), "weight gradient gemm");
    else
        rc = check_cuda(c, run_gemm<T, T, false, true>(c, L->dtype, (const T *)x, L->K,
                                                                (const T *)L->d_prenorm_lp, L->N, L->K, L->N, batch, epi),
                        "weight gradient gemm");
    c->launches++;
    return rc;
}

// Optimiser step on rows [row0, row0 + nrows) of the weight matrix from an averaged gradient of
// the storage type, laid out as those rows only.
template <typename T>
int apply_update_rows_impl(sk_ctx *c, const sk_dense *L, const void *g, uint32_t row0, uint32_t nrows,
                           const sk_optim *lin_, float lr, float clamp, uint32_t step) {
    const Optim lin = make_optim(lin_, step);
    const Hyper hyp{lr, clamp, 1.0f, L->regu, L->regu_coeff};   // the gradient is already averaged
    const size_t off = (size_t)row0 * L->N, len = (size_t)nrows * L->N;
    float *master = master_of<T>(L->master_w, L->w) + off;
    T *w = (T *)L->w + off;
    float *dv = L->dv_w + off, *dm = L->dm_w + off;
    const bool vec = len % 8 == 0 && aligned16(g) && aligned16(w) && aligned16(master) && aligned16(dv) && aligned16(dm);
    size_t blocks = (len / 8 + kRowThreads - 1) / kRowThreads;
    const size_t cap = (size_t)c->num_sms * 8;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    ProfScope ps(c, SK_PROF_UPDATE);
    weight_update_range_kernel<T, T><<<(uint32_t)blocks, kRowThreads, 0, c->stream>>>(
        (const T *)g, kLossScaleInv, w, master, dv, dm, len, lin, hyp, vec);
    c->launches++;
    return check_cuda(c, cudaGetLastError(), "weight step (rows)");
}

template <typename T>
int apply_vector_update_impl(sk_ctx *c, const sk_dense *L, const float *colsums, uint32_t batch_stat,
                             const sk_optim *lin_, const sk_optim *nrm_, float lr, float clamp, uint32_t step) {
    const Optim lin = make_optim(lin_, step), nrm = make_optim(nrm_, step);
    const Hyper hyp{lr, clamp, 1.0f / (float)batch_stat, L->regu, L->regu_coeff};
    return vector_update_launch<T>(c, L, colsums, 1, lin, nrm, hyp);
}

template <typename T>
int reduce_update_broadcast_impl(sk_ctx *c, const sk_dense *L, void *const *peer_grad, uint32_t world, uint32_t rank,
                                 void *const *peer_w, const sk_optim *lin_, float lr, float clamp, uint32_t step) {
    const Optim lin = make_optim(lin_, step);
    const Hyper hyp{lr, clamp, 1.0f, L->regu, L->regu_coeff};   // the staged gradients are already averaged
    const uint32_t rows = L->K / world;
    const size_t off = (size_t)rank * rows * L->N, len = (size_t)rows * L->N;
    PeerPtrs dst{}, src{};
    for (uint32_t r = 0; r < world; ++r) { dst.p[r] = (T *)peer_w[r] + off; src.p[r] = (T *)peer_grad[r] + off; }
    size_t blocks = (len / 8 + kRowThreads - 1) / kRowThreads;
    const size_t cap = (size_t)c->num_sms * 8;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    ProfScope ps(c, SK_PROF_UPDATE);
    reduce_update_broadcast_kernel<T><<<(uint32_t)blocks, kRowThreads, 0, c->stream>>>(
        src, world, len, master_of<T>(L->master_w, L->w) + off, L->dv_w + off, L->dm_w + off, dst, lin, hyp, c->tc_err);
    c->launches++;
    return check_cuda(c, cudaGetLastError(), "reduce + step + broadcast");
}

template <typename T>
int apply_update_impl(sk_ctx *c, const sk_dense *L, const float *dw, const float *colsums, uint32_t batch_stat,
                      const sk_optim *lin_, const sk_optim *nrm_, float lr, float clamp, uint32_t step) {
    const Optim lin = make_optim(lin_, step), nrm = make_optim(nrm_, step);
    const Hyper hyp{lr, clamp, 1.0f / (float)batch_stat, L->regu, L->regu_coeff};
    int rc = vector_update_launch<T>(c, L, colsums, 1, lin, nrm, hyp);
    if (rc) return rc;
    const size_t len = (size_t)L->K * L->N;
    float *master = master_of<T>(L->master_w, L->w);
    const bool vec = len % 4 == 0 && aligned16(dw) && aligned16(L->w) && aligned16(master) && aligned16(L->dv_w) && aligned16(L->dm_w);
    size_t blocks = (len / 4 + kRowThreads - 1) / kRowThreads;
    const size_t cap = (size_t)c->num_sms * 8;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    ProfScope ps(c, SK_PROF_UPDATE);
    weight_update_kernel<T><<<(uint32_t)blocks, kRowThreads, 0, c->stream>>>(dw, (T *)L->w, master, L->dv_w, L->dm_w, len, lin, hyp, vec);
    c->launches++;
    return check_cuda(c, cudaGetLastError(), "weight step");
}

// ---- data-parallel backward in one call ----------------------------------------------------------

// Blocks of rows a [K x N] weight matrix is exchanged in: the largest count <= wanted for which every
// rank owns whole rows of every block and its part is a whole number of 16-byte runs.
uint32_t dp_chunks_for(uint32_t K, uint32_t N, uint32_t world, uint32_t wanted) {
    if (wanted > (uint32_t)kMaxChunks) wanted = kMaxChunks;
    for (uint32_t p = wanted; p >= 1; --p)
        if (K % (p * world) == 0 && ((size_t)(K / (p * world)) * N) % 8 == 0 && (K / p) % 8 == 0) return p;
    return 0;
}

// Rows [row0, row0 + nrows) of dW = X^T . dY in the storage type, divided by batch_stat (loss scale kept).
template <typename T>
int dw_rows_lp(sk_ctx *c, const sk_dense *L, const void *x, uint32_t batch, uint32_t batch_stat, void *g, uint32_t row0,
               uint32_t nrows) {
    T *out = (T *)g + (size_t)row0 * L->N;
    EpiStoreScaled<T> epi{out, L->N, kLpScaleInv / (float)batch_stat, L->N % 8 == 0 && aligned16(out)};
    ProfScope ps(c, SK_PROF_GEMM_DW);
    int rc = check_cuda(c, run_gemm<T, T, false, true>(c, L->dtype, (const T *)x + row0, L->K, (const T *)L->d_prenorm_lp,
                                                        L->N, nrows, L->N, batch, epi), "weight gradient gemm (row block)");
    c->launches++;
    return rc;
}

template <typename T, int W>
cudaError_t launch_exchange(sk_ctx *c, const ExchangeArgs<T> &a) {
    size_t blocks = (a.len / 8 + kRowThreads - 1) / kRowThreads;
    const size_t cap = (size_t)c->num_sms * 8;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    if (a.mc_grad && a.mc_w) exchange_update_kernel<T, W, true><<<(uint32_t)blocks, kRowThreads, 0, c->stream>>>(a);
    else exchange_update_kernel<T, W, false><<<(uint32_t)blocks, kRowThreads, 0, c->stream>>>(a);
    return cudaGetLastError();
}

template <typename T>
int dp_backward_impl(sk_ctx *c, const sk_dense *const *layers, const sk_exchange *ex, uint32_t n, const void *target,
                     uint32_t target_rows, const void *x, uint32_t x_rows, uint32_t loss, uint32_t loss_act,
                     float loss_leaky, const sk_optim *lin_, const sk_optim *nrm_, uint32_t batch, uint32_t batch_stat,
                     uint32_t world, uint32_t rank, uint32_t chunks, uint32_t epoch, float lr, float clamp, uint32_t step) {
    const uint32_t last = n - 1;
    int rc = sk_output_error(c, layers[last], target, target_rows, layers[last]->max_batch, loss, loss_act, loss_leaky);
    uint32_t p_next = 0;   // blocks of layer i + 1
    for (uint32_t ii = n; ii-- > 0 && rc == SK_OK;) {
        const sk_dense *L = layers[ii];
        const sk_exchange &E = ex[ii];
        const void *in = ii == 0 ? x : layers[ii - 1]->out;
        const uint32_t in_rows = ii == 0 ? x_rows : layers[ii - 1]->max_batch;
        if ((rc = check_batch(c, L, in_rows, batch))) break;
        if (ii < last) {
            // delta of this layer from the next layer's weights: the other ranks' rows arrive block by block,
            // this rank's own rows were stepped earlier on this stream
            const sk_dense *nx = layers[ii + 1];
            const uint32_t *flags_b = reinterpret_cast<const uint32_t *>(ex[ii + 1].peer_flags[rank]) + kMaxChunks * kMaxRanks;
            TcGate gate{flags_b, world, rank, (uint32_t)kMaxRanks, p_next, nx->K / p_next, epoch};
            const bool gated = tc_eligible(c, L->dtype, nx->d_prenorm_lp, nx->N, nx->w, nx->N);
            if (!gated) {
                wait_words_kernel<<<1, 64, 0, c->stream>>>(flags_b, p_next, kMaxRanks, world, rank, epoch, c->tc_err);
                c->launches++; c->tc_launches++;
            }
            c->in_ffn_backward = true;
            rc = hidden_error_impl<T>(c, L, nx, batch, batch_stat, gated ? gate : TcGate{});
            c->in_ffn_backward = false;
            if (rc) break;
        }
        // column sums of this rank's rows into its arena (the other ranks read them in the last block's kernel)
        uint32_t nslabs = 0;
        const float *slabs = column_sum_slabs(c, L, batch, &nslabs, &rc);
        if (rc) break;
        colsum_final_kernel<<<(3 * L->N + 255) / 256, 256, 0, c->stream>>>(slabs, (float *)E.peer_colsums[rank], L->N, nslabs);
        c->launches++;
        if ((rc = check_cuda(c, cudaGetLastError(), "column sums (final)"))) break;

        const uint32_t P = dp_chunks_for(L->K, L->N, world, chunks);
        const uint32_t rows_block = L->K / P, rows_own = rows_block / world;
        const Optim lin = make_optim(&lin_[ii], step), nrm = make_optim(&nrm_[ii], step);
        ExchangeArgs<T> a{};
        PeerPtrs pf{};
        for (uint32_t r = 0; r < world; ++r) {
            a.grad.p[r] = E.peer_grad[r]; a.w.p[r] = E.peer_w[r]; a.flags.p[r] = E.peer_flags[r]; a.colsums.p[r] = E.peer_colsums[r];
            pf.p[r] = E.peer_flags[r];
        }
        a.mc_grad = E.mc_grad; a.mc_w = E.mc_w;
        a.world = world; a.rank = rank; a.epoch = epoch;
        a.master = master_of<T>(L->master_w, L->w); a.dv = L->dv_w; a.dm = L->dm_w;
        a.opt = lin; a.hyp = Hyper{lr, clamp, 1.0f, L->regu, L->regu_coeff};   // the staged gradients are already averaged
        a.err = c->tc_err; a.N = L->N;
        a.vp = vector_params<T>(L, lin, nrm, Hyper{lr, clamp, 1.0f / (float)batch_stat, L->regu, L->regu_coeff});
        auto exchange = [&](uint32_t ch) -> int {
            a.chunk = ch;
            a.off = ((size_t)ch * rows_block + (size_t)rank * rows_own) * L->N;
            a.len = (size_t)rows_own * L->N;
            a.done = c->dp_counters + ii * kMaxChunks + ch;
            a.do_vector = ch == P - 1;
            ProfScope ps(c, SK_PROF_EXCHANGE);
            cudaError_t e;
            switch (world) {
            case 2: e = launch_exchange<T, 2>(c, a); break;
            case 4: e = launch_exchange<T, 4>(c, a); break;
            case 8: e = launch_exchange<T, 8>(c, a); break;
            default: e = cudaErrorInvalidValue;
            }
            c->launches++; c->tc_launches++;
            return check_cuda(c, e, "exchange kernel");
        };
        // the exchange of a block is issued after the GEMM of the next one, so that the other ranks' flags of the
        // block have had a GEMM's time to arrive before a kernel waits for them
        for (uint32_t ch = 0; ch < P && rc == SK_OK; ++ch) {
            if ((rc = dw_rows_lp<T>(c, L, in, batch, batch_stat, E.peer_grad[rank], ch * rows_block, rows_block))) break;
            signal_chunk_kernel<<<1, 32, 0, c->stream>>>(pf, world, rank, (0 * kMaxChunks + ch) * kMaxRanks + rank, epoch);
            c->launches++;
            if (ch >= 1) rc = exchange(ch - 1);
        }
        if (rc == SK_OK) rc = exchange(P - 1);
        p_next = P;
    }
    c->fused_colsum_key = nullptr;
    if (rc) return rc;
    // the step is complete when every other rank's rows of the first layer have landed here (the deltas above
    // already waited for the other layers' rows)
    const uint32_t *flags_b0 = reinterpret_cast<const uint32_t *>(ex[0].peer_flags[rank]) + kMaxChunks * kMaxRanks;
    wait_words_kernel<<<1, 64, 0, c->stream>>>(flags_b0, p_next, kMaxRanks, world, rank, epoch, c->tc_err);
    c->launches++; c->tc_launches++;
    return check_cuda(c, cudaGetLastError(), "end of the data-parallel backward pass");
}

#define SK_DISPATCH(dtype, fn, ...)                                        \
    ((dtype) == SK_F32 ? fn<float>(__VA_ARGS__)                            \
     : (dtype) == SK_F16 ? fn<__half>(__VA_ARGS__) : fn<__nv_bfloat16>(__VA_ARGS__))

} // namespace

extern "C" {

int sk_ctx_create(int device, uint32_t tile_dim, void *stream, int create_stream, size_t workspace_bytes, sk_ctx **out) {
    if (!out) return SK_ERR_NULL_POINTER;
    *out = nullptr;
    if (tile_dim == 0 || tile_dim > 32) return SK_ERR_INVALID_CONFIGURATION;
    if (cudaSetDevice(device) != cudaSuccess) return SK_ERR_DRIVER;
    sk_ctx *c = new (std::nothrow) sk_ctx();
    if (!c) return SK_ERR_DRIVER;
    c->device = device;
    c->tile_dim = tile_dim;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) { delete c; return SK_ERR_DRIVER; }
    c->num_sms = prop.multiProcessorCount;
    // dynamic shared memory the row kernels may use for their row cache (static part left free)
    c->smem_optin = prop.sharedMemPerBlockOptin > 8192 ? prop.sharedMemPerBlockOptin - 8192 : 0;
    if (!create_stream) {
        c->stream = reinterpret_cast<cudaStream_t>(stream);
    } else {
        if (cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking) != cudaSuccess) { delete c; return SK_ERR_DRIVER; }
        c->own_stream = true;
    }
    const int optin = (int)c->smem_optin;
    cudaFuncSetAttribute(sk::norm_rows_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, optin);
    cudaFuncSetAttribute(sk::norm_rows_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, optin);
    cudaFuncSetAttribute(sk::norm_rows_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, optin);
    c->cc_major = prop.major;
    if (const char *env = getenv("SK_TC_GROUP_N")) { const int v = atoi(env); if (v >= 1 && v <= 64) c->tc_group_n = (uint32_t)v; }
    c->handover_min_rows = kHandoverMinRows;
    if (const char *env = getenv("SK_HANDOVER_MIN_ROWS")) { const int v = atoi(env); if (v >= 32) c->handover_min_rows = (uint32_t)v; }
    {
        cudaDriverEntryPointQueryResult q;
        void *fn = nullptr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            c->encode_tiled = fn;
        if (cudaMalloc(&c->tc_err, sizeof(int)) == cudaSuccess) cudaMemset(c->tc_err, 0, sizeof(int));
        else c->tc_err = nullptr;
        if (cudaMalloc(&c->dp_counters, kDpCounterWords * sizeof(uint32_t)) == cudaSuccess)
            cudaMemset(c->dp_counters, 0, kDpCounterWords * sizeof(uint32_t));
        else c->dp_counters = nullptr;
        if (cudaMalloc(&c->split_maps, kSplitMapSlots * sizeof(TcSplitMaps)) != cudaSuccess) c->split_maps = nullptr;
    }
    if (workspace_bytes == 0) workspace_bytes = (size_t)64 << 20;
    if (cudaMalloc(&c->workspace, workspace_bytes) != cudaSuccess) {
        if (c->own_stream) cudaStreamDestroy(c->stream);
        if (c->tc_err) cudaFree(c->tc_err);
        if (c->dp_counters) cudaFree(c->dp_counters);
        if (c->split_maps) cudaFree(c->split_maps);
        delete c;
        return SK_ERR_DRIVER;
    }
    c->workspace_bytes = workspace_bytes;
    *out = c;
    return SK_OK;
}

void sk_ctx_destroy(sk_ctx *c) {
    if (!c) return;
    cudaSetDevice(c->device);
    cudaStreamSynchronize(c->stream);
    if (c->workspace) cudaFree(c->workspace);
    if (c->tc_err) cudaFree(c->tc_err);
    if (c->dp_counters) cudaFree(c->dp_counters);
    if (c->split_maps) cudaFree(c->split_maps);
    for (cudaEvent_t e : c->ev_pool) cudaEventDestroy(e);
    for (auto &g : c->step_graphs) if (g.exec) cudaGraphExecDestroy(g.exec);
    if (c->record_stream) cudaStreamDestroy(c->record_stream);
    if (c->own_stream) cudaStreamDestroy(c->stream);
    delete c;
}

int sk_ctx_set_stream(sk_ctx *c, void *stream) {
    if (!c) return SK_ERR_NULL_POINTER;
    if (c->step_capturing) return step_recording(c);
    if (c->own_stream) { cudaStreamSynchronize(c->stream); cudaStreamDestroy(c->stream); c->own_stream = false; }
    c->stream = reinterpret_cast<cudaStream_t>(stream);
    return SK_OK;
}

int sk_ctx_reserve(sk_ctx *c, size_t workspace_bytes) {
    if (!c) return SK_ERR_NULL_POINTER;
    if (c->step_capturing) return step_recording(c);
    c->fused_colsum_key = nullptr;   // column sums handed over by sk_hidden_error are for the very next call only
    if (workspace_bytes <= c->workspace_bytes) return SK_OK;
    cudaSetDevice(c->device);
    cudaStreamSynchronize(c->stream);
    void *p = nullptr;
    int rc = check_cuda(c, cudaMalloc(&p, workspace_bytes), "workspace allocation");
    if (rc) return rc;
    cudaFree(c->workspace);
    c->workspace = p;
    c->workspace_bytes = workspace_bytes;
    return SK_OK;
}

int sk_sync(sk_ctx *c) {
    if (!c) return SK_ERR_NULL_POINTER;
    if (c->step_capturing) return step_recording(c);
    int rc = check_cuda(c, cudaStreamSynchronize(c->stream), "stream synchronize");
    if (rc || !c->tc_err || c->tc_launches == 0) return rc;
    int flag = 0;
    if ((rc = check_cuda(c, cudaMemcpy(&flag, c->tc_err, sizeof(int), cudaMemcpyDeviceToHost), "error flag read"))) return rc;
    if (flag != 0) {
        cudaMemset(c->tc_err, 0, sizeof(int));
        return fail(c, SK_ERR_DEVICE_TIMEOUT, "a bounded device-side wait gave up (code %d: 1 TMA loader, 2 MMA issuer, 3 GEMM epilogue, 5 peer flags)", flag);
    }
    return SK_OK;
}

int sk_step_begin(sk_ctx *c, uint32_t slot) {
    if (!c) return SK_ERR_NULL_POINTER;
    if (slot >= SK_STEP_SLOTS) return fail(c, SK_ERR_INVALID_CONFIGURATION, "step slot %u (there are %d)", slot, (int)SK_STEP_SLOTS);
    if (c->step_open >= 0) return fail(c, SK_ERR_INVALID_CONFIGURATION, "step slot %d is still open", c->step_open);
    sk_ctx::StepGraph &g = c->step_graphs[slot];
    const bool record = g.warmed && !c->profiling && !c->f32_tensor;
    g.warmed = true;
    if (record) {
        cudaSetDevice(c->device);
        int rc;
        if (!c->record_stream && (rc = check_cuda(c, cudaStreamCreateWithFlags(&c->record_stream, cudaStreamNonBlocking), "create recording stream")))
            return rc;
        if ((rc = check_cuda(c, cudaStreamBeginCapture(c->record_stream, cudaStreamCaptureModeThreadLocal), "begin stream capture"))) return rc;
        c->user_stream = c->stream;
        c->stream = c->record_stream;
    }
    c->step_open = (int)slot;
    c->step_capturing = record;
    return SK_OK;
}

int sk_step_abort(sk_ctx *c) {
    if (!c) return SK_ERR_NULL_POINTER;
    if (c->step_open < 0) return SK_OK;
    const bool recording = c->step_capturing;
    c->step_open = -1;
    c->step_capturing = false;
    if (recording) {
        cudaGraph_t graph = nullptr;
        cudaStreamEndCapture(c->record_stream, &graph);   // an invalidated capture reports an error here and is over all the same
        c->stream = c->user_stream;
        if (graph) cudaGraphDestroy(graph);
        cudaGetLastError();
    }
    return SK_OK;
}

int sk_step_end(sk_ctx *c) {
    if (!c) return SK_ERR_NULL_POINTER;
    if (c->step_open < 0) return fail(c, SK_ERR_INVALID_CONFIGURATION, "sk_step_end without sk_step_begin");
    sk_ctx::StepGraph &g = c->step_graphs[c->step_open];
    const bool recording = c->step_capturing;
    c->step_open = -1;
    c->step_capturing = false;
    if (!recording) { c->step_stats[3]++; return SK_OK; }
    cudaGraph_t graph = nullptr;
    int rc = check_cuda(c, cudaStreamEndCapture(c->record_stream, &graph), "end stream capture");
    c->stream = c->user_stream;
    if (rc) { if (graph) cudaGraphDestroy(graph); cudaGetLastError(); return rc; }
    if (g.exec) {
        cudaGraphExecUpdateResultInfo info;
        if (cudaGraphExecUpdate(g.exec, graph, &info) == cudaSuccess) {
            c->step_stats[1]++;
        } else {   // another sequence of kernels than the slot's last step
            cudaGetLastError();
            cudaGraphExecDestroy(g.exec);
            g.exec = nullptr;
        }
    }
    if (!g.exec) {
        rc = check_cuda(c, cudaGraphInstantiate(&g.exec, graph, 0), "instantiate step graph");
        if (rc) { g.exec = nullptr; cudaGraphDestroy(graph); return rc; }
        c->step_stats[0]++;
    }
    cudaGraphDestroy(graph);
    rc = check_cuda(c, cudaGraphLaunch(g.exec, c->stream), "launch step graph");
    if (!rc) c->step_stats[2]++;
    return rc;
}

int sk_step_stats(const sk_ctx *c, uint64_t out[4]) {
    if (!c || !out) return SK_ERR_NULL_POINTER;
    for (int i = 0; i < 4; ++i) out[i] = c->step_stats[i];
    return SK_OK;
}

int sk_ctx_set_option(sk_ctx *c, uint32_t option, uint32_t value) {
    if (!c) return SK_ERR_NULL_POINTER;
    if (c->step_capturing) return step_recording(c);
    if (option == SK_OPTION_GEMM_ENGINE && value <= 1) { c->gemm_engine = value; return SK_OK; }
    if (option == SK_OPTION_COLSUM_HANDOVER && value <= 1) {
        c->colsum_handover = value != 0;
        c->fused_colsum_key = nullptr;
        return SK_OK;
    }
    if (option == SK_OPTION_LEAN_BACKWARD && value <= 1) { c->lean = value != 0; return SK_OK; }
    if (option == SK_OPTION_F32_TENSOR_CORES && value <= 1) { c->f32_tensor = value != 0; return SK_OK; }
    if (option == SK_OPTION_RESERVE_SMS && value < (uint32_t)c->num_sms) { c->reserve_sms = value; return SK_OK; }
    return fail(c, SK_ERR_INVALID_CONFIGURATION, "unknown option %u / value %u", option, value);
}

const char *sk_status_string(int s) {
    switch (s) {
    case SK_OK: return "ok";
    case SK_ERR_DRIVER: return "Driver error";
    case SK_ERR_MISMATCHED_DIMENSIONS: return "Dimension mismatch";
    case SK_ERR_ALLOCATION_LIMIT: return "Allocation limit exceeded";
    case SK_ERR_INVALID_CONFIGURATION: return "Invalid network configuration";
    case SK_ERR_INVALID_BATCH_SIZE: return "Batch size constraint violation";
    case SK_ERR_TRAINING_MODE_REQUIRED: return "Action requires the network to be in training mode";
    case SK_ERR_HARDWARE_CONSTRAINT: return "Hardware acceleration constraint violation";
    case SK_ERR_UNSUPPORTED_CAST: return "Unsupported precision cast operation";
    case SK_ERR_NULL_POINTER: return "Required pointer is NULL";
    case SK_ERR_WORKSPACE: return "Scratch workspace too small";
    case SK_ERR_DEVICE_TIMEOUT: return "Device-side wait timed out";
    case SK_ERR_STATIC_LIMIT: return "Size exceeds the built-in scratch array (N may not exceed 262144 columns)";
    default: return "unknown status";
    }
}

const char *sk_last_error(const sk_ctx *c) { return c ? c->err : ""; }
uint64_t sk_launch_count(const sk_ctx *c) { return c ? c->launches : 0; }

int sk_profile_enable(sk_ctx *c, int on) {
    if (!c) return SK_ERR_NULL_POINTER;
    if (c->step_capturing) return step_recording(c);
    c->profiling = on != 0;
    if (on) {
        c->ev_used = 0;
        while (c->ev_pool.size() < 2 * 1024) {   // create events now, not inside a timed region
            cudaEvent_t a, b;
            if (cudaEventCreate(&a) != cudaSuccess || cudaEventCreate(&b) != cudaSuccess) break;
            c->ev_pool.push_back(a); c->ev_pool.push_back(b); c->ev_class.push_back(0);
        }
    }
    return SK_OK;
}

int sk_profile_read(sk_ctx *c, uint32_t cls, uint64_t *launches, double *total_ms) {
    if (!c || !launches || !total_ms) return SK_ERR_NULL_POINTER;
    if (cls >= SK_PROF_CLASSES) return fail(c, SK_ERR_INVALID_CONFIGURATION, "unknown kernel class %u", cls);
    if (c->step_capturing) return step_recording(c);
    int rc = check_cuda(c, cudaStreamSynchronize(c->stream), "stream synchronize");
    if (rc) return rc;
    *launches = 0;
    *total_ms = 0.0;
    for (size_t i = 0; i < c->ev_used; ++i) {
        if (c->ev_class[i] != cls) continue;
        float ms = 0.0f;
        if (cudaEventElapsedTime(&ms, c->ev_pool[2 * i], c->ev_pool[2 * i + 1]) == cudaSuccess) {
            *total_ms += ms;
            ++*launches;
        }
    }
    return SK_OK;
}

uint32_t sk_scramble_seed(uint32_t step, uint32_t id) {
    uint32_t h = step * 1103515245u + id;
    h = (h ^ (h >> 16)) * 1103515245u;
    return h ^ (h >> 15);
}

int sk_dense_forward(sk_ctx *c, const sk_dense *L, const void *x, uint32_t x_rows, uint32_t batch,
                     uint32_t use_dropout, uint32_t step, uint32_t row_offset) {
    int rc = check_layer(c, L, false);
    if (rc) return rc;
    if (!x) return fail(c, SK_ERR_NULL_POINTER, "input pointer is NULL");
    c->fused_colsum_key = nullptr;   // column sums handed over by sk_hidden_error are for the very next call only
    if ((rc = check_batch(c, L, x_rows, batch))) return rc;
    return SK_DISPATCH(L->dtype, forward_impl, c, L, x, batch, use_dropout, step, row_offset);
}

int sk_dense_forward_batchnorm(sk_ctx *c, const sk_dense *L, const void *x, uint32_t x_rows, uint32_t batch,
                               uint32_t batch_stat, uint32_t phase, float *stats, uint32_t use_dropout, uint32_t step,
                               uint32_t row_offset) {
    int rc = check_layer(c, L, false);
    if (rc) return rc;
    if (!x || !stats) return fail(c, SK_ERR_NULL_POINTER, "input or statistics pointer is NULL");
    c->fused_colsum_key = nullptr;
    if (L->norm != SK_NORM_BATCH) return fail(c, SK_ERR_INVALID_CONFIGURATION, "the block's normalisation is not BatchNorm");
    if (phase > 2) return fail(c, SK_ERR_INVALID_CONFIGURATION, "BatchNorm phase %u (0, 1 or 2)", phase);
    if (batch_stat < batch || batch_stat < 2)
        return fail(c, SK_ERR_INVALID_BATCH_SIZE, "BatchNorm statistics over %u rows with %u local rows", batch_stat, batch);
    if ((rc = check_batch(c, L, x_rows, batch))) return rc;
    return SK_DISPATCH(L->dtype, forward_batchnorm_impl, c, L, x, batch, batch_stat, phase, stats, use_dropout, step, row_offset);
}

int sk_output_error(sk_ctx *c, const sk_dense *L, const void *target, uint32_t target_rows, uint32_t rows,
                    uint32_t loss, uint32_t act, float leaky) {
    int rc = check_layer(c, L, true);
    if (rc) return rc;
    if (!target) return fail(c, SK_ERR_NULL_POINTER, "target pointer is NULL");
    c->fused_colsum_key = nullptr;   // column sums handed over by sk_hidden_error are for the very next call only
    if (target_rows > L->max_batch) return fail(c, SK_ERR_ALLOCATION_LIMIT, "target batches: received %u exceeds max %u", target_rows, L->max_batch);
    if (rows == 0 || rows > L->max_batch || rows > target_rows)
        return fail(c, SK_ERR_MISMATCHED_DIMENSIONS, "rows %u must be within target rows %u and max batch %u", rows, target_rows, L->max_batch);
    if (loss > 2 || act > 7) return fail(c, SK_ERR_INVALID_CONFIGURATION, "ordinal out of range");
    if (loss == SK_LOSS_MSE && act == SK_ACT_SOFTMAX)
        return fail(c, SK_ERR_INVALID_CONFIGURATION, "Mean Squared Loss does not support the Softmax activation function.");
    if (loss == SK_LOSS_CROSS_ENTROPY && act != SK_ACT_SOFTMAX)
        return fail(c, SK_ERR_INVALID_CONFIGURATION, "Cross-Entropy Loss only supports the Softmax activation function.");
    if (loss == SK_LOSS_BINARY_CROSS_ENTROPY && act != SK_ACT_SIGMOID)
        return fail(c, SK_ERR_INVALID_CONFIGURATION, "Binary Cross-Entropy only supports the Sigmoid activation function.");
    return SK_DISPATCH(L->dtype, output_error_impl, c, L, target, rows, loss, act, leaky);
}

int sk_hidden_error(sk_ctx *c, const sk_dense *cur, const sk_dense *next, uint32_t batch, uint32_t batch_stat) {
    int rc = check_layer(c, cur, true);
    if (rc) return rc;
    if ((rc = check_layer(c, next, true))) return rc;
    if (cur->dtype != next->dtype) return fail(c, SK_ERR_INVALID_CONFIGURATION, "adjacent blocks differ in precision");
    if (next->K != cur->N)
        return fail(c, SK_ERR_MISMATCHED_DIMENSIONS, "next layer rows vs current cols: expected %u, found %u", cur->N, next->K);
    if (next->max_batch < batch)
        return fail(c, SK_ERR_MISMATCHED_DIMENSIONS, "next layer gradient rows %u below batch %u", next->max_batch, batch);
    if (cur->act == SK_ACT_SOFTMAX) return fail(c, SK_ERR_INVALID_CONFIGURATION, "Softmax activation can only be passed into the compute_loss function.");
    if (batch == 0 || batch_stat == 0) return fail(c, SK_ERR_INVALID_BATCH_SIZE, "Batch size must be more than zero.");
    if (batch > cur->max_batch) return fail(c, SK_ERR_ALLOCATION_LIMIT, "batch %u exceeds max %u", batch, cur->max_batch);
    if (cur->norm == SK_NORM_BATCH && batch_stat == 1) return fail(c, SK_ERR_INVALID_BATCH_SIZE, "BatchNorm needs a batch size of more than 1.");
    return SK_DISPATCH(cur->dtype, hidden_error_impl, c, cur, next, batch, batch_stat);
}

int sk_backward_update(sk_ctx *c, const sk_dense *L, const void *x, uint32_t x_rows, uint32_t batch,
                       const sk_optim *lin, const sk_optim *nrm, float lr, float clamp, uint32_t step) {
    int rc = check_layer(c, L, true);
    if (rc) return rc;
    if (!x || !lin || !nrm) return fail(c, SK_ERR_NULL_POINTER, "input or optimiser pointer is NULL");
    if ((rc = check_batch(c, L, x_rows, batch))) return rc;
    if (lin->kind > 1 || nrm->kind > 1) return fail(c, SK_ERR_INVALID_CONFIGURATION, "optimiser ordinal out of range");
    return SK_DISPATCH(L->dtype, backward_update_impl, c, L, x, batch, lin, nrm, lr, clamp, step);
}

int sk_ffn_forward(sk_ctx *c, const sk_dense *const *layers, uint32_t n, const void *x, uint32_t x_rows, uint32_t batch,
                   uint32_t use_dropout, uint32_t step, uint32_t row_offset) {
    if (!c || !layers) return SK_ERR_NULL_POINTER;
    c->fused_colsum_key = nullptr;   // column sums handed over by sk_hidden_error are for the very next call only
    if (n == 0) return fail(c, SK_ERR_INVALID_CONFIGURATION, "Cannot execute a forward pass on an empty network");
    const void *cur = x;
    uint32_t rows = x_rows;
    for (uint32_t i = 0; i < n; ++i) {
        if (!layers[i]) return fail(c, SK_ERR_NULL_POINTER, "layer %u is NULL", i);
        if (i > 0 && layers[i]->K != layers[i - 1]->N)
            return fail(c, SK_ERR_MISMATCHED_DIMENSIONS, "forward input feature columns mismatch: expected %u, found %u",
                        layers[i]->K, layers[i - 1]->N);
        int rc = sk_dense_forward(c, layers[i], cur, rows, batch, use_dropout, step, row_offset);
        if (rc) return rc;
        cur = layers[i]->out;                 // the block's output tensor feeds the next block
        rows = layers[i]->max_batch;
    }
    return SK_OK;
}

int sk_ffn_backward(sk_ctx *c, const sk_dense *const *layers, uint32_t n, const void *target, uint32_t target_rows,
                    const void *x, uint32_t x_rows, uint32_t loss, uint32_t loss_act, float loss_leaky,
                    const sk_optim *lin, const sk_optim *nrm, uint32_t batch, float lr, float clamp, uint32_t step) {
    if (!c || !layers || !lin || !nrm) return SK_ERR_NULL_POINTER;
    if (n == 0) return fail(c, SK_ERR_INVALID_CONFIGURATION, "Backward pass on an empty network");
    for (uint32_t i = 0; i < n; ++i)
        if (!layers[i]) return fail(c, SK_ERR_NULL_POINTER, "layer %u is NULL", i);
    const uint32_t last = n - 1;
    auto input_of = [&](uint32_t i, uint32_t &rows) -> const void * {
        if (i == 0) { rows = x_rows; return x; }
        rows = layers[i - 1]->max_batch;
        return layers[i - 1]->out;
    };
    uint32_t rows = 0;
    int rc = sk_output_error(c, layers[last], target, target_rows, layers[last]->max_batch, loss, loss_act, loss_leaky);
    if (rc) return rc;
    const void *in = input_of(last, rows);
    if ((rc = sk_backward_update(c, layers[last], in, rows, batch, &lin[last], &nrm[last], lr, clamp, step))) return rc;
    for (uint32_t i = last; i-- > 0 && rc == SK_OK;) {
        c->in_ffn_backward = true;    // the update of layer i follows its delta directly: sums may be handed over
        rc = sk_hidden_error(c, layers[i], layers[i + 1], batch, batch);
        c->in_ffn_backward = false;
        if (rc) break;
        in = input_of(i, rows);
        rc = sk_backward_update(c, layers[i], in, rows, batch, &lin[i], &nrm[i], lr, clamp, step);
    }
    c->fused_colsum_key = nullptr;
    return rc;
}

int sk_backward_grads(sk_ctx *c, const sk_dense *L, const void *x, uint32_t x_rows, uint32_t batch, float *dw,
                      float *colsums) {
    int rc = check_layer(c, L, true);
    if (rc) return rc;
    if (!x || !dw || !colsums) return fail(c, SK_ERR_NULL_POINTER, "input or output pointer is NULL");
    c->fused_colsum_key = nullptr;   // column sums handed over by sk_hidden_error are for the very next call only
    if ((rc = check_batch(c, L, x_rows, batch))) return rc;
    return SK_DISPATCH(L->dtype, backward_grads_impl, c, L, x, batch, dw, colsums);
}

int sk_apply_update(sk_ctx *c, const sk_dense *L, const float *dw, const float *colsums, uint32_t batch_stat,
                    const sk_optim *lin, const sk_optim *nrm, float lr, float clamp, uint32_t step) {
    int rc = check_layer(c, L, true);
    if (rc) return rc;
    if (!dw || !colsums || !lin || !nrm) return fail(c, SK_ERR_NULL_POINTER, "gradient or optimiser pointer is NULL");
    c->fused_colsum_key = nullptr;   // column sums handed over by sk_hidden_error are for the very next call only
    if (batch_stat == 0) return fail(c, SK_ERR_INVALID_BATCH_SIZE, "Batch size must be more than zero.");
    if (lin->kind > 1 || nrm->kind > 1) return fail(c, SK_ERR_INVALID_CONFIGURATION, "optimiser ordinal out of range");
    return SK_DISPATCH(L->dtype, apply_update_impl, c, L, dw, colsums, batch_stat, lin, nrm, lr, clamp, step);
}

int sk_backward_grads_lp(sk_ctx *c, const sk_dense *L, const void *x, uint32_t x_rows, uint32_t batch,
                         uint32_t batch_stat, void *grad, float *colsums) {
    int rc = check_layer(c, L, true);
    if (rc) return rc;
    if (!x || !grad || !colsums) return fail(c, SK_ERR_NULL_POINTER, "input or output pointer is NULL");
    if ((rc = check_batch(c, L, x_rows, batch))) return rc;
    if (batch_stat == 0) return fail(c, SK_ERR_INVALID_BATCH_SIZE, "Batch size must be more than zero.");
    return SK_DISPATCH(L->dtype, backward_grads_lp_impl, c, L, x, batch, batch_stat, grad, colsums);
}

int sk_apply_update_rows(sk_ctx *c, const sk_dense *L, const void *grad, uint32_t row0, uint32_t nrows,
                         const sk_optim *lin, float lr, float clamp, uint32_t step) {
    int rc = check_layer(c, L, true);
    if (rc) return rc;
    if (!grad || !lin) return fail(c, SK_ERR_NULL_POINTER, "gradient or optimiser pointer is NULL");
    c->fused_colsum_key = nullptr;   // column sums handed over by sk_hidden_error are for the very next call only
    if (nrows == 0 || (uint64_t)row0 + nrows > L->K)
        return fail(c, SK_ERR_MISMATCHED_DIMENSIONS, "rows [%u, %u) outside the %u rows of the weight matrix", row0, row0 + nrows, L->K);
    if (lin->kind > 1) return fail(c, SK_ERR_INVALID_CONFIGURATION, "optimiser ordinal out of range");
    return SK_DISPATCH(L->dtype, apply_update_rows_impl, c, L, grad, row0, nrows, lin, lr, clamp, step);
}

int sk_apply_vector_update(sk_ctx *c, const sk_dense *L, const float *colsums, uint32_t batch_stat,
                           const sk_optim *lin, const sk_optim *nrm, float lr, float clamp, uint32_t step) {
    int rc = check_layer(c, L, true);
    if (rc) return rc;
    if (!colsums || !lin || !nrm) return fail(c, SK_ERR_NULL_POINTER, "column sums or optimiser pointer is NULL");
    c->fused_colsum_key = nullptr;   // column sums handed over by sk_hidden_error are for the very next call only
    if (batch_stat == 0) return fail(c, SK_ERR_INVALID_BATCH_SIZE, "Batch size must be more than zero.");
    if (lin->kind > 1 || nrm->kind > 1) return fail(c, SK_ERR_INVALID_CONFIGURATION, "optimiser ordinal out of range");
    return SK_DISPATCH(L->dtype, apply_vector_update_impl, c, L, colsums, batch_stat, lin, nrm, lr, clamp, step);
}

static int check_exchange(sk_ctx *c, const sk_dense *L, void *const *ptrs, uint32_t world, uint32_t rank) {
    if (!ptrs) return fail(c, SK_ERR_NULL_POINTER, "peer pointer table is NULL");
    if (world == 0 || world > (uint32_t)sk::kMaxRanks || rank >= world)
        return fail(c, SK_ERR_INVALID_CONFIGURATION, "rank %u of %u ranks (at most %d)", rank, world, sk::kMaxRanks);
    if (L->dtype == SK_F32) return fail(c, SK_ERR_INVALID_CONFIGURATION, "the fused exchange carries 16-bit gradients only");
    if (L->K % world != 0 || ((size_t)(L->K / world) * L->N) % 8 != 0)
        return fail(c, SK_ERR_MISMATCHED_DIMENSIONS, "%u weight rows do not split over %u ranks in whole 16-byte runs", L->K, world);
    for (uint32_t r = 0; r < world; ++r)
        if (!ptrs[r] || reinterpret_cast<uintptr_t>(ptrs[r]) % 16 != 0) return fail(c, SK_ERR_NULL_POINTER, "peer pointer %u is NULL or unaligned", r);
    return SK_OK;
}

int sk_reduce_update_broadcast(sk_ctx *c, const sk_dense *L, void *const *peer_grad, uint32_t world, uint32_t rank,
                               void *const *peer_w, const sk_optim *lin, float lr, float clamp, uint32_t step) {
    int rc = check_layer(c, L, true);
    if (rc) return rc;
    if (!lin) return fail(c, SK_ERR_NULL_POINTER, "optimiser pointer is NULL");
    c->fused_colsum_key = nullptr;   // column sums handed over by sk_hidden_error are for the very next call only
    if (lin->kind > 1) return fail(c, SK_ERR_INVALID_CONFIGURATION, "optimiser ordinal out of range");
    if ((rc = check_exchange(c, L, peer_grad, world, rank))) return rc;
    if ((rc = check_exchange(c, L, peer_w, world, rank))) return rc;
    return SK_DISPATCH(L->dtype, reduce_update_broadcast_impl, c, L, peer_grad, world, rank, peer_w, lin, lr, clamp, step);
}

uint32_t sk_dp_blocks(uint32_t K, uint32_t N, uint32_t world, uint32_t wanted) {
    if (world == 0 || wanted == 0) return 0;
    return dp_chunks_for(K, N, world, wanted);
}

uint32_t sk_dp_flag_bytes(void) { return (uint32_t)(kFlagWordsPerLayer * sizeof(uint32_t)); }

int sk_dp_backward(sk_ctx *c, const sk_dense *const *layers, const sk_exchange *ex, uint32_t n, const void *target,
                   uint32_t target_rows, const void *x, uint32_t x_rows, uint32_t loss, uint32_t loss_act, float loss_leaky,
                   const sk_optim *lin, const sk_optim *nrm, uint32_t batch, uint32_t batch_stat, uint32_t world,
                   uint32_t rank, uint32_t blocks, uint32_t epoch, float lr, float clamp, uint32_t step) {
    if (!c || !layers || !ex || !lin || !nrm || !target || !x) return SK_ERR_NULL_POINTER;
    if (n == 0 || n > kDpMaxLayers) return fail(c, SK_ERR_INVALID_CONFIGURATION, "1 to %u layers", kDpMaxLayers);
    if (!(world == 2 || world == 4 || world == 8) || rank >= world)
        return fail(c, SK_ERR_INVALID_CONFIGURATION, "rank %u of %u ranks (2, 4 or 8)", rank, world);
    if (blocks == 0) blocks = 1;
    if (batch == 0 || batch_stat < batch) return fail(c, SK_ERR_INVALID_BATCH_SIZE, "local batch %u of %u rows", batch, batch_stat);
    if (!c->tc_err || !c->dp_counters) return fail(c, SK_ERR_DRIVER, "context has no device error word / counters");
    for (uint32_t i = 0; i < n; ++i) {
        if (!layers[i]) return fail(c, SK_ERR_NULL_POINTER, "layer %u is NULL", i);
        int rc = check_layer(c, layers[i], true);
        if (rc) return rc;
        const sk_dense *L = layers[i];
        if (L->dtype == SK_F32 || L->dtype != layers[0]->dtype)
            return fail(c, SK_ERR_INVALID_CONFIGURATION, "the native exchange carries 16-bit blocks of one precision");
        if (L->norm == SK_NORM_BATCH) return fail(c, SK_ERR_INVALID_CONFIGURATION, "BatchNorm blocks use the phased exchange");
        if (i > 0 && L->K != layers[i - 1]->N)
            return fail(c, SK_ERR_MISMATCHED_DIMENSIONS, "layer %u rows vs layer %u cols: expected %u, found %u", i, i - 1, layers[i - 1]->N, L->K);
        if (lin[i].kind > 1 || nrm[i].kind > 1) return fail(c, SK_ERR_INVALID_CONFIGURATION, "optimiser ordinal out of range");
        if (dp_chunks_for(L->K, L->N, world, blocks) == 0)
            return fail(c, SK_ERR_MISMATCHED_DIMENSIONS, "%u weight rows do not split over %u ranks in whole 16-byte runs", L->K, world);
        if (!ex[i].peer_grad || !ex[i].peer_w || !ex[i].peer_flags || !ex[i].peer_colsums)
            return fail(c, SK_ERR_NULL_POINTER, "exchange tables of layer %u", i);
        for (uint32_t r = 0; r < world; ++r)
            if (!ex[i].peer_grad[r] || !ex[i].peer_w[r] || !ex[i].peer_flags[r] || !ex[i].peer_colsums[r] ||
                reinterpret_cast<uintptr_t>(ex[i].peer_grad[r]) % 16 || reinterpret_cast<uintptr_t>(ex[i].peer_w[r]) % 16 ||
                reinterpret_cast<uintptr_t>(ex[i].peer_colsums[r]) % 16)
                return fail(c, SK_ERR_NULL_POINTER, "exchange pointer of layer %u, rank %u is NULL or unaligned", i, r);
        if (ex[i].peer_w[rank] != L->w) return fail(c, SK_ERR_INVALID_CONFIGURATION, "layer %u: the weight tensor must be this rank's entry of peer_w", i);
    }
    if (cudaSetDevice(c->device) != cudaSuccess) return fail(c, SK_ERR_DRIVER, "cannot select device %d", c->device);
    c->fused_colsum_key = nullptr;
    return layers[0]->dtype == SK_F16
               ? dp_backward_impl<__half>(c, layers, ex, n, target, target_rows, x, x_rows, loss, loss_act, loss_leaky, lin, nrm,
                                          batch, batch_stat, world, rank, blocks, epoch, lr, clamp, step)
               : dp_backward_impl<__nv_bfloat16>(c, layers, ex, n, target, target_rows, x, x_rows, loss, loss_act, loss_leaky,
                                                 lin, nrm, batch, batch_stat, world, rank, blocks, epoch, lr, clamp, step);
}

int sk_peer_alloc(sk_ctx *c, size_t bytes, void **ptr, unsigned char handle_out[64]) {
    if (!c || !ptr || !handle_out) return SK_ERR_NULL_POINTER;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    if (cudaSetDevice(c->device) != cudaSuccess) return fail(c, SK_ERR_DRIVER, "cannot select device %d", c->device);
    void *p = nullptr;
    int rc = check_cuda(c, cudaMalloc(&p, bytes), "exchange arena allocation");
    if (rc) return rc;
    if ((rc = check_cuda(c, cudaMemset(p, 0, bytes), "exchange arena clear"))) { cudaFree(p); return rc; }
    cudaIpcMemHandle_t h;
    if ((rc = check_cuda(c, cudaIpcGetMemHandle(&h, p), "export exchange arena"))) { cudaFree(p); return rc; }
    memcpy(handle_out, &h, 64);
    *ptr = p;
    return SK_OK;
}

int sk_peer_open(sk_ctx *c, const unsigned char handle[64], void **ptr) {
    if (!c || !ptr || !handle) return SK_ERR_NULL_POINTER;
    if (cudaSetDevice(c->device) != cudaSuccess) return fail(c, SK_ERR_DRIVER, "cannot select device %d", c->device);
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, 64);
    void *p = nullptr;
    int rc = check_cuda(c, cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess), "map a peer's exchange arena");
    if (rc) return rc;
    // host-side sanity: the mapping must be device memory that kernels of this device may dereference
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, p) != cudaSuccess || attr.type != cudaMemoryTypeDevice) {
        cudaGetLastError();
        cudaIpcCloseMemHandle(p);
        return fail(c, SK_ERR_DRIVER, "peer mapping is not device memory");
    }
    if (attr.device != c->device) {
        int can = 0;
        if (cudaDeviceCanAccessPeer(&can, c->device, attr.device) != cudaSuccess || !can) {
            cudaGetLastError();
            cudaIpcCloseMemHandle(p);
            return fail(c, SK_ERR_DRIVER, "device %d cannot access memory of device %d", c->device, attr.device);
        }
        cudaError_t e = cudaDeviceEnablePeerAccess(attr.device, 0);
        if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) { cudaIpcCloseMemHandle(p); return check_cuda(c, e, "enable peer access"); }
        cudaGetLastError();
    }
    *ptr = p;
    return SK_OK;
}

int sk_peer_close(sk_ctx *c, void *ptr) {
    if (!c || !ptr) return SK_ERR_NULL_POINTER;
    cudaSetDevice(c->device);
    return check_cuda(c, cudaIpcCloseMemHandle(ptr), "unmap a peer's exchange arena");
}

int sk_peer_free(sk_ctx *c, void *ptr) {
    if (!c || !ptr) return SK_ERR_NULL_POINTER;
    cudaSetDevice(c->device);
    cudaStreamSynchronize(c->stream);
    return check_cuda(c, cudaFree(ptr), "free exchange arena");
}

int sk_copy(sk_ctx *c, void *dst, const void *src, size_t bytes) {
    if (!c || !dst || !src) return SK_ERR_NULL_POINTER;
    c->fused_colsum_key = nullptr;   // column sums handed over by sk_hidden_error are for the very next call only
    return check_cuda(c, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, c->stream), "device copy");
}

int sk_signal_peers(sk_ctx *c, void *const *peer_flags, uint32_t world, uint32_t slot, uint32_t value) {
    if (!c || !peer_flags) return SK_ERR_NULL_POINTER;
    if (world == 0 || world > (uint32_t)sk::kMaxRanks) return fail(c, SK_ERR_INVALID_CONFIGURATION, "at most %d ranks", sk::kMaxRanks);
    sk::PeerPtrs f{};
    for (uint32_t r = 0; r < world; ++r) {
        if (!peer_flags[r]) return fail(c, SK_ERR_NULL_POINTER, "flag pointer %u is NULL", r);
        f.p[r] = peer_flags[r];
    }
    sk::signal_peers_kernel<<<1, 32, 0, c->stream>>>(f, world, slot, value);
    c->launches++;
    return check_cuda(c, cudaGetLastError(), "signal peers");
}

int sk_wait_flags(sk_ctx *c, const uint32_t *flags, uint32_t world, uint32_t value) {
    if (!c || !flags) return SK_ERR_NULL_POINTER;
    if (world == 0 || world > (uint32_t)sk::kMaxRanks || !c->tc_err) return fail(c, SK_ERR_INVALID_CONFIGURATION, "at most %d ranks", sk::kMaxRanks);
    sk::wait_flags_kernel<<<1, 32, 0, c->stream>>>(flags, world, value, c->tc_err);
    c->launches++;
    c->tc_launches++;   // makes sk_sync read the error word
    return check_cuda(c, cudaGetLastError(), "wait for peers");
}

int sk_cast(sk_ctx *c, const void *src, uint32_t sd, void *dst, uint32_t dd, size_t len) {
    if (!c || !src || !dst) return SK_ERR_NULL_POINTER;
    c->fused_colsum_key = nullptr;   // column sums handed over by sk_hidden_error are for the very next call only
    if (len == 0) return SK_OK;
    size_t blocks = (len + 1023) / 1024;
    const size_t cap = (size_t)c->num_sms * 16;
    if (blocks > cap) blocks = cap;
    const uint32_t g = (uint32_t)blocks;
    if (sd == SK_F32 && dd == SK_F16) sk::cast_kernel<float, __half><<<g, 256, 0, c->stream>>>((const float *)src, (__half *)dst, len);
    else if (sd == SK_F16 && dd == SK_F32) sk::cast_kernel<__half, float><<<g, 256, 0, c->stream>>>((const __half *)src, (float *)dst, len);
    else if (sd == SK_F32 && dd == SK_BF16) sk::cast_kernel<float, __nv_bfloat16><<<g, 256, 0, c->stream>>>((const float *)src, (__nv_bfloat16 *)dst, len);
    else if (sd == SK_BF16 && dd == SK_F32) sk::cast_kernel<__nv_bfloat16, float><<<g, 256, 0, c->stream>>>((const __nv_bfloat16 *)src, (float *)dst, len);
    else return fail(c, SK_ERR_UNSUPPORTED_CAST, "cannot convert dtype %u to %u", sd, dd);
    c->launches++;
    return check_cuda(c, cudaGetLastError(), "cast");
}

int sk_fill(sk_ctx *c, void *dst, uint32_t dtype, float value, size_t len) {
    if (!c || !dst) return SK_ERR_NULL_POINTER;
    c->fused_colsum_key = nullptr;   // column sums handed over by sk_hidden_error are for the very next call only
    if (len == 0) return SK_OK;
    size_t blocks = (len + 1023) / 1024;
    const size_t cap = (size_t)c->num_sms * 16;
    if (blocks > cap) blocks = cap;
    const uint32_t g = (uint32_t)blocks;
    if (dtype == SK_F32) sk::fill_kernel<float><<<g, 256, 0, c->stream>>>((float *)dst, value, len);
    else if (dtype == SK_F16) sk::fill_kernel<__half><<<g, 256, 0, c->stream>>>((__half *)dst, value, len);
    else if (dtype == SK_BF16) sk::fill_kernel<__nv_bfloat16><<<g, 256, 0, c->stream>>>((__nv_bfloat16 *)dst, value, len);
    else return fail(c, SK_ERR_INVALID_CONFIGURATION, "unknown dtype %u", dtype);
    c->launches++;
    return check_cuda(c, cudaGetLastError(), "fill");
}

} // extern "C"
