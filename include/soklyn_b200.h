/*
 * soklyn_b200 — C ABI of the B200 (sm_100a) DenseBlock / FeedForwardNetwork hot path.
 *
 * This is the boundary a host binding (Rust `extern "C"`, ctypes, ...) calls in place of
 * the reference's PTX-module launches: every entry point below replaces one
 * `GpuContext::gpu_*` method of Felix1G/soklyn and cites it. All pointers in `sk_dense`
 * are DEVICE pointers borrowed for the duration of the call; the library never frees or
 * keeps them. Calls are ordered on the context's stream and return without waiting for
 * the GPU; `sk_sync` waits. No entry point allocates device memory after `sk_ctx_create`
 * / `sk_ctx_reserve`.
 *
 * Matrices are row-major. Ordinals are the reference's kernel ABI
 * (src/util/function.rs:33-39,65-72,104-116,153-164; LossFunc `as u32`).
 */
#ifndef SOKLYN_B200_H
#define SOKLYN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes; the non-zero ones map onto the variants of src/util/log.rs:15-99. */
enum {
    SK_OK = 0,
    SK_ERR_DRIVER = 1,                 /* Error::DriverError */
    SK_ERR_MISMATCHED_DIMENSIONS = 2,  /* Error::MismatchedDimensions */
    SK_ERR_ALLOCATION_LIMIT = 3,       /* Error::AllocationLimitExceeded */
    SK_ERR_INVALID_CONFIGURATION = 4,  /* Error::InvalidConfiguration */
    SK_ERR_INVALID_BATCH_SIZE = 5,     /* Error::InvalidBatchSize */
    SK_ERR_TRAINING_MODE_REQUIRED = 6, /* Error::TrainingModeRequired */
    SK_ERR_HARDWARE_CONSTRAINT = 7,    /* Error::HardwareConstraintViolation */
    SK_ERR_UNSUPPORTED_CAST = 8,       /* Error::UnsupportedTypeCast */
    SK_ERR_NULL_POINTER = 9,           /* no counterpart: a required pointer is NULL */
    SK_ERR_WORKSPACE = 10,             /* no counterpart: scratch workspace too small */
    SK_ERR_DEVICE_TIMEOUT = 11,        /* no counterpart: a bounded device-side wait gave up */
    SK_ERR_STATIC_LIMIT = 12           /* no counterpart: size beyond the built-in scratch of sk_column_sums_static */
};

enum { SK_F32 = 0, SK_F16 = 1, SK_BF16 = 2 };
enum { SK_ACT_IDENTITY = 0, SK_ACT_SIGMOID = 1, SK_ACT_RELU = 2, SK_ACT_LEAKY_RELU = 3,
       SK_ACT_TANH = 4, SK_ACT_SOFTMAX = 5, SK_ACT_SILU = 6, SK_ACT_MISH = 7 };
enum { SK_NORM_DISABLED = 0, SK_NORM_RMS = 1, SK_NORM_LAYER = 2, SK_NORM_BATCH = 3 };
enum { SK_OPT_SGD = 0, SK_OPT_ADAM = 1 };
enum { SK_REGU_NONE = 0, SK_REGU_L1 = 1, SK_REGU_L2 = 2 };
enum { SK_LOSS_MSE = 0, SK_LOSS_CROSS_ENTROPY = 1, SK_LOSS_BINARY_CROSS_ENTROPY = 2 };

typedef struct sk_ctx sk_ctx;

/* Optimiser hyper-parameters as src/io/device/ffn_device.rs:254-269 unpacks them:
 * SGD{v_coeff, nesterov} -> (beta1, 0, 0, nesterov); Adam{m_coeff, v_coeff, epsilon}
 * -> (beta1, beta2, epsilon, 0). */
typedef struct {
    uint32_t kind;
    float beta1, beta2, epsilon;
    uint32_t nesterov;
} sk_optim;

/* One DenseBlock's device state (src/mlp.rs:14-24, :232-241, :268-288). `T` below is
 * the storage type named by `dtype`. In f32 mode the master_* pointers may be NULL or
 * alias the parameter itself, as src/io/device.rs:262-272 does. Gradient-side pointers
 * may be NULL for an inference-only block (is_training == 0). */
typedef struct {
    uint32_t dtype;                 /* SK_F32 / SK_F16 / SK_BF16 */
    uint32_t K, N, max_batch;       /* inputs, outputs, rows of every cache tensor */
    uint32_t is_training;
    void *w, *b;                    /* T [K x N], T [N] */
    float *master_w, *master_b;     /* f32 copies (16-bit modes) */
    float *dv_w, *dv_b, *dm_w, *dm_b;
    void *norm_w, *norm_b;          /* T [N] */
    float *master_norm_w, *master_norm_b;
    float *dv_norm_w, *dv_norm_b, *dm_norm_w, *dm_norm_b;
    void *out, *predrop, *preact, *centered, *prenorm; /* T [max_batch x N] */
    void *norm_rstd;                /* T [max(max_batch, N)] */
    void *mask;                     /* T [max_batch x N] */
    float *grad, *d_prenorm, *d_norm_w, *d_norm_b;     /* f32 [max_batch x N] */
    void *d_prenorm_lp;             /* T [max_batch x N]: 16-bit copy of d_prenorm feeding the
                                       tensor-core GEMMs; required in 16-bit modes, unused in f32 */
    uint32_t norm, act;
    float leaky_coeff;
    uint32_t regu;
    float regu_coeff, mask_coeff;
    uint32_t tensor_id;             /* id of `w` (src/util/core.rs:84-88); seeds the dropout hash */
} sk_dense;

/* GpuContext::with_device_index (src/io/device.rs:164-183). tile_dim is kept for API
 * compatibility: 16-bit modes still require 16 (src/io/device.rs:248-258), the kernels
 * ignore it. With create_stream != 0 the context creates (and owns) a non-blocking stream,
 * as the reference's GpuContext does; otherwise calls are ordered on the cudaStream_t
 * `stream`, where NULL is the legacy default stream. workspace_bytes of scratch are
 * allocated here (0 = default 64 MiB). Two tuning values are read from the environment here: SK_TC_GROUP_N
 * (tile columns the tensor-core kernels walk together, default 8) and SK_HANDOVER_MIN_ROWS (rows per call from
 * which a hidden block's column sums are taken in the dX epilogue, default 512). */
int sk_ctx_create(int device, uint32_t tile_dim, void *stream, int create_stream, size_t workspace_bytes,
                  sk_ctx **out);
void sk_ctx_destroy(sk_ctx *ctx);
/* Replace the stream later calls are ordered on (no counterpart; the reference owns one stream). */
int sk_ctx_set_stream(sk_ctx *ctx, void *stream);
/* Context options (no counterpart). SK_OPTION_GEMM_ENGINE: 0 = automatic (tcgen05 tensor-core
 * kernel for 16-bit operands whose row pitches are multiples of 16 bytes, FFMA kernel
 * otherwise), 1 = FFMA kernel only.
 * SK_OPTION_COLSUM_HANDOVER: 1 = sk_hidden_error may take the column sums of the layer's d_prenorm /
 * d_norm_w / d_norm_b in its GEMM epilogue and hand them, through the workspace, to the next call if
 * that call is sk_backward_update / sk_backward_grads_lp for the same layer and batch (any other call
 * drops them). The caller promises not to modify those three tensors between the two calls. Off by
 * default; sk_ffn_backward always does this internally, where nothing can come in between.
 * SK_OPTION_LEAN_BACKWARD: 1 = a hidden block whose column sums are taken in the dX epilogue (16-bit,
 * batch >= 512, SiLU+RMSNorm or Mish+LayerNorm) does not store grad, the f32 d_prenorm, d_norm_w and
 * d_norm_b (src/mlp.rs:273-276): nothing in the backward pass reads them again, the GEMMs read the
 * 16-bit d_prenorm_lp. A deviation from the reference, whose getters expose those tensors
 * (src/mlp.rs:446-454): they keep stale contents. Parameters come out bit-identical. Off by default.
 * SK_OPTION_RESERVE_SMS: number of SMs the tensor-core GEMMs leave free, so that a kernel on another
 * stream can run beside them. 0 by default.
 * SK_OPTION_F32_TENSOR_CORES: 1 = f32 products large enough to pay for it (M*N*K >= 2^28, row pitches multiples
 * of 8 elements) run on the tensor cores: both operands are split into three bf16 parts (8 + 8 + 8 significant
 * bits) in the workspace, the six leading partial products are multiplied on the tensor cores and summed over K
 * in registers with round-to-nearest f32 adds, because the tensor pipe truncates when it adds into its own
 * accumulator (src/cuda/kernel/math.cu:8-50 is the FFMA loop this stands in for). Needs 6 bytes of workspace per operand element (sk_ctx_reserve); a
 * product whose parts do not fit runs on the FFMA kernel. Results differ from the FFMA kernel's in the order
 * and rounding of the f32 sums: a single product by up to 3e-6 of its largest element. Off by default. */
enum { SK_OPTION_GEMM_ENGINE = 0, SK_OPTION_COLSUM_HANDOVER = 1, SK_OPTION_LEAN_BACKWARD = 2, SK_OPTION_RESERVE_SMS = 3,
       SK_OPTION_F32_TENSOR_CORES = 4 };
int sk_ctx_set_option(sk_ctx *ctx, uint32_t option, uint32_t value);
/* Grow the scratch workspace; never called implicitly. */
int sk_ctx_reserve(sk_ctx *ctx, size_t workspace_bytes);
/* CudaStream::synchronize as called after every launch in src/io/device/ffn_device.rs:75,110,136.
 * Also reports SK_ERR_DEVICE_TIMEOUT if a tensor-core kernel abandoned a bounded wait. */
int sk_sync(sk_ctx *ctx);
/* Text for a status code, and the detail of the last failure on this context. */
const char *sk_status_string(int status);
const char *sk_last_error(const sk_ctx *ctx);
/* Number of kernels this context has launched since creation (for launch accounting). */
uint64_t sk_launch_count(const sk_ctx *ctx);

/* Whole-step graphs for the launch-bound small networks (no counterpart: the reference launches every kernel
 * by itself and waits for it, src/io/device/ffn_device.rs:75,110,136). The sk_* calls a host makes between
 * sk_step_begin and sk_step_end are recorded by CUDA stream capture (on a stream of the context's own, so the
 * caller's may be the legacy default stream) instead of being launched one by one; sk_step_end turns the record
 * into an executable graph and launches it on the context's stream. Every
 * step is recorded afresh, so kernel arguments that change from step to step (the step number and Adam's bias
 * corrections, the learning rate, the dropout seed, input pointers) need no care; when the sequence of kernels is
 * the one of the slot's previous step, its executable graph is updated in place (cudaGraphExecUpdate), else it is
 * instantiated anew. `slot` (< SK_STEP_SLOTS) names the executable graph to reuse: one per network or phase that
 * alternates on the context. Results are those of the same calls made without the bracket, bit for bit.
 * The first step of a slot runs unrecorded (first launches set function attributes and build tensor maps), and
 * so does every step while profiling or SK_OPTION_F32_TENSOR_CORES is on. Between begin and end the host must
 * not wait for the stream or read results: sk_sync, sk_profile_read, sk_ctx_reserve and sk_ctx_set_stream
 * refuse with SK_ERR_INVALID_CONFIGURATION. If a call in between fails, sk_step_abort drops the record (nothing
 * of the step has run then) and leaves the stream usable. sk_step_stats: out[0] graphs instantiated, out[1]
 * updated in place, out[2] launched, out[3] steps that ran unrecorded. */
enum { SK_STEP_SLOTS = 8 };
int sk_step_begin(sk_ctx *ctx, uint32_t slot);
int sk_step_end(sk_ctx *ctx);
int sk_step_abort(sk_ctx *ctx);
int sk_step_stats(const sk_ctx *ctx, uint64_t out[4]);

/* Per-kernel-class device timing (no counterpart; the reference times phases on the host,
 * examples/mnist_train.rs:180-195). While enabled, every launch of the classes below is
 * bracketed by CUDA events on the context's stream; sk_profile_read waits for the stream and
 * returns launches and total milliseconds of one class since sk_profile_enable(ctx, 1). */
enum { SK_PROF_GEMM_FORWARD = 0, SK_PROF_GEMM_DX = 1, SK_PROF_GEMM_DW = 2, SK_PROF_NORM = 3,
       SK_PROF_OUTPUT_ERROR = 4, SK_PROF_COLSUM = 5, SK_PROF_UPDATE = 6, SK_PROF_EXCHANGE = 7, SK_PROF_CLASSES = 8 };
int sk_profile_enable(sk_ctx *ctx, int on);
int sk_profile_read(sk_ctx *ctx, uint32_t kernel_class, uint64_t *launches, double *total_ms);

/* scramble_seed (src/util/core.rs:90-94). */
uint32_t sk_scramble_seed(uint32_t step, uint32_t tensor_id);

/* GpuContext::gpu_forward_pass (src/io/device/ffn_device.rs:12-139), with the checks of
 * DenseBlock::forward (src/mlp.rs:492-580). x is T [x_rows x K]; the first `batch` rows are
 * used. row_offset is added to the row index hashed by dropout (0 on one device; the first
 * global row of this shard under data parallelism). */
int sk_dense_forward(sk_ctx *ctx, const sk_dense *layer, const void *x, uint32_t x_rows,
                     uint32_t batch, uint32_t use_dropout, uint32_t step, uint32_t row_offset);

/* BatchNorm forward for a batch whose rows are split over several devices (no counterpart: the
 * reference is single-device; arithmetic of src/cuda/kernel/forward.cu's BatchNorm branch with the
 * column statistics taken over all batch_stat rows). stats is device f32 [2 x N]. Three calls with
 * the same arguments, the caller summing over ranks in between:
 *   phase 0: GEMM into prenorm; stats[0][col] = this shard's sum of x          -> sum stats[0] over ranks
 *   phase 1: stats[1][col] = this shard's sum of (x - mean)^2                  -> sum stats[1] over ranks
 *   phase 2: centered, rstd, preact, activation and dropout from the summed statistics.
 * The backward entry points already take batch_stat for BatchNorm's 1/M. */
int sk_dense_forward_batchnorm(sk_ctx *ctx, const sk_dense *layer, const void *x, uint32_t x_rows, uint32_t batch,
                               uint32_t batch_stat, uint32_t phase, float *stats, uint32_t use_dropout,
                               uint32_t step, uint32_t row_offset);

/* GpuContext::gpu_compute_output_layer_error (src/io/device/ffn_device.rs:141-231) with the
 * checks of DenseBlock::compute_loss (src/mlp.rs:756-821). Works on `rows` rows of the block's
 * `out` (the reference always passes out.rows() == max_batch); target is T [>= rows x N].
 * Softmax is applied to `out` in place. */
int sk_output_error(sk_ctx *ctx, const sk_dense *layer, const void *target, uint32_t target_rows,
                    uint32_t rows, uint32_t loss, uint32_t act, float leaky_coeff);

/* First half of GpuContext::gpu_hidden_layer_backward_pass (src/io/device/ffn_device.rs:360-436):
 * delta of `cur` from next.d_prenorm and next's (already updated) weights. batch_stat is the
 * batch size used for BatchNorm's 1/M (the whole batch under data parallelism). */
int sk_hidden_error(sk_ctx *ctx, const sk_dense *cur, const sk_dense *next, uint32_t batch,
                    uint32_t batch_stat);

/* GpuContext::gpu_backward_pass (src/io/device/ffn_device.rs:234-358) with the checks of
 * DenseBlock::backward_output (src/mlp.rs:607-642): dW, dB, sum dNorm and the in-place optimiser
 * step. x is T [x_rows x K] (the block's forward input). */
int sk_backward_update(sk_ctx *ctx, const sk_dense *layer, const void *x, uint32_t x_rows,
                       uint32_t batch, const sk_optim *linear, const sk_optim *norm_opt,
                       float learn_rate, float grad_clamp, uint32_t step);

/* FeedForwardNetwork::forward (src/ffn.rs:40-57) and ::backward (src/ffn.rs:113-166) for a stack of
 * blocks in one call: the same per-layer entry points in the reference's order (output layer
 * first, every hidden delta after the next layer's update), sequenced in native code so that
 * small networks are not bound by per-call host overhead. layers[i+1].K must equal layers[i].N;
 * linear / norm_opt are arrays of n_layers optimisers. */
int sk_ffn_forward(sk_ctx *ctx, const sk_dense *const *layers, uint32_t n_layers, const void *x, uint32_t x_rows,
                   uint32_t batch, uint32_t use_dropout, uint32_t step, uint32_t row_offset);
int sk_ffn_backward(sk_ctx *ctx, const sk_dense *const *layers, uint32_t n_layers, const void *target,
                    uint32_t target_rows, const void *x, uint32_t x_rows, uint32_t loss, uint32_t loss_act,
                    float loss_leaky, const sk_optim *linear, const sk_optim *norm_opt, uint32_t batch,
                    float learn_rate, float grad_clamp, uint32_t step);

/* The two halves of sk_backward_update, for data parallelism (no counterpart in the
 * reference, which is single-device): sk_backward_grads writes the raw batch sums
 * dW f32 [K x N] and colsums f32 [3 x N] (dB, sum dNorm_w, sum dNorm_b; still x512) so
 * that they can be summed across ranks; sk_apply_update divides by loss scale and
 * batch_stat and runs the optimiser on them. */
int sk_backward_grads(sk_ctx *ctx, const sk_dense *layer, const void *x, uint32_t x_rows,
                      uint32_t batch, float *dw, float *colsums);
int sk_apply_update(sk_ctx *ctx, const sk_dense *layer, const float *dw, const float *colsums,
                    uint32_t batch_stat, const sk_optim *linear, const sk_optim *norm_opt,
                    float learn_rate, float grad_clamp, uint32_t step);

/* Sharded form of the same exchange (no counterpart): sk_backward_grads_lp writes dW in the block's
 * storage type, already divided by batch_stat (loss scale x512 kept), so that ranks can
 * reduce-scatter half the bytes; sk_apply_update_rows steps rows [row0, row0 + nrows) of the weight
 * matrix (master, moments and the 16-bit copy) from the summed gradient of just those rows;
 * sk_apply_vector_update steps bias and normalisation parameters from summed column sums. */
int sk_backward_grads_lp(sk_ctx *ctx, const sk_dense *layer, const void *x, uint32_t x_rows, uint32_t batch,
                         uint32_t batch_stat, void *grad, float *colsums);
int sk_apply_update_rows(sk_ctx *ctx, const sk_dense *layer, const void *grad, uint32_t row0, uint32_t nrows,
                         const sk_optim *linear, float learn_rate, float grad_clamp, uint32_t step);
int sk_apply_vector_update(sk_ctx *ctx, const sk_dense *layer, const float *colsums, uint32_t batch_stat,
                           const sk_optim *linear, const sk_optim *norm_opt, float learn_rate, float grad_clamp,
                           uint32_t step);

/* Fused form of the exchange for one process per GPU with peer-mapped buffers (no counterpart).
 * Rank r owns rows [r*K/W, (r+1)*K/W) of each weight matrix. Every rank writes its averaged 16-bit dW
 * (sk_backward_grads_lp) into a gradient buffer T [K][N] inside its exchange arena; sk_signal_peers
 * publishes a value in slot `slot` of every rank's flag array and sk_wait_flags waits (bounded: about two
 * seconds, then SK_ERR_DEVICE_TIMEOUT at the next sk_sync) until all `world` slots of the local array
 * reached it. sk_reduce_update_broadcast is then reduce-scatter + optimiser + all-gather in ONE kernel:
 * it pulls the owned rows out of every rank's gradient buffer over NVLink (peer_grad[i] = gradient
 * buffer of rank i as mapped here), adds them, steps them (f32 master, moments) and stores the new
 * 16-bit rows into every rank's weight tensor (peer_w[i] = weight tensor of rank i, which therefore
 * lives in that rank's arena too). A second handshake releases the dX GEMM of the layer below. */
int sk_reduce_update_broadcast(sk_ctx *ctx, const sk_dense *layer, void *const *peer_grad, uint32_t world,
                               uint32_t rank, void *const *peer_w, const sk_optim *linear, float learn_rate,
                               float grad_clamp, uint32_t step);
/* The same exchange for a whole network in one call: the data-parallel backward pass sequenced in native
 * code (no counterpart; the order kept is the reference's, src/ffn.rs:113-166: every hidden delta reads the
 * next layer's weights after their update). Each weight matrix is exchanged in `blocks` blocks of rows
 * (sk_dp_blocks gives the count actually used for a shape: the largest <= blocks that splits evenly; 0 = the
 * shape cannot be split; blocks = 0 means 1); inside a block rank r owns rows [r*K/(blocks*world),
 * (r+1)*K/(blocks*world)) and keeps f32 masters and moments current for those rows only. Per block: the dW
 * GEMM writes the block of the local 16-bit gradient and raises a flag on the other ranks; one kernel waits
 * for their flags, obtains the sum of the owned rows (peer loads and adds, or one in-switch reduction per 16
 * bytes when mc_grad / mc_w are given), steps them and stores the new 16-bit rows into every rank's weight
 * tensor; and the dX GEMM of the layer below waits, inside its TMA producer, only for the blocks of rows its
 * tile needs. The last block's kernel also adds the [3 x N] column sums of all ranks and steps bias and
 * normalisation parameters. Everything runs on the context's stream; kernels wait only for flags raised by
 * OTHER GPUs, and every such wait is bounded (SK_ERR_DEVICE_TIMEOUT at the next sk_sync; after a wait gave
 * up no weight is changed and no flag raised). Per layer the caller provides, for every rank as mapped into
 * this process: the gradient buffer T [K x N], the weight tensor T [K x N] (this rank's entry must be the
 * block's `w`), sk_dp_flag_bytes() bytes of flag words (zero at set-up), and a column-sum buffer f32 [3 x N].
 * `epoch` must grow by one per call. 16-bit blocks without BatchNorm; world = 2, 4 or 8. */
typedef struct {
    void *const *peer_grad;
    void *const *peer_w;
    void *const *peer_flags;
    void *const *peer_colsums;
    /* Optional: addresses of the gradient buffers / weight tensors inside an NVSwitch multicast mapping that
     * covers the same arenas on all ranks (NULL = plain peer loads and stores). With them the reduction runs
     * inside the switch (multimem.ld_reduce, f32 accumulation, sum returned in the 16-bit type) and a rank's
     * rows are sent once (multimem.st). Do not use in a job in which a rank may leave. */
    void *mc_grad;
    void *mc_w;
} sk_exchange;
uint32_t sk_dp_blocks(uint32_t K, uint32_t N, uint32_t world, uint32_t blocks);
uint32_t sk_dp_flag_bytes(void);
int sk_dp_backward(sk_ctx *ctx, const sk_dense *const *layers, const sk_exchange *exchange, uint32_t n_layers,
                   const void *target, uint32_t target_rows, const void *x, uint32_t x_rows, uint32_t loss,
                   uint32_t loss_act, float loss_leaky, const sk_optim *linear, const sk_optim *norm_opt,
                   uint32_t batch, uint32_t batch_stat, uint32_t world, uint32_t rank, uint32_t blocks,
                   uint32_t epoch, float learn_rate, float grad_clamp, uint32_t step);

/* Exchange arena of one rank: sk_peer_alloc allocates `bytes` of zeroed device memory (set-up time,
 * not the hot path) and returns a 64-byte CUDA IPC handle for it; the other ranks (other processes
 * on the same node) turn that handle into a pointer usable by kernels of THEIR device with
 * sk_peer_open, which maps it with this context's device current and peer access enabled.
 * sk_peer_close / sk_peer_free undo them. */
int sk_peer_alloc(sk_ctx *ctx, size_t bytes, void **ptr, unsigned char handle_out[64]);
int sk_peer_open(sk_ctx *ctx, const unsigned char handle[64], void **ptr);
int sk_peer_close(sk_ctx *ctx, void *ptr);
int sk_peer_free(sk_ctx *ctx, void *ptr);
/* Device-to-device copy of `bytes` on the context's stream (Tensor::clone, src/util/core.rs:686-692). */
int sk_copy(sk_ctx *ctx, void *dst, const void *src, size_t bytes);
int sk_signal_peers(sk_ctx *ctx, void *const *peer_flags, uint32_t world, uint32_t slot, uint32_t value);
int sk_wait_flags(sk_ctx *ctx, const uint32_t *flags, uint32_t world, uint32_t value);

/* No counterpart in the reference. Column sums over the batch of d_prenorm, d_norm_w and
 * d_norm_b, written to colsums f32 [3 x N] exactly as sk_backward_grads writes them, but
 * without a context and without allocating: for callers that are not allowed to allocate
 * device memory (their framework owns the whole device heap, or they only hold raw pointers
 * and a stream and so cannot create an sk_ctx, whose creation allocates). The partial sums
 * live in a 3 MiB array built into the library (present on every GPU that loads it), which
 * limits N to 262144 columns: beyond that the call returns SK_ERR_STATIC_LIMIT. Calls share
 * that array, so calls that overlap on the GPU race and must be serialised by the caller.
 * The first call on a device resolves the array's address; make it before any stream capture, and from
 * one host thread (concurrent first calls on a device all store the same pointer, which is harmless, but
 * it is a data race by the letter).
 * `stream` is a cudaStream_t (NULL = legacy default stream); norm selects which sums are
 * taken (0: dB only, 1: + d_norm_w, 2/3: + d_norm_b), unused inputs may be NULL. */
int sk_column_sums_static(void *stream, const float *d_prenorm, const float *d_norm_w,
                          const float *d_norm_b, float *colsums, uint32_t batch, uint32_t N, uint32_t norm);

/* GpuContext::gpu_cast_t (src/io/device/util_device.rs:7-47): f32 <-> 16-bit, len elements. */
int sk_cast(sk_ctx *ctx, const void *src, uint32_t src_dtype, void *dst, uint32_t dst_dtype, size_t len);
/* GpuContext::gpu_broadcast (src/io/device/util_device.rs:49-78). */
int sk_fill(sk_ctx *ctx, void *dst, uint32_t dtype, float value, size_t len);

#ifdef __cplusplus
}
#endif
#endif /* SOKLYN_B200_H */
