// soklyn_b200.hpp — C++17 host mirror of the reference's DenseBlock / FeedForwardNetwork API
// above the C ABI of soklyn_b200.h. Header-only; link libsoklyn_b200.so and the CUDA runtime.
//
// The reference is a Rust crate; this is its host side for this path restated for a compiled
// host without a Rust toolchain: the same types, method names, argument meaning, checks and
// error variants (src/mlp.rs, src/ffn.rs, src/io/device.rs, src/io/device/ffn_device.rs,
// src/util/{core,context,function,scheduler,log}.rs), with every device operation one call
// into the C ABI. Device memory comes from the CUDA runtime; there is no CPU path.
//
// Differences from the reference, all deliberate:
//   * precision is a run-time value (Precision) instead of a type parameter, because the
//     C ABI is typed at run time;
//   * gpu_* calls return once the work is queued on the context's stream; synchronize()
//     waits (the reference waits inside every call);
//   * a 16-bit training block owns one more tensor, d_prenorm_lp, which takes no tensor id.
#ifndef SOKLYN_B200_HPP
#define SOKLYN_B200_HPP

#include <cuda_runtime_api.h>

#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <memory>
#include <sstream>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "soklyn_b200.h"

namespace soklyn {

// ---------------------------------------------------------------------------------------
// Errors: one class per variant of soklyn::log::Error that this path can raise
// (src/util/log.rs:15-99); what() carries the reference's message text.
// ---------------------------------------------------------------------------------------
struct Error : std::runtime_error {
    using std::runtime_error::runtime_error;
};
struct DriverError : Error {
    using Error::Error;
};
struct MismatchedDimensions : Error {
    size_t expected, found;
    MismatchedDimensions(const std::string &reason, size_t expected_, size_t found_)
        : Error("Dimension mismatch: " + reason + ": expected " + std::to_string(expected_) + ", found " +
                std::to_string(found_) + "."),
          expected(expected_), found(found_) {}
};
struct AllocationLimitExceeded : Error {
    size_t received, max;
    AllocationLimitExceeded(size_t received_, size_t max_, const std::string &reason)
        : Error("Allocation limit exceeded: " + reason + ": items received (" + std::to_string(received_) +
                ") exceeds maximum allowed allocation (" + std::to_string(max_) + ")."),
          received(received_), max(max_) {}
};
struct InvalidConfiguration : Error {
    explicit InvalidConfiguration(const std::string &reason) : Error("Invalid network configuration: " + reason) {}
};
struct InvalidBatchSize : Error {
    explicit InvalidBatchSize(const std::string &reason) : Error("Batch size constraint violation: " + reason) {}
};
struct TrainingModeRequired : Error {
    explicit TrainingModeRequired(const std::string &reason)
        : Error("Invalid operation: " + reason + ": Action requires the network to be in training mode.") {}
};
struct HardwareConstraintViolation : Error {
    HardwareConstraintViolation(const std::string &precision, unsigned expected, unsigned found)
        : Error("Hardware acceleration constraint violation: Precision is " + precision +
                ", which requires a tile dimension of " + std::to_string(expected) + ", but found " +
                std::to_string(found) + ".") {}
};
struct UnsupportedTypeCast : Error {
    UnsupportedTypeCast(const std::string &src, const std::string &dst)
        : Error("Unsupported precision cast operation: Cannot convert data from " + src + " to " + dst) {}
};
// A status of the C ABI without a reference variant (null pointer, workspace, device timeout).
struct NativeError : Error {
    int status;
    NativeError(int status_, const std::string &detail)
        : Error("[status " + std::to_string(status_) + "] " + detail), status(status_) {}
};

namespace detail {
// The mirror checks arguments itself first, with the reference's messages; this maps whatever
// only the native side could see.
[[noreturn]] inline void throw_status(int rc, const std::string &text) {
    const std::string msg = "[status " + std::to_string(rc) + "] " + text;
    switch (rc) {
    case SK_ERR_DRIVER: throw DriverError(msg);
    case SK_ERR_MISMATCHED_DIMENSIONS: {
        MismatchedDimensions e(text, 0, 0);
        throw e;
    }
    case SK_ERR_ALLOCATION_LIMIT: throw AllocationLimitExceeded(0, 0, text);
    case SK_ERR_INVALID_CONFIGURATION: throw InvalidConfiguration(text);
    case SK_ERR_INVALID_BATCH_SIZE: throw InvalidBatchSize(text);
    case SK_ERR_TRAINING_MODE_REQUIRED: throw TrainingModeRequired(text);
    case SK_ERR_HARDWARE_CONSTRAINT: throw HardwareConstraintViolation(text, 16, 0);
    case SK_ERR_UNSUPPORTED_CAST: throw UnsupportedTypeCast(text, "?");
    default: throw NativeError(rc, text);
    }
}
inline void cuda_check(cudaError_t e, const char *what) {
    if (e != cudaSuccess) throw DriverError(std::string(what) + ": " + cudaGetErrorString(e));
}
} // namespace detail

// ---------------------------------------------------------------------------------------
// Hyper-parameter types (src/util/function.rs:1-176); ordinals are the kernel ABI.
// ---------------------------------------------------------------------------------------
enum class Precision : uint32_t { FP32 = SK_F32, FP16 = SK_F16, BF16 = SK_BF16 }; // BF16: extension of this build
inline const char *precision_name(Precision p) {
    return p == Precision::FP32 ? "FP32" : p == Precision::FP16 ? "FP16" : "BF16";
}
inline size_t element_size(Precision p) { return p == Precision::FP32 ? 4 : 2; }

struct Regularisation { // None_ / L1Regular{regu_coeff} / L2Regular{regu_coeff}
    uint32_t kind = SK_REGU_NONE;
    float regu_coeff = 0.f;
    static Regularisation None() { return {SK_REGU_NONE, 0.f}; }
    static Regularisation L1Regular(float c) { return {SK_REGU_L1, c}; }
    static Regularisation L2Regular(float c) { return {SK_REGU_L2, c}; }
    uint32_t ordinal() const { return kind; }
};

enum class Normalisation : uint32_t { Disabled = 0, RMSNorm = 1, LayerNorm = 2, BatchNorm = 3 };

struct Optimiser { // SGD{v_coeff, nesterov} (ordinal 0) / Adam{m_coeff, v_coeff, epsilon} (ordinal 1)
    uint32_t kind = SK_OPT_SGD;
    float m_coeff = 0.f, v_coeff = 0.f, epsilon = 0.f;
    bool nesterov = false;
    static Optimiser SGD(float v_coeff = 0.f, bool nesterov = false) { return {SK_OPT_SGD, 0.f, v_coeff, 0.f, nesterov}; }
    static Optimiser Adam(float m_coeff = 0.9f, float v_coeff = 0.999f, float epsilon = 1e-8f) {
        return {SK_OPT_ADAM, m_coeff, v_coeff, epsilon, false};
    }
    uint32_t ordinal() const { return kind; }
    // (beta1, beta2, epsilon, nesterov) as src/io/device/ffn_device.rs:254-264 unpacks them
    sk_optim kernel_args() const {
        if (kind == SK_OPT_SGD) return sk_optim{kind, v_coeff, 0.f, 0.f, nesterov ? 1u : 0u};
        return sk_optim{kind, m_coeff, v_coeff, epsilon, 0u};
    }
};

struct Activation { // LeakyReLU carries its coefficient
    uint32_t kind = SK_ACT_IDENTITY;
    float coeff = 0.f;
    static Activation Identity() { return {SK_ACT_IDENTITY, 0.f}; }
    static Activation Sigmoid() { return {SK_ACT_SIGMOID, 0.f}; }
    static Activation ReLU() { return {SK_ACT_RELU, 0.f}; }
    static Activation LeakyReLU(float c) { return {SK_ACT_LEAKY_RELU, c}; }
    static Activation Tanh() { return {SK_ACT_TANH, 0.f}; }
    static Activation Softmax() { return {SK_ACT_SOFTMAX, 0.f}; }
    static Activation SiLU() { return {SK_ACT_SILU, 0.f}; }
    static Activation Mish() { return {SK_ACT_MISH, 0.f}; }
    uint32_t ordinal() const { return kind; }
    bool operator==(const Activation &o) const { return kind == o.kind; }
    bool operator!=(const Activation &o) const { return kind != o.kind; }
};

enum class LossFunc : uint32_t { MeanSquareLoss = 0, CrossEntropyLoss = 1, BinaryCrossEntropy = 2 };

// ---------------------------------------------------------------------------------------
// Configuration records (src/util/context.rs:1-85)
// ---------------------------------------------------------------------------------------
struct LayerInitConfig {
    Normalisation normalisation = Normalisation::Disabled;
    Activation activation = Activation::Identity();
    Regularisation regularisation = Regularisation::None();
    float mask_coeff = 0.f;
};
struct TrainContext {
    Optimiser optimiser, norm_optimiser;
    size_t batch_size = 0;
    float learn_rate = 0.f;
    float grad_clamp = std::numeric_limits<float>::max();
};
struct MultiLayerTrainContext {
    std::vector<Optimiser> optimisers, norm_optimisers;
    size_t batch_size = 0;
    float learn_rate = 0.f;
    float grad_clamp = std::numeric_limits<float>::max();
    TrainContext get_train_context(size_t idx) const {
        return TrainContext{optimisers.at(idx), norm_optimisers.at(idx), batch_size, learn_rate, grad_clamp};
    }
};
struct LossConfig {
    LossFunc loss_func = LossFunc::MeanSquareLoss;
    Activation activation = Activation::Identity();
};

// ---------------------------------------------------------------------------------------
// Learning-rate schedulers (src/util/scheduler.rs), all arithmetic in f32 like the reference.
// ---------------------------------------------------------------------------------------
class CosineDecayLR { // linear warm-up min->max, then cosine decay back to min (scheduler.rs:3-78)
  public:
    CosineDecayLR(float min_lr, float max_lr, size_t total_step, size_t warmup_steps)
        : min_lr_(min_lr), max_lr_(max_lr), cur_lr_(min_lr), total_(total_step), warmup_(warmup_steps) {
        update();
    }
    void reset() { cur_step_ = 0; update(); }
    float get_learning_rate() const { return cur_lr_; }
    float step() { ++cur_step_; update(); return cur_lr_; }

  private:
    void update() {
        if (cur_step_ < warmup_) {
            const float progress = (float)cur_step_ / (float)warmup_;
            cur_lr_ = min_lr_ + progress * (max_lr_ - min_lr_);
            return;
        }
        const size_t decay_total = total_ - warmup_;
        if (decay_total == 0) { cur_lr_ = min_lr_; return; }
        const float progress = (float)(cur_step_ - warmup_) / (float)decay_total;
        cur_lr_ = min_lr_ + 0.5f * (max_lr_ - min_lr_) * (1.0f + std::cos(progress * 3.14159265358979323846f));
    }
    float min_lr_, max_lr_, cur_lr_;
    size_t cur_step_ = 0, total_, warmup_;
};

class ExponentialLR { // lr *= factor each step (scheduler.rs:81-123)
  public:
    ExponentialLR(float lr_initial, float lr_factor) : ori_(lr_initial), cur_(lr_initial), factor_(lr_factor) {}
    void reset() { cur_ = ori_; }
    float get_learning_rate() const { return cur_; }
    float step() { cur_ *= factor_; return cur_; }

  private:
    float ori_, cur_, factor_;
};

enum class SchedulerMode { Minimize, Maximize };
class ReduceLROnPlateauScheduler { // scheduler.rs:127-231
  public:
    ReduceLROnPlateauScheduler(size_t patience, SchedulerMode mode, float lr_factor, float min_lr)
        : mode_(mode), patience_(patience), factor_(lr_factor), min_lr_(min_lr), best_(worst()) {
        if (patience == 0) throw InvalidConfiguration("Patience must be non-zero.");
    }
    void reset(float learning_rate) { cur_ = learning_rate; timer_ = 0; best_ = worst(); }
    float get_learning_rate() const { return cur_; }
    float step(float test_val) {
        if (std::isnan(test_val)) return cur_;
        const bool improved = mode_ == SchedulerMode::Maximize ? test_val > best_ : test_val < best_;
        if (improved) { best_ = test_val; timer_ = 0; }
        else if (++timer_ == patience_) { timer_ = 0; cur_ = std::max(cur_ * factor_, min_lr_); }
        return cur_;
    }

  private:
    float worst() const {
        const float m = std::numeric_limits<float>::max();
        return mode_ == SchedulerMode::Maximize ? -m : m;
    }
    SchedulerMode mode_;
    size_t patience_, timer_ = 0;
    float factor_, min_lr_, cur_ = 0.f, best_;
};

// ---------------------------------------------------------------------------------------
// Weight initialisers (InitFunc, src/util/function.rs:190-319). The reference draws from
// rand_chacha's ChaCha8Rng, which is not part of its source tree; these draw the same
// distributions (uniform in +-limit, Box-Muller normal) from a SplitMix64 stream, so the values
// differ from a reference run with the same seed. Load weights with InitGivenFunc when
// bit-equal weights are needed.
// ---------------------------------------------------------------------------------------
struct InitFunc {
    virtual ~InitFunc() = default;
    virtual std::vector<float> init(size_t fan_in, size_t fan_out, size_t length) = 0;
};
struct InitZeroFunc : InitFunc {
    std::vector<float> init(size_t, size_t, size_t length) override { return std::vector<float>(length, 0.f); }
};
struct InitGivenFunc : InitFunc { // hands back a prepared matrix (weights are loaded, not drawn)
    std::vector<float> values;
    explicit InitGivenFunc(std::vector<float> v) : values(std::move(v)) {}
    std::vector<float> init(size_t, size_t, size_t length) override {
        if (values.size() != length) throw MismatchedDimensions("given weights vs layer shape", length, values.size());
        return values;
    }
};
// ChaCha with 8 rounds as rand_chacha::ChaCha8Rng runs it (src/util/function.rs:196-213 holds one per
// initialiser): 64-bit block counter in words 12-13, stream id zero, the keystream read as little-endian
// 32-bit words from block 0 on. seed_from_u64 is rand_core's: the eight key words are PCG32 (XSH-RR)
// outputs, multiplier 6364136223846793005, increment 11634580027462260723, state advanced before each
// output. Restated from the published algorithms; the crates' sources are not part of the reference tree.
class ChaCha8Rng {
  public:
    static ChaCha8Rng seed_from_u64(uint64_t state) {
        ChaCha8Rng r;
        for (int i = 0; i < 8; ++i) {
            state = state * 6364136223846793005ull + 11634580027462260723ull;
            const uint32_t xorshifted = (uint32_t)(((state >> 18) ^ state) >> 27);
            const uint32_t rot = (uint32_t)(state >> 59);
            r.key_[i] = (xorshifted >> rot) | (xorshifted << ((32u - rot) & 31u));
        }
        return r;
    }
    uint32_t next_u32() {
        if (index_ == 16) { block(); index_ = 0; }
        return buf_[index_++];
    }

  private:
    static uint32_t rotl(uint32_t x, int n) { return (x << n) | (x >> (32 - n)); }
    static void quarter(uint32_t *s, int a, int b, int c, int d) {
        s[a] += s[b]; s[d] = rotl(s[d] ^ s[a], 16);
        s[c] += s[d]; s[b] = rotl(s[b] ^ s[c], 12);
        s[a] += s[b]; s[d] = rotl(s[d] ^ s[a], 8);
        s[c] += s[d]; s[b] = rotl(s[b] ^ s[c], 7);
    }
    void block() {
        uint32_t in[16] = {0x61707865u, 0x3320646Eu, 0x79622D32u, 0x6B206574u};
        for (int i = 0; i < 8; ++i) in[4 + i] = key_[i];
        in[12] = (uint32_t)counter_; in[13] = (uint32_t)(counter_ >> 32); in[14] = 0; in[15] = 0;
        uint32_t s[16];
        for (int i = 0; i < 16; ++i) s[i] = in[i];
        for (int r = 0; r < 4; ++r) {   // 8 rounds = 4 column + diagonal pairs
            quarter(s, 0, 4, 8, 12); quarter(s, 1, 5, 9, 13); quarter(s, 2, 6, 10, 14); quarter(s, 3, 7, 11, 15);
            quarter(s, 0, 5, 10, 15); quarter(s, 1, 6, 11, 12); quarter(s, 2, 7, 8, 13); quarter(s, 3, 4, 9, 14);
        }
        for (int i = 0; i < 16; ++i) buf_[i] = s[i] + in[i];
        ++counter_;
    }
    uint32_t key_[8] = {0}, buf_[16] = {0};
    uint64_t counter_ = 0;
    int index_ = 16;
};

// normal_dist / uniform_dist of src/util/function.rs:219-248, in f32 arithmetic, operation for operation
// (`u32::MAX as f32` is 2^32 after rounding, and so is `u32::MAX as f32 + 1.0`).
class InitRandomBase : public InitFunc {
  public:
    explicit InitRandomBase(uint64_t seed, float factor = 1.f) : rng_(ChaCha8Rng::seed_from_u64(seed)), factor_(factor) {}
    uint32_t next_u32() { return rng_.next_u32(); }

  protected:
    std::vector<float> uniform(size_t n, float limit) {
        std::vector<float> v(n);
        for (auto &x : v) {
            const float raw = (float)next_u32() / 4294967296.0f;
            x = factor_ * (-limit + raw * (2.0f * limit));
        }
        return v;
    }
    std::vector<float> normal(size_t n, float std_dev) {
        std::vector<float> v(n);
        for (auto &x : v) {
            const float u1 = ((float)next_u32() + 1.0f) / 4294967296.0f;
            const float u2 = (float)next_u32() / 4294967296.0f;
            const float z = std::sqrt(-2.0f * std::log(u1)) * std::cos((2.0f * 3.14159274101257324219f) * u2);
            x = factor_ * z * std_dev;
        }
        return v;
    }

  private:
    ChaCha8Rng rng_;
    float factor_;
};
struct InitXavierUniformFunc : InitRandomBase {
    using InitRandomBase::InitRandomBase;
    std::vector<float> init(size_t fi, size_t fo, size_t n) override { return uniform(n, std::sqrt(6.0f / (float)(fi + fo))); }
};
struct InitXavierNormalFunc : InitRandomBase {
    using InitRandomBase::InitRandomBase;
    std::vector<float> init(size_t fi, size_t fo, size_t n) override { return normal(n, std::sqrt(2.0f / (float)(fi + fo))); }
};
struct InitHeUniformFunc : InitRandomBase {
    using InitRandomBase::InitRandomBase;
    std::vector<float> init(size_t fi, size_t, size_t n) override { return uniform(n, std::sqrt(6.0f / (float)fi)); }
};
struct InitHeNormalFunc : InitRandomBase {
    using InitRandomBase::InitRandomBase;
    std::vector<float> init(size_t fi, size_t, size_t n) override { return normal(n, std::sqrt(2.0f / (float)fi)); }
};

class Tensor;
class DenseBlock;

// ---------------------------------------------------------------------------------------
// GpuContext (src/io/device.rs:150-272 and src/io/device/{ffn,util}_device.rs): the device,
// its stream and the native context. Each gpu_* method is one call into the C ABI.
// ---------------------------------------------------------------------------------------
class GpuContext {
  public:
    // GpuContext::new(tile_dim) / with_device_index(ordinal, tile_dim). The context owns a
    // non-blocking stream like the reference's unless `stream` is given.
    explicit GpuContext(uint32_t tile_dim = 16, int ordinal = 0, cudaStream_t stream = nullptr, bool own_stream = true,
                        size_t workspace_bytes = 0)
        : tile_dim_(tile_dim), ordinal_(ordinal) {
        int count = 0;
        if (cudaGetDeviceCount(&count) != cudaSuccess || ordinal >= count)
            throw DriverError("Failed to create CUDA context: no CUDA device " + std::to_string(ordinal) +
                              " (there is no CPU path)");
        detail::cuda_check(cudaSetDevice(ordinal), "cudaSetDevice");
        if (own_stream && stream == nullptr) {
            detail::cuda_check(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking), "cudaStreamCreate");
            owns_stream_ = true;
        } else {
            stream_ = stream;
        }
        const int rc = sk_ctx_create(ordinal, tile_dim, stream_, 0, workspace_bytes, &ctx_);
        if (rc != SK_OK) {
            if (owns_stream_) cudaStreamDestroy(stream_);
            throw DriverError(std::string("sk_ctx_create failed: ") + sk_status_string(rc));
        }
    }
    static GpuContext with_device_index(int ordinal, uint32_t tile_dim) { return GpuContext(tile_dim, ordinal); }
    GpuContext(const GpuContext &) = delete;
    GpuContext &operator=(const GpuContext &) = delete;
    GpuContext(GpuContext &&o) noexcept { *this = std::move(o); }
    GpuContext &operator=(GpuContext &&o) noexcept {
        if (this != &o) {
            release();
            ctx_ = o.ctx_; stream_ = o.stream_; owns_stream_ = o.owns_stream_; tile_dim_ = o.tile_dim_; ordinal_ = o.ordinal_;
            o.ctx_ = nullptr; o.stream_ = nullptr; o.owns_stream_ = false;
        }
        return *this;
    }
    ~GpuContext() { release(); }

    uint32_t get_tile_dim() const { return tile_dim_; }
    int ordinal() const { return ordinal_; }
    cudaStream_t stream() const { return stream_; }
    sk_ctx *native() const { return ctx_; }
    void synchronize() const { check(sk_sync(ctx_)); }
    uint64_t launch_count() const { return sk_launch_count(ctx_); }
    void reserve(size_t workspace_bytes) { check(sk_ctx_reserve(ctx_, workspace_bytes)); }
    // One training step as one CUDA graph (sk_step_begin / sk_step_end): the calls made while the guard lives
    // are recorded and launched together when it is closed. No counterpart in the reference.
    class StepGraph {
      public:
        StepGraph(const GpuContext &c, uint32_t slot = 0) : c_(c) { c_.check(sk_step_begin(c_.ctx_, slot)); }
        void launch() { open_ = false; c_.check(sk_step_end(c_.ctx_)); }   // throws on failure
        ~StepGraph() { if (open_) sk_step_abort(c_.ctx_); }                // left by an exception: drop the record
        StepGraph(const StepGraph &) = delete;
        StepGraph &operator=(const StepGraph &) = delete;
      private:
        const GpuContext &c_;
        bool open_ = true;
    };
    // force the FFMA GEMM (true) or let the library use the tensor-core kernel where it can (false)
    void set_gemm_engine(bool ffma_only) { check(sk_ctx_set_option(ctx_, SK_OPTION_GEMM_ENGINE, ffma_only ? 1u : 0u)); }

    // src/io/device.rs:248-258
    void check_tile_dim(Precision p) const {
        if (p != Precision::FP32 && tile_dim_ != 16) throw HardwareConstraintViolation(precision_name(p), 16, tile_dim_);
    }

    // src/io/device/util_device.rs:7-78
    inline void gpu_cast_t(const Tensor &src, Tensor &dst) const;
    inline void gpu_broadcast(Tensor &dst, float value) const;

    // src/io/device/ffn_device.rs:12-139, 141-231, 234-358, 360-436
    inline void gpu_forward_pass(DenseBlock &cur, const Tensor &input, size_t batch_size, bool use_dropout, size_t step,
                                 uint32_t row_offset = 0) const;
    inline void gpu_compute_output_layer_error(DenseBlock &cur, const Tensor &target, LossFunc err_mode,
                                               Activation activation) const;
    inline void gpu_backward_pass(DenseBlock &cur, const Tensor &input, const TrainContext &train_ctx, size_t step) const;
    inline void gpu_hidden_layer_backward_pass(DenseBlock &cur, DenseBlock &next, const Tensor &input,
                                               const TrainContext &train_ctx, size_t step) const;
    // whole-network calls: the layer loop of src/ffn.rs:40-57 and :113-166 sequenced natively
    inline void gpu_ffn_forward(std::vector<DenseBlock> &layers, const Tensor &input, size_t batch_size, bool use_dropout,
                                size_t step, uint32_t row_offset = 0) const;
    inline void gpu_ffn_backward(std::vector<DenseBlock> &layers, const Tensor &target, const Tensor &input,
                                 const LossConfig &loss_config, const MultiLayerTrainContext &train_ctx, size_t step) const;

    void check(int rc) const {
        if (rc != SK_OK) detail::throw_status(rc, ctx_ ? sk_last_error(ctx_) : sk_status_string(rc));
    }

  private:
    void release() {
        if (ctx_) sk_ctx_destroy(ctx_);
        if (owns_stream_ && stream_) cudaStreamDestroy(stream_);
        ctx_ = nullptr; stream_ = nullptr; owns_stream_ = false;
    }
    sk_ctx *ctx_ = nullptr;
    cudaStream_t stream_ = nullptr;
    bool owns_stream_ = false;
    uint32_t tile_dim_ = 16;
    int ordinal_ = 0;
};

// ---------------------------------------------------------------------------------------
// Tensor (src/util/core.rs:414-693): a row-major device buffer, its shape and a process-wide
// id. The id of a block's weight tensor seeds the dropout hash (core.rs:84-94), so ids are
// handed out in allocation order like the reference's global counter.
// ---------------------------------------------------------------------------------------
namespace detail {
inline std::atomic<uint64_t> &tensor_id_counter() {
    static std::atomic<uint64_t> c{0};
    return c;
}
} // namespace detail
// Restart the id counter (to reproduce the ids of a fresh reference process).
inline void reset_tensor_ids(uint64_t start = 0) { detail::tensor_id_counter().store(start); }
// scramble_seed (core.rs:90-94)
inline uint32_t scramble_seed(uint32_t step, uint32_t layer_id) { return sk_scramble_seed(step, layer_id); }

class Tensor {
  public:
    Tensor() = default;
    Tensor(const Tensor &) = delete;
    Tensor &operator=(const Tensor &) = delete;
    Tensor(Tensor &&o) noexcept { *this = std::move(o); }
    Tensor &operator=(Tensor &&o) noexcept {
        if (this != &o) {
            free_();
            ptr_ = o.ptr_; rows_ = o.rows_; cols_ = o.cols_; precision_ = o.precision_; id_ = o.id_;
            o.ptr_ = nullptr; o.rows_ = o.cols_ = 0;
        }
        return *this;
    }
    ~Tensor() { free_(); }

    // -- constructors (core.rs:557-645) --
    static Tensor zeros(const GpuContext &ctx, size_t rows, size_t cols, Precision p = Precision::FP32, bool take_id = true) {
        Tensor t = alloc(ctx, rows, cols, p, take_id);
        detail::cuda_check(cudaMemsetAsync(t.ptr_, 0, t.bytes(), ctx.stream()), "cudaMemsetAsync");
        return t;
    }
    static Tensor fill(const GpuContext &ctx, size_t rows, size_t cols, float value, Precision p = Precision::FP32) {
        Tensor t = alloc(ctx, rows, cols, p, true);
        ctx.gpu_broadcast(t, value);
        return t;
    }
    // Host f32 values -> device tensor of precision p (rounded to nearest even for 16-bit).
    static Tensor from_cpu_vector(const GpuContext &ctx, const float *values, size_t length, size_t rows, size_t cols,
                                  Precision p = Precision::FP32) {
        if (length != rows * cols) throw MismatchedDimensions("host vector length vs tensor shape", rows * cols, length);
        Tensor t = alloc(ctx, rows, cols, p, true);
        if (p == Precision::FP32) {
            t.upload(ctx, values, length * sizeof(float));
            ctx.synchronize();
        } else {
            Tensor staging = alloc(ctx, rows, cols, Precision::FP32, false);
            staging.upload(ctx, values, length * sizeof(float));
            ctx.gpu_cast_t(staging, t);
            ctx.synchronize(); // staging is released on return
        }
        return t;
    }
    static Tensor from_cpu_vector(const GpuContext &ctx, const std::vector<float> &v, size_t rows, size_t cols,
                                  Precision p = Precision::FP32) {
        return from_cpu_vector(ctx, v.data(), v.size(), rows, cols, p);
    }
    // Tensor::clone (core.rs:686-692): a new tensor (new id) with the same contents.
    Tensor clone(const GpuContext &ctx) const {
        Tensor t = alloc(ctx, rows_, cols_, precision_, true);
        ctx.check(sk_copy(ctx.native(), t.ptr_, ptr_, bytes()));
        return t;
    }
    // type.rs:140-177: f32 <-> 16-bit
    Tensor cast(const GpuContext &ctx, Precision p) const {
        Tensor t = zeros(ctx, rows_, cols_, p);
        ctx.gpu_cast_t(*this, t);
        return t;
    }
    void broadcast(const GpuContext &ctx, float value) { ctx.gpu_broadcast(*this, value); }

    // Raw copy of `nbytes` in the tensor's own storage type, queued on the context's stream.
    void upload(const GpuContext &ctx, const void *host, size_t nbytes) {
        if (nbytes > bytes()) throw AllocationLimitExceeded(nbytes, bytes(), "upload bytes");
        detail::cuda_check(cudaMemcpyAsync(ptr_, host, nbytes, cudaMemcpyHostToDevice, ctx.stream()), "cudaMemcpyAsync");
    }
    // Device -> host as f32 (16-bit tensors are widened on the device first); waits for the stream.
    std::vector<float> download(const GpuContext &ctx) const {
        std::vector<float> host(len());
        if (len() == 0) return host;
        if (precision_ == Precision::FP32) {
            detail::cuda_check(cudaMemcpyAsync(host.data(), ptr_, bytes(), cudaMemcpyDeviceToHost, ctx.stream()), "cudaMemcpyAsync");
            ctx.synchronize();
        } else {
            Tensor wide = alloc(ctx, rows_, cols_, Precision::FP32, false);
            ctx.gpu_cast_t(*this, wide);
            detail::cuda_check(cudaMemcpyAsync(host.data(), wide.ptr_, wide.bytes(), cudaMemcpyDeviceToHost, ctx.stream()), "cudaMemcpyAsync");
            ctx.synchronize();
        }
        return host;
    }

    // -- accessors --
    int64_t get_id() const { return id_; }
    size_t rows() const { return rows_; }
    size_t cols() const { return cols_; }
    size_t len() const { return rows_ * cols_; }
    size_t bytes() const { return len() * element_size(precision_); }
    Precision precision() const { return precision_; }
    void *ptr() const { return ptr_; }
    bool empty() const { return ptr_ == nullptr; }

  private:
    static Tensor alloc(const GpuContext &ctx, size_t rows, size_t cols, Precision p, bool take_id) {
        Tensor t;
        t.rows_ = rows; t.cols_ = cols; t.precision_ = p;
        t.id_ = take_id ? (int64_t)detail::tensor_id_counter().fetch_add(1) : -1;
        detail::cuda_check(cudaSetDevice(ctx.ordinal()), "cudaSetDevice");
        detail::cuda_check(cudaMalloc(&t.ptr_, t.bytes() ? t.bytes() : 1), "cudaMalloc");
        return t;
    }
    void free_() {
        if (ptr_) cudaFree(ptr_);
        ptr_ = nullptr;
    }
    void *ptr_ = nullptr;
    size_t rows_ = 0, cols_ = 0;
    Precision precision_ = Precision::FP32;
    int64_t id_ = -1;
};
using Tensor1D = Tensor; // a vector is a tensor of one row
using Tensor2D = Tensor;

// ---------------------------------------------------------------------------------------
// ParamState (src/mlp.rs:14-160): a parameter pair w, b with, for training, the f32 masters
// (16-bit modes only) and the two optimiser moments.
// ---------------------------------------------------------------------------------------
struct ParamState {
    Tensor w, b;
    std::unique_ptr<Tensor> master_w, master_b, dv_w, dv_b, dm_w, dm_b;

    static ParamState new_linear(const GpuContext &ctx, const std::vector<float> &w_vec, size_t inputs, size_t outputs,
                                 bool is_training, Precision p) {
        ParamState s;
        const bool half = p != Precision::FP32;
        s.w = Tensor::from_cpu_vector(ctx, w_vec, inputs, outputs, p);
        s.b = Tensor::zeros(ctx, 1, outputs, p);
        // the master copy holds the weights as the 16-bit tensor stores them (mlp.rs:27-43)
        if (half) {
            s.master_w = std::make_unique<Tensor>(s.w.cast(ctx, Precision::FP32));
            s.master_b = std::make_unique<Tensor>(Tensor::zeros(ctx, 1, outputs));
        }
        if (is_training) {
            s.dv_w = std::make_unique<Tensor>(Tensor::zeros(ctx, inputs, outputs));
            s.dv_b = std::make_unique<Tensor>(Tensor::zeros(ctx, 1, outputs));
            s.dm_w = std::make_unique<Tensor>(Tensor::zeros(ctx, inputs, outputs));
            s.dm_b = std::make_unique<Tensor>(Tensor::zeros(ctx, 1, outputs));
        }
        return s;
    }
    static ParamState new_norm(const GpuContext &ctx, size_t outputs, bool is_training, Precision p) {
        ParamState s;
        const bool half = p != Precision::FP32;
        s.w = Tensor::fill(ctx, 1, outputs, 1.0f, p);
        s.b = Tensor::zeros(ctx, 1, outputs, p);
        if (half) {
            s.master_w = std::make_unique<Tensor>(Tensor::fill(ctx, 1, outputs, 1.0f));
            s.master_b = std::make_unique<Tensor>(Tensor::zeros(ctx, 1, outputs));
        }
        if (is_training) {
            s.dv_w = std::make_unique<Tensor>(Tensor::zeros(ctx, 1, outputs));
            s.dv_b = std::make_unique<Tensor>(Tensor::zeros(ctx, 1, outputs));
            s.dm_w = std::make_unique<Tensor>(Tensor::zeros(ctx, 1, outputs));
            s.dm_b = std::make_unique<Tensor>(Tensor::zeros(ctx, 1, outputs));
        }
        return s;
    }
    // ParamState<f32>::cast_f16 (mlp.rs:203-220): 16-bit copies of w / b, the f32 values become the
    // masters, the moments move over. Consumes the state.
    ParamState cast_f16(const GpuContext &ctx, Precision p = Precision::FP16) && {
        ParamState s;
        s.w = w.clone(ctx).cast(ctx, p);
        s.b = b.clone(ctx).cast(ctx, p);
        s.master_w = std::make_unique<Tensor>(w.clone(ctx));
        s.master_b = std::make_unique<Tensor>(b.clone(ctx));
        s.dv_w = std::move(dv_w); s.dv_b = std::move(dv_b); s.dm_w = std::move(dm_w); s.dm_b = std::move(dm_b);
        ctx.synchronize(); // the temporaries of clone().cast() are released here
        return s;
    }
    // ParamState<f16>::cast_f32 (mlp.rs:185-200): the masters become w / b.
    ParamState cast_f32(const GpuContext &ctx) && {
        if (!master_w || !master_b) throw InvalidConfiguration("16-bit parameter state without f32 masters");
        ParamState s;
        s.w = master_w->clone(ctx);
        s.b = master_b->clone(ctx);
        s.dv_w = std::move(dv_w); s.dv_b = std::move(dv_b); s.dm_w = std::move(dm_w); s.dm_b = std::move(dm_b);
        return s;
    }
    // mlp.rs:112-160: the optional tensors must have the shape of w / b
    void validate() const {
        auto same = [](const char *name, const std::unique_ptr<Tensor> &t, const Tensor &ref) {
            if (t && (t->rows() != ref.rows() || t->cols() != ref.cols()))
                throw MismatchedDimensions(std::string("parameter state tensor ") + name, ref.len(), t->len());
        };
        same("master_w", master_w, w); same("dv_w", dv_w, w); same("dm_w", dm_w, w);
        same("master_b", master_b, b); same("dv_b", dv_b, b); same("dm_b", dm_b, b);
    }
};

// ---------------------------------------------------------------------------------------
// DenseBlock (src/mlp.rs:232-821)
// ---------------------------------------------------------------------------------------
class DenseBlock {
  public:
    // DenseBlock::new / new_with_config (mlp.rs:309-375)
    DenseBlock(const GpuContext &ctx, bool is_training, size_t inputs, size_t outputs, size_t max_batch_size, InitFunc &init,
               const LayerInitConfig &cfg = LayerInitConfig(), Precision p = Precision::FP32) {
        if (inputs == 0 || outputs == 0) throw InvalidConfiguration("Input or output size cannot be 0.");
        if (max_batch_size == 0) throw InvalidConfiguration("Batch size cannot be 0.");
        const std::vector<float> w_vec = init.init(inputs, outputs, inputs * outputs);
        ParamState linear = ParamState::new_linear(ctx, w_vec, inputs, outputs, is_training, p);
        ParamState norm = ParamState::new_norm(ctx, outputs, is_training, p);
        build(ctx, is_training, std::move(linear), std::move(norm), max_batch_size, cfg, p);
    }
    static DenseBlock new_with_config(const GpuContext &ctx, bool is_training, size_t inputs, size_t outputs,
                                      size_t max_batch_size, InitFunc &init, const LayerInitConfig &cfg,
                                      Precision p = Precision::FP32) {
        return DenseBlock(ctx, is_training, inputs, outputs, max_batch_size, init, cfg, p);
    }
    // DenseBlock::from_tensors (mlp.rs:377-427)
    static DenseBlock from_tensors(const GpuContext &ctx, bool is_training, ParamState linear, ParamState norm,
                                   size_t max_batch_size, const LayerInitConfig &cfg, Precision p = Precision::FP32) {
        DenseBlock b;
        b.build(ctx, is_training, std::move(linear), std::move(norm), max_batch_size, cfg, p);
        return b;
    }
    DenseBlock(DenseBlock &&) noexcept = default;
    DenseBlock &operator=(DenseBlock &&) noexcept = default;

    // ---- getters / setters (mlp.rs:429-480) ----
    const Tensor &get_weights() const { return linear_.w; }
    const Tensor &get_biases() const { return linear_.b; }
    const Tensor *get_master_weights() const { return linear_.master_w.get(); }
    const Tensor *get_master_biases() const { return linear_.master_b.get(); }
    const Tensor *get_dv_weights() const { return linear_.dv_w.get(); }
    const Tensor *get_dv_biases() const { return linear_.dv_b.get(); }
    const Tensor *get_dm_weights() const { return linear_.dm_w.get(); }
    const Tensor *get_dm_biases() const { return linear_.dm_b.get(); }
    const Tensor &get_norm_weights() const { return norm_.w; }
    const Tensor &get_norm_biases() const { return norm_.b; }
    const Tensor *get_master_norm_weights() const { return norm_.master_w.get(); }
    const Tensor *get_master_norm_biases() const { return norm_.master_b.get(); }
    const Tensor *get_dv_norm_weights() const { return norm_.dv_w.get(); }
    const Tensor *get_dv_norm_biases() const { return norm_.dv_b.get(); }
    const Tensor *get_dm_norm_weights() const { return norm_.dm_w.get(); }
    const Tensor *get_dm_norm_biases() const { return norm_.dm_b.get(); }
    const Tensor *get_norm_weights_grad() const { return d_norm_w_.get(); }
    const Tensor *get_norm_biases_grad() const { return d_norm_b_.get(); }
    const Tensor &get_outputs() const { return out_; }
    const Tensor &get_predrop_outputs() const { return predrop_; }
    const Tensor &get_preact_outputs() const { return preact_; }
    const Tensor &get_centered_outputs() const { return centered_; }
    const Tensor &get_prenorm_outputs() const { return prenorm_; }
    const Tensor &get_norm_rstd() const { return norm_rstd_; }
    const Tensor *get_grads() const { return grad_.get(); }
    const Tensor *get_delta_prenorm_out() const { return d_prenorm_.get(); }
    const Tensor &get_masks() const { return mask_; }
    size_t get_max_batch_size() const { return max_batch_; }
    float get_mask_coeff() const { return cfg_.mask_coeff; }
    Normalisation get_normalisation() const { return cfg_.normalisation; }
    Activation get_activation() const { return cfg_.activation; }
    Regularisation get_regularisation() const { return cfg_.regularisation; }
    bool is_training_mode() const { return is_training_; }
    Precision precision() const { return precision_; }

    // DenseBlock<f32>::convert_f16 (mlp.rs:835-858) and DenseBlock<f16>::convert_f32 (mlp.rs:861-888):
    // parameters through the ParamState casts, forward cache and mask through a device cast, the
    // f32 gradient tensors move over. Both consume the block: call as std::move(block).convert_f16(ctx).
    DenseBlock convert_f16(const GpuContext &ctx, Precision p = Precision::FP16) && {
        if (precision_ != Precision::FP32 || p == Precision::FP32)
            throw UnsupportedTypeCast(precision_name(precision_), precision_name(p));
        ParamState lin = std::move(linear_).cast_f16(ctx, p), nrm = std::move(norm_).cast_f16(ctx, p);
        return std::move(*this).converted(ctx, std::move(lin), std::move(nrm), p);
    }
    DenseBlock convert_f32(const GpuContext &ctx) && {
        if (precision_ == Precision::FP32) throw UnsupportedTypeCast(precision_name(precision_), "FP32");
        ParamState lin = std::move(linear_).cast_f32(ctx), nrm = std::move(norm_).cast_f32(ctx);
        return std::move(*this).converted(ctx, std::move(lin), std::move(nrm), Precision::FP32);
    }

    void set_mask_coeff(float v) { cfg_.mask_coeff = v; refresh(); }
    void set_normalisation(Normalisation v) { cfg_.normalisation = v; refresh(); }
    void set_activation(Activation v) { cfg_.activation = v; refresh(); }
    void set_regularisation(Regularisation v) { cfg_.regularisation = v; refresh(); }
    void reset_mask(const GpuContext &ctx) { mask_.broadcast(ctx, 1.0f); }

    // The block as the C ABI sees it: borrowed device pointers + configuration.
    const sk_dense &desc() const { return desc_; }

    // ---- checks (mlp.rs:492-519) ----
    void check_input_dimension(const Tensor &input, size_t batch_size) const {
        if (input.rows() < batch_size)
            throw MismatchedDimensions("forward input rows vs explicit batch size", batch_size, input.rows());
        if (input.rows() > max_batch_)
            throw AllocationLimitExceeded(input.rows(), max_batch_, "input batches");
        if (input.cols() != linear_.w.rows())
            throw MismatchedDimensions("forward input feature columns mismatch", linear_.w.rows(), input.cols());
    }
    void check_mode(size_t batch_size) const {
        if (cfg_.activation == Activation::Softmax())
            throw InvalidConfiguration("Softmax activation can only be passed into the compute_loss function.");
        if (batch_size == 0) throw InvalidBatchSize("Batch size must be more than zero.");
        if (cfg_.normalisation == Normalisation::BatchNorm && batch_size == 1)
            throw InvalidBatchSize("Normalisation is set to BatchNorm, but given batch size is 1. "
                                   "Batch size must be more than 1.");
    }
    static void check_loss(const LossConfig &lc) {
        const LossFunc lf = lc.loss_func;
        const Activation act = lc.activation;
        if (lf == LossFunc::MeanSquareLoss && act == Activation::Softmax())
            throw InvalidConfiguration("Mean Squared Loss does not support the Softmax activation function.");
        if (lf == LossFunc::CrossEntropyLoss && act != Activation::Softmax())
            throw InvalidConfiguration("Cross-Entropy Loss only supports the Softmax activation function.");
        if (lf == LossFunc::BinaryCrossEntropy && act != Activation::Sigmoid())
            throw InvalidConfiguration("Binary Cross-Entropy only supports the Sigmoid activation function.");
    }

    // ---- hot path (mlp.rs:548-821) ----
    const Tensor &forward(const GpuContext &ctx, const Tensor &input, size_t batch_size, bool use_dropout, size_t step,
                          uint32_t row_offset = 0) {
        check_input_dimension(input, batch_size);
        check_mode(batch_size);
        ctx.gpu_forward_pass(*this, input, batch_size, use_dropout, step, row_offset);
        return out_;
    }
    void backward_output(const GpuContext &ctx, const Tensor &input, const TrainContext &train_ctx, size_t step) {
        if (!is_training_) throw TrainingModeRequired("output layer backward pass");
        check_input_dimension(input, train_ctx.batch_size);
        check_mode(train_ctx.batch_size);
        ctx.gpu_backward_pass(*this, input, train_ctx, step);
    }
    void backward_hidden(const GpuContext &ctx, DenseBlock &next_layer, const Tensor &input, const TrainContext &train_ctx,
                         size_t step) {
        if (!is_training_) throw TrainingModeRequired("hidden layer backward pass");
        check_input_dimension(input, train_ctx.batch_size);
        const size_t cur_cols = linear_.w.cols(), next_rows = next_layer.get_weights().rows();
        if (next_rows != cur_cols)
            throw MismatchedDimensions("backward pass weight adjacency (next layer rows vs current cols)", cur_cols, next_rows);
        if (!next_layer.get_grads() || next_layer.get_grads()->rows() < input.rows())
            throw MismatchedDimensions("backward pass activation gradient rows should be more than or equal to batch rows",
                                       input.rows(), next_layer.get_grads() ? next_layer.get_grads()->rows() : 0);
        check_mode(train_ctx.batch_size);
        ctx.gpu_hidden_layer_backward_pass(*this, next_layer, input, train_ctx, step);
    }
    void compute_loss(const GpuContext &ctx, const Tensor &target, const LossConfig &loss_config) {
        if (!is_training_) throw TrainingModeRequired("compute loss");
        check_target(target);
        check_loss(loss_config);
        ctx.gpu_compute_output_layer_error(*this, target, loss_config.loss_func, loss_config.activation);
    }
    void check_target(const Tensor &target) const {
        if (target.cols() != linear_.w.cols()) throw MismatchedDimensions("target columns", linear_.w.cols(), target.cols());
        if (target.rows() > max_batch_) throw AllocationLimitExceeded(target.rows(), max_batch_, "target batches");
    }

  private:
    DenseBlock() = default;
    // mlp.rs:377-427; the allocation order fixes the tensor ids
    void build(const GpuContext &ctx, bool is_training, ParamState linear, ParamState norm, size_t max_batch,
               const LayerInitConfig &cfg, Precision p) {
        linear.validate();
        norm.validate();
        precision_ = p; is_training_ = is_training; max_batch_ = max_batch; cfg_ = cfg;
        linear_ = std::move(linear);
        norm_ = std::move(norm);
        const size_t wc = linear_.w.cols();
        out_ = Tensor::zeros(ctx, max_batch, wc, p);
        predrop_ = Tensor::zeros(ctx, max_batch, wc, p);
        preact_ = Tensor::zeros(ctx, max_batch, wc, p);
        centered_ = Tensor::zeros(ctx, max_batch, wc, p);
        prenorm_ = Tensor::zeros(ctx, max_batch, wc, p);
        norm_rstd_ = Tensor::zeros(ctx, 1, std::max(max_batch, wc), p);
        if (is_training) {
            grad_ = std::make_unique<Tensor>(Tensor::zeros(ctx, max_batch, wc));
            d_prenorm_ = std::make_unique<Tensor>(Tensor::zeros(ctx, max_batch, wc));
            d_norm_w_ = std::make_unique<Tensor>(Tensor::zeros(ctx, max_batch, wc));
            d_norm_b_ = std::make_unique<Tensor>(Tensor::zeros(ctx, max_batch, wc));
        }
        mask_ = Tensor::fill(ctx, max_batch, wc, 1.0f, p);
        // 16-bit copy of d_prenorm feeding the tensor-core GEMMs; not a reference tensor, takes no id
        if (is_training && p != Precision::FP32)
            d_prenorm_lp_ = std::make_unique<Tensor>(Tensor::zeros(ctx, max_batch, wc, p, false));
        refresh();
    }
    DenseBlock converted(const GpuContext &ctx, ParamState lin, ParamState nrm, Precision p) && {
        DenseBlock b;
        b.precision_ = p; b.is_training_ = is_training_; b.max_batch_ = max_batch_; b.cfg_ = cfg_;
        b.linear_ = std::move(lin);
        b.norm_ = std::move(nrm);
        b.out_ = out_.cast(ctx, p); b.predrop_ = predrop_.cast(ctx, p); b.preact_ = preact_.cast(ctx, p);
        b.centered_ = centered_.cast(ctx, p); b.prenorm_ = prenorm_.cast(ctx, p); b.norm_rstd_ = norm_rstd_.cast(ctx, p);
        b.grad_ = std::move(grad_); b.d_prenorm_ = std::move(d_prenorm_);
        b.d_norm_w_ = std::move(d_norm_w_); b.d_norm_b_ = std::move(d_norm_b_);
        b.mask_ = mask_.cast(ctx, p);
        if (is_training_ && p != Precision::FP32)
            b.d_prenorm_lp_ = std::make_unique<Tensor>(Tensor::zeros(ctx, max_batch_, b.out_.cols(), p, false));
        b.refresh();
        ctx.synchronize(); // the casts read this block's tensors, which go away with it
        return b;
    }
    void refresh() {
        auto f = [](const std::unique_ptr<Tensor> &t) { return t ? (float *)t->ptr() : nullptr; };
        sk_dense d;
        std::memset(&d, 0, sizeof d);
        d.dtype = (uint32_t)precision_;
        d.K = (uint32_t)linear_.w.rows(); d.N = (uint32_t)linear_.w.cols();
        d.max_batch = (uint32_t)max_batch_; d.is_training = is_training_ ? 1u : 0u;
        d.w = linear_.w.ptr(); d.b = linear_.b.ptr();
        d.master_w = f(linear_.master_w); d.master_b = f(linear_.master_b);
        d.dv_w = f(linear_.dv_w); d.dv_b = f(linear_.dv_b); d.dm_w = f(linear_.dm_w); d.dm_b = f(linear_.dm_b);
        d.norm_w = norm_.w.ptr(); d.norm_b = norm_.b.ptr();
        d.master_norm_w = f(norm_.master_w); d.master_norm_b = f(norm_.master_b);
        d.dv_norm_w = f(norm_.dv_w); d.dv_norm_b = f(norm_.dv_b); d.dm_norm_w = f(norm_.dm_w); d.dm_norm_b = f(norm_.dm_b);
        d.out = out_.ptr(); d.predrop = predrop_.ptr(); d.preact = preact_.ptr();
        d.centered = centered_.ptr(); d.prenorm = prenorm_.ptr(); d.norm_rstd = norm_rstd_.ptr(); d.mask = mask_.ptr();
        d.grad = f(grad_); d.d_prenorm = f(d_prenorm_); d.d_norm_w = f(d_norm_w_); d.d_norm_b = f(d_norm_b_);
        d.d_prenorm_lp = d_prenorm_lp_ ? d_prenorm_lp_->ptr() : nullptr;
        d.norm = (uint32_t)cfg_.normalisation; d.act = cfg_.activation.ordinal(); d.leaky_coeff = cfg_.activation.coeff;
        d.regu = cfg_.regularisation.ordinal(); d.regu_coeff = cfg_.regularisation.regu_coeff;
        d.mask_coeff = cfg_.mask_coeff;
        d.tensor_id = (uint32_t)(linear_.w.get_id() & 0xFFFFFFFF);
        desc_ = d;
    }

    ParamState linear_, norm_;
    Tensor out_, predrop_, preact_, centered_, prenorm_, norm_rstd_, mask_;
    std::unique_ptr<Tensor> grad_, d_prenorm_, d_norm_w_, d_norm_b_, d_prenorm_lp_;
    size_t max_batch_ = 0;
    LayerInitConfig cfg_;
    Precision precision_ = Precision::FP32;
    bool is_training_ = false;
    sk_dense desc_{};
};

// ---------------------------------------------------------------------------------------
// FeedForwardNetwork (src/ffn.rs)
// ---------------------------------------------------------------------------------------
class FeedForwardNetwork {
  public:
    FeedForwardNetwork(std::vector<DenseBlock> layers, size_t inputs) : layers_(std::move(layers)), inputs_(inputs) {}

    // ffn.rs:40-57 — every layer's output tensor, borrowed. With `fused` the checks run first
    // and then the whole stack is one native call; without it each layer is called in turn.
    std::vector<const Tensor *> forward(const GpuContext &ctx, const Tensor &input, size_t batch_size, bool use_dropout,
                                        size_t step, uint32_t row_offset = 0, bool fused = true) {
        std::vector<const Tensor *> outputs;
        if (fused && !layers_.empty()) {
            const Tensor *cur = &input;
            for (auto &l : layers_) {
                l.check_input_dimension(*cur, batch_size);
                l.check_mode(batch_size);
                cur = &l.get_outputs();
            }
            ctx.gpu_ffn_forward(layers_, input, batch_size, use_dropout, step, row_offset);
            for (auto &l : layers_) outputs.push_back(&l.get_outputs());
            return outputs;
        }
        const Tensor *cur = &input;
        for (auto &l : layers_) {
            cur = &l.forward(ctx, *cur, batch_size, use_dropout, step, row_offset);
            outputs.push_back(cur);
        }
        return outputs;
    }

    // ffn.rs:73-94 — host vector in, copy of the last layer's output back
    Tensor forward_raw(const GpuContext &ctx, const std::vector<float> &raw_pixels, size_t batch_size, bool use_dropout,
                       size_t step) {
        if (layers_.empty())
            throw InvalidConfiguration("Cannot execute raw forward pass on an empty network matrix architecture");
        Tensor x = Tensor::from_cpu_vector(ctx, raw_pixels, batch_size, inputs_, layers_[0].precision());
        Tensor out = forward(ctx, x, batch_size, use_dropout, step).back()->clone(ctx);
        ctx.synchronize(); // x is released on return
        return out;
    }

    // ffn.rs:113-166 — output layer first, then the hidden layers in reverse; each hidden delta
    // reads the next layer's weights after that layer's update.
    void backward(const GpuContext &ctx, const std::vector<const Tensor *> &outputs, const Tensor &target, const Tensor &input,
                  const LossConfig &loss_config, const MultiLayerTrainContext &train_ctx, size_t step, bool fused = true) {
        const size_t n = layers_.size();
        if (outputs.size() != n || train_ctx.optimisers.size() != n || train_ctx.norm_optimisers.size() != n)
            throw InvalidConfiguration("Backward pass expects exactly " + std::to_string(n) +
                                       " activation vectors and optimizers. Found " + std::to_string(outputs.size()) +
                                       " outputs, " + std::to_string(train_ctx.optimisers.size()) + " optimisers.");
        if (n == 0) return;
        const size_t last = n - 1;
        bool own_outputs = true;
        for (size_t i = 0; i < n; ++i) own_outputs = own_outputs && outputs[i] == &layers_[i].get_outputs();
        if (fused && own_outputs) {
            check_backward(target, input, loss_config, train_ctx);
            ctx.gpu_ffn_backward(layers_, target, input, loss_config, train_ctx, step);
            return;
        }
        const Tensor &head_input = last > 0 ? *outputs[last - 1] : input;
        layers_[last].compute_loss(ctx, target, loss_config);
        layers_[last].backward_output(ctx, head_input, train_ctx.get_train_context(last), step);
        for (size_t i = last; i-- > 0;) {
            const Tensor &layer_input = i > 0 ? *outputs[i - 1] : input;
            layers_[i].backward_hidden(ctx, layers_[i + 1], layer_input, train_ctx.get_train_context(i), step);
        }
    }

    std::vector<DenseBlock> &get_layers() { return layers_; }
    const std::vector<DenseBlock> &get_layers() const { return layers_; }
    size_t len() const { return layers_.size(); }
    bool is_empty() const { return layers_.empty(); }

  private:
    // the host-side checks of compute_loss / backward_output / backward_hidden (mlp.rs:607-821)
    void check_backward(const Tensor &target, const Tensor &input, const LossConfig &lc,
                        const MultiLayerTrainContext &tc) const {
        for (auto &l : layers_)
            if (!l.is_training_mode()) throw TrainingModeRequired("backward pass");
        layers_.back().check_target(target);
        DenseBlock::check_loss(lc);
        const Tensor *cur = &input;
        for (size_t i = 0; i < layers_.size(); ++i) {
            const DenseBlock &l = layers_[i];
            l.check_input_dimension(*cur, tc.batch_size);
            l.check_mode(tc.batch_size);
            if (i + 1 < layers_.size() && layers_[i + 1].get_weights().rows() != l.get_weights().cols())
                throw MismatchedDimensions("backward pass weight adjacency (next layer rows vs current cols)",
                                           l.get_weights().cols(), layers_[i + 1].get_weights().rows());
            cur = &l.get_outputs();
        }
    }
    std::vector<DenseBlock> layers_;
    size_t inputs_;
};

// ---------------------------------------------------------------------------------------
// GpuContext methods: one C-ABI call each
// ---------------------------------------------------------------------------------------
inline void GpuContext::gpu_cast_t(const Tensor &src, Tensor &dst) const {
    if (src.len() != dst.len())
        throw MismatchedDimensions("GPU precision cast source vs destination buffer sizes", dst.len(), src.len());
    if ((src.precision() == Precision::FP32) == (dst.precision() == Precision::FP32))
        throw UnsupportedTypeCast(precision_name(src.precision()), precision_name(dst.precision()));
    check(sk_cast(ctx_, src.ptr(), (uint32_t)src.precision(), dst.ptr(), (uint32_t)dst.precision(), src.len()));
}
inline void GpuContext::gpu_broadcast(Tensor &dst, float value) const {
    check(sk_fill(ctx_, dst.ptr(), (uint32_t)dst.precision(), value, dst.len()));
}
inline void GpuContext::gpu_forward_pass(DenseBlock &cur, const Tensor &input, size_t batch_size, bool use_dropout, size_t step,
                                         uint32_t row_offset) const {
    check_tile_dim(cur.precision());
    check(sk_dense_forward(ctx_, &cur.desc(), input.ptr(), (uint32_t)input.rows(), (uint32_t)batch_size, use_dropout ? 1u : 0u,
                           (uint32_t)(step & 0xFFFFFFFFu), row_offset));
}
inline void GpuContext::gpu_compute_output_layer_error(DenseBlock &cur, const Tensor &target, LossFunc err_mode,
                                                       Activation activation) const {
    check(sk_output_error(ctx_, &cur.desc(), target.ptr(), (uint32_t)target.rows(), (uint32_t)cur.get_outputs().rows(),
                          (uint32_t)err_mode, activation.ordinal(), activation.coeff));
}
inline void GpuContext::gpu_backward_pass(DenseBlock &cur, const Tensor &input, const TrainContext &tc, size_t step) const {
    const sk_optim lin = tc.optimiser.kernel_args(), nrm = tc.norm_optimiser.kernel_args();
    check(sk_backward_update(ctx_, &cur.desc(), input.ptr(), (uint32_t)input.rows(), (uint32_t)tc.batch_size, &lin, &nrm,
                             tc.learn_rate, tc.grad_clamp, (uint32_t)(step & 0xFFFFFFFFu)));
}
inline void GpuContext::gpu_hidden_layer_backward_pass(DenseBlock &cur, DenseBlock &next, const Tensor &input,
                                                       const TrainContext &tc, size_t step) const {
    check_tile_dim(cur.precision());
    check(sk_hidden_error(ctx_, &cur.desc(), &next.desc(), (uint32_t)tc.batch_size, (uint32_t)tc.batch_size));
    gpu_backward_pass(cur, input, tc, step);
}
inline void GpuContext::gpu_ffn_forward(std::vector<DenseBlock> &layers, const Tensor &input, size_t batch_size,
                                        bool use_dropout, size_t step, uint32_t row_offset) const {
    if (layers.empty()) return;
    check_tile_dim(layers[0].precision());
    std::vector<const sk_dense *> ptrs;
    for (auto &l : layers) ptrs.push_back(&l.desc());
    check(sk_ffn_forward(ctx_, ptrs.data(), (uint32_t)ptrs.size(), input.ptr(), (uint32_t)input.rows(), (uint32_t)batch_size,
                         use_dropout ? 1u : 0u, (uint32_t)(step & 0xFFFFFFFFu), row_offset));
}
inline void GpuContext::gpu_ffn_backward(std::vector<DenseBlock> &layers, const Tensor &target, const Tensor &input,
                                         const LossConfig &lc, const MultiLayerTrainContext &tc, size_t step) const {
    std::vector<const sk_dense *> ptrs;
    std::vector<sk_optim> lin, nrm;
    for (size_t i = 0; i < layers.size(); ++i) {
        ptrs.push_back(&layers[i].desc());
        lin.push_back(tc.optimisers[i].kernel_args());
        nrm.push_back(tc.norm_optimisers[i].kernel_args());
    }
    check(sk_ffn_backward(ctx_, ptrs.data(), (uint32_t)ptrs.size(), target.ptr(), (uint32_t)target.rows(), input.ptr(),
                          (uint32_t)input.rows(), (uint32_t)lc.loss_func, lc.activation.ordinal(), lc.activation.coeff,
                          lin.data(), nrm.data(), (uint32_t)tc.batch_size, tc.learn_rate, tc.grad_clamp,
                          (uint32_t)(step & 0xFFFFFFFFu)));
}

} // namespace soklyn
#endif // SOKLYN_B200_HPP
