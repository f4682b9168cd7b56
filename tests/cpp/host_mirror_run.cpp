// Test driver for the C++ host mirror (include/soklyn_b200.hpp).
//
//   host_mirror_run checks               host-only checks, no GPU needed: error variants raised before
//                                        any device work, schedulers, seeds. Prints "ok <n>".
//   host_mirror_run train IN OUT         builds the network described by IN on device 0, trains it for the
//                                        given steps through DenseBlock / FeedForwardNetwork, and writes the
//                                        last layer's output of every step plus the final state of every
//                                        layer to OUT. tests/test_cpp_host_gpu.py compares OUT with the same
//                                        run through the Python mirror (bit for bit) and the CPU oracle.
//
// IN  (little endian): u32 magic 'SKLN', precision, layers, batch, max_batch, steps, loss, loss_act,
//      optimiser (0 SGD, 1 Adam), use_dropout, fused (bit 0: whole-network native calls, bit 1: every step as one CUDA graph), cosine (0/1),
//      cosine_total, cosine_warmup; f32 lr, loss_act_coeff, cosine_min, cosine_max;
//      u32 dims[layers+1]; per layer {u32 norm, u32 act, f32 act_coeff, f32 mask_coeff, u32 regu, f32 regu_coeff};
//      f32 weights of every layer [K x N]; f32 x [batch x dims[0]]; f32 target [batch x dims[layers]].
// OUT: a sequence of records {u32 name_len, name, u64 count, f32 values[count]}.
#include <cstdio>
#include <cstring>
#include <fstream>
#include <iostream>

#include "soklyn_b200.hpp"

using namespace soklyn;

namespace {

struct Reader {
    std::ifstream f;
    explicit Reader(const char *path) : f(path, std::ios::binary) {
        if (!f) throw std::runtime_error(std::string("cannot open ") + path);
    }
    uint32_t u32() { uint32_t v; f.read((char *)&v, 4); return v; }
    float f32() { float v; f.read((char *)&v, 4); return v; }
    std::vector<float> floats(size_t n) {
        std::vector<float> v(n);
        f.read((char *)v.data(), (std::streamsize)(n * 4));
        if (!f) throw std::runtime_error("input file too short");
        return v;
    }
};

struct Writer {
    std::ofstream f;
    explicit Writer(const char *path) : f(path, std::ios::binary) {}
    void record(const std::string &name, const std::vector<float> &v) {
        const uint32_t n = (uint32_t)name.size();
        const uint64_t c = v.size();
        f.write((const char *)&n, 4);
        f.write(name.data(), n);
        f.write((const char *)&c, 8);
        f.write((const char *)v.data(), (std::streamsize)(c * 4));
    }
};

template <class E, class F> int expect_throw(const char *what, F &&fn) {
    try {
        fn();
    } catch (const E &e) {
        return 1;
    } catch (const std::exception &e) {
        std::fprintf(stderr, "%s: wrong exception: %s\n", what, e.what());
        return -1000;
    }
    std::fprintf(stderr, "%s: no exception\n", what);
    return -1000;
}

int host_checks() {
    int ok = 0;
    // scramble_seed (src/util/core.rs:90-94) restated independently
    for (uint32_t step : {0u, 1u, 7u, 123456u})
        for (uint32_t id : {0u, 23u, 54u}) {
            uint32_t h = step * 1103515245u + id;
            h = (h ^ (h >> 16)) * 1103515245u;
            h ^= h >> 15;
            if (scramble_seed(step, id) != h) { std::fprintf(stderr, "scramble_seed mismatch\n"); return 1; }
            ++ok;
        }
    // schedulers (src/util/scheduler.rs)
    {
        CosineDecayLR s(1e-5f, 1e-3f, 100, 10);
        if (s.get_learning_rate() != 1e-5f) return 2;
        for (int i = 0; i < 10; ++i) s.step();
        if (std::fabs(s.get_learning_rate() - 1e-3f) > 1e-9f) return 3;
        for (int i = 0; i < 90; ++i) s.step();
        if (std::fabs(s.get_learning_rate() - 1e-5f) > 1e-9f) return 4;
        ExponentialLR e(0.1f, 0.5f);
        e.step(); e.step();
        if (e.get_learning_rate() != 0.025f) return 5;
        e.reset();
        if (e.get_learning_rate() != 0.1f) return 6;
        ReduceLROnPlateauScheduler r(2, SchedulerMode::Minimize, 0.5f, 0.01f);
        r.reset(0.1f);
        r.step(1.0f); r.step(2.0f);
        if (r.get_learning_rate() != 0.1f) return 7;
        r.step(2.0f);
        if (r.get_learning_rate() != 0.05f) return 8;
        r.step(std::nanf(""));
        if (r.get_learning_rate() != 0.05f) return 9;
        for (int i = 0; i < 20; ++i) r.step(3.0f);
        if (r.get_learning_rate() != 0.01f) return 10;
        ok += 9;
        ok += expect_throw<InvalidConfiguration>("zero patience", [] { ReduceLROnPlateauScheduler(0, SchedulerMode::Maximize, .5f, 0.f); });
    }
    // optimiser unpacking (src/io/device/ffn_device.rs:254-264)
    {
        const sk_optim a = Optimiser::Adam(0.8f, 0.99f, 1e-6f).kernel_args();
        const sk_optim s = Optimiser::SGD(0.9f, true).kernel_args();
        if (a.kind != 1 || a.beta1 != 0.8f || a.beta2 != 0.99f || a.epsilon != 1e-6f || a.nesterov != 0) return 11;
        if (s.kind != 0 || s.beta1 != 0.9f || s.beta2 != 0.f || s.nesterov != 1) return 12;
        ok += 2;
    }
    // initialisers: sizes, bounds, determinism
    {
        InitXavierUniformFunc u1(42), u2(42);
        auto a = u1.init(64, 32, 2048), b = u2.init(64, 32, 2048);
        const float lim = std::sqrt(6.0f / 96.0f);
        for (size_t i = 0; i < a.size(); ++i)
            if (a[i] != b[i] || std::fabs(a[i]) > lim) return 13;
        InitHeNormalFunc n(7);
        auto c = n.init(256, 64, 16384);
        double m = 0, v = 0;
        for (float x : c) m += x;
        m /= c.size();
        for (float x : c) v += (x - m) * (x - m);
        v /= c.size();
        if (std::fabs(m) > 5e-3 || std::fabs(v - 2.0 / 256) > 1e-3) return 14;
        ok += 2;
        ok += expect_throw<MismatchedDimensions>("given weights", [] { InitGivenFunc g({1.f, 2.f}); g.init(2, 2, 4); });
    }
    // error messages carry the reference's text
    {
        const MismatchedDimensions e("target columns", 10, 12);
        if (std::string(e.what()) != "Dimension mismatch: target columns: expected 10, found 12.") return 15;
        const TrainingModeRequired t("compute loss");
        if (std::string(t.what()) != "Invalid operation: compute loss: Action requires the network to be in training mode.") return 16;
        ok += 2;
        ok += expect_throw<InvalidConfiguration>("loss/activation", [] {
            DenseBlock::check_loss(LossConfig{LossFunc::CrossEntropyLoss, Activation::Sigmoid()});
        });
        ok += expect_throw<InvalidConfiguration>("mse softmax", [] {
            DenseBlock::check_loss(LossConfig{LossFunc::MeanSquareLoss, Activation::Softmax()});
        });
        ok += expect_throw<InvalidConfiguration>("bce", [] {
            DenseBlock::check_loss(LossConfig{LossFunc::BinaryCrossEntropy, Activation::Tanh()});
        });
    }
    if (ok < 0) return 17;
    std::printf("ok %d\n", ok);
    return 0;
}

// Error behaviour that needs a device: the same cases tests/test_api_gpu.py runs through Python.
int device_checks(const GpuContext &ctx) {
    int ok = 0;
    InitZeroFunc zero;
    ok += expect_throw<InvalidConfiguration>("zero inputs", [&] { DenseBlock(ctx, true, 0, 4, 8, zero); });
    ok += expect_throw<InvalidConfiguration>("zero batch", [&] { DenseBlock(ctx, true, 4, 4, 0, zero); });
    DenseBlock a(ctx, true, 8, 16, 4, zero), b(ctx, true, 16, 8, 4, zero), infer(ctx, false, 8, 16, 4, zero);
    Tensor x = Tensor::zeros(ctx, 4, 8), wide = Tensor::zeros(ctx, 4, 9), tall = Tensor::zeros(ctx, 5, 8);
    Tensor t = Tensor::zeros(ctx, 4, 16);
    const TrainContext tc{Optimiser::SGD(), Optimiser::SGD(), 4, 0.1f};
    ok += expect_throw<MismatchedDimensions>("columns", [&] { a.forward(ctx, wide, 4, false, 1); });
    ok += expect_throw<AllocationLimitExceeded>("rows", [&] { a.forward(ctx, tall, 4, false, 1); });
    ok += expect_throw<MismatchedDimensions>("batch > rows", [&] { a.forward(ctx, x, 5, false, 1); });
    ok += expect_throw<InvalidBatchSize>("batch 0", [&] { a.forward(ctx, x, 0, false, 1); });
    ok += expect_throw<TrainingModeRequired>("inference loss", [&] { infer.compute_loss(ctx, t, LossConfig{}); });
    ok += expect_throw<TrainingModeRequired>("inference backward", [&] { infer.backward_output(ctx, x, tc, 1); });
    ok += expect_throw<MismatchedDimensions>("adjacency", [&] { a.backward_hidden(ctx, a, x, tc, 1); });
    a.set_normalisation(Normalisation::BatchNorm);
    ok += expect_throw<InvalidBatchSize>("batchnorm 1", [&] { a.forward(ctx, x, 1, false, 1); });
    a.set_normalisation(Normalisation::Disabled);
    a.set_activation(Activation::Softmax());
    ok += expect_throw<InvalidConfiguration>("softmax forward", [&] { a.forward(ctx, x, 4, false, 1); });
    a.set_activation(Activation::ReLU());
    ok += expect_throw<UnsupportedTypeCast>("cast f32->f32", [&] { Tensor y = Tensor::zeros(ctx, 4, 8); ctx.gpu_cast_t(x, y); });
    {
        GpuContext odd(8, 0);
        DenseBlock hb(odd, true, 8, 16, 4, zero, LayerInitConfig(), Precision::FP16);
        Tensor hx = Tensor::zeros(odd, 4, 8, Precision::FP16);
        ok += expect_throw<HardwareConstraintViolation>("tile dim", [&] { hb.forward(odd, hx, 4, false, 1); });
    }
    {   // convert_f16 / convert_f32 (src/mlp.rs:835-888): the f32 parameters survive the round trip bit for bit
        InitXavierUniformFunc init(5);
        DenseBlock f(ctx, true, 8, 16, 4, init);
        const std::vector<float> w0 = f.get_weights().download(ctx);
        DenseBlock h = std::move(f).convert_f16(ctx);
        bool good = h.precision() == Precision::FP16 && h.get_master_weights() && h.get_master_weights()->download(ctx) == w0 &&
                    h.get_weights().precision() == Precision::FP16 && h.get_grads() && h.desc().d_prenorm_lp;
        Tensor hx = Tensor::zeros(ctx, 4, 8, Precision::FP16);
        h.forward(ctx, hx, 4, false, 1);
        ok += expect_throw<UnsupportedTypeCast>("f16 -> f16", [&] { DenseBlock again = std::move(h).convert_f16(ctx); });
        DenseBlock back = std::move(h).convert_f32(ctx);
        good = good && back.precision() == Precision::FP32 && !back.get_master_weights() && back.get_weights().download(ctx) == w0;
        ok += good ? 1 : -1000;
    }
    std::vector<DenseBlock> layers;
    layers.push_back(std::move(a));
    layers.push_back(std::move(b));
    FeedForwardNetwork net(std::move(layers), 8);
    auto outs = net.forward(ctx, x, 4, false, 1);
    MultiLayerTrainContext one{{Optimiser::SGD()}, {Optimiser::SGD()}, 4, 0.1f};
    Tensor t8 = Tensor::zeros(ctx, 4, 8);
    ok += expect_throw<InvalidConfiguration>("optimiser count", [&] { net.backward(ctx, outs, t8, x, LossConfig{}, one, 1); });
    ctx.synchronize();
    if (ok != 16) std::fprintf(stderr, "%d of 16 device checks passed\n", ok);
    return ok == 16 ? 0 : 1;
}

int train(const char *in_path, const char *out_path) {
    Reader in(in_path);
    if (in.u32() != 0x4E4C4B53u) throw std::runtime_error("bad magic");
    const Precision prec = (Precision)in.u32();
    const uint32_t n_layers = in.u32(), batch = in.u32(), max_batch = in.u32(), steps = in.u32();
    const LossFunc loss = (LossFunc)in.u32();
    const uint32_t loss_act = in.u32(), optimiser = in.u32(), use_dropout = in.u32(), fused = in.u32();
    const uint32_t cosine = in.u32(), cos_total = in.u32(), cos_warm = in.u32();
    const float lr = in.f32(), loss_act_coeff = in.f32(), cos_min = in.f32(), cos_max = in.f32();
    std::vector<uint32_t> dims(n_layers + 1);
    for (auto &d : dims) d = in.u32();
    std::vector<LayerInitConfig> cfgs(n_layers);
    for (auto &c : cfgs) {
        c.normalisation = (Normalisation)in.u32();
        c.activation.kind = in.u32();
        c.activation.coeff = in.f32();
        c.mask_coeff = in.f32();
        c.regularisation.kind = in.u32();
        c.regularisation.regu_coeff = in.f32();
    }
    GpuContext ctx(16, 0);
    if (int rc = device_checks(ctx)) { std::fprintf(stderr, "device checks failed\n"); return rc; }

    reset_tensor_ids(0);
    std::vector<DenseBlock> layers;
    for (uint32_t i = 0; i < n_layers; ++i) {
        InitGivenFunc init(in.floats((size_t)dims[i] * dims[i + 1]));
        layers.emplace_back(ctx, true, dims[i], dims[i + 1], max_batch, init, cfgs[i], prec);
    }
    const std::vector<float> xh = in.floats((size_t)batch * dims[0]), th = in.floats((size_t)batch * dims[n_layers]);
    Tensor x = Tensor::from_cpu_vector(ctx, xh, batch, dims[0], prec);
    Tensor t = Tensor::from_cpu_vector(ctx, th, batch, dims[n_layers], prec);
    FeedForwardNetwork net(std::move(layers), dims[0]);

    const Optimiser opt = optimiser == 0 ? Optimiser::SGD(0.f, false) : Optimiser::Adam(0.9f, 0.999f, 1e-8f);
    MultiLayerTrainContext tc{std::vector<Optimiser>(n_layers, opt), std::vector<Optimiser>(n_layers, opt), batch, lr};
    const LossConfig lc{loss, Activation{loss_act, loss_act_coeff}};
    CosineDecayLR sched(cos_min, cos_max, cos_total, cos_warm);

    Writer out(out_path);
    for (uint32_t s = 1; s <= steps; ++s) {
        if (cosine) tc.learn_rate = sched.step();
        if (fused & 2u) {   // forward and backward recorded and launched as one graph; the output is read afterwards
            GpuContext::StepGraph graph(ctx);
            auto outs = net.forward(ctx, x, batch, use_dropout != 0, s, 0, (fused & 1u) != 0);
            net.backward(ctx, outs, t, x, lc, tc, s, (fused & 1u) != 0);
            graph.launch();
            out.record("step_out", outs.back()->download(ctx));
            continue;
        }
        auto outs = net.forward(ctx, x, batch, use_dropout != 0, s, 0, (fused & 1u) != 0);
        out.record("step_out", outs.back()->download(ctx));
        net.backward(ctx, outs, t, x, lc, tc, s, (fused & 1u) != 0);
    }
    ctx.synchronize();
    for (uint32_t i = 0; i < n_layers; ++i) {
        const DenseBlock &l = net.get_layers()[i];
        const std::string p = "l" + std::to_string(i) + ".";
        const bool half = prec != Precision::FP32;
        out.record(p + "id", {(float)l.get_weights().get_id()});
        out.record(p + "w", (half ? *l.get_master_weights() : l.get_weights()).download(ctx));
        out.record(p + "b", (half ? *l.get_master_biases() : l.get_biases()).download(ctx));
        out.record(p + "norm_w", (half ? *l.get_master_norm_weights() : l.get_norm_weights()).download(ctx));
        out.record(p + "norm_b", (half ? *l.get_master_norm_biases() : l.get_norm_biases()).download(ctx));
        out.record(p + "dm_w", l.get_dm_weights()->download(ctx));
        out.record(p + "dv_w", l.get_dv_weights()->download(ctx));
        out.record(p + "out", l.get_outputs().download(ctx));
        out.record(p + "preact", l.get_preact_outputs().download(ctx));
        out.record(p + "mask", l.get_masks().download(ctx));
        out.record(p + "grad", l.get_grads()->download(ctx));
        out.record(p + "d_prenorm", l.get_delta_prenorm_out()->download(ctx));
    }
    std::printf("trained %u steps, %llu kernel launches\n", steps, (unsigned long long)ctx.launch_count());
    return 0;
}

} // namespace

int main(int argc, char **argv) {
    try {
        if (argc == 2 && std::string(argv[1]) == "checks") return host_checks();
        if (argc == 4 && std::string(argv[1]) == "train") return train(argv[2], argv[3]);
        if (argc == 7 && std::string(argv[1]) == "draws") {
            // draws KIND SEED FAN_IN FAN_OUT N: the initialiser's values as hexadecimal bit patterns, one per line,
            // after the generator's first eight raw 32-bit draws
            const std::string kind = argv[2];
            const uint64_t seed = std::strtoull(argv[3], nullptr, 10);
            const size_t fi = std::strtoull(argv[4], nullptr, 10), fo = std::strtoull(argv[5], nullptr, 10);
            const size_t n = std::strtoull(argv[6], nullptr, 10);
            InitXavierUniformFunc raw(seed);
            for (int i = 0; i < 8; ++i) std::printf("%08x\n", raw.next_u32());
            std::vector<float> v;
            if (kind == "xavier_uniform") { InitXavierUniformFunc f(seed, 0.5f); v = f.init(fi, fo, n); }
            else if (kind == "xavier_normal") { InitXavierNormalFunc f(seed); v = f.init(fi, fo, n); }
            else if (kind == "he_uniform") { InitHeUniformFunc f(seed); v = f.init(fi, fo, n); }
            else if (kind == "he_normal") { InitHeNormalFunc f(seed, 2.0f); v = f.init(fi, fo, n); }
            else return 2;
            for (float x : v) { uint32_t b; std::memcpy(&b, &x, 4); std::printf("%08x\n", b); }
            return 0;
        }
        std::fprintf(stderr, "usage: %s checks | train IN OUT | draws KIND SEED FAN_IN FAN_OUT N\n", argv[0]);
        return 2;
    } catch (const std::exception &e) {
        std::fprintf(stderr, "error: %s\n", e.what());
        return 3;
    }
}
