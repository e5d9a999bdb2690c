// Test program for the C++ host mirror (include/train_station_b200.hpp): trains an MLP for a number of steps exactly
// as the Python tests do and writes every result to a file the pytest side compares with the oracle; then times the
// same step in a loop, which measures the step rate of a compiled host (no interpreter between the launches).
//
//   mirror_step <in.bin> <out.bin> <steps> <loss: sum|mean|mse> <relu_last: 0|1> <timed steps>
//
// in.bin : int32 n_layers, batch, d[0..n_layers]; then f32 x[batch*d0], target[batch*dn], and per layer W, b.
// out.bin: f32 loss, y[batch*dn], then per layer gW, gb (of the last step), W, b, m(W), v(W) after the last step.
// stdout : one line "steps_per_s <value>" when timed steps > 0.
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "train_station_b200.hpp"

namespace tsn = train_station;

static std::vector<float> read_f32(FILE* f, size_t n) {
    std::vector<float> v(n);
    if (n && fread(v.data(), sizeof(float), n, f) != n) throw tsn::Error("short input file");
    return v;
}
static void write_f32(FILE* f, const std::vector<float>& v) {
    if (!v.empty() && fwrite(v.data(), sizeof(float), v.size(), f) != v.size()) throw tsn::Error("short write");
}

struct Net {
    std::vector<tsn::Tensor> W, B;
    tsn::Tensor x, target;
    std::string loss_kind;
    bool relu_last = false;

    // one forward pass and the loss, written the way the reference's examples write it
    std::pair<tsn::Tensor, tsn::Tensor> forward() const {
        tsn::Tensor h = x;
        for (size_t i = 0; i < W.size(); ++i) {
            h = h.matmul(W[i]).add_tensor(B[i]);
            if (i + 1 < W.size() || relu_last) h = h.relu();
        }
        tsn::Tensor loss = loss_kind == "sum" ? h.sum() : loss_kind == "mean" ? h.mean() : h.sub_tensor(target).pow_scalar(2.0f).mean();
        return {h, loss};
    }
};

int main(int argc, char** argv) {
    if (argc != 7) {
        fprintf(stderr, "usage: %s in.bin out.bin steps sum|mean|mse relu_last timed_steps\n", argv[0]);
        return 2;
    }
    try {
        const int steps = std::stoi(argv[3]), timed = std::stoi(argv[6]);
        if (!tsn::cuda_is_available()) throw tsn::Error("no CUDA device: this library has no CPU fallback");
        tsn::set_default_device(0);
        FILE* in = fopen(argv[1], "rb");
        if (!in) throw tsn::Error(std::string("cannot open ") + argv[1]);
        int32_t head[2];
        if (fread(head, sizeof(int32_t), 2, in) != 2) throw tsn::Error("short header");
        const int layers = head[0];
        const size_t batch = (size_t)head[1];
        std::vector<int32_t> d((size_t)layers + 1);
        if (fread(d.data(), sizeof(int32_t), d.size(), in) != d.size()) throw tsn::Error("short header");
        Net net;
        net.loss_kind = argv[4];
        net.relu_last = std::stoi(argv[5]) != 0;
        net.x = tsn::Tensor::from_slice(read_f32(in, batch * d[0]), {batch, (size_t)d[0]});
        net.target = tsn::Tensor::from_slice(read_f32(in, batch * d[layers]), {batch, (size_t)d[layers]});
        for (int i = 0; i < layers; ++i) {
            net.W.push_back(tsn::Tensor::from_slice(read_f32(in, (size_t)d[i] * d[i + 1]), {(size_t)d[i], (size_t)d[i + 1]}).with_requires_grad());
            net.B.push_back(tsn::Tensor::from_slice(read_f32(in, (size_t)d[i + 1]), {(size_t)d[i + 1]}).with_requires_grad());
        }
        fclose(in);

        tsn::Adam opt = tsn::Adam::with_learning_rate(1e-3f);
        std::vector<tsn::Tensor*> params;
        for (int i = 0; i < layers; ++i) {
            params.push_back(&net.W[i]);
            params.push_back(&net.B[i]);
        }
        for (tsn::Tensor* p : params) opt.add_parameter(*p);

        FILE* out = fopen(argv[2], "wb");
        if (!out) throw tsn::Error(std::string("cannot open ") + argv[2]);
        for (int s = 0; s < steps; ++s) {
            auto [y, loss] = net.forward();
            loss.backward();
            if (s + 1 == steps) {
                write_f32(out, {loss.value()});
                write_f32(out, y.data());
                for (int i = 0; i < layers; ++i) {
                    write_f32(out, net.W[i].grad_by_value().value().data());
                    write_f32(out, net.B[i].grad_by_value().value().data());
                }
            }
            opt.step(params);
            opt.zero_grad(params);
        }
        for (int i = 0; i < layers; ++i) {
            write_f32(out, net.W[i].data());
            write_f32(out, net.B[i].data());
            auto [m, v] = opt.state(net.W[i]);
            write_f32(out, m.data());
            write_f32(out, v.data());
        }
        fclose(out);

        {   // NoGradTrack: nothing is recorded while it lives, and inference leaves no gradient behind
            tsn::NoGradTrack guard;
            auto [y, loss] = net.forward();
            if (loss.requires_grad() || tsn::is_grad_enabled()) throw tsn::Error("NoGradTrack did not switch gradient tracking off");
        }
        if (!tsn::is_grad_enabled()) throw tsn::Error("NoGradTrack did not restore gradient tracking");
        bool threw = false;
        try { tsn::Tensor::ones({2, 3}).matmul(tsn::Tensor::ones({4, 2})); } catch (const tsn::Error&) { threw = true; }
        if (!threw) throw tsn::Error("a shape mismatch in matmul did not throw");

        if (timed > 0) {
            for (int s = 0; s < 20; ++s) {       // warm-up: allocator and clocks
                auto [y, loss] = net.forward();
                loss.backward();
                opt.step(params);
                opt.zero_grad(params);
            }
            tsn::synchronize();
            const auto t0 = std::chrono::steady_clock::now();
            for (int s = 0; s < timed; ++s) {
                auto [y, loss] = net.forward();
                loss.backward();
                opt.step(params);
                opt.zero_grad(params);
            }
            tsn::synchronize();
            const double sec = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
            printf("steps_per_s %.1f\n", timed / sec);
        }
        return 0;
    } catch (const std::exception& e) {
        fprintf(stderr, "mirror_step: %s\n", e.what());
        return 1;
    }
}
