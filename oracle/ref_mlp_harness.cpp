// TEST INFRASTRUCTURE.  C wrapper around the reference's own host MLP, mlp_cpp::MLP<double>
// (test/mlp.h of intel/tiny-dpcpp-nn), which is compiled UNMODIFIED from where it lies in the
// reference checkout (-I<reference>/test).  It is the oracle the reference's own tests use
// (test/doctest_swiftnet.cpp:112-232).  Output goes to oracle/_ref/ only.
//
// mlp.h keeps its weights private and has no setter; the harness reaches them by compiling the
// header with `private` spelled `public`, so seeded weights can be injected without touching it.
#include <cmath>
#include <iostream>
#include <random>
#include <sstream>
#include <string>
#include <vector>

#include "common.h" // shim
#define private public
#include "mlp.h"
#undef private

using mlp_cpp::MLP;

static std::streambuf *const g_cout_buf = std::cout.rdbuf();

static Activation to_act(int a) { return a == 0 ? Activation::ReLU : a == 4 ? Activation::Sigmoid : Activation::None; }

extern "C" {

// One sample through forward + backward of the reference MLP.
//   weights: n_mat matrices (in x out, row-major, unpacked) or null to keep mlp.h's own init
//            (init_mode 0 linspace, 1 random (mt19937 seed 42), 2 constant 0.1)
//   x, target: `width` doubles.  n_mat = n_hidden_layers + 1 (mlp.h's 4th constructor argument).
// Outputs (any may be null): fwd ((n_mat + 1) x width), weights_out (n_mat x width x width, in x out),
//   grads (n_mat x width x width, out x in), loss_grads (n_mat x width, already divided by batch),
//   dl_dinput (width, divided by batch), loss (width).
int ref_mlp_sample(int in_dim, int width, int out_dim, int n_mat, int batch, int act, int out_act,
                   const double *weights, int init_mode, const double *x, const double *target, double loss_scale,
                   double *fwd, double *weights_out, double *grads, double *loss_grads, double *dl_dinput,
                   double *loss) {
    try {
        std::ostringstream sink; // mlp.h prints from forward(); keep the test output clean
        auto *old = std::cout.rdbuf(sink.rdbuf());
        MLP<double> mlp(in_dim, width, out_dim, n_mat, batch, to_act(act), to_act(out_act),
                        (mlp_cpp::WeightInitMode)init_mode);
        if (weights) {
            for (int l = 0; l < n_mat; ++l)
                for (int k = 0; k < width; ++k)
                    for (int n = 0; n < width; ++n)
                        mlp.weights[l].data[n][k] = weights[((size_t)l * width + k) * width + n]; // stored (out x in)
        }
        std::vector<double> xin(x, x + width), tgt(target, target + width);
        auto outs = mlp.forward(xin, true);
        if (fwd)
            for (int l = 0; l <= n_mat; ++l)
                for (int n = 0; n < width; ++n) fwd[l * width + n] = outs[l][n];
        if (weights_out) {
            auto wv = mlp.getUnpackedWeights();
            for (size_t i = 0; i < wv.size(); ++i) weights_out[i] = wv[i];
        }
        if (grads || loss_grads || dl_dinput || loss) {
            std::vector<mlp_cpp::Matrix<double>> wg(n_mat);
            std::vector<std::vector<double>> lg;
            std::vector<double> lv, dldo, dldi;
            mlp.backward(xin, tgt, wg, lg, lv, dldo, dldi, loss_scale);
            if (grads)
                for (int l = 0; l < n_mat; ++l)
                    for (int o = 0; o < width; ++o)
                        for (int i = 0; i < width; ++i) grads[((size_t)l * width + o) * width + i] = wg[l].data[o][i];
            if (loss_grads)
                for (int l = 0; l < n_mat; ++l)
                    for (int n = 0; n < width; ++n) loss_grads[l * width + n] = lg[l][n];
            if (dl_dinput)
                for (int n = 0; n < width; ++n) dl_dinput[n] = dldi[n];
            if (loss)
                for (int n = 0; n < width; ++n) loss[n] = lv[n];
        }
        std::cout.rdbuf(old);
        return 0;
    } catch (const std::exception &e) {
        std::cout.rdbuf(g_cout_buf);
        std::cerr << "ref_mlp_sample: " << e.what() << std::endl;
        return 1;
    }
}

// Throughput helper for the CPU baseline: `batch` samples through forward (and backward when
// do_backward != 0) of one shared MLP instance; returns the number of samples processed.
long ref_mlp_run_batch(int width, int n_mat, int act, int out_act, const double *weights, const double *x,
                       const double *target, long batch, int do_backward, double *checksum) {
    // called from several threads at once: std::cout is left alone here (with equal widths mlp.h prints nothing)
    MLP<double> mlp(width, width, width, n_mat, 1, to_act(act), to_act(out_act), mlp_cpp::WeightInitMode::constant);
    for (int l = 0; l < n_mat; ++l)
        for (int k = 0; k < width; ++k)
            for (int n = 0; n < width; ++n) mlp.weights[l].data[n][k] = weights[((size_t)l * width + k) * width + n];
    double acc = 0.0;
    for (long b = 0; b < batch; ++b) {
        std::vector<double> xin(x + b * width, x + (b + 1) * width);
        if (!do_backward) {
            auto out = mlp.forward(xin, false);
            acc += out[0][0];
        } else {
            std::vector<double> tgt(target + b * width, target + (b + 1) * width);
            std::vector<mlp_cpp::Matrix<double>> wg(n_mat);
            std::vector<std::vector<double>> lg;
            std::vector<double> lv, dldo, dldi;
            mlp.backward(xin, tgt, wg, lg, lv, dldo, dldi, 1.0);
            acc += wg[0].data[0][0];
        }
    }
    if (checksum) *checksum = acc;
    return batch;
}

} // extern "C"
