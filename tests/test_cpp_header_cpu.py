"""The header-only C++ layer (tiny-dpcpp-nn_b200/cpp/tnn_api.h) compiles, links against the C-ABI library
and reports host-side errors as exceptions - no device needed."""
import os
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SRC = r"""
#include <cstdio>
#include <cstring>
#include "tnn_api.h"
int main() {
    std::printf("%s\n", tnn_version());
    try {
        tnn::Network<tnn::half> bad(64, 64, 4, tnn::Activation::ReLU, tnn::Activation::None, /*width*/ 48, true);
        return 1;
    } catch (const std::runtime_error &e) {
        if (!std::strstr(e.what(), "power of 2")) return 2;
    }
    try {
        tnn::EncodingModule bad("{\"otype\": \"Nope\"}");
        return 3;
    } catch (const std::runtime_error &e) {
        if (!std::strstr(e.what(), "Unknown encoding type")) return 4;
    }
    // the whole surface instantiates: Network<T>, SwiftNetMLP<T>, Encoding, Loss<T>, Optimizer, Trainer<T>, DataParallel
    using Net = tnn::SwiftNetMLP<tnn::bf16>;
    void (Net::*inf)(const void *, void *, size_t, void *) = &Net::inference;
    void (tnn::Trainer<tnn::bf16>::*step)(const void *, const float *, int, size_t, void *) = &tnn::Trainer<tnn::bf16>::training_step;
    void (*loss)(void *, float, const void *, const float *, int, float *, void *, size_t, int, float *) = &tnn::Loss<tnn::half>::evaluate;
    tnn::Optimizer opt;
    return (inf && step && loss && opt.lr > 0 && sizeof(tnn::DataParallel) && sizeof(tnn::EncodingModule)) ? 0 : 5;
}
"""


def test_cpp_layer_compiles_links_and_throws(tnn_lib, tmp_path):
    pkg = os.path.join(ROOT, "tiny-dpcpp-nn_b200")
    src = tmp_path / "main.cpp"
    src.write_text(SRC)
    exe = tmp_path / "main"
    subprocess.run(["g++", "-std=c++17", "-I", os.path.join(pkg, "cpp"), str(src), "-o", str(exe), "-L", pkg,
                    "-ltnn_b200", f"-Wl,-rpath,{pkg}"], check=True)
    r = subprocess.run([str(exe)], capture_output=True, text=True)
    assert r.returncode == 0, (r.returncode, r.stdout, r.stderr)
    assert "tnn_b200" in r.stdout
