"""A training step through the header-only C++ layer (tiny-dpcpp-nn_b200/cpp/tnn_api.h): a stand-alone C++ program
(g++, cudart for memory only) builds a Network, an Identity Encoding and a Trainer with the reference's class names,
runs training steps on the image-regression shapes and prints the losses; the same steps through the Python front
end must give the same numbers (both are thin layers over the same C ABI)."""
import os
import subprocess

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SRC = r"""
#include <cstdio>
#include <cuda_runtime.h>
#include <vector>
#include "tnn_api.h"
int main() {
    const size_t batch = 128 * 20 + 8;
    tnn::Network<tnn::bf16> net(64, 3, 4, tnn::Activation::ReLU, tnn::Activation::None, 64, true, /*seed*/ 11);
    tnn::Encoding enc("{\"otype\": \"Identity\", \"n_dims_to_encode\": 2, \"scale\": 1.0, \"offset\": 0.0}", 64);
    tnn::Trainer<tnn::bf16> trainer(net, &enc, tnn::Optimizer{1e-2f, 0.9f, 0.99f, 1e-15f});
    std::vector<float> q(batch * 2), t(batch * 3);
    for (size_t i = 0; i < batch; ++i) {
        q[2 * i] = (float)((i * 37) % 1000) / 1000.0f;
        q[2 * i + 1] = (float)((i * 91) % 1000) / 1000.0f;
        for (int c = 0; c < 3; ++c) t[3 * i + c] = q[2 * i] * (c + 1) - q[2 * i + 1];
    }
    float *dq, *dt;
    cudaMalloc(&dq, q.size() * 4);
    cudaMalloc(&dt, t.size() * 4);
    cudaMemcpy(dq, q.data(), q.size() * 4, cudaMemcpyHostToDevice);
    cudaMemcpy(dt, t.data(), t.size() * 4, cudaMemcpyHostToDevice);
    for (int s = 0; s < 20; ++s) {
        trainer.training_step(dq, dt, 3, batch, nullptr);
        float loss = 0;
        cudaMemcpy(&loss, trainer.loss(), 4, cudaMemcpyDeviceToHost);
        std::printf("%.9g\n", loss);
    }
    if (net.sync_status(nullptr) != 0 || trainer.step_count() != 20) return 1;
    return 0;
}
"""


def test_training_through_the_cpp_layer_matches_the_python_front_end(tnn_lib, tmp_path):
    from tiny_dpcpp_nn.trainer import Trainer

    pkg = os.path.join(ROOT, "tiny-dpcpp-nn_b200")
    src = tmp_path / "train.cpp"
    src.write_text(SRC)
    exe = tmp_path / "train"
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    subprocess.run(["g++", "-std=c++17", "-I", os.path.join(pkg, "cpp"), "-I", os.path.join(cuda, "include"), str(src),
                    "-o", str(exe), "-L", pkg, "-ltnn_b200", "-L", os.path.join(cuda, "lib64"), "-lcudart",
                    f"-Wl,-rpath,{pkg}", f"-Wl,-rpath,{os.path.join(cuda, 'lib64')}"], check=True)
    r = subprocess.run([str(exe)], capture_output=True, text=True)
    assert r.returncode == 0, (r.returncode, r.stdout[-500:], r.stderr[-500:])
    cpp_losses = np.array([float(x) for x in r.stdout.split()])
    assert len(cpp_losses) == 20 and cpp_losses[-1] < 0.8 * cpp_losses[0]

    batch = 128 * 20 + 8
    i = np.arange(batch)
    q = np.stack([((i * 37) % 1000) / 1000.0, ((i * 91) % 1000) / 1000.0], 1).astype(np.float32)
    t = np.stack([q[:, 0] * (c + 1) - q[:, 1] for c in range(3)], 1).astype(np.float32)
    net = tnn_lib.create_network(64, 3, 4, 0, 8, 64, "torch.bfloat16", True, seed=11)
    enc = tnn_lib.create_encoding("Identity", dict(n_dims_to_encode=2, scale=1.0, offset=0.0), 64)
    tr = Trainer(net, lr=1e-2, encoding=enc)
    qt, tt = torch.from_numpy(q).cuda(), torch.from_numpy(t).cuda()
    py_losses = np.array([tr.training_step(qt, tt).item() for _ in range(20)])
    assert np.allclose(cpp_losses, py_losses, rtol=1e-6), (cpp_losses[:3], py_losses[:3])
