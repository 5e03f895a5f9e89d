"""Headline benchmark: samples/s of one SwiftNet training step (and of inference) at width 64,
4 hidden layers, batch 2^22 per GPU, on the 2-D image-regression workload: fp32 coordinates in [0, 1]^2 ->
identity encoding padded to 64 -> 4 x 64 ReLU network -> 3 outputs, targets = nearest-texel lookup of a seeded
2048 x 2048 x 3 image (sum of 16 random sinusoids), L2 loss, Adam; data parallel over N GPUs.

  python bench.py --gpus N --steps K --warmup W            # this library on N GPUs (N > 1: under torchrun)
  python bench.py --impl reference --steps K --warmup W    # the reference's CPU path on the host cores

A step = ONE fused kernel (identity encoding folded into the first-layer load -> forward -> L2 loss -> backward ->
weight-gradient reduction; activations never leave the SM) + ONE kernel that finishes the gradient sums, applies
Adam to the fp32 master weights and refreshes the bf16 weights (N > 1: slab reduction, one NCCL all-reduce of the
80 KiB gradient buffer, Adam kernel).
`--only train|infer|c5|grid|sweep|c4` runs just that part and prints a short line: the small, single-kernel
commands the profiler captures are taken from (with `--log2-batch` below the headline size).
Prints ONE JSON line.  `value` = whole-job training samples/s with inputs resident in HBM; `e2e` = the same
through the public API from pinned HOST buffers (H2D of coordinates and targets, D2H of the loss inside the timed
region).  Extra keys: `roofline` (dominant kernel of the step), `rooflines` (each kernel), `swiftnet_64x64` (the
same network fed 64 bf16 inputs and 64 fp32 targets per sample), `sweep`, `cpu_baseline`, `clocks`, `gpu_launches`,
`infer` (inference throughput, last).
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "tiny-dpcpp-nn_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import numpy as np  # noqa: E402

WIDTH, N_HIDDEN, LOG2_BATCH = 64, 4, 22
N_IN, N_OUT = 2, 3
IMAGE_RES, IMAGE_WAVES, IMAGE_FMAX = 2048, 16, 32.0
N_MAT = N_HIDDEN + 1
METRIC = "train_samples_per_s"
UNIT = "samples/s"
# algorithmic work per sample (benchmarks/common_benchmarks.h:87-88, 120-121 of the reference: padded widths count)
FLOPS_FWD = 2 * WIDTH * WIDTH * N_MAT            # 40 960
FLOPS_BWD = 2 * FLOPS_FWD - 2 * WIDTH * WIDTH    # delta chain over L matrices + L+1 weight gradients
FLOPS_TRAIN = 3 * FLOPS_FWD                      # 122 880 (the reference's 3x model)
BYTES_TRAIN_C5 = N_IN * 4 + N_OUT * 4            # coordinates + targets, fp32
BYTES_INFER_C5 = N_IN * 4 + WIDTH * 2            # coordinates in, padded bf16 output row out
BYTES_INFER_64 = 2 * WIDTH * 2                   # x in + y out, bf16
BYTES_TRAIN_64 = WIDTH * 2 + WIDTH * 4           # x bf16 + targets fp32
# DRAM bytes (read + write) per sample of the fused training kernel from profiler captures at batch 2^19
# (the traffic is proportional to the batch: inputs and targets are read once, nothing else is streamed)
TRAIN_DRAM_BYTES_PER_SAMPLE = {"c5": 20.26, "64x64": 391.0}
TRAIN_DRAM_SOURCE = "ncu dram__bytes_read.sum + dram__bytes_write.sum at batch 2^19, scaled by the batch"
N_ROTATE = 4  # distinct input batches used in turn: 4 x 84 MB > 126 MB of L2, so no step finds its inputs cached


def workload_name(batch_log2):
    return (f"image_regression_2d_identity_pad{WIDTH}_swiftnet_w{WIDTH}_l{N_HIDDEN}_relu_none_out{N_OUT}_bf16_"
            f"batch2^{batch_log2}_per_gpu (train step: L2 loss, Adam lr 1e-3 b 0.9/0.99 eps 1e-15; coords uniform[0,1]^2, "
            f"targets = nearest texel of a seeded {IMAGE_RES}^2 image of {IMAGE_WAVES} sinusoids)")


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm_gbs=p["hbm_gbs"], tflops=p["bf16_tflops"], tflops_sustained=p["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm_gbs=6650.0, tflops=1590.0, tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.gpu)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, power, reasons = [], [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); smax.append(float(f[2])); power.append(float(f[3]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        busy = [s for s, p in zip(sm, power) if p >= 0.5 * max(power)] or sm
        return {"sm_mhz": float(np.median(busy)), "sm_max_mhz": max(smax), "power_w_max": max(power),
                "samples": len(sm), "reasons": sorted(reasons)}


# --------------------------------------------------------------------------------- synthetic workload
def xavier_weights(n_mat, width, seed):
    """n_mat matrices (in x out), uniform(+-sqrt(6 / (2 width))), numpy PCG64 - same draw as tests/synth.py."""
    rng = np.random.default_rng(seed)
    bound = np.sqrt(6.0 / (2 * width))
    return rng.uniform(-bound, bound, (n_mat, width, width)).astype(np.float32)


def c5_weights():
    """Xavier-uniform weights (seed 6, identical on every rank); output columns beyond the 3 real outputs are zero,
    as Network::set_weights_matrices leaves them (Network.h:171-233)."""
    w = xavier_weights(N_MAT, WIDTH, 6)
    w[-1][:, N_OUT:] = 0.0
    return w


def image_waves(seed=7):
    """Parameters of the target image I_c(u, v) = sum_k a_kc sin(2 pi f_k . (u, v) + phi_k), k < 16, f ~ U[1, 32]^2."""
    rng = np.random.default_rng(seed)
    f = rng.uniform(1.0, IMAGE_FMAX, (IMAGE_WAVES, N_IN))
    phi = rng.uniform(0.0, 2 * np.pi, IMAGE_WAVES)
    a = rng.uniform(-1.0, 1.0, (IMAGE_WAVES, N_OUT)) / IMAGE_WAVES
    return f, phi, a


def nearest_texel_targets_np(q, res=IMAGE_RES):
    """Targets of the coordinates q (n x 2, in [0, 1)): the image value at the centre of the texel q falls into."""
    f, phi, a = image_waves()
    ij = np.minimum((q.astype(np.float64) * res).astype(np.int64), res - 1)
    uv = (ij + 0.5) / res
    return (np.sin(2 * np.pi * uv @ f.T + phi) @ a).astype(np.float32)


def _packed(w):
    """(in x out) matrices -> the packed parameter order the optimiser sees."""
    from tiny_dpcpp_nn.modules import to_packed_layout_coord

    idx = np.array([to_packed_layout_coord(i, WIDTH, WIDTH) for i in range(WIDTH * WIDTH)])
    flat = w.reshape(w.shape[0], -1)
    out = np.empty_like(flat)
    out[:, idx] = flat
    return out.reshape(-1)


# --------------------------------------------------------------------------------- CPU reference arm
def _cpu_train_rate(n_samples, threads, seed=0):
    """samples/s of forward + backward of the reference's own host MLP (test/mlp.h through oracle/_ref)
    or, where that library is absent, of the oracle port, on `threads` host threads, on the same workload:
    identity-encoded coordinates (2 values, then ones) into the 4 x 64 network, 3 targets (the rest zero)."""
    from oracle import oracle as O  # the CPU legs are the one place bench.py runs the oracle

    w = c5_weights().astype(np.float64)
    rng = np.random.default_rng(100 + seed)
    q = rng.uniform(0, 1, (n_samples, N_IN))
    x = np.ones((n_samples, WIDTH))
    x[:, :N_IN] = q
    t = np.zeros((n_samples, WIDTH))
    t[:, :N_OUT] = nearest_texel_targets_np(q)
    if O.ref_lib() is not None:
        kind = "reference"
        chunks = np.array_split(np.arange(n_samples), threads)
        t0 = time.perf_counter()
        ths = [threading.Thread(target=O.ref_mlp_run_batch,
                                args=(WIDTH, N_MAT, "relu", "none", w, x[c], t[c], True)) for c in chunks if len(c)]
        [th.start() for th in ths]
        [th.join() for th in ths]
        dt = time.perf_counter() - t0
    else:
        kind = "port"
        t0 = time.perf_counter()
        interm = O.mlp_forward(x, w, N_MAT, WIDTH, "relu", "none", bf16=True, n_threads=threads)
        dy = (2 * (interm[-1] - t) / (n_samples * WIDTH)).astype(np.float32)
        O.mlp_backward(dy, interm, w, N_MAT, WIDTH, "relu", "none", bf16=True, want_dx=False, n_threads=threads)
        dt = time.perf_counter() - t0
    return n_samples / dt, kind


def cpu_baseline(target_seconds=12.0):
    threads = os.cpu_count() or 1
    rate, kind = _cpu_train_rate(256 * threads, threads)          # calibration
    n = int(max(256 * threads, min(rate * target_seconds, 1 << 22)))
    rate, kind = _cpu_train_rate(n, threads, seed=1)
    return {"value": rate, "unit": UNIT, "cores": threads, "kind": kind,
            "sample": f"{n} samples of the same training step (forward + L2 + backward, weights fixed) through "
                      + ("the reference's test/mlp.h, double precision" if kind == "reference" else "the oracle port")}


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    rate0, kind = _cpu_train_rate(128 * threads, threads)
    per_step = int(max(128 * threads, min(rate0 * 4.0, 1 << 20)))   # about 4 s of CPU work per step
    for i in range(args.warmup):
        _cpu_train_rate(max(per_step // 8, threads), threads, seed=10 + i)
    t0 = time.perf_counter()
    for i in range(args.steps):
        _cpu_train_rate(per_step, threads, seed=20 + i)
    dt = time.perf_counter() - t0
    value = per_step * args.steps / dt
    sample = f"{per_step} samples per step of the batch-2^{LOG2_BATCH} step, {threads} host threads"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f64" if kind == "reference" else "bf16", "data": "synthetic",
        "config": {"workload": workload_name(LOG2_BATCH), "global_batch": args.gpus << LOG2_BATCH,
                   "parallelism": f"dp{args.gpus}" if args.gpus > 1 else "single", "l2_flush": "n/a (CPU)"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# --------------------------------------------------------------------------------- GPU helpers
GRID_CFG = dict(otype="HashGrid", n_dims_to_encode=3, n_levels=16, n_features_per_level=2, log2_hashmap_size=19,
                base_resolution=16, per_level_scale=2.0)
IDENTITY_CFG = dict(otype="Identity", n_dims_to_encode=N_IN, scale=1.0, offset=0.0)


def launch_count(L):
    return int(L.load().tnn_launch_count())


def make_c5(L, torch, batch, rank, n_batches):
    """Network, encoding and `n_batches` distinct (coords, targets) batches of the image-regression workload."""
    net = L.create_network(WIDTH, N_OUT, N_HIDDEN, 0, 8, WIDTH, "torch.bfloat16", True, seed=0)
    enc = L.create_encoding("Identity", IDENTITY_CFG, WIDTH)
    f, phi, a = image_waves()
    ft, phit, at = (torch.from_numpy(v.astype(np.float32)).cuda() for v in (f, phi, a))
    # the target image, held on the device: value at the texel centres
    axis = (torch.arange(IMAGE_RES, device="cuda", dtype=torch.float32) + 0.5) / IMAGE_RES
    image = torch.empty((IMAGE_RES, IMAGE_RES, N_OUT), device="cuda")
    for i0 in range(0, IMAGE_RES, 256):  # in slabs: the phase tensor of the whole image would be 1 GiB
        u = axis[i0:i0 + 256, None, None] * ft[None, None, :, 0]
        v = axis[None, :, None] * ft[None, None, :, 1]
        image[i0:i0 + 256] = (torch.sin(2 * np.pi * (u + v) + phit)[..., None] * at).sum(-2)
    batches = []
    gen = torch.Generator(device="cuda").manual_seed(100 + rank)
    for _ in range(n_batches):
        q = torch.rand((batch, N_IN), device="cuda", generator=gen)
        ij = (q * IMAGE_RES).long().clamp_(max=IMAGE_RES - 1)
        t = image[ij[:, 0], ij[:, 1]].contiguous()
        batches.append((q, t))
    del image
    return net, enc, batches


def grid_leg(L, torch, batch, steps, timed, n_levels=16, base_resolution=16):
    """Forward and parameter-gradient backward of the hash grid (3-D inputs, 2 features per level; 16 levels from
    resolution 16 unless told otherwise: `--grid-levels 13 --grid-base-resolution 128` are the hashed levels of the
    same grid alone, `--grid-levels 1` its coarsest level alone)."""
    cfg = dict(GRID_CFG, n_levels=n_levels, base_resolution=base_resolution)
    enc = L.create_encoding("HashGrid", cfg, 2 * n_levels, seed=3)
    gen = torch.Generator(device="cuda").manual_seed(7)
    pos = torch.rand((batch, 3), device="cuda", generator=gen)
    dy = torch.rand((batch, 2 * n_levels), device="cuda", generator=gen) - 0.5
    res = {}
    fwd = lambda: enc.fwd(pos)  # noqa: E731
    for name, fn in (("grid_fwd", fwd),
                     ("grid_bwd_deterministic", lambda: enc.bwd_with_encoding_grad(dy, pos, False, False, deterministic=True)),
                     ("grid_bwd_segmented_atomic_free", lambda: enc.bwd_with_encoding_grad(dy, pos, False, False, deterministic=2)),
                     ("grid_bwd_atomic", lambda: enc.bwd_with_encoding_grad(dy, pos, False, False, deterministic=False))):
        for _ in range(2):
            fn()
        res[name] = timed(fn, steps) / steps
    # Adam over the whole table (fp32 parameters, two moments, gradient: 28 bytes per parameter and step)
    n = enc.n_params()
    table = torch.zeros(n, device="cuda")
    m, v = torch.zeros_like(table), torch.zeros_like(table)
    g = torch.rand(n, device="cuda", generator=gen) - 0.5
    adam = lambda: L.adam_step(table, m, v, g, 1)  # noqa: E731
    for _ in range(2):
        adam()
    res["grid_adam"] = timed(adam, steps) / steps
    res["grid_adam_gbs"] = 28.0 * n / (res["grid_adam"] * 1e-3) * 1e-9
    return res


def grid_rooflines(grid_ms, grid_batch, peaks):
    """Algorithmic bytes per sample of the 3-D, 16-level, 2-feature grid: forward 12 (position) + 128 (32 fp32
    features written) + 16 x 8 x 8 gathered = 1 164; backward 12 + 128 (dL/dy read) + 2 x 1 024 (read-modify-write of
    the gathered entries) = 2 188."""
    fwd_bytes = 3 * 4 + 32 * 4 + 16 * 8 * 2 * 4
    bwd_bytes = 3 * 4 + 32 * 4 + 2 * 16 * 8 * 2 * 4
    adam_gbs = grid_ms.pop("grid_adam_gbs", None)
    adam_ms = grid_ms.pop("grid_adam", None)
    out = []
    for k, v in grid_ms.items():
        b = fwd_bytes if k == "grid_fwd" else bwd_bytes
        gbs = b * grid_batch / (v * 1e-3) * 1e-9
        out.append({"kernel": k, "ms": v, "batch": grid_batch, "bytes_per_sample": b, "gbs": gbs,
                    "frac_hbm": gbs / peaks["hbm_gbs"]})
    if adam_ms is not None:
        out.append({"kernel": "adam_vec4_kernel (grid table, 14.2 M parameters)", "ms": adam_ms, "gbs": adam_gbs,
                    "frac_hbm": adam_gbs / peaks["hbm_gbs"], "bytes_per_parameter": 28})
    return out


def sweep_rows(L, torch, Trainer, batch, steps, timed, peaks, widths=(16, 32, 64, 128), layers=(2, 4, 8)):
    """The reference's sweep (benchmarks/benchmark_all.cpp:53-104): widths 16..128, 2 / 4 / 8 hidden layers."""
    rows = []
    for width in widths:
        gen = torch.Generator(device="cuda").manual_seed(100)
        x = (torch.rand((batch, width), device="cuda", generator=gen) * 2 - 1).to(torch.bfloat16)
        targets = torch.rand((batch, width), device="cuda", generator=gen) * 2 - 1
        for n_hidden in layers:
            net = L.create_network(width, width, n_hidden, 0, 8, width, "torch.bfloat16", True, seed=0)
            net.set_params(torch.from_numpy(xavier_weights(n_hidden + 1, width, 2).reshape(-1)).cuda(), False)
            tr = Trainer(net)
            inf = lambda: net.inference(x)  # noqa: E731
            trn = lambda: tr.forward_backward(x, targets)  # noqa: E731
            for fn in (inf, trn):
                for _ in range(2):
                    fn()
            ms_i = timed(inf, steps) / steps
            ms_t = timed(trn, steps) / steps
            flops = 2 * width * width * (n_hidden + 1)
            tf_i, tf_t = flops * batch / ms_i * 1e-9, 3 * flops * batch / ms_t * 1e-9
            hbm_i = 4 * width * batch / ms_i * 1e-6 / peaks["hbm_gbs"]
            hbm_t = 6 * width * batch / ms_t * 1e-6 / peaks["hbm_gbs"]
            rows.append({"w": width, "l": n_hidden, "infer_ms": round(ms_i, 4), "train_ms": round(ms_t, 4),
                         "infer_tflops": round(tf_i, 1), "train_tflops": round(tf_t, 1),
                         # fraction of the roof that binds: the larger of the tensor and the HBM fraction
                         "infer_frac": round(max(tf_i / peaks["tflops"], hbm_i), 3),
                         "train_frac": round(max(tf_t / peaks["tflops"], hbm_t), 3), "status": net.status()})
            del tr, net
        del x, targets
    return rows


def run_only(args):
    """One kernel, few launches: what a profiler capture is taken from."""
    import torch

    from tiny_dpcpp_nn import _lib as L
    from tiny_dpcpp_nn.trainer import Trainer

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback for the product path")
    batch = 1 << args.log2_batch
    peaks = load_peaks()

    def timed(fn, steps):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)

    out = {"only": args.only, "log2_batch": args.log2_batch, "steps": args.steps}
    if args.only == "grid":
        out.update(grid_leg(L, torch, batch, args.steps, timed, args.grid_levels, args.grid_base_resolution))
    elif args.only == "c4":
        # hash grid (3-D, 16 levels x 2 features, 2^19 entries per level) feeding a width-64 network with 2 hidden
        # layers and 3 outputs: through the C ABI trainer, and through the torch.nn.Module front end
        import tiny_dpcpp_nn as tnn

        net_cfg = {"n_neurons": 64, "n_hidden_layers": 2, "activation": "relu", "output_activation": "none"}
        model = tnn.NetworkWithInputEncoding(3, 3, net_cfg, GRID_CFG, seed=3)
        gen = torch.Generator(device="cuda").manual_seed(7)
        pos = torch.rand((batch, 3), device="cuda", generator=gen)
        target = torch.rand((batch, 3), device="cuda", generator=gen)

        def fwd():
            with torch.no_grad():
                return model(pos)

        def fwd_bwd():
            model.zero_grad(set_to_none=True)
            loss = ((model(pos).float() - target) ** 2).mean()
            loss.backward()
            return loss

        model.eval()
        for _ in range(2):
            fwd()
        out["c4_inference_ms"] = timed(fwd, args.steps) / args.steps
        model.train()
        for _ in range(2):
            fwd_bwd()
        out["c4_module_forward_backward_ms"] = timed(fwd_bwd, args.steps) / args.steps
        net = L.create_network(64, 3, 2, 0, 8, 64, "torch.bfloat16", True, seed=4)
        enc = L.create_encoding("HashGrid", GRID_CFG, 64, seed=3)
        tr = Trainer(net, encoding=enc)
        step = lambda: tr.training_step(pos, target)  # noqa: E731
        for _ in range(2):
            step()
        out["c4_trainer_step_ms"] = timed(step, args.steps) / args.steps
        out["c4_inference_samples_per_s"] = batch / out["c4_inference_ms"] * 1e3
        out["c4_training_samples_per_s"] = batch / out["c4_trainer_step_ms"] * 1e3
        out["kernel_status"] = net.status()
    elif args.only == "sweep":
        out["sweep"] = sweep_rows(L, torch, Trainer, batch, args.steps, timed, peaks,
                                  widths=(args.sweep_width,) if args.sweep_width else (16, 32, 64, 128),
                                  layers=(args.sweep_layers,) if args.sweep_layers else (2, 4, 8))
    elif args.only == "c5":
        net, enc, batches = make_c5(L, torch, batch, 0, 1)
        net.set_params(torch.from_numpy(c5_weights().reshape(-1)).cuda(), False)
        q, t = batches[0]
        tr = Trainer(net, encoding=enc)
        fn = lambda: tr.forward_backward(q, t)  # noqa: E731
        for _ in range(max(args.warmup, 1)):
            fn()
        out["ms"] = timed(fn, args.steps) / args.steps
        inf = lambda: L.nwe_inference(net, enc, q)  # noqa: E731
        for _ in range(2):
            inf()
        out["infer_ms"] = timed(inf, args.steps) / args.steps
        out["kernel_status"] = net.status()
    else:
        w = xavier_weights(N_MAT, WIDTH, 0)
        net = L.create_network(WIDTH, WIDTH, N_HIDDEN, 0, 8, WIDTH, "torch.bfloat16", True, seed=0)
        net.set_params(torch.from_numpy(w.reshape(-1)).cuda(), False)
        gen = torch.Generator(device="cuda").manual_seed(100)
        x = (torch.rand((batch, WIDTH), device="cuda", generator=gen) * 2 - 1).to(torch.bfloat16)
        if args.only == "infer":
            fn = lambda: net.inference(x)  # noqa: E731
        else:
            targets = torch.rand((batch, WIDTH), device="cuda", generator=gen) * 2 - 1
            tr = Trainer(net)
            fn = lambda: tr.forward_backward(x, targets)  # noqa: E731
        for _ in range(max(args.warmup, 1)):
            fn()
        out["ms"] = timed(fn, args.steps) / args.steps
        out["kernel_status"] = net.status()
    print(json.dumps(out))


# --------------------------------------------------------------------------------- GPU arm
def run_gpu_arm(args):
    import torch
    import torch.distributed as dist

    from tiny_dpcpp_nn import _lib as L
    from tiny_dpcpp_nn.trainer import Trainer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback for the product path")
    torch.cuda.set_device(local_rank)
    # The one JSON line must be the only thing on stdout: libraries (NCCL prints its version when a communicator is
    # created) write there at C level, so stdout points at stderr until the line is printed.
    sys.stdout.flush()
    saved_stdout = os.dup(1)
    os.dup2(2, 1)
    pg = None
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        pg = dist.group.WORLD
    batch = 1 << args.log2_batch
    peaks = load_peaks()
    lib = L.load()

    # synthetic data of the configuration's shapes: weights Xavier-uniform seed 6 (same on every rank), coordinates
    # uniform[0, 1)^2 with per-rank seeds 100 + rank, targets looked up in the seeded image
    net, enc, batches = make_c5(L, torch, batch, rank, N_ROTATE)
    trainer = Trainer(net, lr=1e-3, betas=(0.9, 0.99), eps=1e-15, process_group=pg, world_size=world, encoding=enc)
    trainer.set_master_params(torch.from_numpy(_packed(c5_weights())).cuda())

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def timed(fn, steps):
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        sync_all()
        ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item()

    # -------- training step, inputs resident in HBM; the step's batch rotates over N_ROTATE distinct batches
    # (together larger than L2), so no step finds its coordinates or targets in the cache
    turn = [0]

    def step():
        q, t = batches[turn[0] % N_ROTATE]
        turn[0] += 1
        return trainer.training_step(q, t)

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()  # nvidia-smi needs a moment to start: it runs from before the warm-up on
    t_load = time.perf_counter()
    for _ in range(max(args.warmup, 3)):
        step()
    n0 = launch_count(L)
    ms_total = timed(step, args.steps)
    launches = launch_count(L) - n0
    # keep the same load on the GPU (untimed) until the sampler has seen about two seconds of it
    # (the number of extra steps is agreed between the ranks: a step holds a collective)
    remaining = torch.tensor([2.0 - (time.perf_counter() - t_load)], device="cuda")
    if world > 1:
        dist.all_reduce(remaining, op=dist.ReduceOp.MAX)
    ms_guess = max(ms_total / args.steps, 1e-3)
    for _ in range(int(min(max(remaining.item(), 0.0) * 1e3 / ms_guess, 20000))):
        step()
    torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None
    status = net.status()
    loss_value = float(trainer._loss.item())
    ms_step = ms_total / args.steps
    value = world * batch / (ms_step * 1e-3)
    # the same step with the gradient exchange as reduction kernel + ncclAllReduce + Adam kernel, for comparison
    windowed = bool(trainer.peer_window)
    dp_exchange = None
    if world > 1:
        dp_exchange = {"used": "peer_window" if windowed else "nccl_allreduce", "ms_per_step": round(ms_step, 5)}
        if windowed:
            trainer.set_peer_window(False)
            for _ in range(3):
                step()
            dp_exchange["ms_per_step_nccl_allreduce"] = round(timed(step, args.steps) / args.steps, 5)
            trainer.set_peer_window(True)
        # and with no exchange at all, per rank: what each GPU alone needs for the step (a second trainer without
        # a communicator on the same network; the data-parallel trainer's next step rewrites the weights from its
        # own master copy, so the ranks stay replicas)
        alone_tr = Trainer(net, lr=1e-3, betas=(0.9, 0.99), eps=1e-15, encoding=enc)

        def step_alone():
            q, t = batches[turn[0] % N_ROTATE]
            turn[0] += 1
            alone_tr.training_step(q, t)

        for _ in range(3):
            step_alone()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            step_alone()
        e1.record()
        torch.cuda.synchronize()
        alone = torch.tensor([e0.elapsed_time(e1) / args.steps], device="cuda")
        every = [torch.zeros_like(alone) for _ in range(world)]
        dist.all_gather(every, alone)
        dp_exchange["ms_per_step_without_exchange_by_rank"] = [round(v.item(), 5) for v in every]
        del alone_tr
        step()

    # -------- inference at the same batch: coordinates in, padded bf16 output rows out (512 MiB written per call)
    q0, t0_ = batches[0]
    y = torch.empty((batch, WIDTH), dtype=torch.bfloat16, device="cuda")
    infer = lambda: L.nwe_inference(net, enc, q0, out=y)  # noqa: E731
    for _ in range(3):
        infer()
    ms_inf = timed(infer, args.steps) / args.steps
    infer_value = world * batch / (ms_inf * 1e-3)

    # -------- per-kernel durations (CUDA events around one call at a time, same stream); the 64-in / 64-target legs
    # run the same network as a plain SwiftNet (bf16 rows in, 64 fp32 targets per row)
    s = L.stream_ptr()
    gen = torch.Generator(device="cuda").manual_seed(100 + rank)
    net64 = L.create_network(WIDTH, WIDTH, N_HIDDEN, 0, 8, WIDTH, "torch.bfloat16", True, seed=0)
    net64.set_params(torch.from_numpy(xavier_weights(N_MAT, WIDTH, 0).reshape(-1)).cuda(), False)
    x64 = (torch.rand((batch, WIDTH), device="cuda", generator=gen) * 2 - 1).to(torch.bfloat16)
    t64 = torch.rand((batch, WIDTH), device="cuda", generator=gen) * 2 - 1
    tr64 = Trainer(net64)
    interm = torch.empty((N_MAT + 1, batch, WIDTH), dtype=torch.bfloat16, device="cuda")
    dy = torch.empty((batch, WIDTH), dtype=torch.bfloat16, device="cuda")
    grads = torch.empty(net.n_params(), dtype=torch.float32, device="cuda")
    loss1 = torch.zeros(1, dtype=torch.float32, device="cuda")

    def k_train_c5():  # the fused kernel of the step (+ two tiny reductions: loss partials, gradient slabs)
        L.check(lib.tnn_network_with_encoding_train_step(net._h, enc._h, L.dptr(q0), L.dptr(t0_), N_OUT, batch, 1.0,
                                                         L.dptr(grads), L.DTYPE_FP32, 1, None, 0, L.dptr(loss1), s))

    def k_train_64():
        L.check(lib.tnn_network_train_step(net64._h, L.dptr(x64), L.dptr(t64), WIDTH, batch, 1.0, L.dptr(grads),
                                           L.DTYPE_FP32, 1, L.dptr(loss1), s))

    def k_fwd():
        L.check(lib.tnn_network_forward(net64._h, L.dptr(x64), None, L.dptr(interm), batch, s))

    def k_bwd():
        L.check(lib.tnn_network_backward(net64._h, L.dptr(dy), L.dptr(interm), L.dptr(grads), L.DTYPE_FP32, 1, None,
                                         None, batch, s))

    def k_bwd_from_input():
        L.check(lib.tnn_network_backward_from_input(net64._h, L.dptr(x64), L.dptr(dy), L.dptr(grads), L.DTYPE_FP32, 1,
                                                    None, batch, s))

    def k_loss():
        L.check(lib.tnn_l2_loss(L.dptr(interm[N_MAT]), L.dptr(t64), WIDTH, None, L.dptr(dy), batch, WIDTH, 1.0,
                                L.dptr(loss1), s))

    infer64 = lambda: net64.inference(x64)  # noqa: E731
    step64 = lambda: tr64.training_step(x64, t64)  # noqa: E731
    kernel_ms = {}
    for name, fn in (("mlp_train_fused_c5", k_train_c5), ("mlp_inference_c5", infer), ("mlp_train_fused_64x64", k_train_64),
                     ("train_step_64x64", step64), ("mlp_inference_64x64", infer64), ("mlp_fwd_store", k_fwd),
                     ("l2_loss", k_loss), ("mlp_bwd", k_bwd), ("mlp_bwd_from_input", k_bwd_from_input)):
        for _ in range(2):
            fn()
        kernel_ms[name] = timed(fn, args.steps) / args.steps

    def roof(name, flops_per_sample, bytes_per_sample, note):
        t = kernel_ms[name] * 1e-3
        tf = flops_per_sample * batch / t * 1e-12
        gb = bytes_per_sample * batch / t * 1e-9
        return {"kernel": name, "ms": round(kernel_ms[name], 5), "tflops": round(tf, 1),
                "frac_tensor": round(tf / peaks["tflops"], 4), "gbs": round(gb, 1),
                "frac_hbm": round(gb / peaks["hbm_gbs"], 4), "note": note}

    act_bytes = WIDTH * 2
    rooflines = [
        roof("mlp_train_fused_c5", FLOPS_TRAIN, BYTES_TRAIN_C5, "the step's kernel: 2 fp32 coords + 3 fp32 targets in"),
        roof("mlp_inference_c5", FLOPS_FWD, BYTES_INFER_C5, "coords in, padded bf16 y out"),
        roof("mlp_train_fused_64x64", FLOPS_TRAIN, BYTES_TRAIN_64, "x bf16 in, 64 fp32 targets in"),
        roof("mlp_inference_64x64", FLOPS_FWD, BYTES_INFER_64, "x in, y out"),
        roof("mlp_fwd_store", FLOPS_FWD, act_bytes * (N_MAT + 2), "unfused path: x in, input copy + every activation out"),
        roof("mlp_bwd", FLOPS_BWD, act_bytes * (N_MAT + 1), "unfused path: dy + a_L..a_0 in"),
        roof("mlp_bwd_from_input", FLOPS_TRAIN - 2 * WIDTH * WIDTH, act_bytes * 2,
             "backward pass of the autograd module: x and dy in, hidden activations recomputed on chip "
             "(forward without the output layer + backward flop)"),
        roof("l2_loss", 0, act_bytes * 2 + WIDTH * 4, "unfused path: y in, dy out, targets in"),
    ]
    swiftnet = {"workload": f"swiftnet_w{WIDTH}_l{N_HIDDEN}_in64_out64_batch2^{args.log2_batch}: 64 bf16 inputs, 64 fp32 targets",
                "train_step_ms": round(kernel_ms["train_step_64x64"], 5),
                "train_samples_per_s": world * batch / (kernel_ms["train_step_64x64"] * 1e-3),
                "infer_ms": round(kernel_ms["mlp_inference_64x64"], 5),
                "infer_samples_per_s": world * batch / (kernel_ms["mlp_inference_64x64"] * 1e-3),
                "infer_frac_of_hbm_peak": round(BYTES_INFER_64 * batch / (kernel_ms["mlp_inference_64x64"] * 1e-3) * 1e-9
                                                / peaks["hbm_gbs"], 4)}

    # (rank 0 only, so it is timed locally: `timed` holds collectives that every rank would have to join)
    def timed_local(fn, steps):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)

    del interm, dy, x64, t64, tr64, net64
    grid_batch = 1 << 20
    grid_roofs, sweep = [], None
    if rank == 0 and not args.brief:
        grid_ms = grid_leg(L, torch, grid_batch, max(3, min(args.steps, 10)), timed_local)
        grid_roofs = grid_rooflines(grid_ms, grid_batch, peaks)
        if world == 1:
            sweep = sweep_rows(L, torch, Trainer, batch, max(3, min(args.steps, 5)), timed_local, peaks)
    dom_r = rooflines[0]
    tps = TRAIN_DRAM_BYTES_PER_SAMPLE["c5"]
    roofline = {"bound": "tensor", "kernel": "mlp_train_pipe_kernel<64, narrow targets, bf16> (identity encoding folded in, 3 targets per sample)",
                "achieved": dom_r["tflops"], "peak": peaks["tflops"],
                "unit": "TFLOP/s", "frac": dom_r["frac_tensor"],
                "traffic": tps * batch if tps else None, "traffic_source": TRAIN_DRAM_SOURCE if tps else None,
                "peak_source": peaks["source"],
                "frac_of_sustained_peak": round(dom_r["tflops"] / peaks["tflops_sustained"], 4),
                "hbm_frac_same_kernel": dom_r["frac_hbm"]}

    # -------- end to end through the public API with HOST buffers: coordinates and targets of every step come from
    # pinned host memory (20 bytes per sample), the loss is read back every step.  The copy of the next step's batch
    # runs on a second stream while the current step computes (two device buffers), as a data loader would do.
    hq = [b[0].cpu().pin_memory() for b in batches[:2]]
    ht = [b[1].cpu().pin_memory() for b in batches[:2]]
    dq = [torch.empty_like(batches[0][0]) for _ in range(2)]
    dt_ = [torch.empty_like(batches[0][1]) for _ in range(2)]
    copy_stream = torch.cuda.Stream()
    main_stream = torch.cuda.current_stream()
    ready = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]

    def enqueue_copy(i):
        b = i & 1
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed[b])  # the step that last read this buffer is done
            dq[b].copy_(hq[b], non_blocking=True)
            dt_[b].copy_(ht[b], non_blocking=True)
            ready[b].record(copy_stream)

    def e2e_run(n):
        for b in range(2):
            consumed[b].record(main_stream)
        enqueue_copy(0)
        for i in range(n):
            b = i & 1
            if i + 1 < n:
                enqueue_copy(i + 1)
            main_stream.wait_event(ready[b])
            loss = trainer.training_step(dq[b], dt_[b])
            consumed[b].record(main_stream)
            float(loss.item())  # device -> host read of the step's result

    e2e_steps = max(4, min(args.steps, 20))
    e2e_run(3)
    sync_all()
    t0 = time.perf_counter()
    e2e_run(e2e_steps)
    sync_all()
    dt_e2e = torch.tensor([time.perf_counter() - t0], device="cuda")
    if world > 1:
        dist.all_reduce(dt_e2e, op=dist.ReduceOp.MAX)
    e2e_value = world * batch * e2e_steps / dt_e2e.item()

    cpu = cpu_baseline() if (rank == 0 and world == 1 and not args.no_cpu) else None

    if rank == 0:
        out = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": workload_name(args.log2_batch), "global_batch": world * batch,
                       "parallelism": f"dp{world}" if world > 1 else "single",
                       "l2_flush": f"{N_ROTATE} distinct input batches used in turn ({N_ROTATE * BYTES_TRAIN_C5 * batch >> 20} MiB "
                                   "of coordinates and targets, larger than the 126 MB L2)"},
            "train_tflops": FLOPS_TRAIN * value * 1e-12,
            "train_frac_of_bf16_peak": FLOPS_TRAIN * value * 1e-12 / world / peaks["tflops"],
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": batch * BYTES_TRAIN_C5,
                    "d2h_bytes_per_step": 4, "steps": e2e_steps,
                    "note": "copy of step i + 1 overlaps the compute of step i (two streams, two device buffers)"},
            "gpu_launches": launches,
            "kernels_per_step": (["mlp_train_pipe_kernel", "adam_refresh_kernel"] if world == 1 else
                                 ["mlp_train_pipe_kernel", "dp_adam_refresh_kernel (gradient exchange over peer windows inside)"]
                                 if windowed else
                                 ["mlp_train_pipe_kernel", "reduce_dw_kernel", "ncclAllReduce (80 KiB)",
                                  "adam_refresh_kernel"]),
            "roofline": roofline, "rooflines": rooflines, "swiftnet_64x64": swiftnet, "grid_rooflines": grid_roofs,
            "clocks": clocks, "kernel_status": status, "final_loss_sum": loss_value,
        }
        if dp_exchange is not None:
            out["dp_exchange"] = dp_exchange
        if sweep is not None:
            out["sweep"] = sweep
        if cpu is not None:
            out["cpu_baseline"] = cpu
        # inference last, so that it survives a reader that keeps only the end of the line
        out["infer"] = {"value": infer_value, "unit": UNIT, "n_gpus": world, "ms": round(ms_inf, 5),
                        "tflops": round(FLOPS_FWD * infer_value * 1e-12, 1),
                        "frac_of_bf16_peak": round(FLOPS_FWD * infer_value * 1e-12 / world / peaks["tflops"], 4),
                        "hbm_gbs": round(BYTES_INFER_C5 * infer_value * 1e-9 / world, 1),
                        "frac_of_hbm_peak": round(BYTES_INFER_C5 * infer_value * 1e-9 / world / peaks["hbm_gbs"], 4),
                        "scaling": "batch sharded over the GPUs, no communication"}
        sys.stdout.flush()
        os.dup2(saved_stdout, 1)
        print(json.dumps(out), flush=True)
        os.dup2(2, 1)
    if world > 1:
        dist.destroy_process_group()


def _watchdog(seconds):
    """A run that is still going after `seconds` is stuck (a rank that never joined a collective): leave loudly."""
    def fire():
        sys.stderr.write(f"bench.py: still running after {seconds} s, giving up\n")
        sys.stderr.flush()
        os._exit(3)

    t = threading.Timer(seconds, fire)
    t.daemon = True
    t.start()


def main():
    _watchdog(1200)
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--log2-batch", type=int, default=LOG2_BATCH)
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--brief", action="store_true", help="skip the hash-grid and sweep legs")
    ap.add_argument("--grid-levels", type=int, default=16, help="levels of the grid of `--only grid`")
    ap.add_argument("--sweep-width", type=int, default=0, help="`--only sweep`: this width alone (16, 32, 64, 128)")
    ap.add_argument("--sweep-layers", type=int, default=0, help="`--only sweep`: this number of hidden layers alone")
    ap.add_argument("--grid-base-resolution", type=int, default=16, help="coarsest resolution of that grid")
    ap.add_argument("--only", choices=["train", "infer", "c5", "grid", "sweep", "c4"],
                    help="run one part only: a single kernel (profiler captures), the width / depth sweep, or the "
                         "grid -> MLP model")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.only:
        run_only(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
