"""Headline benchmark: samples/s of one SwiftNet training step (and of inference) at width 64,
4 hidden layers, batch 2^22 per GPU, synthetic inputs.

  python bench.py --gpus N --steps K --warmup W            # this library on N GPUs (N > 1: under torchrun)
  python bench.py --impl reference --steps K --warmup W    # the reference's CPU path on the host cores

A step = one fused kernel (forward -> L2 loss -> backward -> weight-gradient reduction, activations never
leave the SM) -> (N > 1: one NCCL all-reduce of the fp32 gradient buffer) -> Adam + weight refresh.
`--only train|infer|grid` runs just that kernel a few times and prints a short line: the small, single-kernel
command the profiler captures are taken from (with `--log2-batch` below the headline size).
Prints ONE JSON line.  `value` = whole-job training samples/s with inputs resident in HBM; `e2e` =
the same through the public API from pinned HOST buffers (H2D of inputs and targets, D2H of the
loss inside the timed region).  Extra keys: `infer` (inference throughput), `roofline` (dominant
kernel of the step), `rooflines` (each kernel), `cpu_baseline`, `clocks`, `gpu_launches`.
"""
import argparse
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
N_MAT = N_HIDDEN + 1
METRIC = "train_samples_per_s"
UNIT = "samples/s"
# algorithmic work per sample (benchmarks/common_benchmarks.h:87-88, 120-121 of the reference)
FLOPS_FWD = 2 * WIDTH * WIDTH * N_MAT            # 40 960
FLOPS_BWD = 2 * FLOPS_FWD - 2 * WIDTH * WIDTH    # delta chain over L matrices + L+1 weight gradients
FLOPS_TRAIN = 3 * FLOPS_FWD                      # 122 880 (the reference's 3x model)
BYTES_INFER = 2 * WIDTH * 2                      # x in + y out, bf16
# DRAM bytes (read + write) per sample of the fused training kernel from a profiler capture at batch 2^19
# (the traffic is proportional to the batch: inputs and targets are read once, nothing else is streamed)
TRAIN_DRAM_BYTES_PER_SAMPLE = 391.0
TRAIN_DRAM_SOURCE = "ncu dram__bytes_read.sum + dram__bytes_write.sum at batch 2^19, scaled by the batch"


def workload_name(batch_log2):
    return (f"swiftnet_train_step_w{WIDTH}_l{N_HIDDEN}_relu_none_bf16_batch2^{batch_log2}_per_gpu "
            "(L2 loss, Adam lr 1e-3 b 0.9/0.99 eps 1e-15; inputs/targets uniform[-1,1])")


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


# --------------------------------------------------------------------------------- CPU reference arm
def _cpu_train_rate(n_samples, threads, seed=0):
    """samples/s of forward + backward of the reference's own host MLP (test/mlp.h through oracle/_ref)
    or, where that library is absent, of the oracle port, on `threads` host threads."""
    from oracle import oracle as O  # the CPU legs are the one place bench.py runs the oracle

    w = xavier_weights(N_MAT, WIDTH, 0).astype(np.float64)
    rng = np.random.default_rng(100 + seed)
    x = rng.uniform(-1, 1, (n_samples, WIDTH))
    t = rng.uniform(-1, 1, (n_samples, WIDTH))
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
        "config": {"workload": workload_name(LOG2_BATCH), "l2_flush": "n/a (CPU)"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# --------------------------------------------------------------------------------- single-kernel runs
GRID_CFG = dict(otype="HashGrid", n_dims_to_encode=3, n_levels=16, n_features_per_level=2, log2_hashmap_size=19,
                base_resolution=16, per_level_scale=2.0)


def grid_leg(L, torch, batch, steps, timed):
    """Forward and parameter-gradient backward of the 16-level hash grid (3-D inputs, 2 features per level)."""
    enc = L.create_encoding("HashGrid", GRID_CFG, 32, seed=3)
    gen = torch.Generator(device="cuda").manual_seed(7)
    pos = torch.rand((batch, 3), device="cuda", generator=gen)
    dy = torch.rand((batch, 32), device="cuda", generator=gen) - 0.5
    res = {}
    fwd = lambda: enc.fwd(pos)  # noqa: E731
    for name, fn in (("grid_fwd", fwd),
                     ("grid_bwd_deterministic", lambda: enc.bwd_with_encoding_grad(dy, pos, False, False, deterministic=True)),
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


def run_only(args):
    """One kernel, few launches: what a profiler capture is taken from."""
    import torch

    from tiny_dpcpp_nn import _lib as L
    from tiny_dpcpp_nn.trainer import Trainer

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback for the product path")
    batch = 1 << args.log2_batch

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
        out.update(grid_leg(L, torch, batch, args.steps, timed))
    elif args.only == "c4":
        # hash grid (3-D, 16 levels x 2 features, 2^19 entries per level) feeding a width-64 network with 2 hidden
        # layers and 3 outputs, through the torch.nn.Module front end: forward, and forward + backward of an L2 loss
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
        out["c4_forward_backward_ms"] = timed(fwd_bwd, args.steps) / args.steps
        out["c4_inference_samples_per_s"] = batch / out["c4_inference_ms"] * 1e3
        out["c4_training_samples_per_s"] = batch / out["c4_forward_backward_ms"] * 1e3
    elif args.only == "sweep":
        # the reference's sweep (benchmarks/benchmark_all.cpp): widths 16..128, 2 / 4 / 8 hidden layers
        peaks = load_peaks()
        rows = []
        for width in (16, 32, 64, 128):
            gen = torch.Generator(device="cuda").manual_seed(100)
            x = (torch.rand((batch, width), device="cuda", generator=gen) * 2 - 1).to(torch.bfloat16)
            targets = torch.rand((batch, width), device="cuda", generator=gen) * 2 - 1
            for n_hidden in (2, 4, 8):
                net = L.create_network(width, width, n_hidden, 0, 8, width, "torch.bfloat16", True, seed=0)
                net.set_params(torch.from_numpy(xavier_weights(n_hidden + 1, width, 0).reshape(-1)).cuda(), False)
                tr = Trainer(net)
                inf = lambda: net.inference(x)  # noqa: E731
                trn = lambda: tr.forward_backward(x, targets)  # noqa: E731
                for fn in (inf, trn):
                    for _ in range(2):
                        fn()
                ms_i = timed(inf, args.steps) / args.steps
                ms_t = timed(trn, args.steps) / args.steps
                flops = 2 * width * width * (n_hidden + 1)
                rows.append({"width": width, "n_hidden": n_hidden, "infer_ms": ms_i, "train_ms": ms_t,
                             "infer_samples_per_s": batch / ms_i * 1e3, "train_samples_per_s": batch / ms_t * 1e3,
                             "infer_tflops": flops * batch / ms_i * 1e-9, "train_tflops": 3 * flops * batch / ms_t * 1e-9,
                             "infer_frac_hbm": 4 * width * batch / ms_i * 1e-6 / peaks["hbm_gbs"],
                             "status": net.status()})
                del tr, net
            del x, targets
        out["sweep"] = rows
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
    pg = None
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        pg = dist.group.WORLD
    batch = 1 << args.log2_batch
    peaks = load_peaks()

    # synthetic data of the configuration's shapes: weights Xavier-uniform seed 0 (same on every rank),
    # inputs / targets uniform[-1, 1], per-rank seeds
    w = xavier_weights(N_MAT, WIDTH, 0)
    net = L.create_network(WIDTH, WIDTH, N_HIDDEN, 0, 8, WIDTH, "torch.bfloat16", True, seed=0)
    net.set_params(torch.from_numpy(w.reshape(-1)).cuda(), False)
    gen = torch.Generator(device="cuda").manual_seed(100 + rank)
    x = (torch.rand((batch, WIDTH), device="cuda", generator=gen) * 2 - 1).to(torch.bfloat16)
    gen.manual_seed(1 + 1000 * rank)
    targets = torch.rand((batch, WIDTH), device="cuda", generator=gen) * 2 - 1
    trainer = Trainer(net, lr=1e-3, betas=(0.9, 0.99), eps=1e-15, process_group=pg, world_size=world)
    trainer.set_master_params(torch.from_numpy(_packed(w)).cuda())

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

    # -------- training step, inputs resident in HBM (every step streams 1.5 GiB of inputs and targets, far
    # more than the 126 MB L2, so no explicit flush is needed)
    step = lambda: trainer.training_step(x, targets)  # noqa: E731
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()  # nvidia-smi needs a moment to start: it runs from before the warm-up on
    t_load = time.perf_counter()
    for _ in range(max(args.warmup, 3)):
        step()
    ms_total = timed(step, args.steps)
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

    # -------- inference at the same batch
    infer = lambda: net.inference(x)  # noqa: E731
    for _ in range(3):
        infer()
    ms_inf = timed(infer, args.steps) / args.steps
    infer_value = world * batch / (ms_inf * 1e-3)

    # -------- per-kernel durations (CUDA events around one call at a time, same stream)
    lib = L.load()
    s = L.stream_ptr()
    tr = trainer
    interm = torch.empty((N_MAT + 1, batch, WIDTH), dtype=torch.bfloat16, device="cuda")
    dy = torch.empty((batch, WIDTH), dtype=torch.bfloat16, device="cuda")

    def k_train():  # the fused kernel (+ two tiny reductions: loss partials, gradient slabs)
        L.check(lib.tnn_network_train_step(net._h, L.dptr(x), L.dptr(targets), WIDTH, batch, 1.0, L.dptr(tr.grads),
                                           L.DTYPE_FP32, 1, L.dptr(tr._loss), s))

    def k_fwd():
        L.check(lib.tnn_network_forward(net._h, L.dptr(x), None, L.dptr(interm), batch, s))

    def k_bwd():
        L.check(lib.tnn_network_backward(net._h, L.dptr(dy), L.dptr(interm), L.dptr(tr.grads), L.DTYPE_FP32, 1, None,
                                         None, batch, s))

    def k_loss():
        L.check(lib.tnn_l2_loss(L.dptr(interm[N_MAT]), L.dptr(targets), WIDTH, None, L.dptr(dy), batch, WIDTH, 1.0,
                                L.dptr(tr._loss), s))

    kernel_ms = {}
    for name, fn in (("mlp_train_fused", k_train), ("mlp_inference", infer), ("mlp_fwd_store", k_fwd),
                     ("l2_loss", k_loss), ("mlp_bwd", k_bwd)):
        for _ in range(2):
            fn()
        kernel_ms[name] = timed(fn, args.steps) / args.steps

    def roof(name, flops_per_sample, bytes_per_sample, note):
        t = kernel_ms[name] * 1e-3
        tf = flops_per_sample * batch / t * 1e-12
        gb = bytes_per_sample * batch / t * 1e-9
        return {"kernel": name, "ms": kernel_ms[name], "tflops": tf, "frac_tensor": tf / peaks["tflops"], "gbs": gb,
                "frac_hbm": gb / peaks["hbm_gbs"], "note": note}

    act_bytes = WIDTH * 2
    rooflines = [
        roof("mlp_train_fused", FLOPS_TRAIN, act_bytes + WIDTH * 4, "the step's kernel: x in, targets in"),
        roof("mlp_inference", FLOPS_FWD, BYTES_INFER, "x in, y out"),
        roof("mlp_fwd_store", FLOPS_FWD, act_bytes * (N_MAT + 2), "unfused path: x in, input copy + every activation out"),
        roof("mlp_bwd", FLOPS_BWD, act_bytes * (N_MAT + 1), "unfused path: dy + a_L..a_0 in"),
        roof("l2_loss", 0, act_bytes * 2 + WIDTH * 4, "unfused path: y in, dy out, targets in"),
    ]
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

    grid_batch = 1 << 20
    grid_ms = grid_leg(L, torch, grid_batch, max(3, min(args.steps, 10)), timed_local) if rank == 0 else {}
    # per sample and level: 8 corners x 2 features (4 B each) read, position read once, 2 features written
    grid_fwd_bytes = 16 * (8 * 2 * 4) + 3 * 4 + 32 * 4
    grid_adam_gbs = grid_ms.pop("grid_adam_gbs", None)
    grid_adam_ms = grid_ms.pop("grid_adam", None)
    grid_rooflines = [{"kernel": k, "ms": v, "batch": grid_batch,
                       "gbs": grid_fwd_bytes * grid_batch / (v * 1e-3) * 1e-9,
                       "frac_hbm": grid_fwd_bytes * grid_batch / (v * 1e-3) * 1e-9 / peaks["hbm_gbs"],
                       "note": "16 levels x 8 corners x 2 fp32 features gathered (or scattered) per sample; "
                               "the fine levels' tables exceed L2"} for k, v in grid_ms.items()]
    if grid_adam_ms is not None:
        grid_rooflines.append({"kernel": "adam_kernel (grid table, 14.2 M parameters)", "ms": grid_adam_ms,
                               "gbs": grid_adam_gbs, "frac_hbm": grid_adam_gbs / peaks["hbm_gbs"],
                               "note": "28 bytes per parameter and step: parameter, two moments read and written, gradient read"})
    dom_r = rooflines[0]
    roofline = {"bound": "tensor", "kernel": "mlp_train_pipe_kernel", "achieved": dom_r["tflops"], "peak": peaks["tflops"],
                "unit": "TFLOP/s", "frac": dom_r["frac_tensor"],
                "traffic": TRAIN_DRAM_BYTES_PER_SAMPLE * batch, "traffic_source": TRAIN_DRAM_SOURCE,
                "peak_source": peaks["source"],
                "frac_of_sustained_peak": dom_r["tflops"] / peaks["tflops_sustained"],
                "hbm_frac_same_kernel": dom_r["frac_hbm"]}
    del interm, dy

    # -------- end to end through the public API with HOST buffers
    hx = torch.empty((batch, WIDTH), dtype=torch.bfloat16).pin_memory()
    ht = torch.empty((batch, WIDTH), dtype=torch.float32).pin_memory()
    hx.copy_(x.cpu()); ht.copy_(targets.cpu())
    dx_, dt_ = torch.empty_like(x), torch.empty_like(targets)

    def e2e_step():
        dx_.copy_(hx, non_blocking=True)
        dt_.copy_(ht, non_blocking=True)
        loss = trainer.training_step(dx_, dt_)
        return float(loss.item())  # device -> host read of the step's result

    e2e_steps = max(2, min(args.steps, 5))
    for _ in range(2):
        e2e_step()
    sync_all()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
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
                       "l2_flush": "inputs larger than L2 (1.5 GiB streamed per step)"},
            "train_tflops": FLOPS_TRAIN * value * 1e-12, "train_frac_of_bf16_peak": FLOPS_TRAIN * value * 1e-12 / world / peaks["tflops"],
            "infer": {"value": infer_value, "unit": UNIT, "ms": ms_inf, "tflops": FLOPS_FWD * infer_value * 1e-12,
                      "frac_of_bf16_peak": FLOPS_FWD * infer_value * 1e-12 / world / peaks["tflops"],
                      "hbm_gbs": BYTES_INFER * infer_value * 1e-9 / world,
                      "frac_of_hbm_peak": BYTES_INFER * infer_value * 1e-9 / world / peaks["hbm_gbs"]},
            "roofline": roofline, "rooflines": rooflines, "grid_rooflines": grid_rooflines,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": batch * WIDTH * (2 + 4),
                    "d2h_bytes_per_step": 4, "steps": e2e_steps},
            "gpu_launches": 5 * args.steps,
            "kernels_per_step": ["mlp_train_pipe_kernel", "sum_partials_kernel", "reduce_dw_kernel", "adam_kernel",
                                 "set_params_kernel"] + (["ncclAllReduce (80 KiB)"] if world > 1 else []),
            "clocks": clocks, "kernel_status": status, "final_loss_sum": loss_value,
        }
        if cpu is not None:
            out["cpu_baseline"] = cpu
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


def xavier_weights(n_mat, width, seed):
    """n_mat matrices (in x out), uniform(+-sqrt(6 / (2 width))), numpy PCG64 - same draw as tests/synth.py."""
    rng = np.random.default_rng(seed)
    bound = np.sqrt(6.0 / (2 * width))
    return rng.uniform(-bound, bound, (n_mat, width, width)).astype(np.float32)


def _packed(w):
    """(in x out) matrices -> the packed parameter order the optimiser sees."""
    from tiny_dpcpp_nn.modules import to_packed_layout_coord

    idx = np.array([to_packed_layout_coord(i, WIDTH, WIDTH) for i in range(WIDTH * WIDTH)])
    flat = w.reshape(N_MAT, -1)
    out = np.empty_like(flat)
    out[:, idx] = flat
    return out.reshape(-1)


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
    ap.add_argument("--only", choices=["train", "infer", "grid", "sweep", "c4"],
                    help="run one kernel only (profiler captures), the width / depth sweep, or the grid -> MLP model")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.only:
        run_only(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
