"""Benchmark of the int8 training step (NITI VGG-small on synthetic 32x32 data).

    python bench.py [--gpus N] [--steps K] [--warmup W]            # this library on N B200s (VGG-small-7, 128 images per GPU)
    python bench.py --config vgg9_wide --global-batch 256 ...      # VGG-small-9 (…P-512-512), fixed global batch (strong scaling)
    python bench.py --config vgg13 --global-batch 1024 --gpus 8    # VGG-13-style, global batch 1024
    python bench.py --impl reference [--gpus N] [--steps K] ...    # the reference's integer path on the host cores

One "step" = one integer training step (forward, integer loss, error back-propagation, weight
gradients, integer SGD update) over one synthetic batch.  The default line is weak scaling: every GPU
trains its own shard of 128 images; the int32 weight gradients of the ranks are summed exactly once per step.
Prints ONE JSON line (rank 0).  Fields:
  value      images/s with the batch already resident in HBM (CUDA events, max over ranks)
  e2e        images/s through Trainer.step with pinned host buffers in and the logits read back
  roofline   the tensor-core contraction kernels (conv forward / error-backward with the requantisation inside),
             each call timed alone as ten back-to-back launches replayed from a CUDA graph: algorithmic int8 ops / time
             against 2x the measured bf16 burst peak (also given against the sustained and the nominal figure)
  sustained  the same step replayed back to back for two seconds, with the clocks seen
  cpu_baseline  the reference's own Python (or, without it, the oracle port) on the host cores (rank 0, N=1)
  config.parity_vs_oracle  N > 1: a short run through the SAME exchange route, checked against oracle replicas
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CONFIGS = {
    # name: (layer list, description, default per-GPU batch (weak) or None, default global batch (strong) or None)
    "vgg7": ([128, 128, "M", 256, 256, "M", 512, 512, "M"],
             "VGG-small-7 integer training step (conv 128-128-P-256-256-P-512-512-P, FC 8192->10)", 128, None),
    "vgg9_wide": ([128, 128, "M", 256, 256, "M", 512, 512, "M", 512, 512],
                  "VGG-small-9 integer training step (conv 128-128-P-256-256-P-512-512-P-512-512, FC 8192->10)", None, 256),
    "vgg13": ([64, 64, "M", 128, 128, "M", 256, 256, "M", 512, 512, "M", 512, 512, "M"],
              "VGG-13-style integer training step (conv 64-64-P-128-128-P-256-256-P-512-512-P-512-512-P, FC 512->10)", None, 1024),
}
VGG7 = CONFIGS["vgg7"][0]
PER_GPU_BATCH = 128
UNIT = "images/s"
WORKLOAD_TAIL = ", 3x32x32 synthetic images, 10 classes, dropout on, grad bit-width 5"
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel, recorded from an ncu capture of
# that launch (the 256->256 @16x16 forward call at batch 128; algorithmic bytes 8.98e6)
NCU_TRAFFIC_BYTES = 9.04e6
NCU_TRAFFIC_OF = "fprop 256->256 @16x16, batch 128 (ncu, one launch); algorithmic 8.98e6 bytes"
NOMINAL_INT8_TOPS = 4500.0


def metric_name(config):
    return {"vgg7": "int8 VGG-small-7 training throughput", "vgg9_wide": "int8 VGG-small-9 training throughput",
            "vgg13": "int8 VGG-13 training throughput"}[config]


def workload_name(config):
    return CONFIGS[config][1] + WORKLOAD_TAIL


def plan_batches(args, world):
    """(per-GPU batch, global batch, scaling) for the chosen config and flags."""
    cfg, _, per_gpu, glob = CONFIGS[args.config]
    if args.global_batch:
        if args.global_batch % world:
            raise SystemExit("--global-batch must be a multiple of the number of GPUs")
        return args.global_batch // world, args.global_batch, "strong"
    if per_gpu is not None and args.scaling != "strong":
        return per_gpu, per_gpu * world, "weak"
    g = glob if glob is not None else per_gpu
    if g % world:
        raise SystemExit("the config's global batch is not a multiple of the number of GPUs")
    return g // world, g, "strong"


def synth_batch(rng, B):
    mean = np.array([0.49139968, 0.48215827, 0.44653124], dtype=np.float32)
    std = np.array([0.24703233, 0.24348505, 0.26158768], dtype=np.float32)
    u8 = rng.integers(0, 256, size=(B, 3, 32, 32), dtype=np.uint8)
    x = (u8.astype(np.float32) / np.float32(255.0) - mean[None, :, None, None]) / std[None, :, None, None]
    return x.astype(np.float32), rng.integers(0, 10, size=B).astype(np.int64)


def vgg_shapes(cfg):
    shapes, cin = [], 3
    for c in cfg:
        if c != "M":
            shapes.append((c, 3, 3, cin))
            cin = c
    shapes.append((10, cin * (32 // 2 ** cfg.count("M")) ** 2))
    return shapes


def xavier_exp(shape):
    if len(shape) == 4:
        K, R, S, C = shape
        fan_in, fan_out = C * R * S, K * R * S
    else:
        fan_out, fan_in = shape
    return int(np.ceil(np.log2(np.sqrt(6.0 / (fan_in + fan_out))))) - 7


def step_ops_per_image(cfg):
    """Algorithmic int8 ops (2 per MAC) of one training step per image: forward + error-backward
    (not for the first layer) + weight gradient of every convolution, and the three FC products."""
    ops, cin, hw = 0, 3, 32
    first = True
    for c in cfg:
        if c == "M":
            hw //= 2
            continue
        mac = hw * hw * c * 9 * cin
        ops += 2 * mac * (2 if first else 3)
        first = False
        cin = c
    ops += 2 * (cin * hw * hw * 10) * 3
    return ops


# ------------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    """SM clock and throttle reasons while the timed regions run: NVML polled every 5 ms from a thread (read-only
    queries); falls back to `nvidia-smi -lms` when the NVML module is missing."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    REASON_BITS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown"}

    def __init__(self, gpu_index):
        self.samples, self.proc, self.idx = [], None, gpu_index
        self.sm, self.mx, self.reasons, self._stop, self._thread = [], 0, set(), False, None

    def _nvml_loop(self, nv, handle):
        while not self._stop:
            try:
                self.sm.append(float(nv.nvmlDeviceGetClockInfo(handle, nv.NVML_CLOCK_SM)))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(handle)
                except AttributeError:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(handle)
                for bit, name in self.REASON_BITS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.005)

    def start(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            idx = self.idx
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            if vis:
                try:
                    idx = int(vis.split(",")[self.idx])
                except (ValueError, IndexError):
                    idx = self.idx
            handle = nv.nvmlDeviceGetHandleByIndex(idx)
            self.mx = float(nv.nvmlDeviceGetMaxClockInfo(handle, nv.NVML_CLOCK_SM))
            self._thread = threading.Thread(target=self._nvml_loop, args=(nv, handle), daemon=True)
            self._thread.start()
            return
        except Exception:
            self._thread = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.idx), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append(line.strip())

    def stop(self):
        self._stop = True
        if self._thread is not None:
            self._thread.join(timeout=2)
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = list(self.sm), self.mx, set(self.reasons)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            f = [t.strip() for t in s.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx = max(mx, float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        busy = [v for v in sm if v >= 0.5 * max(sm)]
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(sm),
                "source": "nvml, 5 ms period" if self._thread is not None else "nvidia-smi -lms 100"}


# ------------------------------------------------------------------------------------------------
# the reference's integer path on the host cores: its own Python when oracle/_ref holds it, else the oracle port
# ------------------------------------------------------------------------------------------------
def synth_weights(cfg, seed):
    rng = np.random.default_rng(seed)
    shapes = vgg_shapes(cfg)
    return shapes, [rng.integers(-127, 128, size=s).astype(np.int8) for s in shapes], [xavier_exp(s) for s in shapes], rng


def cpu_port_images_per_s(cfg, batch, steps, warmup, seed=1234):
    """The oracle's NumPy restatement (contractions through torch._int_mm) on all host cores."""
    import torch
    from oracle import niti_oracle as O
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    O.set_backend("int_mm")  # exact int8 x int8 -> int32 products on the CPU's VNNI/AMX units
    shapes, weights, wexps, rng = synth_weights(cfg, seed)
    net = O.Net(cfg, weights, wexps, dropout=True, mu=5, seed=seed)
    times = []
    for i in range(warmup + steps):
        x, t = synth_batch(rng, batch)
        t0 = time.perf_counter()
        x8, xe = O.float_to_int8(x)
        net.forward(np.ascontiguousarray(x8.transpose(0, 2, 3, 1)), xe, step=i)
        net.backward(t, step=i)
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
    O.set_backend("int64")
    total = sum(times)
    return batch * len(times) / total, cores, total / len(times)


def cpu_reference_images_per_s(cfg, batch, steps, warmup, seed=1234, budget_s=None):
    """The reference's own ti_torch / ti_loss / ti_net / ti_vgg (oracle/_ref, unmodified) on all host cores, its four
    CUDA extensions replaced by exact CPU stand-ins whose contractions run through torch._int_mm.  The first step's
    logits are checked against the oracle port.  Returns (images/s, cores, s per step, steps timed) or None when
    oracle/_ref is absent.  `budget_s` ends the timed loop early once that much time has been spent."""
    import torch
    from oracle import make_ref, niti_oracle as O, philox, ref_harness
    if not make_ref.available():
        return None
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    O.set_backend("int_mm")
    try:
        H = ref_harness.load()
        shapes, weights, wexps, rng = synth_weights(cfg, seed)
        port = O.Net(cfg, weights, wexps, dropout=True, mu=5, seed=seed)
        feat = shapes[-1][1]
        times = []
        with H.active(grad_bitwidth=5, training=True) as mode:
            net = H.ti_vgg.TiVGG_cifar.__new__(H.ti_vgg.TiVGG_cifar)
            H.ti_net.TiNet.__init__(net)
            net.forward_layers = H.ti_vgg.TiVGG_cifar._make_layers(net, cfg)
            wl = [l for l in net.forward_layers if hasattr(l, "weight")]
            for l, w, e in zip(wl, weights, wexps):
                l.weight, l.weight_exp = torch.from_numpy(w.copy()), torch.tensor(float(e))
            t_start = time.perf_counter()
            for i in range(warmup + steps):
                x, t = synth_batch(rng, batch)
                calls = [philox.random_u32_tensor(seed + i, 0xFFFE, (feat,)), philox.random_u32_tensor(seed + i, 0xFFFF, (batch, 10))]
                mode.rand_calls = 0
                mode.rand_provider = lambda k, size, high, calls=calls: calls[k]
                t0 = time.perf_counter()
                out, out_exp = net.forward(torch.from_numpy(x))
                net.backward(torch.from_numpy(t))
                dt = time.perf_counter() - t0
                if i == 0:
                    x8, xe = O.float_to_int8(x)
                    want, want_e = port.forward(np.ascontiguousarray(x8.transpose(0, 2, 3, 1)), xe, step=0)
                    if not (np.array_equal(out.numpy(), want) and int(out_exp) == want_e):
                        raise RuntimeError("the reference's logits differ from the oracle port's on the first step")
                if i >= warmup:
                    times.append(dt)
                    if budget_s is not None and time.perf_counter() - t_start > budget_s:
                        break
    finally:
        O.set_backend("int64")
    total = sum(times)
    return batch * len(times) / total, cores, total / len(times), len(times)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    cfg = CONFIGS[args.config][0]
    per_gpu, glob, scaling = plan_batches(args, max(world, args.gpus))
    batch = per_gpu  # one step of the arm = one GPU's share of a step, on the host cores
    warm = min(args.warmup, 1)
    r = cpu_reference_images_per_s(cfg, batch, args.steps, warm, budget_s=150.0)
    if r is not None:
        v, cores, sec, timed = r
        kind = "reference"
        what = "the reference's own ti_torch/ti_loss/ti_net/ti_vgg (unmodified, oracle/_ref), extension calls served by exact CPU stand-ins over torch._int_mm"
    else:
        v, cores, sec = cpu_port_images_per_s(cfg, batch, min(args.steps, 3), warm)
        timed, kind = min(args.steps, 3), "port"
        what = "oracle port of ti_torch/ti_loss/ti_net with torch._int_mm contractions (oracle/_ref is absent)"
    sample = (f"{timed} training steps of {args.config} on batches of {batch} synthetic images ({sec:.2f} s per step, "
              f"{warm} warm-up), {what}, {cores} threads; ONE CPU process whatever --gpus says")
    line = {"impl": "reference", "metric": metric_name(args.config), "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": scaling,
            "vs_baseline": None, "dtype": "int8", "data": "synthetic",
            "config": {"workload": workload_name(args.config), "per_gpu_batch": per_gpu, "global_batch": glob, "batch_per_step": batch,
                       "steps_timed": timed, "processes": 1},
            "cpu_baseline": {"value": v, "unit": UNIT, "cores": cores, "kind": kind, "sample": sample},
            "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# this library
# ------------------------------------------------------------------------------------------------
def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return p.get("hbm_gbs", 6650.0), p.get("bf16_tflops_sustained", 1400.0), p.get("bf16_tflops", 1590.0), "measured"
    return 6650.0, 1400.0, 1590.0, "fallback"


PARITY_CFG = [128, "M", 128, "M", 512, "M"]


def dp_parity_check(dev, rank, world, exchange, dist):
    """N > 1: two steps of a small net (global batch 8 x N, sharded) through the SAME exchange route the timed run is about
    to use, every rank's logits and final weights compared with oracle replicas whose int32 gradients are summed before
    one update.  Returns (all ranks agree with the oracle, route name)."""
    import torch
    from niti_b200 import ti_torch, ti_vgg
    from niti_b200.dp import shard_range
    from niti_b200.trainer import Trainer
    from oracle import dp_oracle
    seed, steps, glob = 31, 2, 8 * world
    rng = np.random.default_rng(seed)
    shapes = vgg_shapes(PARITY_CFG)
    weights = [rng.integers(-127, 128, size=s).astype(np.int8) for s in shapes]
    wexps = [xavier_exp(s) for s in shapes]
    batches = [synth_batch(rng, glob) for _ in range(steps)]
    ti_torch.GRAD_BITWIDTH, ti_torch.TRAINING = 5, True
    group_was, ti_torch.WGRAD_GROUP = ti_torch.WGRAD_GROUP, 2  # two layers fill a group here: their gradient slices are pushed, as in the timed net
    model = ti_vgg.TiVGG_cifar(list(PARITY_CFG), dropout=True, fuse_relu=True)
    for l, w, e in zip(model.weighted_layers(), weights, wexps):
        l.weight = torch.from_numpy(w).to(dev)
        l.weight_exp = ti_torch.exp_tensor(e, dev)
    lo, hi = shard_range(glob, rank, world)
    tr = Trainer(model, hi - lo, dev, rank=rank, world=world, use_graph=True, seed=seed, warmup_steps=1,
                 peer_update="auto" if exchange == "auto" else False, sample_offset=lo)
    route = "peer-memory update kernel" if tr.peer is not None else "NCCL all-reduce + update"
    logits = []
    for x, t in batches:
        out, exp = tr.step(torch.from_numpy(x[lo:hi].copy()).pin_memory(), torch.from_numpy(t[lo:hi].copy()).pin_memory())
        tr.sync()
        logits.append((out.numpy().copy(), int(exp)))
    got_w = [l.weight.cpu().numpy() for l in model.weighted_layers()]
    tr.close()
    ti_torch.WGRAD_GROUP = group_was
    spans = [shard_range(glob, r, world) for r in range(world)]
    want, want_w = dp_oracle.expected(PARITY_CFG, weights, wexps, batches, spans, seed)
    ok = all(np.array_equal(logits[s][0], want[(s, lo)][0]) and logits[s][1] == want[(s, lo)][1] for s in range(steps))
    ok = ok and all(np.array_equal(a, b) for a, b in zip(got_w, want_w))
    flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    return bool(flag.item()), route


def run_ours(args):
    import torch
    import torch.distributed as dist
    from niti_b200 import ops, ti_torch, ti_vgg
    from niti_b200.trainer import Trainer

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    # libraries (NCCL's version banner) write to stdout; keep stdout for the one JSON line
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N>1 must be launched with torch.distributed.run --nproc-per-node N")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def max_over_ranks(v):
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    cfg = CONFIGS[args.config][0]
    B, global_batch, scaling = plan_batches(args, world)

    # --- N > 1: the exchange route that is about to be timed, against the oracle
    parity, parity_route = None, None
    if world > 1 and not args.no_parity_check:
        parity, parity_route = dp_parity_check(dev, rank, world, args.exchange, dist)
        if not parity:
            if rank == 0:
                sys.stderr.write("bench.py: the data-parallel exchange does not reproduce the oracle replicas; no value is reported\n")
            dist.destroy_process_group()
            raise SystemExit(3)

    rng = np.random.default_rng(1235)
    shapes = vgg_shapes(cfg)
    weights = [rng.integers(-127, 128, size=s).astype(np.int8) for s in shapes]
    ti_torch.GRAD_BITWIDTH, ti_torch.TRAINING = 5, True
    model = ti_vgg.TiVGG_cifar(list(cfg), dropout=True, fuse_relu=True)
    for l, w, s in zip(model.weighted_layers(), weights, shapes):
        l.weight = torch.from_numpy(w).to(dev)
        l.weight_exp = ti_torch.exp_tensor(xavier_exp(s), dev)
    trainer = Trainer(model, B, dev, rank=rank, world=world, use_graph=True, seed=1235,
                      peer_update="auto" if args.exchange == "auto" else False, push_gradients=False if args.no_push else (True if args.push else "auto"))
    peer_exchange = trainer.peer is not None
    data_rng = np.random.default_rng(5000 + rank)
    batches = []
    for _ in range(4):
        x, t = synth_batch(data_rng, B)
        batches.append((torch.from_numpy(x).pin_memory(), torch.from_numpy(t).pin_memory()))

    # --- per-kernel timing of one eager step (before graph capture)
    trainer.step(*batches[0])
    trainer.sync()
    launches0 = ops.LAUNCHES
    ops.PROFILE = []
    trainer.step(*batches[1])
    trainer.sync()
    prof, ops.PROFILE = ops.PROFILE, None
    launches_per_step = ops.LAUNCHES - launches0
    per_kernel = {}
    for name, aops, abytes, a, b in prof:
        d = per_kernel.setdefault(name, [0, 0.0, 0, 0])
        d[0] += 1
        d[1] += a.elapsed_time(b) * 1e-3
        d[2] += aops
        d[3] += abytes

    # --- warm-up (captures the CUDA graphs), then the timed regions
    for i in range(max(args.warmup, 3)):
        trainer.step(*batches[i % 4])
    trainer.sync()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)  # > 126 MB L2

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    # (1) inputs resident in HBM, L2 flushed between steps, per-step CUDA events
    trainer.x.copy_(batches[0][0])
    trainer.t.copy_(batches[0][1])
    barrier()
    evs = []
    for i in range(args.steps):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        trainer.run_device_step()
        b.record()
        evs.append((a, b))
    barrier()
    dev_s = max_over_ranks(sum(a.elapsed_time(b) for a, b in evs) * 1e-3)
    # (2) end to end through Trainer.step: pinned host batch in, logits out, every step
    barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    a.record()
    trainer.prefetch(*batches[0])
    prev = None
    for i in range(args.steps):
        # Every step's batch crosses PCIe inside the timed region (the copy of batch i+1 runs beside step i's kernels)
        # and every step's logits are read on the host: those of step i-1 while step i runs, so that neither the
        # PCIe round trips nor the host's enqueue time leave the GPU idle.
        cur = trainer.step(*batches[i % 4], prefetch_next=batches[(i + 1) % 4])
        if prev is not None:
            out_h, exp_h = prev.wait()
            _ = int(out_h[0, 0])
        prev = cur
    out_h, exp_h = prev.wait()
    _ = int(out_h[0, 0])
    b.record()
    barrier()
    e2e_s = max_over_ranks(max(a.elapsed_time(b) * 1e-3, time.perf_counter() - t0 if world == 1 else 0.0))
    if rank == 0:
        sampler.stop()
    trainer.sync()

    # (3) sustained: the same device step replayed back to back (no L2 flush, no pauses) for about two seconds
    sus = None
    if args.sustained_s > 0:
        sus_sampler = ClockSampler(local)
        n_chunk = max(50, int(0.25 / max(dev_s / args.steps, 1e-5)))
        barrier()
        if rank == 0:
            sus_sampler.start()
        chunks, total, t_begin = [], 0.0, time.perf_counter()
        n_rounds = max(1, int(args.sustained_s / (n_chunk * dev_s / args.steps)))
        for _ in range(n_rounds):  # the same number of steps on every rank
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(n_chunk):
                trainer.run_device_step()
            b.record()
            b.synchronize()
            chunks.append(a.elapsed_time(b) * 1e-3 / n_chunk)
        barrier()
        if rank == 0:
            sus_sampler.stop()
        trainer.sync()
        last = chunks[len(chunks) // 2:]
        sus_ms = max_over_ranks(sum(last) / len(last)) * 1e3
        if rank == 0:
            cs = sus_sampler.summary()
            sus = {"ms_per_step": sus_ms, "value": B * world / (sus_ms * 1e-3), "unit": UNIT, "seconds": time.perf_counter() - t_begin,
                   "steps": n_rounds * n_chunk, "first_chunk_ms_per_step": chunks[0] * 1e3,
                   "how": "graph-replayed device steps back to back, no L2 flush; mean of the second half of the chunks",
                   "clocks": cs, "ms_x_mhz": (sus_ms * cs["sm_mhz"] if cs.get("sm_mhz") else None)}

    redos, downs = {}, {}
    for i, l in enumerate(model.weighted_layers()):
        for name in ("_fwd_state", "_bwd_state"):
            stt = getattr(l, name, None)
            if stt is not None:
                redos[f"conv{i + 1}{name[:4]}"] = int(stt[3].item())
                if int(stt[2].item()) >> 8:
                    downs[f"conv{i + 1}{name[:4]}"] = int(stt[2].item()) >> 8
    checksum = trainer.replica_checksum()
    if world > 1:
        cs = torch.tensor([checksum], dtype=torch.int64, device=dev)
        lo, hi = cs.clone(), cs.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        replicas_equal = bool(lo.item() == hi.item())
    else:
        replicas_equal = True

    # --- the dominant kernel (tensor-core conv forward / error-backward with fused requantisation), per layer:
    # ten back-to-back calls replayed from a CUDA graph, CUDA events around the replay on the launching stream
    tc_ops, tc_time, tc_calls, per_layer = 0, 0.0, 0, []
    if rank == 0:
        convs = [l for l in model.weighted_layers() if hasattr(l, "padding")]
        for l in convs[1:]:
            K, R, S, C = l.weight.shape
            hw = l.act.shape[1]
            x = l.act
            err = torch.randint(-127, 128, (B, hw, hw, K), dtype=torch.int8, device=dev)
            ea = torch.zeros((), dtype=torch.int32, device=dev)
            for name, fn in (("fprop", lambda: ops.conv_fprop_fused(x, l.weight, l._fwd_state, 1, 0, None, 0, 0, True, ea, ea)),
                             ("dgrad", lambda: ops.conv_dgrad_fused(err, l.weight, st_b, 1, 0, None, 0, 0, ea, ea))):
                st_b = ops.new_requant_state(dev)
                t = time_graph(fn)
                gop = 2 * B * hw * hw * K * R * S * C
                tc_ops += gop; tc_time += t; tc_calls += 1
                per_layer.append({"layer": f"{name} {C}->{K} @{hw}x{hw}", "us": t * 1e6, "tops": gop / t / 1e12})

    if rank == 0:
        hbm, bf16_sus, bf16_burst, src = measured_peaks()
        images = B * world * args.steps
        peak_tops = 2.0 * bf16_burst  # every call is timed alone: the burst figure is the one that applies
        achieved = tc_ops / tc_time / 1e12 if tc_time > 0 else 0.0
        line = {
            "metric": metric_name(args.config), "value": images / dev_s, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": dev_s / args.steps * 1e3, "higher_is_better": True,
            "scaling": scaling, "vs_baseline": None, "dtype": "int8", "data": "synthetic",
            "config": {"workload": workload_name(args.config),
                       "per_gpu_batch": B, "global_batch": B * world, "parallelism": f"dp{world}",
                       "l2": "256 MB buffer written between timed steps (L2 flush); per-step CUDA events",
                       "graph": "step replayed from CUDA graphs", "replicas_bit_identical": replicas_equal,
                       "exchange": ("none" if world == 1 else "reduce-scatter + update + weight broadcast in one kernel over peer memory"
                                    + ("; gradient slices of the grouped layers pushed to their owners by copy engines under the backward pass"
                                       if trainer.push_stream is not None else "")
                                    if peer_exchange else "NCCL all-reduce of the int32 gradients, then the update launch"),
                       "parity_vs_oracle": parity,
                       "parity_check": (None if parity is None else f"2 steps of a conv128-P-conv128-P-conv512-P-FC net, global batch {8 * world} "
                                        f"sharded over {world} ranks, through the {parity_route}: logits and final weights of every rank "
                                        "equal oracle replicas with summed int32 gradients and one update"),
                       "shift_mispredictions_per_layer_since_start": redos,
                       "shift_step_downs_per_layer_since_start": downs,
                       "effective_int8_tops": step_ops_per_image(cfg) * images / dev_s / 1e12},
            "e2e": {"value": images / e2e_s, "unit": UNIT, "h2d_bytes_per_step": trainer.h2d_bytes,
                    "d2h_bytes_per_step": trainer.d2h_bytes, "ms_per_step": e2e_s / args.steps * 1e3},
            "gpu_launches": launches_per_step * args.steps,
            "roofline": {"bound": "tensor", "kernel": "umma_parked_kernel / umma_gemm_kernel<fused> (conv forward + error-backward, "
                                                       f"requantisation in the kernel, tcgen05 kind::i8), all {tc_calls} such calls of a step",
                         "achieved": achieved, "peak": peak_tops, "unit": "TOP/s", "frac": achieved / peak_tops,
                         "frac_of_2x_bf16_sustained": achieved / (2.0 * bf16_sus), "frac_of_nominal_4500": achieved / NOMINAL_INT8_TOPS,
                         "traffic": NCU_TRAFFIC_BYTES, "traffic_of": NCU_TRAFFIC_OF, "traffic_source": "recorded ncu capture (constant)",
                         "launches_timed": tc_calls * 10, "avg_launch_us": tc_time / max(tc_calls, 1) * 1e6,
                         "per_layer": per_layer,
                         "timing": "each call (one launch; two for the layers whose tiles do not fit in tensor memory) x10 in a CUDA graph, CUDA events around the replay",
                         "peak_source": f"2 x bf16_tflops burst ({src}): each call is timed alone; dense int8 rate is twice bf16 on this part"},
            "kernels_eager_step": {k: {"launches": v[0], "ms": v[1] * 1e3,
                                       "tops": (v[2] / v[1] / 1e12 if v[1] > 0 and v[2] else None),
                                       "gbs": (v[3] / v[1] / 1e9 if v[1] > 0 else None)} for k, v in per_kernel.items()},
            "clocks": sampler.summary(),
        }
        if sus is not None:
            line["sustained"] = sus
        if world == 1 and not args.no_cpu_baseline:
            r = cpu_reference_images_per_s(cfg, B, 2, 1)
            if r is not None:
                v, cores, sec, timed = r
                line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": cores, "kind": "reference",
                                        "sample": f"{timed} training steps of {args.config} on batches of {B} images ({sec:.2f} s per step, 1 warm-up): "
                                                  f"the reference's own ti_torch/ti_loss/ti_net/ti_vgg, extension calls served by exact CPU "
                                                  f"stand-ins over torch._int_mm, {cores} threads; first-step logits equal the oracle port's"}
            else:
                v, cores, sec = cpu_port_images_per_s(cfg, 16, 3, 1)
                line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": cores, "kind": "port",
                                        "sample": f"3 training steps of {args.config} on 16 of the {B} images per step "
                                                  f"({sec:.2f} s per step), oracle port with torch._int_mm, {cores} threads"}
        os.write(real_stdout, (json.dumps(line) + "\n").encode())
    if world > 1:
        trainer.close()
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------------
# single kernel cases (profiling) and the GEMM / conv sweep
# ------------------------------------------------------------------------------------------------
def time_graph(fn, reps=10):
    """Average device time of fn(): `reps` back-to-back calls replayed from a CUDA graph, CUDA events around the replay."""
    import torch
    fn(); fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(reps):
            fn()
    g.replay()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    g.replay()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) * 1e-3 / reps


def make_case(name, shape):
    """Returns (callable, algorithmic ops, algorithmic bytes) for one kernel case on cuda:0.
    conv cases: shape = N,H,W,C,K (3x3, pad 1); gemm cases: shape = M,N,K."""
    import torch
    from niti_b200 import ops
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(7)

    def r8(*s):
        return torch.randint(-127, 128, s, dtype=torch.int8, generator=g).to(dev)

    if name == "train_step":
        # one whole training step of the default workload (VGG-small-7), eager launches: shape = (batch,)
        from niti_b200 import ti_torch, ti_vgg
        from niti_b200.trainer import Trainer
        B = shape[0]
        cfg = CONFIGS["vgg7"][0]
        shapes_, weights, wexps, rng = synth_weights(cfg, 1235)
        ti_torch.GRAD_BITWIDTH, ti_torch.TRAINING = 5, True
        model = ti_vgg.TiVGG_cifar(list(cfg), dropout=True, fuse_relu=True)
        for l, w, e in zip(model.weighted_layers(), weights, wexps):
            l.weight = torch.from_numpy(w).to(dev)
            l.weight_exp = ti_torch.exp_tensor(e, dev)
        trainer = Trainer(model, B, dev, use_graph=False, seed=1235)
        x, t = synth_batch(rng, B)
        trainer.x.copy_(torch.from_numpy(x))
        trainer.t.copy_(torch.from_numpy(t))
        return trainer.run_device_step, step_ops_per_image(cfg) * B, 0
    if name == "conv_wgrad_multi":
        # the four weight gradients of a VGG-small-7 step that leave as one launch: shape = (batch,)
        B = shape[0]
        layers = [(8, 512, 512), (8, 256, 512), (16, 256, 256), (16, 128, 256)]
        jobs = [(r8(B, hw, hw, C), r8(B, hw, hw, K), torch.zeros((K, 3, 3, C), dtype=torch.int32, device=dev), 3, 3, 1) for hw, C, K in layers]
        gop = sum(2 * B * hw * hw * K * 9 * C for hw, C, K in layers)
        nbytes = sum(j[0].numel() + j[1].numel() + 4 * j[2].numel() for j in jobs)
        return (lambda: ops.conv_wgrad_accumulate_multi(jobs)), gop, nbytes
    if name.startswith("gemm"):
        M, N, K = shape
        ta, tb = {"gemm_tn": (False, True), "gemm_nn": (False, False), "gemm_tn_a": (True, False)}[name]
        a, b = r8(*((K, M) if ta else (M, K))), r8(*((N, K) if tb else (K, N)))
        return (lambda: ops.gemm_acc(a, b, ta, tb)), 2 * M * N * K, M * K + N * K + 4 * M * N
    N, H, W, C, K = shape
    x, w, err = r8(N, H, W, C), r8(K, 3, 3, C), r8(N, H, W, K)
    gop = 2 * N * H * W * K * 9 * C
    ea = torch.zeros((), dtype=torch.int32, device=dev)
    if name == "conv_fprop_fused":
        st = ops.new_requant_state(dev)
        return (lambda: ops.conv_fprop_fused(x, w, st, 1, 0, None, 0, 0, True, ea, ea)), gop, x.numel() + w.numel() + N * H * W * K
    if name == "conv_dgrad_fused":
        st = ops.new_requant_state(dev)
        return (lambda: ops.conv_dgrad_fused(err, w, st, 1, 0, None, 0, 0, ea, ea)), gop, err.numel() + w.numel() + x.numel()
    if name == "conv_fprop":
        return (lambda: ops.conv_fprop_acc(x, w)), gop, x.numel() + w.numel() + 4 * N * H * W * K
    if name == "conv_dgrad":
        return (lambda: ops.conv_dgrad_acc(err, w)), gop, err.numel() + w.numel() + 4 * x.numel()
    if name == "conv_wgrad":
        return (lambda: ops.conv_wgrad_acc(x, err)), gop, x.numel() + err.numel() + 4 * w.numel()
    raise SystemExit(f"unknown case {name}")


def run_step_down_case(shape):
    """Error-backward + requantisation of one layer when the shift guess is right, one too high every call, and
    alternately right / one too high, without and with the per-layer side buffer: microseconds per call (both launches)."""
    import torch
    from niti_b200 import ops
    dev = torch.device("cuda", 0)
    N, H, W, C, K = shape
    g = torch.Generator().manual_seed(7)
    w = torch.randint(-127, 128, (K, 3, 3, C), dtype=torch.int8, generator=g).to(dev)
    big = torch.randint(-127, 128, (N, H, W, K), dtype=torch.int8, generator=g).to(dev)
    small = (big.int() // 2).to(torch.int8)          # every sum about half as large: one bit less
    mask = torch.randint(-127, 128, (N, H, W, C), dtype=torch.int8, generator=g).to(dev).clamp_(min=0)
    ea = torch.zeros((), dtype=torch.int32, device=dev)
    out = {"case": "dgrad_step_down", "shape": shape}
    for use_side in (False, True):
        st = ops.new_requant_state(dev)
        nbytes = ops.conv_dgrad_side_bytes(N, H, W, C, K, 3, 3, 1)
        side = torch.empty(nbytes, dtype=torch.uint8, device=dev) if use_side and nbytes else None

        def f(e):
            return ops.conv_dgrad_fused(e, w, st, 1, 0, None, 0, 0, ea, ea, relu_mask=mask, side=side)
        for _ in range(3):
            f(big)
        key = "with_side" if use_side else "without_side"
        out[key] = {"right_us": time_graph(lambda: f(big)) * 1e6}
        f(big)
        # every second call is one shift below the guess: repaired with the side buffer, contracted again without it
        # (there the guess follows the last value, so both calls of a pair miss)
        out[key]["alternating_us"] = time_graph(lambda: (f(big), f(small))) * 1e6 / 2
        out[key]["verdict_of_last_call"] = int(st[2].item()) & 3
    ops.check_status("cuda:0")
    print(json.dumps(out))


def run_case(args):
    import torch
    from niti_b200 import ops
    torch.cuda.set_device(0)
    shape = tuple(int(v) for v in args.shape.split(","))
    if args.case == "dgrad_step_down":
        return run_step_down_case(shape)
    fn, aops, abytes = make_case(args.case, shape)
    if args.plain_launches:
        for _ in range(args.plain_launches):  # eager launches only: what a profiler should see
            fn()
        torch.cuda.synchronize()
        ops.check_status("cuda:0")
        print(json.dumps({"case": args.case, "shape": shape, "launched": args.plain_launches}))
        return
    t = time_graph(fn)
    ops.check_status("cuda:0")
    print(json.dumps({"case": args.case, "shape": shape, "us": t * 1e6, "tops": aops / t / 1e12, "gbs": abytes / t / 1e9}))


def run_sweep(args):
    import torch
    from niti_b200 import ops
    torch.cuda.set_device(0)
    _, bf16_sus, bf16_burst, src = measured_peaks()
    for n in (1024, 4096, 8192, 16384):
        a = torch.randint(-127, 128, (n, n), dtype=torch.int8).cuda()
        t_lib = time_graph(lambda: torch._int_mm(a, a), reps=3 if n > 8192 else 10)
        for name in ("gemm_tn", "gemm_nn", "gemm_tn_a"):
            fn, aops, _ = make_case(name, (n, n, n))
            t = time_graph(fn, reps=3 if n > 8192 else 10)
            print(json.dumps({"case": name, "n": n, "us": t * 1e6, "tops": aops / t / 1e12, "frac_of_2x_bf16_burst": aops / t / 1e12 / (2 * bf16_burst),
                              "cublaslt_int_mm_tops": 2 * n ** 3 / t_lib / 1e12}), flush=True)
        del a
    for c in (64, 256, 512):
        for hw in (8, 16, 32):
            for name in ("conv_fprop_fused", "conv_dgrad_fused", "conv_wgrad"):
                if c % 128 and name != "conv_wgrad":
                    name = name.replace("_fused", "")
                fn, aops, _ = make_case(name, (256, hw, hw, c, c))
                t = time_graph(fn, reps=3)
                print(json.dumps({"case": name, "C=K": c, "HW": hw, "batch": 256, "us": t * 1e6, "tops": aops / t / 1e12,
                                  "frac_of_2x_bf16_burst": aops / t / 1e12 / (2 * bf16_burst)}), flush=True)
    ops.check_status("cuda:0")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="vgg7", choices=sorted(CONFIGS), help="network: vgg7 (default), vgg9_wide, vgg13")
    ap.add_argument("--global-batch", type=int, default=0, help="fixed global batch split over the GPUs (strong scaling)")
    ap.add_argument("--scaling", default="auto", choices=["auto", "weak", "strong"])
    ap.add_argument("--sustained-s", type=float, default=2.0, help="seconds of back-to-back steps after the timed regions (0: skip)")
    ap.add_argument("--no-parity-check", action="store_true", help="N > 1: skip the oracle check of the exchange route")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--push", action="store_true", help="N>2: push gradient slices as at N=2 (default there only)")
    ap.add_argument("--no-push", action="store_true",
                    help="ablation (N>1, peer-memory route): no gradient slices pushed under the backward pass; the update kernel reads every layer from the peers' buckets")
    ap.add_argument("--no-step-down-codes", action="store_true",
                    help="ablation: error-backward layers that guess their shift contract again on every wrong guess")
    ap.add_argument("--exchange", default="auto", choices=["auto", "nccl"],
                    help="N>1: 'auto' = the peer-memory update kernel when the ranks share a node, else NCCL; 'nccl' = all-reduce")
    ap.add_argument("--case", help="time one kernel case instead of the training step (see make_case; 'train_step' with "
                                   "--shape BATCH runs whole eager steps of the default workload)")
    ap.add_argument("--shape", default="128,16,16,256,256")
    ap.add_argument("--plain-launches", type=int, default=0, help="with --case: just launch it this many times (for ncu)")
    ap.add_argument("--sweep", action="store_true", help="GEMM and conv roofline sweep, one JSON line per case")
    args = ap.parse_args()
    if args.case:
        return run_case(args)
    if args.sweep:
        return run_sweep(args)
    if args.no_step_down_codes:
        from niti_b200 import ti_torch
        ti_torch.STEP_DOWN_CODES = False
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
