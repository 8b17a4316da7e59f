#!/usr/bin/env python
"""Benchmark of the Dense-layer training step.

    python bench.py --gpus N --steps K --warmup W            # this library, N ranks (torchrun for N > 1)
    python bench.py --impl reference --steps K --warmup W    # the reference's CPU path (oracle port), host cores

Workload (config.workload): BASELINE configs[3], the data-parallel wide MLP
4096-8192-8192-8192-4096 (ReLU hidden, linear output), bf16 operands with fp32
accumulation and fp32 master weights, MSE against N(0,1) targets, Adam, GLOBAL
batch 65536 split evenly over the ranks (strong scaling), one fp32 gradient
all-reduce per layer per step.  Inputs are seeded synthetic N(0,1) blocks; the
weights are drawn in the reference's distribution, U(-1,1)*scale(act).

One JSON line on stdout (rank 0).  `value` times steps whose inputs already sit in
HBM; `e2e` times the same steps fed from pinned host memory through the pipelined
C-ABI call (host->device copies and the loss read-back inside the timed region).
"""
import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

DIMS = [(4096, 8192), (8192, 8192), (8192, 8192), (8192, 4096)]
ACTS = ["relu", "relu", "relu", "linear"]
GLOBAL_BATCH = 65536
# Data parallel: from this many ranks on, the parameter update is split over the ranks (reduce-scatter, update of the
# own piece, all-gather) unless --shard-update says otherwise.  Measured, sharded against replicated, each pair in one
# call on one box: 8 ranks 8.242 against 8.390 ms per step, 4 ranks 15.137 against 15.876, 2 ranks 28.99 against 28.69.
SHARD_UPDATE_FROM_RANKS = 4
SEED = 3
LR = 1e-3
BLOCK_ROWS = 1024                     # data is generated in blocks of rows keyed by (seed, stream, block)
SUM_IO = sum(a * b for a, b in DIMS)  # 201,326,592
PARAMS = SUM_IO + sum(b for _, b in DIMS)
FLOP_PER_SAMPLE = 6.0 * SUM_IO        # forward + dX + dW GEMMs, the reference's dX of layer 0 included
# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum, ncu, --clock-control none) of the step's twelve GEMM
# launches, captured on this network with 8192 rows per launch, in launch order: forward of layers 0-3, then per
# layer from the last to the first the weight-gradient product (TN) and the input-gradient product (NT).  Rows are
# M of the NN / NT products and K of the TN products, and both the tiles a launch walks and the strips it streams
# grow in proportion to them, so a launch with R rows moves R / 8192 times these bytes.
NCU_ROWS = 8192
NCU_GEMM_DRAM_BYTES = {   # (orientation, m, n, k at 8192 rows): measured DRAM bytes
    ("NN", "rows", 8192, 4096): 333.6e6, ("NN", "rows", 8192, 8192): 1080.4e6, ("NN", "rows", 4096, 8192): 715.0e6,
    ("TN", 8192, 4096, "rows"): 715.2e6, ("TN", 8192, 8192, "rows"): 1339.4e6, ("TN", 4096, 8192, "rows"): 634.3e6,
    ("NT", "rows", 8192, 4096): 534.6e6, ("NT", "rows", 8192, 8192): 1285.8e6, ("NT", "rows", 4096, 8192): 640.2e6,
}


def step_gemms(rows, bf16_out=2, f32=4):
    """The twelve GEMM launches of one step on `rows` rows: (orientation, key into NCU_GEMM_DRAM_BYTES, flops,
    algorithmic bytes = every operand read once + the output written once, bf16 operands, the relu mask of the
    input-gradient products included)."""
    out = []
    L = len(DIMS)
    for i, (a, b) in enumerate(DIMS):                      # forward: rows x b x a
        last = i + 1 == L
        alg = 2 * (rows * a + a * b) + (f32 if last else bf16_out) * rows * b
        out.append(("NN", ("NN", "rows", b, a), 2.0 * rows * a * b, alg))
    for i in range(L - 1, -1, -1):
        a, b = DIMS[i]
        out.append(("TN", ("TN", a, b, "rows"), 2.0 * rows * a * b, 2 * (rows * a + rows * b) + f32 * a * b))
        mask = 2 * rows * a if i > 0 else 0
        out.append(("NT", ("NT", "rows", a, b), 2.0 * rows * a * b, 2 * (rows * b + a * b) + mask + 2 * rows * a))
    return out


def layer_weights(layer):
    """U(-1,1) * scale(act): sqrt(2/in) for relu, sqrt(1/in) for linear (src/layer.zig:330-338)."""
    (n_in, n_out), act = DIMS[layer], ACTS[layer]
    rng = np.random.default_rng([SEED, 100 + layer])
    scale = np.float32(np.sqrt((2.0 if act == "relu" else 1.0) / n_in))
    w = rng.random((n_in, n_out), dtype=np.float32)
    w *= np.float32(2.0)
    w -= np.float32(1.0)
    w *= scale
    return w


def fill_rows(dst, stream, row0):
    """dst[i] = global row row0+i of N(0,1) stream `stream` (0 inputs, 1 targets); same data for any rank count."""
    rows, cols = dst.shape
    assert row0 % BLOCK_ROWS == 0
    for off in range(0, rows, BLOCK_ROWS):
        n = min(BLOCK_ROWS, rows - off)
        rng = np.random.default_rng([SEED, stream, (row0 + off) // BLOCK_ROWS])
        dst[off:off + n] = rng.standard_normal((BLOCK_ROWS, cols), dtype=np.float32)[:n]


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        d = json.load(open(path))
        return {"bf16_sustained": float(d["bf16_tflops_sustained"]), "bf16_burst": float(d["bf16_tflops"]),
                "hbm": float(d["hbm_gbs"]), "source": "measured"}
    except Exception:
        return {"bf16_sustained": 1400.0, "bf16_burst": 1590.0, "hbm": 6650.0, "source": "fallback"}


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while the timed regions run."""

    def __init__(self, device):
        super().__init__(daemon=True)
        self.device, self.samples, self.reasons, self.max_mhz, self.stop_flag = device, [], set(), None, False
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(device)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
            self.ok = True
        except Exception:
            pass

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40,
                 "hw_power_brake_slowdown": 0x80}
        while not self.stop_flag:
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(0.05)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["unavailable"]}
        return {"sm_mhz": int(np.median(self.samples)), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


def bind_to_gpu_numa_node(device):
    """Pins this process to the CPUs of the NUMA node the GPU hangs off, BEFORE any pinned host memory is
    allocated, so that the step's input buffers land in memory local to the GPU's PCIe root.  Returns what was
    found and done (reported under e2e.numa)."""
    info = {"gpu_node": None, "bound": False}
    try:
        import pynvml
        pynvml.nvmlInit()
        bus = pynvml.nvmlDeviceGetPciInfo(pynvml.nvmlDeviceGetHandleByIndex(device)).busId
        bus = (bus.decode() if isinstance(bus, bytes) else bus).lower()
        if len(bus.split(":")[0]) == 8:          # NVML prints an 8-digit PCI domain, sysfs a 4-digit one
            bus = bus[4:]
        base = f"/sys/bus/pci/devices/{bus}"
        node = int(open(f"{base}/numa_node").read())
        info["gpu_node"] = node
        cpus = set()
        for part in open(f"{base}/local_cpulist").read().strip().split(","):
            if part:
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = os.sched_getaffinity(0)
        info["allowed_cpus"] = len(allowed)
        if node >= 0 and cpus & allowed and (cpus & allowed) != allowed:
            os.sched_setaffinity(0, cpus & allowed)
            info["bound"] = True
        info["local_cpus"] = len(cpus & allowed)
    except Exception as e:                       # no NVML / sysfs entry: nothing is bound, say so
        info["error"] = type(e).__name__
    return info


def block_hash(a):
    """Order-sensitive 64-bit digest of a float32 block (bit patterns, not values: -0.0 and NaN payloads count)."""
    u = np.ascontiguousarray(a).view(np.uint32).astype(np.uint64)
    idx = np.arange(1, u.size + 1, dtype=np.uint64)
    with np.errstate(over="ignore"):
        return int((u * (idx | np.uint64(1))).sum(dtype=np.uint64))


DP_CHECK_DIMS, DP_CHECK_ACTS = [(64, 128), (128, 96), (96, 32)], ["relu", "relu", "linear"]


def dp_check(zn, be, dist, rank, world, local, shard_update):
    """Correctness of the data-parallel path in the run that is being timed: a small network (64-128-96-32, Adam,
    MSE, 4 steps, global batch 8 rows per rank) trained across all ranks through the same communicator as the
    benchmark, and on rank 0 the same network on ONE GPU through a second context.  Every rank must end with
    bit-identical parameters, and they must agree with the one-GPU run."""
    import torch
    rows = 8 * world + 3                                   # not a multiple of the rank count: uneven shards
    rng = np.random.default_rng(17)
    x = rng.standard_normal((rows, 64)).astype(np.float32)
    t = rng.standard_normal((rows, 32)).astype(np.float32)
    Ws = [(rng.uniform(-1, 1, (a, b)) * np.sqrt(2.0 / a)).astype(np.float32) for a, b in DP_CHECK_DIMS]
    bs = [rng.uniform(-0.1, 0.1, b).astype(np.float32) for _, b in DP_CHECK_DIMS]

    def build(backend):
        net = zn.Network(backend, zn.Precision.FP32_SIMT)
        for i, ((a, b), act) in enumerate(zip(DP_CHECK_DIMS, DP_CHECK_ACTS)):
            net.addDense(a, b, act)
            net.setWeights(i, Ws[i], bs[i])
        net.setOptimizer(zn.Adam())
        return net

    net = build(be)
    net.setDataParallel(rows)
    if shard_update:
        net.setUpdateSharding(True)          # the same exchange pattern as the timed network
    lo, hi = zn.Backend.distributeWorkload(rows, world, rank)
    losses = [net.trainStep(np.ascontiguousarray(x[lo:hi]), np.ascontiguousarray(t[lo:hi]), 0.01, zn.Loss.mse) for _ in range(4)]
    params = [net.getWeights(i) for i in range(3)]
    digest = [block_hash(np.concatenate([w.ravel(), b])) & 0x7FFFFFFFFFFFFFFF for w, b in params] + \
             [block_hash(np.array(losses, np.float32)) & 0x7FFFFFFFFFFFFFFF]
    net.deinit()
    all_digests = [torch.zeros(len(digest), dtype=torch.int64) for _ in range(world)]
    dist.all_gather(all_digests, torch.tensor(digest, dtype=torch.int64))
    identical = all(bool(torch.equal(all_digests[0], d)) for d in all_digests)
    result = {"ranks_bit_identical": identical, "tolerance": 1e-5, "steps": 4, "rows": rows, "update_sharded": bool(shard_update)}
    if rank == 0:
        solo_be = zn.Backend(local, zn.Precision.FP32_SIMT)
        solo = build(solo_be)
        solo_losses = [solo.trainStep(x, t, 0.01, zn.Loss.mse) for _ in range(4)]
        dev = 0.0
        for i in range(3):
            w, b = solo.getWeights(i)
            for got, want in ((params[i][0], w), (params[i][1], b)):
                dev = max(dev, float(np.linalg.norm(got.astype(np.float64) - want) / np.linalg.norm(want.astype(np.float64))))
        result["vs_one_gpu_rel_l2"] = dev
        result["loss_rel_dev"] = float(np.max(np.abs(np.array(losses) - np.array(solo_losses)) / np.abs(solo_losses)))
        solo.deinit()
        solo_be.deinit()
    return result


def gemm_sweep_summary(zn, be, peaks):
    """BASELINE configs[4] in brief, for the N = 1 line: bf16 on the six stated sizes x {NN+bias+ReLU, NT, TN},
    tf32 and fp32 on 4096^3 only; 3 warm-up + 10 timed launches each (the reference's scheme is 10 + 100,
    src/benchmark/cuda_benchmark.zig:17-25).  TFLOP/s = 2*M*N*K / average launch time."""
    out = []
    rng = np.random.default_rng(4)
    precs = {"bf16": zn.Precision.BF16_TC, "tf32": zn.Precision.TF32_TC, "fp32": zn.Precision.FP32_SIMT}
    sizes = [(256, 256, 256), (1024, 1024, 1024), (4096, 4096, 4096), (8192, 8192, 8192), (16384, 16384, 16384), (65536, 512, 512)]
    for (m, n, k) in sizes:
        a = be.tensor(rng.standard_normal(m * k, dtype=np.float32))
        b = be.tensor(rng.standard_normal(k * n, dtype=np.float32))
        bias = be.tensor(rng.uniform(-0.1, 0.1, n).astype(np.float32))
        c = be.tensor(m * n)
        for pname in (["bf16", "tf32", "fp32"] if (m, n, k) == (4096, 4096, 4096) else ["bf16"]):
            be.set_precision(precs[pname])
            fam = 1 if pname == "fp32" else 0
            calls = {"NN+bias+relu": lambda: be.matMulBiasRelu(a, b, bias, c, m, n, k),
                     "NT": lambda: be.matMulTransposeB(a, b, c, m, n, k), "TN": lambda: be.matMulTransposeA(a, b, c, m, n, k)}
            for oname, call in calls.items():
                for _ in range(3):
                    call()
                be.endCommandBatch()
                be.profile(True)
                be.profile_reset()
                for _ in range(10):
                    call()
                p = be.profile_get(fam)
                be.profile(False)
                tf = p["flops"] / (p["ms"] * 1e-3) / 1e12
                out.append({"mnk": [m, n, k], "orient": oname, "precision": pname, "ms": round(p["ms"] / p["launches"], 5),
                            "tflops": round(tf, 2),
                            "frac_of_measured_bf16_burst": round(tf / peaks["bf16_burst"], 4) if pname == "bf16" else None})
        for tt in (a, b, bias, c):
            tt.free()
    be.set_precision(zn.Precision.BF16_TC)
    return out


# --------------------------------------------------------------------------------------- CPU side

def oracle_net():
    from oracle import zn_oracle as zo
    net = zo.Net()
    for i, ((a, b), act) in enumerate(zip(DIMS, ACTS)):
        net.add_dense(a, b, zo.RELU if act == "relu" else zo.LINEAR)
        net.set_params(i, layer_weights(i), np.zeros(b, np.float32))
        net.set_adam(i)
    return net, zo


def cpu_sample(net, zo, rows, x, t):
    """One bounded sample of the workload on one host core: gradients of `rows` rows of the global batch
    (the per-row part of a step) and one clip + Adam pass over all parameters (the per-step part).
    Returns (seconds per row, seconds per step-fixed part)."""
    t0 = time.perf_counter()
    net.shard_gradients(x[:rows], t[:rows], rows, GLOBAL_BATCH, zo.MSE)
    t1 = time.perf_counter()
    net.clip_and_update(LR)
    t2 = time.perf_counter()
    return (t1 - t0) / rows, t2 - t1


def cpu_rows_for_budget(net, zo, x, t, seconds):
    per_row, _ = cpu_sample(net, zo, 2, x, t)
    return int(max(2, min(x.shape[0], round(seconds / max(per_row, 1e-3)))))


def cpu_baseline(budget_s=12.0):
    net, zo = oracle_net()
    x = np.empty((64, DIMS[0][0]), np.float32)
    t = np.empty((64, DIMS[-1][1]), np.float32)
    fill_rows(x, 0, 0)
    fill_rows(t, 1, 0)
    rows = cpu_rows_for_budget(net, zo, x, t, budget_s)
    per_row, fixed = cpu_sample(net, zo, rows, x, t)
    value = GLOBAL_BATCH / (GLOBAL_BATCH * per_row + fixed)
    return {"value": value, "unit": "samples/s", "cores": 1, "kind": "port",
            "sample": f"oracle (single-threaded restatement of the reference CPU path): forward+backward of {rows} rows "
                      f"of the global batch ({per_row * 1e3:.1f} ms/row) plus one clip+Adam pass over {PARAMS} parameters "
                      f"({fixed:.2f} s); extrapolated to a {GLOBAL_BATCH}-row step as rows*per_row + fixed"}


def run_reference(args):
    """--impl reference: the reference's own CPU Dense path (its restatement in oracle/, the reference being
    Zig with no toolchain here), on the host cores it can use: one, the path has no threads."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    net, zo = oracle_net()
    x = np.empty((64, DIMS[0][0]), np.float32)
    t = np.empty((64, DIMS[-1][1]), np.float32)
    fill_rows(x, 0, 0)
    fill_rows(t, 1, 0)
    total_budget = 150.0
    rows = cpu_rows_for_budget(net, zo, x, t, total_budget / (args.steps + args.warmup) * 0.6)
    for _ in range(max(0, args.warmup - 1)):
        cpu_sample(net, zo, rows, x, t)
    step_s = []
    for _ in range(args.steps):
        per_row, fixed = cpu_sample(net, zo, rows, x, t)
        step_s.append(GLOBAL_BATCH * per_row + fixed)
    ms = 1e3 * float(np.mean(step_s))
    value = GLOBAL_BATCH / (ms / 1e3)
    sample = (f"each step = gradients of {rows} rows of the global batch + one clip+Adam pass over all parameters, "
              f"extrapolated to {GLOBAL_BATCH} rows (rows are independent in the reference loops)")
    line = {
        "impl": "reference", "metric": "train_samples_per_sec", "value": value, "unit": "samples/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.gpus, args.gpus >= SHARD_UPDATE_FROM_RANKS if args.shard_update is None
                                  else bool(args.shard_update) and args.gpus > 1),
        "cpu_baseline": {"value": value, "unit": "samples/s", "cores": 1, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(n_gpus, shard_update=False):
    return {"update": "split over the ranks (reduce-scatter, own piece, all-gather)" if shard_update else "replicated on every rank",
            "workload": "wide_mlp_dp: BASELINE configs[3], MLP 4096-8192-8192-8192-4096 relu/linear, MSE, Adam lr 1e-3, seed 3",
            "global_batch": GLOBAL_BATCH, "per_gpu_batch": GLOBAL_BATCH // n_gpus, "parallelism": f"dp{n_gpus}",
            "params": PARAMS, "allreduce_bytes_per_step": 4 * PARAMS if n_gpus > 1 else 0,   # a reduce-scatter + all-gather pair moves the same bytes
            "l2": "inputs (>= 256 MB per rank and step) and weights (805 MB) exceed the 126 MB L2; no flush needed"}


# --------------------------------------------------------------------------------------- GPU side

def run_ours(args):
    import zigneuron_b200 as zn

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N > 1")
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist_mod
        dist = dist_mod
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("gloo", rank=rank, world_size=world)

    def barrier():
        if dist:
            dist.barrier()

    def max_over_ranks(v):
        if not dist:
            return v
        import torch
        tt = torch.tensor([v], dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        return float(tt[0])

    numa = bind_to_gpu_numa_node(local)
    be = zn.Backend(local, zn.Precision.BF16_TC)
    check = None
    if world > 1:
        ids = [zn.Backend.dp_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        be.dp_init(rank, world, ids[0])
    shard_update = world >= SHARD_UPDATE_FROM_RANKS if args.shard_update is None else (bool(args.shard_update) and world > 1)
    if world > 1:
        check = dp_check(zn, be, dist, rank, world, local, shard_update)

    net = zn.Network(be, zn.Precision.BF16_TC)
    for i, ((a, b), act) in enumerate(zip(DIMS, ACTS)):
        net.addDense(a, b, act)
        net.setWeights(i, layer_weights(i), np.zeros(b, np.float32))
    net.setOptimizer(zn.Adam(beta1=0.9, beta2=0.999, eps=1e-8))
    if world > 1:
        net.setDataParallel(GLOBAL_BATCH)
        if shard_update:
            net.setUpdateSharding(True)

    lo, hi = zn.Backend.distributeWorkload(GLOBAL_BATCH, world, rank)
    rows = hi - lo
    hx = be.host_alloc((rows, DIMS[0][0]))
    ht = be.host_alloc((rows, DIMS[-1][1]))
    fill_rows(hx, 0, lo)
    fill_rows(ht, 1, lo)
    dx, dt = be.tensor(hx), be.tensor(ht)

    sampler = ClockSampler(local)
    loss = zn.Loss.mse

    # ---- leg 1: inputs resident in HBM
    for _ in range(args.warmup):
        net.trainStep(dx, dt, LR, loss, rows=rows)
    barrier()
    be.endCommandBatch()
    sampler.start()
    be.profile(True)
    be.profile_reset()
    launches0 = be.launch_count()
    be.timer_start()
    last_loss = None
    for _ in range(args.steps):
        last_loss = net.trainStep(dx, dt, LR, loss, rows=rows)
    ms_total = be.timer_stop()
    barrier()
    launches = be.launch_count() - launches0
    prof = {name: be.profile_get(fam) for name, fam in
            [("gemm", 0), ("loss", 2), ("bias_reduce", 3), ("grad_norm", 4), ("optimizer", 5), ("convert", 6)]}
    be.profile(False)
    ms_total = max_over_ranks(ms_total)
    ms_per_step = ms_total / args.steps
    value = GLOBAL_BATCH / (ms_per_step / 1e3)

    # ---- leg 2: end to end from pinned host memory, two steps in flight
    e2e_warm = max(1, min(2, args.warmup))
    for _ in range(e2e_warm):
        net.submitStep(hx, ht, rows, LR, loss)
        net.waitStep()
    # steady state of the two-deep pipeline: one step is in flight when the clock starts, and every timed iteration
    # submits one step (its host->device copy included) and waits for the oldest one (its loss read back), so the
    # timed region holds exactly `steps` copies, `steps` steps and `steps` read-backs
    net.submitStep(hx, ht, rows, LR, loss)
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        net.submitStep(hx, ht, rows, LR, loss)
        e2e_loss = net.waitStep()
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    net.waitStep()
    be.endCommandBatch()
    barrier()
    sampler.stop_flag = True
    if sampler.is_alive():
        sampler.join(timeout=2)
    e2e_value = GLOBAL_BATCH * args.steps / e2e_s

    # ---- leg 3: the copies of leg 2 alone (same pinned buffers, all ranks at once, no compute): the ceiling the
    # host side sets for the end-to-end number
    be.copyData(hx, dx, hx.size)
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        be.copyData(hx, dx, hx.size)
        be.copyData(ht, dt, ht.size)
    copy_s = max_over_ranks(time.perf_counter() - t0)
    barrier()
    h2d_bytes = int(hx.nbytes + ht.nbytes) * world
    h2d_ceiling_gbs = h2d_bytes * args.steps / copy_s / 1e9

    # every rank must hold the same parameters after the timed steps
    if world > 1:
        import torch
        mine = torch.tensor([block_hash(np.concatenate([w.ravel(), b])) & 0x7FFFFFFFFFFFFFFF
                             for w, b in (net.getWeights(i) for i in range(len(DIMS)))], dtype=torch.int64)
        everyone = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(everyone, mine)
        check["bench_net_ranks_bit_identical"] = all(bool(torch.equal(everyone[0], d)) for d in everyone)

    if rank != 0:
        if dist:
            dist.destroy_process_group()
        return

    peaks = measured_peaks()
    g = prof["gemm"]
    achieved = g["flops"] / (g["ms"] * 1e-3) / 1e12 if g["ms"] > 0 else 0.0
    peak = peaks["bf16_sustained"]
    line = {
        "metric": "train_samples_per_sec", "value": value, "unit": "samples/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": workload_config(world, shard_update),
        "step_tflops": FLOP_PER_SAMPLE * value / 1e12 / world,
        "step_frac_of_bf16_peak": {"per_gpu_tflops": FLOP_PER_SAMPLE * value / 1e12 / world,
                                   "of_measured_sustained": FLOP_PER_SAMPLE * value / 1e12 / world / peaks["bf16_sustained"],
                                   "of_measured_burst": FLOP_PER_SAMPLE * value / 1e12 / world / peaks["bf16_burst"],
                                   "of_datasheet_2250": FLOP_PER_SAMPLE * value / 1e12 / world / 2250.0},
        "roofline": {"kernel": "gemm_tc_pair_kernel<bf16> (tcgen05 cta_group::2, 12 launches per step: NN, TN, NT per layer)",
                     "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                     "frac": achieved / peak if peak else None, "peak_source": f"{peaks['source']}, sustained bf16",
                     "launches": g["launches"], "avg_launch_ms": g["ms"] / max(1, g["launches"]),
                     **gemm_traffic(rows)},
        "kernel_ms_per_step": {k: v["ms"] / args.steps for k, v in prof.items()},
        "kernel_ms_note": "gemm, loss and convert run on the main stream and add up to the step; optimizer, bias_reduce and "
                          "grad_norm run on side streams underneath the GEMMs, so their durations (and GB/s) are stretched "
                          "by sharing the GPU and do not add to the step",
        "hbm_kernels": {k: {"achieved_gbs": v["bytes"] / (v["ms"] * 1e-3) / 1e9 if v["ms"] > 0 else None,
                            "frac_of_measured_hbm": (v["bytes"] / (v["ms"] * 1e-3) / 1e9 / peaks["hbm"]) if v["ms"] > 0 else None}
                        for k, v in prof.items() if k != "gemm"},
        "e2e": {"value": e2e_value, "unit": "samples/s", "h2d_bytes_per_step": h2d_bytes,
                "d2h_bytes_per_step": 12 * world, "ms_per_step": 1e3 * e2e_s / args.steps,
                "how": "zn_net_submit_step / zn_net_wait_step from pinned host buffers, two steps in flight; timed in the "
                       "pipeline's steady state: each timed iteration = one submit (with its copies) + one wait",
                "h2d_ceiling_gbs": h2d_ceiling_gbs, "h2d_only_ms_per_step": 1e3 * copy_s / args.steps,
                "h2d_ceiling_how": "the same buffers copied host->device by every rank at once, nothing else running",
                "bound_ms_per_step": max(ms_per_step, 1e3 * copy_s / args.steps),
                "frac_of_bound": max(ms_per_step, 1e3 * copy_s / args.steps) / (1e3 * e2e_s / args.steps),
                "numa": numa},
        "gpu_launches": int(launches),
        "clocks": sampler.summary(),
        "loss": {"resident_last": last_loss, "e2e_last": e2e_loss},
    }
    clk = line["clocks"].get("sm_mhz")
    if clk:
        # what the step achieves of the datasheet peak AT THE CLOCK THE GPU RAN AT (the 1 kW cap holds the SM clock
        # well below its maximum under a dense GEMM)
        line["roofline"]["clock_normalised"] = achieved / (2250.0 * clk / line["clocks"]["sm_max_mhz"])
    if check is not None:
        line["dp_check"] = check
    if world == 1 and not args.no_sweep:
        net.deinit()
        for tt in (dx, dt):
            tt.free()
        line["gemm_sweep"] = gemm_sweep_summary(zn, be, peaks)
    if world == 1 and not args.no_cpu:
        line["cpu_baseline"] = cpu_baseline()
    print(json.dumps(line), flush=True)
    failed = check is not None and not (check["ranks_bit_identical"] and check.get("bench_net_ranks_bit_identical", True)
                                        and check.get("vs_one_gpu_rel_l2", 0.0) <= check["tolerance"])
    if dist:
        dist.destroy_process_group()
    if failed:
        raise SystemExit("dp_check failed: " + json.dumps(check))


def gemm_traffic(rows):
    """roofline.traffic: measured DRAM bytes per launch (average over the step's twelve GEMMs) beside the algorithmic
    bytes, and the same per orientation."""
    gemms = step_gemms(rows)
    scale = rows / NCU_ROWS
    per = {}
    for orient, key, _, alg in gemms:
        d = per.setdefault(orient, {"launches": 0, "traffic": 0.0, "algorithmic": 0.0})
        d["launches"] += 1
        d["traffic"] += NCU_GEMM_DRAM_BYTES[key] * scale
        d["algorithmic"] += alg
    total = sum(d["traffic"] for d in per.values())
    total_alg = sum(d["algorithmic"] for d in per.values())
    for d in per.values():
        d["ratio"] = d["traffic"] / d["algorithmic"]
    return {"traffic": total / len(gemms), "algorithmic_bytes": total_alg / len(gemms), "traffic_over_algorithmic": total / total_alg,
            "traffic_unit": f"DRAM bytes per launch, average of the 12 GEMMs of a step; ncu capture at {NCU_ROWS} rows per launch "
                            f"scaled by rows / {NCU_ROWS} (bytes are linear in the rows at fixed layer widths)",
            "traffic_by_orientation": per}


def run_gemm_sweep(args):
    """BASELINE configs[4]: standalone Dense GEMMs, NN/NT/TN, fused bias+ReLU on NN, operands N(0,1) seed 4.
    Not the headline line: prints one JSON line per (size, orientation, precision) for the results table and is
    the small case the ncu captures run."""
    import zigneuron_b200 as zn
    be = zn.Backend(0)
    peaks = measured_peaks()
    sizes = [tuple(int(v) for v in s.split("x")) for s in args.sizes.split(",")]
    precs = {"bf16": zn.Precision.BF16_TC, "tf32": zn.Precision.TF32_TC, "fp32": zn.Precision.FP32_SIMT}
    rng = np.random.default_rng(4)
    for (m, n, k) in sizes:
        a = be.tensor(rng.standard_normal(m * k, dtype=np.float32))
        b = be.tensor(rng.standard_normal(k * n, dtype=np.float32))
        bias = be.tensor(rng.uniform(-0.1, 0.1, n).astype(np.float32))
        c = be.tensor(m * n)
        for pname in args.precisions.split(","):
            be.set_precision(precs[pname])
            fam = 1 if pname == "fp32" else 0
            calls = {"NN+bias+relu": lambda: be.matMulBiasRelu(a, b, bias, c, m, n, k),
                     "NT": lambda: be.matMulTransposeB(a, b, c, m, n, k), "TN": lambda: be.matMulTransposeA(a, b, c, m, n, k)}
            for oname, call in calls.items():
                for _ in range(args.warmup):
                    call()
                be.endCommandBatch()
                be.profile(True)
                be.profile_reset()
                for _ in range(args.steps):
                    call()
                p = be.profile_get(fam)
                be.profile(False)
                tf = p["flops"] / (p["ms"] * 1e-3) / 1e12
                peak = peaks["bf16_burst"] if pname == "bf16" else None
                print(json.dumps({"workload": "gemm_sweep", "mnk": [m, n, k], "orient": oname, "precision": pname,
                                  "ms": p["ms"] / p["launches"], "tflops": tf,
                                  "frac_of_measured_bf16_burst": tf / peak if peak else None}), flush=True)
        for t in (a, b, bias, c):
            t.free()
    be.deinit()


def run_other_config(args):
    """BASELINE configs[1] (784-512-256-10, batch 1024, Adam, CE with logits, seed 1) and configs[2] (the wide MLP at
    batch 8192 with SGD, seed 2), inputs resident on the device.  Extra lines for the results table.
    wide_mlp_adam_shard is the same wide MLP with Adam at batch 8192: what ONE rank of the 8-GPU data-parallel
    step computes, without the exchange; with --trace it gives the lane timeline of that step."""
    if args.trace:
        os.environ["ZN_TRACE_FILE"] = os.path.abspath(args.trace)
        if os.path.exists(args.trace):
            os.remove(args.trace)
    import zigneuron_b200 as zn
    if args.workload == "mlp784":
        dims, acts, B, seed, loss, lr = [(784, 512), (512, 256), (256, 10)], ["relu", "relu", "linear"], 1024, 1, zn.Loss.cross_entropy_logits, 1e-3
        precisions = [("fp32_simt", zn.Precision.FP32_SIMT), ("tf32", zn.Precision.TF32_TC), ("bf16", zn.Precision.BF16_TC)]
    else:
        dims, acts, B, seed, loss, lr = DIMS, ACTS, 8192, 2, zn.Loss.mse, 1e-3
        precisions = [("bf16", zn.Precision.BF16_TC), ("tf32", zn.Precision.TF32_TC)]
        if args.workload == "wide_mlp_adam_shard":
            precisions = precisions[:1]
    rng = np.random.default_rng(seed)
    if args.workload == "mlp784":
        x = rng.random((B, 784), dtype=np.float32)
        t = np.eye(10, dtype=np.float32)[rng.integers(0, 10, B)]
    else:
        x = rng.standard_normal((B, dims[0][0]), dtype=np.float32)
        t = rng.standard_normal((B, dims[-1][1]), dtype=np.float32)
    be = zn.Backend(0)
    flop = 6.0 * B * sum(a * b for a, b in dims)
    for pname, prec in precisions:
        net = zn.Network(be, prec)
        wr = np.random.default_rng([seed, 7])
        for i, ((a, b), act) in enumerate(zip(dims, acts)):
            net.addDense(a, b, act)
            scale = np.sqrt((2.0 if act == "relu" else 1.0) / a) if args.workload != "mlp784" else np.sqrt(2.0 / (a + b))
            net.setWeights(i, ((wr.random((a, b), dtype=np.float32) * 2 - 1) * np.float32(scale)).astype(np.float32), np.zeros(b, np.float32))
        if args.workload in ("mlp784", "wide_mlp_adam_shard"):
            net.setOptimizer(zn.Adam())
        dx, dt = be.tensor(x), be.tensor(t)
        losses = [net.trainStep(dx, dt, lr, loss, rows=B) for _ in range(args.warmup)]
        be.endCommandBatch()
        launches0 = be.launch_count()
        be.timer_start()
        for _ in range(args.steps):
            losses.append(net.trainStep(dx, dt, lr, loss, rows=B))
        ms = be.timer_stop() / args.steps
        launches = (be.launch_count() - launches0) / args.steps
        # the same step through the pipelined calls, inputs in pinned host memory: the host issues step i + 1
        # while step i runs, so what is left is the longer of the device's and the host's time per step
        ms_pipe = None
        if args.workload == "mlp784":
            hx, ht = be.host_alloc(x.shape), be.host_alloc(t.shape)
            hx[:], ht[:] = x, t
            for _ in range(3):
                net.submitStep(hx, ht, B, lr, loss)
                net.waitStep()
            net.submitStep(hx, ht, B, lr, loss)
            be.timer_start()
            for _ in range(args.steps):
                net.submitStep(hx, ht, B, lr, loss)
                losses.append(net.waitStep())
            ms_pipe = be.timer_stop() / args.steps
            net.waitStep()
        print(json.dumps({"workload": args.workload, "precision": pname, "batch": B, "ms_per_step": ms,
                          "ms_per_step_pipelined_from_host": ms_pipe,
                          "launches_per_step": launches,
                          "samples_per_s": B / (ms / 1e3), "tflops": flop / (ms / 1e3) / 1e12,
                          "loss_first": losses[0], "loss_last": losses[-1]}), flush=True)
        if args.trace:
            be.profile(True)
            for _ in range(3):
                net.trainStep(dx, dt, lr, loss, rows=B)
            be.profile(False)
        net.deinit()
        dx.free()
        dt.free()
    be.deinit()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="wide_mlp_dp", choices=["wide_mlp_dp", "gemm_sweep", "mlp784", "wide_mlp_sgd", "wide_mlp_adam_shard"])
    ap.add_argument("--trace", default=None, help="after timing, run 3 more steps with every launch written to this file "
                    "as 'family lane start_ms end_ms' (lanes: 0 main, 1 comm, 2 opt, 3 aux)")
    ap.add_argument("--sizes", default="1024x1024x1024,4096x4096x4096,8192x8192x8192,65536x512x512")
    ap.add_argument("--precisions", default="bf16,tf32,fp32")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU-baseline leg")
    ap.add_argument("--no-sweep", action="store_true", help="N = 1: skip the GEMM sweep appended to the line")
    ap.add_argument("--shard-update", type=int, default=None, choices=[0, 1],
                    help="N > 1: split the parameter update over the ranks (reduce-scatter / update / all-gather)")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    if args.workload == "gemm_sweep":
        run_gemm_sweep(args)
    elif args.workload in ("mlp784", "wide_mlp_sgd", "wide_mlp_adam_shard"):
        run_other_config(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
