#!/usr/bin/env python
"""Benchmark of the E1 Elman-cell hot path (forward + BPTT backward).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one forward + backward pass of the E1 cell over one batch of seeded
synthetic input at the benchmark's configs[1]: bf16, d=1280, B=32 sequences per
GPU, T=512 (16 384 tokens per GPU and step).  For N > 1 the launcher starts one
process per GPU (torchrun); the batch is sharded by rank with no data-path
collective (each sequence's recurrence is independent): weak scaling.

Prints ONE JSON line (rank 0).  `value` is whole-job tokens/s with inputs
resident in HBM; `e2e` is the same pass through the public API with pinned host
buffers copied in and results copied out inside the timed region.
`--impl reference` times the reference's own CPU algorithm (the Python time loop
with autograd, restated in oracle/) on the host cores instead.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC = "E1 layer fwd+bwd tokens/s @ d1280 B32 T512"
UNIT = "tokens/s"
T, B, D = 512, 32, 1280
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
# DRAM bytes per launch of the dominant kernel from the committed ncu capture
# (profiles/), or None while no capture of the current kernel exists.
NCU_TRAFFIC_BYTES = {"rec_tc_kernel<fwd>": 170.1e6, "rec_tc_kernel<bwd>": 231.1e6}  # profiles/rec_tc_kernel_e1_c1.md


def host_topology():
    """What the ranks share on the host side: CPUs this process may run on and NUMA nodes visible."""
    import glob
    try:
        cpus = len(os.sched_getaffinity(0))
    except (AttributeError, OSError):
        cpus = os.cpu_count()
    return {"cpus": cpus, "numa_nodes": len(glob.glob("/sys/devices/system/node/node[0-9]*"))}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference_cuda"],
                    help="ours | reference (the reference's CPU path) | reference_cuda (the "
                         "reference's own CUDA kernels rebuilt for sm_100, if oracle/_ref exists)")
    ap.add_argument("--workload", default="cell", choices=["cell", "lm", "e5", "c4"],
                    help="cell = configs[1] (the headline line); lm = configs[2] training step; "
                         "e5 = configs[3] low-rank cell")
    ap.add_argument("--pipeline-chunks", type=int, default=10,
                    help="lm workload, our arm: time chunks of the (layer, time chunk) pipeline "
                         "over CUDA streams; 0 or 1 = layers one after another as the reference")
    ap.add_argument("--pipeline-streams", type=int, default=0, help="0 = from the SM count")
    ap.add_argument("--cuda-graph", type=int, default=-1,
                    help="lm workload, our arm: capture the training step (with the gradient "
                         "all-reduce for N > 1) into a CUDA graph (default); 0 = eager step, "
                         "DistributedDataParallel for N > 1")
    ap.add_argument("--lm-level", type=int, default=1, choices=[0, 1, 5],
                    help="lm workload: ladder level of the layers (configs[2] is level 1)")
    ap.add_argument("--time-steps", type=int, default=0,
                    help="c4 workload: sequence length instead of 2048 (small captures)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-sub-records", action="store_true",
                    help="skip the reference_cuda and lm sub-records of the default line")
    ap.add_argument("--cpu-seconds", type=float, default=12.0,
                    help="CPU work to spend on the cpu_baseline leg (whole passes, at least 2)")
    ap.add_argument("--cpu-sample-steps", type=int, default=0,
                    help="time steps of the workload the CPU baseline runs")
    return ap.parse_args()


def make_inputs(seed: int):
    """configs[1] recipe: x~N(0,1); W_x,W_h~N(0,1/d), W_h rescaled to spectral radius 0.9;
    b=0; z = x W_gx^T with W_gx~N(0,1/(2d)); h0=0; d_output~N(0,1)."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, B, D, generator=g)
    W_x = torch.randn(D, D, generator=g) / math.sqrt(D)
    W_h = torch.randn(D, D, generator=g) / math.sqrt(D)
    rho = float(torch.linalg.eigvals(W_h.double()).abs().max())
    W_h = W_h * (0.9 / rho)
    b = torch.zeros(D)
    W_gx = torch.randn(D, D, generator=g) / math.sqrt(2 * D)
    z = (x.reshape(T * B, D) @ W_gx.T).reshape(T, B, D)
    r = torch.randn(T, B, D, generator=g)
    return {"x": x, "z": z, "h0": torch.zeros(B, D), "W_x": W_x, "W_h": W_h, "b": b, "d_output": r}


def read_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return p, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU while the timed region runs: an
    NVML polling thread (read-only queries, every 20 ms) started before the warm-up, with
    the timed region marked by begin()/end() so only samples taken inside it count.  Falls
    back to an `nvidia-smi -lms` child process when NVML cannot be loaded."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
               0x4: "sw_power_cap"}

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.path = None
        self.thread = None
        self.samples = []      # (time, sm_mhz, reasons bitmask)
        self.windows = []
        self.max_mhz = None
        self._stop = False

    def _nvml_loop(self, nv, handle):
        while not self._stop:
            try:
                mhz = nv.nvmlDeviceGetClockInfo(handle, nv.NVML_CLOCK_SM)
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(handle)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(handle)
                self.samples.append((time.perf_counter(), float(mhz), int(mask)))
            except Exception:
                pass
            time.sleep(0.02)

    def start(self):
        try:
            import pynvml as nv
            import threading
            nv.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(self.gpu).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            handle = nv.nvmlDeviceGetHandleByUUID(uuid)
            self.max_mhz = float(nv.nvmlDeviceGetMaxClockInfo(handle, nv.NVML_CLOCK_SM))
            self.thread = threading.Thread(target=self._nvml_loop, args=(nv, handle), daemon=True)
            self.thread.start()
            return
        except Exception:
            self.thread = None
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.out = open(self.path, "w")
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu), f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=self.out, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def begin(self):
        self._t0 = time.perf_counter()

    def end(self):
        self.windows.append((self._t0, time.perf_counter()))

    def stop(self):
        if self.thread is not None:
            self._stop = True
            self.thread.join(timeout=2)
            inside = [s for s in self.samples if any(a <= s[0] <= b for a, b in self.windows)]
            where = "timed regions"
            if not inside:  # a timed region shorter than one polling interval
                inside, where = self.samples, "warm-up and timed regions"
            reasons = set()
            for _, _, mask in inside:
                for bit, nm in self.REASONS.items():
                    if mask & bit:
                        reasons.add(nm)
            return {"sm_mhz": statistics.median([s[1] for s in inside]) if inside else None,
                    "sm_max_mhz": self.max_mhz, "samples": len(inside), "sampled": where,
                    "source": "nvml", "reasons": sorted(reasons)}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.out.close()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        with open(self.path) as f:
            for line in f:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 9:
                    continue
                try:
                    sm.append(float(parts[1])); mx.append(float(parts[2]))
                except ValueError:
                    continue
                for nm, val in zip(names, parts[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(nm)
        os.unlink(self.path)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "samples": len(sm),
                "sampled": "warm-up and timed regions", "source": "nvidia-smi",
                "reasons": sorted(reasons)}


def cpu_reference_pass(inp, steps):
    """The reference's CPU path for this workload: the Python time loop of its E1 cell
    with autograd for BPTT, fp32, on the first `steps` time steps.  Returns seconds."""
    from oracle import elman_oracle as orc
    sub = {k: (v[:steps].contiguous() if v.dim() == 3 else v) for k, v in inp.items()}
    t0 = time.perf_counter()
    orc.e1_autograd(sub["x"], sub["z"], sub["h0"], sub["W_x"], sub["W_h"], sub["b"],
                    sub["d_output"])
    return time.perf_counter() - t0


def run_reference(args, rank):
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    inp = make_inputs(1234)
    # one step = one pass over the workload; whole T when the run then stays near 90 s of
    # CPU work (about a second per pass on 16 cores), else a prefix of the time steps
    cpu_reference_pass(inp, 32)
    probe = cpu_reference_pass(inp, 128)
    budget = 90.0 / max(1, args.steps + max(1, min(args.warmup, 2)))
    sample = T if probe * (T / 128) <= budget else max(32, int(budget / probe * 128) // 32 * 32)
    sample = min(T, sample)
    for _ in range(max(1, min(args.warmup, 2))):
        cpu_reference_pass(inp, sample)
    times = [cpu_reference_pass(inp, sample) for _ in range(args.steps)]
    sec = sum(times) / len(times)
    value = B * sample / sec
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3 * (T / sample),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": "configs[1]: E1 cell fwd+bwd, d=1280, B=32, T=512 (fp32 on CPU)"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": f"each step is one pass over the first {sample} of {T} time "
                                   "steps, full B and d, fp32, forward + autograd backward; "
                                   "ms_per_step is scaled to T=512"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def measure_reference_cuda_cell(inp, steps, warmup):
    """The reference's unmodified CUDA kernels (cuBLAS GEMM + elementwise kernels per time
    step, rebuilt for sm_100 into oracle/_ref) on the current GPU and the given inputs.
    Returns {"ms_per_step", "value"} or {"unavailable": why}."""
    from oracle import ref_cuda
    if not (torch.cuda.is_available() and ref_cuda.available()):
        return {"unavailable": "oracle/_ref/libelman_ref_cuda.so not built or no GPU"}
    d = {k: v.to(torch.bfloat16).cuda().contiguous() for k, v in inp.items()}
    flush_buf = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")

    def step():
        h, out, v, _ = ref_cuda.e1_forward(True, d["x"], d["z"], d["h0"], d["W_x"], d["W_h"], d["b"])
        return ref_cuda.e1_backward(d["W_x"], d["W_h"], d["x"], d["z"], h, v, d["d_output"])

    for _ in range(max(warmup, 3)):
        step()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(steps):
        flush_buf.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record(); step(); e.record(); e.synchronize()
        total += s.elapsed_time(e)
    return {"ms_per_step": total / steps, "value": B * T * steps / (total / 1e3), "unit": UNIT,
            "steps": steps,
            "what": "reference kernels (elman/cuda/lib, unmodified) compiled for sm_100, same "
                    "inputs, same GPU, L2 flushed between iterations"}


def run_reference_cuda(args, rank, local_rank):
    """Prints the headline JSON line for the reference's own CUDA kernels (impl=reference_cuda)."""
    if rank != 0:
        return
    if torch.cuda.is_available():
        torch.cuda.set_device(local_rank)
    rec = measure_reference_cuda_cell(make_inputs(1234), args.steps, args.warmup)
    if "unavailable" in rec:
        print(json.dumps({"impl": "reference_cuda", "unavailable": rec["unavailable"]}))
        return
    print(json.dumps({
        "impl": "reference_cuda", "metric": METRIC, "value": rec["value"], "unit": UNIT, "n_gpus": 1,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": rec["ms_per_step"],
        "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "configs[1]: E1 cell fwd+bwd, bf16, d=1280, B=32, T=512",
                   "what": rec["what"]}}), flush=True)


class _RefCudaBackend:
    """Routes the E1 extension functions to the reference's own CUDA kernels (oracle/_ref);
    used only by `--workload lm --impl reference_cuda` to time the reference LM step."""

    @staticmethod
    def mamba_gated_elman_forward(training, x, z, h0, W_x, W_h, b):
        from oracle import ref_cuda
        h, out, v, ws = ref_cuda.e1_forward(training, x, z, h0, W_x, W_h, b)
        ws.record_stream(torch.cuda.current_stream())
        return [h, out, v]

    @staticmethod
    def mamba_gated_elman_backward(W_x, W_h, x, z, h, v, d_output):
        from oracle import ref_cuda
        r = ref_cuda.e1_backward(W_x, W_h, x, z, h, v, d_output)
        r[5].record_stream(torch.cuda.current_stream())
        return list(r[:5])


def run_e5(args, rank, world, local_rank):
    """configs[3]: E5 low-rank cell forward + backward, bf16, d=1536, rank 270, B=32, T=512.
    U,V ~ N(0, 1/sqrt(d r)) with U_h V_h rescaled to spectral radius 0.9, x ~ N(0,1).
    `--impl reference_cuda` runs the reference's fused E5 kernels on the same inputs."""
    from elman_b200 import _lib
    from elman_b200 import hasty_pytorch_lib as H
    Td, Bd, d, r = 512, 32, 1536, 270
    torch.cuda.set_device(local_rank)
    g = torch.Generator().manual_seed(1237 + rank)
    s = (d * r) ** -0.25
    mats = {}
    for nm in ("h", "x", "z"):
        mats["U_" + nm] = torch.randn(d, r, generator=g) * s
        mats["V_" + nm] = torch.randn(r, d, generator=g) * s
    rho = float(torch.linalg.eigvals((mats["V_h"] @ mats["U_h"]).double()).abs().max())
    mats["U_h"] *= math.sqrt(0.9 / rho)
    mats["V_h"] *= math.sqrt(0.9 / rho)
    dev = {k: v.to(torch.bfloat16).cuda().contiguous() for k, v in mats.items()}
    x = torch.randn(Td, Bd, d, generator=g).to(torch.bfloat16).cuda()
    dy = torch.randn(Td, Bd, d, generator=g).to(torch.bfloat16).cuda()
    h0 = torch.zeros(Bd, d, dtype=torch.bfloat16, device="cuda")
    b = torch.zeros(d, dtype=torch.bfloat16, device="cuda")
    w = [dev[k] for k in ("U_h", "V_h", "U_x", "V_x", "U_z", "V_z")]
    if args.impl == "reference_cuda":
        from oracle import ref_cuda
        if not ref_cuda.available():
            if rank == 0:
                print(json.dumps({"impl": "reference_cuda", "unavailable": "oracle/_ref not built"}))
            return

        def step():
            h, out, v, _ = ref_cuda.e5_forward(True, x, h0, *w, b)
            return ref_cuda.e5_backward(*w, x, h, v, dy)
    else:
        def step():
            h, out, v = H.pure_lowrank_elman_forward(True, x, h0, *w, b)
            return H.pure_lowrank_elman_backward(*w, x, h, v, dy)
    flush_buf = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    launches0 = _lib.launch_count()
    total = 0.0
    for _ in range(args.steps):
        flush_buf.zero_()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record(); step(); s1.record(); s1.synchronize()
        total += s0.elapsed_time(s1)
    if rank == 0:
        print(json.dumps({
            "impl": args.impl, "metric": "E5 layer fwd+bwd tokens/s @ d1536 r270 B32 T512",
            "value": Bd * Td * args.steps / (total / 1e3), "unit": UNIT, "n_gpus": 1,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": total / args.steps,
            "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "configs[3]: E5 low-rank cell fwd+bwd, bf16, d=1536, r=270, "
                                   "B=32, T=512"},
            "gpu_launches": _lib.launch_count() - launches0,
            "device_status": _lib.device_status()[0]}), flush=True)


def run_c4(args, rank, world, local_rank):
    """configs[4]: E1 forward only (inference), bf16, d=2048, B=256, T=2048: the large-batch
    shape, where the recurrence pipelines several batch groups through each resident tile of
    W_h.  x, z ~ N(0,1)/2, W_x Xavier-scaled, W_h at spectral radius about 0.5.
    `--impl reference_cuda` runs the reference's forward kernels on the same inputs."""
    from elman_b200 import _lib
    from elman_b200 import hasty_pytorch_lib as H
    Td, Bd, d = (args.time_steps if args.time_steps > 0 else 2048), 256, 2048
    torch.cuda.set_device(local_rank)
    g = torch.Generator().manual_seed(1239 + rank)
    x = torch.empty(Td, Bd, d, dtype=torch.bfloat16, device="cuda")
    z = torch.empty(Td, Bd, d, dtype=torch.bfloat16, device="cuda")
    for t0 in range(0, Td, 256):  # generated in slices: the fp32 host copy stays small
        n = min(256, Td - t0)
        x[t0:t0 + n] = (torch.randn(n, Bd, d, generator=g) * 0.5).to(torch.bfloat16).cuda()
        z[t0:t0 + n] = (torch.randn(n, Bd, d, generator=g) * 0.5).to(torch.bfloat16).cuda()
    W_x = (torch.randn(d, d, generator=g) / math.sqrt(d)).to(torch.bfloat16).cuda()
    W_h = (torch.randn(d, d, generator=g) * 0.5 / math.sqrt(d)).to(torch.bfloat16).cuda()
    b = torch.zeros(d, dtype=torch.bfloat16, device="cuda")
    h0 = torch.zeros(Bd, d, dtype=torch.bfloat16, device="cuda")
    if args.impl == "reference_cuda":
        from oracle import ref_cuda
        if not ref_cuda.available():
            if rank == 0:
                print(json.dumps({"impl": "reference_cuda", "unavailable": "oracle/_ref not built"}))
            return

        def step():
            return ref_cuda.e1_forward(False, x, z, h0, W_x, W_h, b)
    else:
        def step():
            return H.mamba_gated_elman_forward(False, x, z, h0, W_x, W_h, b)
    for _ in range(max(args.warmup, 3)):
        out = step()
    torch.cuda.synchronize()
    del out
    launches0 = _lib.launch_count()
    total = 0.0
    for _ in range(args.steps):  # 4.3 GB of inputs per pass: far beyond L2, no flush needed
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record(); out = step(); s1.record(); s1.synchronize()
        del out
        total += s0.elapsed_time(s1)
    if rank == 0:
        print(json.dumps({
            "impl": args.impl, "metric": "E1 forward tokens/s @ d2048 B256 T2048",
            "value": Bd * Td * args.steps / (total / 1e3), "unit": UNIT, "n_gpus": 1,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": total / args.steps,
            "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "configs[4]: E1 cell forward (inference), bf16, d=2048, B=256, "
                                   f"T={Td}; inputs larger than L2"},
            "gpu_launches": _lib.launch_count() - launches0,
            "device_status": _lib.device_status()[0]}), flush=True)


def measure_lm(args, rank, world, local_rank, impl, steps, warmup):
    """configs[2]: full E1 byte-level LM (d=1280 x 6 layers, 49.5M parameters), bf16, AdamW,
    T=512, 32 sequences per GPU, seeded Zipf(1.1) token ids; one step = forward, loss,
    backward, gradient all-reduce (N > 1), gradient clipping, optimizer step.  Every step's
    tokens come from pinned host memory and the loss is read back at the end of the timed
    region.  The process group, if any, must exist already.  Returns the record (rank 0) or
    None; the step graph is released before returning."""
    import torch.distributed as dist
    from elman_b200 import _lib
    from elman_b200 import ladder_lm, mamba_gated_elman

    dev = torch.device("cuda", local_rank)
    saved_backend = mamba_gated_elman.hasty_pytorch_lib
    if impl == "reference_cuda":
        from oracle import ref_cuda
        if not ref_cuda.available():
            return {"unavailable": "oracle/_ref not built"} if rank == 0 else None
        mamba_gated_elman.hasty_pytorch_lib = _RefCudaBackend
    try:
        torch.manual_seed(1234)
        chunks = args.pipeline_chunks if impl == "ours" else 0
        model = ladder_lm.LadderLM(vocab_size=256, dim=D, depth=6, level=args.lm_level,
                                   expansion=1.0, pipeline_chunks=chunks,
                                   pipeline_streams=args.pipeline_streams,
                                   fused_ops=(impl == "ours"))
        if impl != "ours":   # the reference arm: framework ops around the reference's kernels
            for layer in model.layers:
                layer.fused = False
        model = model.to(dev).bfloat16()
        net = model
        graphed = impl == "ours" and args.cuda_graph != 0
        if world > 1 and not graphed:
            net = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local_rank],
                                                            find_unused_parameters=False)
        host_tokens = ladder_lm.zipf_tokens(B, T + 1, seed=1234 + rank).pin_memory()
        gstep = None
        reducer = None
        if graphed:
            # gradients, parameters and optimizer state in flat buffers: one memset, one
            # all-reduce per layer while backward runs (N > 1), one AdamW launch with the
            # clipping factor folded in; the whole step captured into a CUDA graph
            from elman_b200 import train_step
            reducer = train_step.make_gradient_reducer(model)
            opt = train_step.FlatAdamW(reducer, lr=3e-4, betas=(0.9, 0.95), eps=1e-8,
                                       weight_decay=0.1)
            if world > 1:  # same initial weights on every rank
                dist.broadcast(reducer.flat_params, src=0)
            gstep = train_step.GraphedTrainStep(net, opt, host_tokens.to(dev), max_grad_norm=1.0,
                                                autocast_dtype=torch.bfloat16, reducer=reducer)
        else:
            opt = torch.optim.AdamW(model.parameters(), lr=3e-4, betas=(0.9, 0.95),
                                    weight_decay=0.1)

        def step():
            if graphed:
                return gstep(host_tokens)
            tok = host_tokens.to(dev, non_blocking=True)
            opt.zero_grad(set_to_none=True)
            with torch.autocast(device_type="cuda", dtype=torch.bfloat16):
                loss = net(tok, return_loss=True)
            loss.backward()
            torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
            opt.step()
            return loss

        def barrier():
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()

        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        for _ in range(max(warmup, 3)):
            step()
        barrier()
        launches0 = _lib.launch_count()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sampler.begin()
        ev0.record()
        for _ in range(steps):
            loss = step()
        ev1.record()
        loss_val = float(loss.detach())  # device -> host read of the step's result
        barrier()
        sampler.end()
        clocks = sampler.stop() if rank == 0 else None
        status = _lib.device_status()[0]
        ms = ev0.elapsed_time(ev1)
        t_all = torch.tensor([ms], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t_all, op=dist.ReduceOp.MAX)
        ms = float(t_all.cpu())
        rec = None
        if rank == 0:
            rec = {
                "impl": impl,
                "metric": f"E{args.lm_level} d1280x6 LM training tokens/s (B32 x T512 per GPU)",
                "value": B * T * world * steps / (ms / 1e3), "unit": UNIT, "n_gpus": world,
                "steps": steps, "warmup": max(warmup, 3), "ms_per_step": ms / steps,
                "higher_is_better": True, "scaling": "weak", "dtype": "bf16", "data": "synthetic",
                "config": {"workload": f"configs[2]: LadderLM level {args.lm_level}, d=1280, depth 6, "
                                       "AdamW, Zipf(1.1) tokens from pinned host memory each step, "
                                       "data parallel",
                           "params": model.get_num_params(),
                           "pipeline_chunks": chunks, "cuda_graph": bool(graphed)},
                "allreduce": (None if world == 1 else
                              (reducer.describe() if reducer is not None else
                               "DistributedDataParallel over NCCL")),
                "final_loss": loss_val, "clocks": clocks, "device_status": status,
                "gpu_launches": (gstep.library_launches_per_step * steps if graphed
                                 else _lib.launch_count() - launches0)}
        if graphed:
            # NCCL cannot tear a communicator down while a CUDA graph that captured its
            # kernels is alive: release the graph before anybody destroys the group
            gstep.graph = None
            gstep = None
        del model, net, opt
        import gc
        gc.collect()
        torch.cuda.synchronize()
        return rec
    finally:
        mamba_gated_elman.hasty_pytorch_lib = saved_backend


def init_process_group(world, local_rank):
    import torch.distributed as dist
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("TORCH_NCCL_ASYNC_ERROR_HANDLING", "0")  # required to capture NCCL
        dist.init_process_group(backend="nccl", device_id=torch.device("cuda", local_rank))


def run_lm(args, rank, world, local_rank):
    import torch.distributed as dist
    torch.cuda.set_device(local_rank)
    init_process_group(world, local_rank)
    rec = measure_lm(args, rank, world, local_rank, args.impl, args.steps, args.warmup)
    if rank == 0:
        print(json.dumps(rec), flush=True)
    if world > 1:
        torch.cuda.synchronize()
        dist.barrier()
        _destroy_process_group_bounded(20.0)


def _destroy_process_group_bounded(seconds):
    """destroy_process_group in a helper thread; if it has not returned in time the process
    exits directly (all results are printed by then)."""
    import threading
    import torch.distributed as dist
    t = threading.Thread(target=dist.destroy_process_group, daemon=True)
    t.start()
    t.join(seconds)
    if t.is_alive():
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def main():
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.workload == "lm":
        run_lm(args, rank, world, local_rank)
        return
    if args.workload == "e5":
        run_e5(args, rank, world, local_rank)
        return
    if args.workload == "c4":
        if rank == 0:
            run_c4(args, rank, world, local_rank)
        return
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if args.impl == "reference_cuda":
        run_reference_cuda(args, rank, local_rank)
        return

    import torch.distributed as dist
    from elman_b200 import _lib
    from elman_b200 import hasty_pytorch_lib as H

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    init_process_group(world, local_rank)

    inp = make_inputs(1234 + rank)
    host = {k: v.to(torch.bfloat16).contiguous().pin_memory() for k, v in inp.items()}
    d = {k: v.to(dev, non_blocking=True) for k, v in host.items()}
    torch.cuda.synchronize()
    flush_buf = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)

    def step_device():
        h, out, v = H.mamba_gated_elman_forward(True, d["x"], d["z"], d["h0"], d["W_x"],
                                                d["W_h"], d["b"])
        return H.mamba_gated_elman_backward(d["W_x"], d["W_h"], d["x"], d["z"], h, v,
                                            d["d_output"]), out

    out_host = {k: torch.empty_like(host["x"]).pin_memory() for k in ("y", "dx", "dz")}
    dw_host = {k: torch.empty(D, D, dtype=torch.bfloat16).pin_memory() for k in ("dW_x", "dW_h")}

    def step_e2e():
        x = host["x"].to(dev, non_blocking=True)
        z = host["z"].to(dev, non_blocking=True)
        r = host["d_output"].to(dev, non_blocking=True)
        h, out, v = H.mamba_gated_elman_forward(True, x, z, d["h0"], d["W_x"], d["W_h"], d["b"])
        dx, dz, dWx, dWh, db = H.mamba_gated_elman_backward(d["W_x"], d["W_h"], x, z, h, v, r)
        out_host["y"].copy_(out, non_blocking=True)
        out_host["dx"].copy_(dx, non_blocking=True)
        out_host["dz"].copy_(dz, non_blocking=True)
        dw_host["dW_x"].copy_(dWx, non_blocking=True)
        dw_host["dW_h"].copy_(dWh, non_blocking=True)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, phases=False):
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
              for _ in range(steps)]
        phase_ms = [[], [], [], []]
        barrier()
        wall0 = time.perf_counter()
        for s, e in ev:
            flush_buf.zero_()          # evict L2 between timed iterations (not timed)
            s.record()
            fn()
            e.record()
            if phases:
                e.synchronize()
                for ph in range(4):
                    phase_ms[ph].append(_lib.last_timing_ms(ph))
        barrier()
        wall = time.perf_counter() - wall0
        total_ms = sum(s.elapsed_time(e) for s, e in ev)
        return total_ms, wall, phase_ms

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(max(args.warmup, 3)):
        step_device()
    torch.cuda.synchronize()
    if _lib.device_status()[0] != 0:
        raise SystemExit("a device-side wait timed out during warm-up: " + str(_lib.device_status()))

    _lib.set_option("time_kernels", 1)
    launches0, tc0 = _lib.launch_count(), _lib.tc_launch_count()
    sampler.begin()
    total_ms, wall, phase_ms = timed(step_device, args.steps, phases=True)
    sampler.end()
    launches = _lib.launch_count() - launches0
    tc_launches = _lib.tc_launch_count() - tc0
    _lib.set_option("time_kernels", 0)

    for _ in range(3):
        step_e2e()
    torch.cuda.synchronize()
    sampler.begin()
    e2e_serial_ms, _, _ = timed(step_e2e, args.steps)
    sampler.end()

    # The same calls through the package's host-buffer front end: uploads, kernels and
    # downloads of consecutive steps overlap on three streams.  Every step still moves its
    # own inputs up and its own results down inside the timed region.
    from elman_b200.host_io import E1HostPipeline
    pipe = E1HostPipeline(T, B, D, d["W_x"], d["W_h"], d["b"], d["h0"], device=dev)
    pipe.pre_compute = flush_buf.zero_      # L2 eviction before each step's kernels (timed)
    for _ in range(3):
        pipe.submit(host["x"], host["z"], host["d_output"])
    pipe.wait()
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler.begin()
    ev0.record()
    for _ in range(args.steps):
        res = pipe.submit(host["x"], host["z"], host["d_output"])
    pipe.wait()
    ev1.record()
    barrier()
    sampler.end()
    e2e_ms = ev0.elapsed_time(ev1)
    clocks = sampler.stop() if rank == 0 else None
    if _lib.device_status()[0] != 0:
        raise SystemExit("a device-side wait timed out: " + str(_lib.device_status()))

    # every rank's own end-to-end time: the host's PCIe / memory system is shared by the ranks
    e2e_each = torch.zeros(world, dtype=torch.float64, device=dev)
    e2e_each[rank] = e2e_ms
    t_all = torch.tensor([total_ms, e2e_ms, e2e_serial_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(e2e_each, op=dist.ReduceOp.SUM)
        dist.all_reduce(t_all, op=dist.ReduceOp.MAX)
    e2e_each = [float(v) / args.steps for v in e2e_each.cpu()]
    total_ms, e2e_ms, e2e_serial_ms = (float(v) for v in t_all.cpu())

    # Beside the headline, outside its timed region (as the CPU baseline is): the same cell
    # through the reference's own CUDA kernels on this GPU (rank 0), and the configs[2] LM
    # training step on all N ranks, with its gradient all-reduce — the workload that has a
    # collective — plus, at N = 1, the same LM step through the reference's kernels.
    del pipe, res
    sub = {}
    if not args.no_sub_records:
        if rank == 0:
            sub["reference_cuda"] = measure_reference_cuda_cell(inp, min(args.steps, 10), 3)
        lm_steps = max(5, min(args.steps, 20))
        lm = measure_lm(args, rank, world, local_rank, "ours", lm_steps, 3)
        if rank == 0 and lm is not None:
            keep = ("ms_per_step", "value", "unit", "n_gpus", "steps", "allreduce", "clocks",
                    "final_loss", "gpu_launches", "device_status", "config")
            sub["lm"] = {k: lm[k] for k in keep if k in lm}
            if world == 1:
                ref_lm = measure_lm(args, rank, world, local_rank, "reference_cuda", 5, 3)
                sub["lm"]["reference_cuda_ms_per_step"] = (
                    ref_lm.get("ms_per_step") if ref_lm else None)
                if ref_lm and "unavailable" in ref_lm:
                    sub["lm"]["reference_cuda_unavailable"] = ref_lm["unavailable"]

    if rank == 0:
        tokens = B * T * world * args.steps
        value = tokens / (total_ms / 1e3)
        e2e_value = tokens / (e2e_ms / 1e3)
        peaks, peaks_kind = read_peaks()
        mean = lambda xs: sum(xs) / max(len(xs), 1)
        rec_fwd_ms, rec_bwd_ms, proj_ms, bgemm_ms = (mean(p) for p in phase_ms)
        dom = "fwd" if rec_fwd_ms >= rec_bwd_ms else "bwd"
        dom_ms = max(rec_fwd_ms, rec_bwd_ms)
        rec_flops = 2.0 * T * B * D * D               # per launch of either recurrence kernel
        # algorithmic HBM bytes per launch: forward reads pre, z and writes h, v, y;
        # backward reads h, v, z, dy and writes dv, dz
        rec_bytes = (6.0 if dom == "bwd" else 5.0) * B * D * 2 * T
        achieved_tf = rec_flops / (dom_ms / 1e3) / 1e12 if dom_ms > 0 else 0.0
        peak_tf = float(peaks.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"]))
        roofline = {
            "kernel": f"rec_tc_kernel<{dom}>", "bound": "tensor",
            "achieved": achieved_tf, "peak": peak_tf, "unit": "TFLOP/s",
            "frac": achieved_tf / peak_tf if peak_tf else None,
            "traffic": NCU_TRAFFIC_BYTES.get(f"rec_tc_kernel<{dom}>"),
            "peak_source": f"{peaks_kind} (bf16_tflops burst; sustained "
                           f"{peaks.get('bf16_tflops_sustained')})",
            "note": "per-step recurrence at B=32 is latency-bound (grid-wide dependency every "
                    "step); us_per_step is the figure of merit",
            "hbm_view": {"achieved_gbs": rec_bytes / (dom_ms / 1e3) / 1e9 if dom_ms > 0 else 0.0,
                         "peak_gbs": peaks.get("hbm_gbs")},
        }
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": total_ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": "configs[1]: E1 cell fwd+bwd, bf16, d=1280, B=32 per GPU, T=512",
                       "tokens_per_step_per_gpu": B * T, "sharding": "batch (no collective)",
                       "l2": "256 MiB buffer written between timed iterations",
                       "seed": "1234+rank"},
            "e2e": {"value": e2e_value, "unit": UNIT,
                    "h2d_bytes_per_step": 3 * T * B * D * 2,
                    "d2h_bytes_per_step": 3 * T * B * D * 2 + 2 * D * D * 2 + D * 2,
                    "ms_per_step": e2e_ms / args.steps,
                    "per_rank": {
                        "ms_per_step": e2e_each,
                        "h2d_gbs": [3 * T * B * D * 2 / (ms * 1e6) for ms in e2e_each],
                        "d2h_gbs": [(3 * T * B * D * 2 + 2 * D * D * 2 + D * 2) / (ms * 1e6)
                                    for ms in e2e_each],
                        "host": host_topology()},
                    "how": "E1HostPipeline: pinned host buffers in and out every step; upload, "
                           "kernels and download of consecutive steps overlap on 3 streams",
                    "one_call_at_a_time": {"value": tokens / (e2e_serial_ms / 1e3),
                                           "ms_per_step": e2e_serial_ms / args.steps}},
            "gpu_launches": launches, "tensor_core_launches": tc_launches,
            "clocks": clocks, "roofline": roofline,
            "phases_ms": {"recurrence_fwd": rec_fwd_ms, "recurrence_bwd": rec_bwd_ms,
                          "projection_fwd": proj_ms, "gemms_bwd": bgemm_ms,
                          "recurrence_fwd_us_per_step": rec_fwd_ms * 1e3 / T,
                          "recurrence_bwd_us_per_step": rec_bwd_ms * 1e3 / T},
            # tensor-core view of the time-parallel phases and of the whole call (algorithmic
            # flops: one 2*T*B*d^2 GEMM forward, three backward, 12*T*B*d^2 per call)
            "tensor_view": {
                "projection_fwd_tflops": rec_flops / (proj_ms / 1e3) / 1e12 if proj_ms > 0 else None,
                "gemms_bwd_tflops": 3 * rec_flops / (bgemm_ms / 1e3) / 1e12 if bgemm_ms > 0 else None,
                "whole_call_tflops": 6 * rec_flops / (total_ms / args.steps / 1e3) / 1e12,
                "projection_fwd_frac": rec_flops / (proj_ms / 1e3) / 1e12 / peak_tf if proj_ms > 0 else None,
                "gemms_bwd_frac": 3 * rec_flops / (bgemm_ms / 1e3) / 1e12 / peak_tf if bgemm_ms > 0 else None,
                "whole_call_frac": 6 * rec_flops / (total_ms / args.steps / 1e3) / 1e12 / peak_tf,
                "peak_tflops": peak_tf},
            "wall_s_timed_region": wall,
        }
        line.update(sub)
        if world == 1 and not args.no_cpu_baseline:
            cores = os.cpu_count() or 1
            torch.set_num_threads(cores)
            fp32 = {k: v.float() for k, v in host.items()}
            cpu_reference_pass(fp32, 8)
            n_t = T if args.cpu_sample_steps <= 0 else min(T, args.cpu_sample_steps)
            passes, spent = 0, 0.0
            while passes < 2 or (spent < args.cpu_seconds and passes < 64):
                spent += cpu_reference_pass(fp32, n_t)
                passes += 1
            line["cpu_baseline"] = {
                "value": B * n_t * passes / spent, "unit": UNIT, "cores": cores,
                "kind": "port",
                "sample": f"{passes} passes over the first {n_t} of {T} time steps, full B and d, "
                          f"fp32, forward + autograd backward ({spent:.1f} s of CPU work)"}
        else:
            line["cpu_baseline"] = None
        print(json.dumps(line), flush=True)

    if world > 1:
        torch.cuda.synchronize()
        dist.barrier()
        _destroy_process_group_bounded(20.0)


if __name__ == "__main__":
    main()
