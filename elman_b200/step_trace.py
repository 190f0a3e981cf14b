"""Per-step phase table of the persistent recurrence kernels, from their own cycle stamps.

With the library option ``rec_trace`` set, CTA 0 of ``rec_tc_kernel`` (E0/E1 dense recurrence) and of
``lowrank_tc_kernel`` (E5) stores ``clock64`` stamps for the first 64 steps of a launch, 16 slots per
step; ``elman_b200_recurrence_trace`` copies them to the host.  This module runs one traced forward
(and backward) launch on seeded inputs and prints the median time between consecutive stamps of the
critical path, the same table the kernel restructurings were steered by.

    python -m elman_b200.step_trace --level 1 --dim 1280 --batch 32
    python -m elman_b200.step_trace --level 5 --dim 1536 --rank 270 --batch 32

It is a diagnostic of this library (the reference has no counterpart); the stamps cost a few percent,
so a traced launch is never a benchmark number.
"""
import argparse
import ctypes
import statistics

import torch

from . import _lib
from . import hasty_pytorch_lib as H

SLOTS = 16
STEPS = 64

# (slot, label) in the order of the critical path of one step.
DENSE_PATH = [(0, "step counter satisfied"), (11, "proxy fence done"), (1, "TMA issued"),
              (2, "state tile landed"), (3, "MMAs issued"), (4, "accumulators complete"),
              (5, "partials scattered to cluster peers"), (6, "all partials landed"),
              (14, "partial sums read"), (7, "new state stored"), (9, "step published")]
LOWRANK_PATH = [(0, "state ready"), (1, "phase-1 MMAs issued"), (2, "rank accumulator complete"),
                (3, "partials sent"), (4, "partials landed"), (5, "summed"),
                (6, "rank vector sent to every CTA"), (7, "rank vector landed"),
                (8, "phase-2 MMAs issued"), (9, "state accumulator complete"),
                (10, "state written")]


def read_trace():
    buf = (ctypes.c_longlong * (STEPS * SLOTS))()
    rc = _lib.load().elman_b200_recurrence_trace(buf, STEPS * SLOTS)
    if rc != 0:
        raise RuntimeError(f"elman_b200_recurrence_trace returned {rc}")
    return [[buf[s * SLOTS + k] for k in range(SLOTS)] for s in range(STEPS)]


def phase_table(trace, path, steps=range(8, 60)):
    """Median cycles between consecutive stamps of `path`, plus the wrap to the next step's first."""
    rows = []
    for (a, la), (b, lb) in zip(path[:-1], path[1:]):
        d = [trace[s][b] - trace[s][a] for s in steps if trace[s][a] and trace[s][b]]
        if d:
            rows.append((f"{la} -> {lb}", statistics.median(d)))
    # the last stamp of the path that this launch wrote (the forward dense kernel has no
    # separate publishing stamp: its finalising warps release the counter themselves)
    first = path[0][0]
    last, last_label = next((k, lb) for k, lb in reversed(path) if trace[steps[0]][k])
    d = [trace[s + 1][first] - trace[s][last] for s in steps]
    rows.append((f"{last_label} -> next step's {path[0][1]}", statistics.median(d)))
    per = statistics.median(trace[s + 1][first] - trace[s][first] for s in steps)
    return per, rows


def print_table(title, per, rows, mhz):
    print(f"{title}: {per:.0f} cycles per step = {per / mhz:.2f} us at {mhz:.0f} MHz")
    for label, cyc in rows:
        print(f"  {label:<64s} {cyc:7.0f} cyc {1e3 * cyc / mhz:6.0f} ns")


def traced(fn):
    _lib.set_option("rec_trace", 1)
    try:
        out = fn()
        torch.cuda.synchronize()
        return out, read_trace()
    finally:
        _lib.set_option("rec_trace", 0)


def main():
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--level", type=int, default=1, choices=[1, 5])
    ap.add_argument("--dim", type=int, default=1280)
    ap.add_argument("--rank", type=int, default=270)
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--time-steps", type=int, default=128)
    ap.add_argument("--sm-mhz", type=float, default=0.0, help="0 = the device's current maximum")
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("step_trace needs a CUDA device")
    mhz = args.sm_mhz or torch.cuda.get_device_properties(0).clock_rate / 1e3
    T, B, d = args.time_steps, args.batch, args.dim
    g = torch.Generator(device="cuda").manual_seed(5)

    def rnd(*shape, scale=1.0):
        return (torch.randn(*shape, device="cuda", generator=g) * scale).bfloat16()

    if args.level == 1:
        x, z, dy = rnd(T, B, d), rnd(T, B, d), rnd(T, B, d)
        h0 = torch.zeros(B, d, device="cuda", dtype=torch.bfloat16)
        W_x, W_h, b = rnd(d, d, scale=d ** -0.5), rnd(d, d, scale=0.5 * d ** -0.5), rnd(d, scale=0.1)
        (h, y, v), tr = traced(lambda: H.mamba_gated_elman_forward(True, x, z, h0, W_x, W_h, b))
        print_table(f"E1 forward  d={d} B={B}", *phase_table(tr, DENSE_PATH), mhz)
        _, tr = traced(lambda: H.mamba_gated_elman_backward(W_x, W_h, x, z, h, v, dy))
        print_table(f"E1 backward d={d} B={B}", *phase_table(tr, DENSE_PATH), mhz)
    else:
        r = args.rank
        x, dy = rnd(T, B, d), rnd(T, B, d)
        h0 = torch.zeros(B, d, device="cuda", dtype=torch.bfloat16)
        s = 0.5 * (d * r) ** -0.25       # U [d, r], V [r, d]; small enough that the state stays bounded
        w = [rnd(d, r, scale=s) if k % 2 == 0 else rnd(r, d, scale=s) for k in range(6)]
        b = rnd(d, scale=0.1)
        (h, out, v), tr = traced(lambda: H.pure_lowrank_elman_forward(True, x, h0, *w, b))
        print_table(f"E5 forward  d={d} r={r} B={B}", *phase_table(tr, LOWRANK_PATH), mhz)
        _, tr = traced(lambda: H.pure_lowrank_elman_backward(*w, x, h, v, dy))
        print_table(f"E5 backward d={d} r={r} B={B}", *phase_table(tr, LOWRANK_PATH), mhz)
    print("device status", _lib.device_status())


if __name__ == "__main__":
    main()
