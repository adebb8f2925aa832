"""Headline benchmark: forward + backward of the sparse attention operator on the reference's
window configuration, reported as effective TFLOP/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (N = 1): batch 2, seqlen 4096, 32 query / 8 KV heads, head_dim 128, bf16, causal with a
1024-token left window on every head (window_sizes = [[0, 1024, 0, 0]] * 8), softmax_threshold 1.0,
is_split_kv = is_split_qo = True. Q/K/V/dO are iid N(0, 1) from a fixed seed (synthetic). One step =
one forward and one backward through the public operator (``flash_sparse_attn_func`` + autograd).
With N > 1 every rank runs its own copy of that batch (independent (batch, head) slices, no
collective in the data path): weak scaling, value = sum over ranks / max time over ranks.

metric  fwd_bwd_effective_tflops = dense-causal-equivalent FLOPs of the step (4*D*B*Hq*S(S+1)/2 for the
        forward, 2.5x that for the backward) / device time of the step.
e2e     the same with HOST buffers: pinned Q/K/V/dO copied in, out/dQ/dK/dV copied back, every step.
roofline the backward main kernel (the dominant one): executed FLOPs at 128x128 tile granularity /
        its CUDA-event duration inside the timed steps, against the measured dense bf16 peak.
cpu_baseline  the CPU oracle (eager fp32 forward + autograd backward) on a bounded number of
        (batch, head) slices of the same workload, scaled to the same metric.

``--impl reference`` prints the CPU arm alone on the same metric / config.
"""

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for p in (os.path.join(ROOT, "flash-sparse-attention_b200"), ROOT):
    if p not in sys.path:
        sys.path.insert(0, p)

import torch  # noqa: E402

B, S, HQ, HKV, D = 2, 4096, 32, 8, 128
WINDOW = 1024
THRESHOLD = 1.0
METRIC = "fwd_bwd_effective_tflops"
UNIT = "TFLOP/s"


def effective_flops(batch=B, heads=HQ):
    fwd = 4.0 * D * batch * heads * S * (S + 1) / 2
    return 3.5 * fwd


def executed_pairs_tile_granular():
    """(query, key) pairs inside visited 128x128 tiles, per (batch, head): with a causal band of WINDOW keys,
    query tile m visits its diagonal tile and the min(m, WINDOW / 128) tiles before it (a tile WINDOW / 128 + 1
    back has no pair with q - k < WINDOW)."""
    return sum(min(mb, WINDOW // 128) + 1 for mb in range(S // 128)) * 128 * 128


def config_dict(n_gpus):
    return {
        "workload": "C2 sparse causal local-window attention fwd+bwd",
        "batch_per_gpu": B, "seqlen": S, "heads_q": HQ, "heads_kv": HKV, "head_dim": D,
        "window_sizes": [0, WINDOW, 0, 0], "softmax_threshold": THRESHOLD, "is_split_kv": True,
        "is_split_qo": True, "global_batch": B * n_gpus, "parallelism": f"dp{n_gpus} (independent batch slices)",
        "l2": "inputs (168 MB) and working set (>450 MB) exceed the 126 MB L2; no flush needed",
    }


# --------------------------------------------------------------------------------------------------
# CPU arm (oracle): eager fp32 forward + autograd backward on (batch, head) slices
# --------------------------------------------------------------------------------------------------
def cpu_slice_step(seed):
    from oracle import eager

    g = torch.Generator().manual_seed(seed)
    q = torch.randn(1, S, 1, D, generator=g).to(torch.bfloat16)
    k = torch.randn(1, S, 1, D, generator=g).to(torch.bfloat16)
    v = torch.randn(1, S, 1, D, generator=g).to(torch.bfloat16)
    do = torch.randn(1, S, 1, D, generator=g).to(torch.bfloat16)
    ws = torch.tensor([[0, WINDOW, 0, 0]], dtype=torch.int32)
    t0 = time.perf_counter()
    eager.backward(q, k, v, do, None, True, is_local=True, window_sizes=ws)  # forward + backward
    return time.perf_counter() - t0


def cpu_baseline(budget_s=20.0):
    cores = torch.get_num_threads()
    cpu_slice_step(0)  # warm-up
    times = []
    t_start = time.perf_counter()
    while len(times) < 2 or (time.perf_counter() - t_start < budget_s and len(times) < 16):
        times.append(cpu_slice_step(len(times) + 1))
    per_slice = sorted(times)[len(times) // 2]
    value = effective_flops(1, 1) / per_slice / 1e12
    return {"value": value, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"{len(times)} (batch, head) slices of the same workload (S={S}, D={D}, window {WINDOW}), "
                      f"eager fp32 forward + autograd backward; median {per_slice:.2f} s per slice"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    cores = torch.get_num_threads()
    total = max(1, args.steps + args.warmup)
    probe = cpu_slice_step(0)
    slices = max(1, min(8, int(150.0 / total / max(probe, 1e-3))))
    for i in range(args.warmup):
        for j in range(slices):
            cpu_slice_step(100 + i * slices + j)
    t0 = time.perf_counter()
    for i in range(args.steps):
        for j in range(slices):
            cpu_slice_step(1000 + i * slices + j)
    dt = time.perf_counter() - t0
    ms = dt / max(args.steps, 1) * 1e3
    value = effective_flops(1, 1) * slices / (ms / 1e3) / 1e12
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": config_dict(args.gpus),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": f"each step = {slices} (batch, head) slice(s) of the workload through the CPU "
                                   "oracle (eager fp32 forward + autograd backward)"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# --------------------------------------------------------------------------------------------------
# clocks
# --------------------------------------------------------------------------------------------------
class ClockSampler(threading.Thread):
    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._stop_evt = threading.Event()
        self.ok = False
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.ok = False

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop_evt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.05)

    def stop(self):
        self._stop_evt.set()

    def summary(self):
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


# --------------------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------------------
def traffic_from_profile():
    """DRAM bytes per launch of the backward main kernel, from the committed ncu summary (or None)."""
    path = os.path.join(ROOT, "profiles", "bwd_kernel_c2.txt")
    try:
        for line in open(path):
            if line.startswith("traffic_bytes_per_launch:"):
                return float(line.split(":")[1].strip())
    except OSError:
        pass
    return None


def run_gpu(args):
    import torch.distributed as dist

    import flash_sparse_attn as fsa
    from flash_sparse_attn import _lib

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    _lib.load()  # fail loudly if the CUDA library is missing

    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    mk = lambda *shape: torch.randn(*shape, generator=g, device=dev, dtype=torch.bfloat16)  # noqa: E731
    q, k, v, do = mk(B, S, HQ, D), mk(B, S, HKV, D), mk(B, S, HKV, D), mk(B, S, HQ, D)
    ws = torch.tensor([[0, WINDOW, 0, 0]] * HKV, dtype=torch.int32, device=dev)

    def step(qq, kk, vv, dd):
        qq.grad = kk.grad = vv.grad = None
        out = fsa.flash_sparse_attn_func(qq, kk, vv, is_causal=True, window_sizes=ws, softmax_threshold=THRESHOLD,
                                         is_split_kv=True, is_split_qo=True)
        out.backward(dd)
        return out

    qg, kg, vg = (t.requires_grad_(True) for t in (q, k, v))

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident throughput ("value") + per-kernel events for the roofline ----------------
    for _ in range(max(args.warmup, 3)):
        step(qg, kg, vg, do)
    n_ev = args.steps
    ev_b = [torch.cuda.Event(enable_timing=True) for _ in range(n_ev)]
    ev_a = [torch.cuda.Event(enable_timing=True) for _ in range(n_ev)]
    for e in ev_b + ev_a:
        e.record()  # creates the handles
    sampler = ClockSampler(local_rank)
    barrier()
    sampler.start()
    t_start, t_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_start.record()
    for i in range(args.steps):
        qg.grad = kg.grad = vg.grad = None
        out = fsa.flash_sparse_attn_func(qg, kg, vg, is_causal=True, window_sizes=ws, softmax_threshold=THRESHOLD,
                                         is_split_kv=True, is_split_qo=True)
        _lib.set_profile_events(ev_b[i], ev_a[i])  # around the backward main kernel of this step
        out.backward(do)
        _lib.set_profile_events(None, None)
    t_stop.record()
    barrier()
    sampler.stop()
    fsa.check_status()
    ms_total = t_start.elapsed_time(t_stop)
    kern_ms = sorted(b.elapsed_time(a) for b, a in zip(ev_b, ev_a))
    kern_ms_avg = sum(kern_ms) / len(kern_ms)

    # ---- end to end with host buffers --------------------------------------------------------------
    # Every step copies its inputs from pinned host memory and its results back, as the contract asks. The three
    # phases of consecutive steps overlap the way a host-side caller with a prefetching loader runs them: inputs of
    # step i + 1 travel on a copy-in stream and results of step i - 1 on a copy-out stream while the kernels of
    # step i run (two sets of device and host buffers); PCIe is full duplex, so a step costs max(in, out, kernels).
    hq, hk, hv, hdo = (t.detach().cpu().pin_memory() for t in (q, k, v, do))
    host_out = [tuple(torch.empty_like(t).pin_memory() for t in (hq, hq, hk, hv)) for _ in range(2)]
    dev_in = [tuple(torch.empty_like(t) for t in (q, k, v, do)) for _ in range(2)]
    s_cur, s_in, s_out = torch.cuda.current_stream(), torch.cuda.Stream(), torch.cuda.Stream()
    ev_in = [torch.cuda.Event() for _ in range(2)]    # inputs of the slot have landed
    ev_comp = [torch.cuda.Event() for _ in range(2)]  # kernels of the slot are done (inputs free, results ready)
    ev_out = [torch.cuda.Event() for _ in range(2)]   # results of the slot have reached the host
    results = [None, None]

    def copy_in(i):
        b = i & 1
        with torch.cuda.stream(s_in):
            if i >= 2:
                s_in.wait_event(ev_comp[b])  # step i - 2 has finished reading this slot
            for d, h in zip(dev_in[b], (hq, hk, hv, hdo)):
                d.copy_(h, non_blocking=True)
            ev_in[b].record(s_in)

    def compute(i):
        b = i & 1
        s_cur.wait_event(ev_in[b])
        a, b_, c = (t.detach().requires_grad_(True) for t in dev_in[b][:3])
        out = step(a, b_, c, dev_in[b][3])
        results[b] = (out.detach(), a.grad, b_.grad, c.grad)
        ev_comp[b].record(s_cur)

    def copy_out(i):
        b = i & 1
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_comp[b])  # the host slot was last written by step i - 2 on this same stream
            for h, d in zip(host_out[b], results[b]):
                d.record_stream(s_out)
                h.copy_(d, non_blocking=True)
            ev_out[b].record(s_out)

    def e2e_run(n):
        copy_in(0)
        for i in range(n):
            if i + 1 < n:
                copy_in(i + 1)
            compute(i)
            copy_out(i)
        s_cur.wait_stream(s_out)
        s_cur.wait_stream(s_in)

    e2e_run(3)
    torch.cuda.synchronize()
    barrier()
    e_steps = max(3, min(args.steps, 10))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    e2e_run(e_steps)
    e1.record()
    barrier()
    fsa.check_status()
    e2e_ms = e0.elapsed_time(e1) / e_steps
    torch.cuda.synchronize()
    if not torch.equal(host_out[(e_steps - 1) & 1][0], out.detach().cpu()):  # same inputs, same forward bits
        raise RuntimeError("end-to-end leg: the output that reached the host differs from the device-resident run")

    # ---- reduce over ranks: max time ------------------------------------------------------------------
    times = torch.tensor([ms_total, e2e_ms, kern_ms_avg], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_total, e2e_ms, kern_ms_avg = times.tolist()
    ms_per_step = ms_total / args.steps
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    flops_step = effective_flops() * world
    value = flops_step / (ms_per_step / 1e3) / 1e12
    e2e_value = flops_step / (e2e_ms / 1e3) / 1e12
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        pass
    peak = peaks.get("bf16_tflops_sustained") or 1590.0 * 0.88
    peak_src = "measured (sustained cuBLAS bf16, MEASURED_PEAKS.json)" if peaks else "fallback"
    exec_flops_bwd = 2.5 * 4.0 * D * executed_pairs_tile_granular() * B * HQ
    achieved = exec_flops_bwd / (kern_ms_avg / 1e3) / 1e12
    h2d = sum(t.numel() * t.element_size() for t in (hq, hk, hv, hdo))
    d2h = sum(t.numel() * t.element_size() for t in host_out[0])
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "config": config_dict(world),
        "clocks": sampler.summary(),
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_ms,
                "overlap": "copy-in of step i+1 and copy-out of step i-1 run on their own streams beside the kernels of step i"},
        "gpu_launches": 4 * args.steps,
        "roofline": {"bound": "tensor", "kernel": "bwd_kernel<128, bf16, sparse>", "achieved": achieved, "peak": peak,
                     "unit": "TFLOP/s", "frac": achieved / peak, "traffic": traffic_from_profile(),
                     "peak_source": peak_src, "kernel_ms": kern_ms_avg,
                     "flops_per_launch": exec_flops_bwd,
                     "note": "executed FLOPs = 2.5 * 4*D*(pairs in visited 128x128 tiles); of measured peak"},
    }
    if world == 1 and not args.no_cpu:
        torch.set_num_threads(max(1, os.cpu_count() or 1))
        line["cpu_baseline"] = cpu_baseline()
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg (profiling runs)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
