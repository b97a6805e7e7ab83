"""Benchmark of the GL-SDM memory operator on B200: memory-op tokens/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c4] [--impl ours|reference]

A step is one pass of the operator over one batch of synthetic input of the chosen
configuration (default c4: 16,777,216-slot bf16 bank, d_v 256, top-32, 64 x 8192 tokens =
16 commit epochs of 32,768 tokens): per epoch a query route+read, a write route + prediction
read + delta proposal, and the buffered commit. Rank 0 prints one JSON line.

  value         device-resident throughput (inputs already in HBM), CUDA events, max over ranks
  e2e           the same work through the public operator with pinned HOST inputs: per epoch
                the factor scores / targets / gates are copied host->device and the readings
                device->host inside the timed region
  roofline      the dominant kernel's algorithmic bytes / its measured duration vs the measured
                HBM copy peak (MEASURED_PEAKS.json)
  cpu_baseline  the PyTorch CPU port of the reference path (oracle/torch_port.py) timed on this
                machine's cores on a bounded token sample of the same workload
--impl reference times that CPU port alone (the reference's own CPU path cannot travel to the
GPU machine; the port is pinned to its outputs by tests/test_oracle_golden.py).
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

FALLBACK_HBM_GBS = 6650.0
NOMINAL_HBM_GBS = 8000.0


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            data = json.load(f)
        return float(data["hbm_gbs"]), "measured"
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index):
        self.rows, self.proc, self.index = [], None, device_index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._drain, daemon=True).start()
        except OSError:
            self.proc = None

    def _drain(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        clocks, maxes, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                clocks.append(float(r[1])), maxes.append(float(r[2]))
            except (ValueError, IndexError):
                continue
            for name, cell in zip(names, r[5:9]):
                if cell.lower().startswith("active"):
                    reasons.add(name)
        if not clocks:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        busy = sorted(clocks)[len(clocks) // 2:]  # upper half: samples taken under load
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": max(maxes), "reasons": sorted(reasons),
                "samples": len(clocks)}


def dist_setup(args):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        if args.impl == "reference":
            return rank, world, local, None
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        return rank, world, local, dist
    return rank, world, local, None


def barrier(dist):
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(dist, ms, device):
    if dist is None:
        return ms
    t = torch.tensor([ms], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


# ------------------------------------------------------------------------------------------------

def run_cpu_port(w, steps, warmup, sample_tokens, threads):
    """Time the CPU port on `sample_tokens` tokens of one epoch per step. Returns tokens/s."""
    from gl_sdm_b200 import workloads
    from oracle import torch_port as port
    torch.set_num_threads(threads)
    gen_device = "cuda" if torch.cuda.is_available() else "cpu"
    bank = workloads.make_bank(w, gen_device, banks=1).cpu()
    seqs = max(1, sample_tokens // w.chunk)
    tokens = min(w.chunk, sample_tokens)
    times = []
    for i in range(warmup + steps):
        x = {k: v.cpu() for k, v in workloads.make_epoch_inputs(w, gen_device, 7000 + i, sequences=seqs, tokens=tokens).items()}
        t0 = time.perf_counter()
        port.routed_read(bank, x["q_scores"], w.width)
        a, d, k = port.propose(bank, x["k_scores"], w.width, x["target"].float(), x["beta"], x["log_decay"], None, 0, 0,
                               w.chunk, 1)
        port.commit(bank, a, d, k, in_place=True)
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
    n = seqs * tokens
    return n / statistics.median(times), n, statistics.median(times)


def reference_arm(args, w, rank):
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    value, n, sec = run_cpu_port(w, args.steps, args.warmup, args.cpu_sample_tokens, threads)
    line = {
        "impl": "reference", "metric": "memory-op tokens/s", "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(w, args, 1),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port",
                         "sample": f"{n} tokens of one commit epoch per step (route+read, propose, in-place commit) on the "
                                   f"full {w.slots}-slot bank; PyTorch CPU port of the reference path"},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def workload_config(w, args, world):
    return {"workload": f"{w.name}: {w.description}", "routing": "product-key factor scores (fp32) -> fused top-k",
            "slots": w.slots, "d_v": w.dim, "top_k": w.width, "tokens_per_step": w.tokens_per_step,
            "commit_epochs": w.epochs, "tokens_per_epoch": w.tokens_per_epoch, "bank_dtype": str(w.bank_dtype).split(".")[-1],
            "sharding": f"slots over {world} GPU(s)" if world > 1 else "single GPU",
            "l2": "inputs larger than L2 (per-epoch factor scores alone exceed 126 MB)"}


def ours(args, w, rank, world, local, dist):
    from gl_sdm_b200 import _native, workloads
    from gl_sdm_b200.operator import SharedBankOperator
    if world > 1:
        from gl_sdm_b200.sharded import ShardedBankOperator
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    lib = _native.library()
    if w.per_request_banks:
        raise SystemExit("per-request-bank workloads (c1, c2) are measured by tests/bench of the stack API; use c3-c5 here")

    bank = workloads.make_bank(w, dev)
    if world > 1:
        op = ShardedBankOperator(bank, w.width, w.width, dist, chunk_size=w.chunk)
        del bank
    else:
        op = SharedBankOperator(bank, w.width, w.width, chunk_size=w.chunk)
    seqs_local = w.sequences // world
    epochs = [workloads.make_epoch_inputs(w, dev, 1000 * (rank + 1) + e, sequences=seqs_local) for e in range(w.epochs)]

    def step():
        out = None
        for x in epochs:
            out = op.epoch(x["q_scores"], x["k_scores"], x["target"], x["beta"], x["log_decay"])
        return out

    for _ in range(args.warmup):
        step()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = lib.glsdm_kernel_launches()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier(dist)
    start.record()
    for _ in range(args.steps):
        step()
    stop.record()
    barrier(dist)
    ms = max_over_ranks(dist, start.elapsed_time(stop), dev)
    launches = lib.glsdm_kernel_launches() - launches0
    clocks = sampler.stop() if rank == 0 else None
    _native.raise_on_device_status(dev)
    ms_per_step = ms / args.steps
    value = w.tokens_per_step / (ms_per_step / 1e3)

    # -- per-phase device times (separate pass; events between the three calls of an epoch) ----
    phase = {"read": 0.0, "propose": 0.0, "commit": 0.0}
    marks = []
    for x in epochs:
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        ev[0].record()
        op.read(x["q_scores"])
        ev[1].record()
        prop = op.propose(x["k_scores"], x["target"], x["beta"], x["log_decay"])
        ev[2].record()
        op.commit(*prop)
        ev[3].record()
        marks.append(ev)
    torch.cuda.synchronize()
    for ev in marks:
        for i, name in enumerate(("read", "propose", "commit")):
            phase[name] += ev[i].elapsed_time(ev[i + 1])
    calls = len(marks)
    # unique touched rows / entries of the last epoch, for the commit's algorithmic bytes
    addresses = prop[0]
    unique_fraction = float(torch.unique(addresses).numel()) / max(1, addresses.numel())
    peak, peak_kind = measured_peaks()
    algo = workloads.algorithmic_bytes(w, w.tokens_per_epoch // world, unique_fraction, layers=1)
    dominant = max(phase, key=phase.get)
    per_launch_ms = phase[dominant] / calls
    achieved = algo[dominant] / (per_launch_ms / 1e3) / 1e9
    kernel_names = {"read": "pk_select_read_kernel", "propose": "pk_propose_kernel",
                    "commit": "commit (radix sort + reduce_kernel)"}
    roofline = {"bound": "hbm", "kernel": kernel_names[dominant], "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak, "peak_kind": f"of {peak_kind}", "frac_of_nominal_8TBs": achieved / NOMINAL_HBM_GBS,
                "traffic": load_traffic(dominant, w),
                "algorithmic_bytes_per_launch": algo[dominant], "ms_per_launch": per_launch_ms,
                "phases": {k: {"ms_per_epoch": phase[k] / calls, "algorithmic_GBs": algo[k] / (phase[k] / calls / 1e3) / 1e9,
                               "frac": algo[k] / (phase[k] / calls / 1e3) / 1e9 / peak} for k in phase},
                "unique_row_fraction": unique_fraction}

    # -- end to end from pinned host memory ------------------------------------------------------
    e2e = None if args.no_e2e else end_to_end(args, w, op, epochs[0], dev, dist, world)

    if rank != 0:
        return
    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        cv, n, sec = run_cpu_port(w, 1, 1, args.cpu_sample_tokens, threads)
        cpu = {"value": cv, "unit": "tokens/s", "cores": threads, "kind": "port",
               "sample": f"{n} tokens of one commit epoch (route+read, propose, in-place commit), full {w.slots}-slot bank, "
                         f"{sec:.2f} s; PyTorch CPU port of the reference path"}
    line = {
        "metric": "memory-op tokens/s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32 accumulate over %s bank" % str(w.bank_dtype).split(".")[-1], "data": "synthetic",
        "config": workload_config(w, args, world), "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e,
        "gpu_launches": int(launches), "clocks": clocks,
    }
    print(json.dumps(line), flush=True)


def load_traffic(phase, w):
    """DRAM bytes per launch of the dominant kernel from the committed ncu summary, if any."""
    path = os.path.join(ROOT, "profiles", "traffic.json")
    if not os.path.exists(path):
        return None
    with open(path) as f:
        table = json.load(f)
    entry = table.get(f"{w.name}:{phase}")
    return None if entry is None else entry.get("dram_bytes_per_launch")


def end_to_end(args, w, op, template, dev, dist, world):
    """Host-resident inputs: per epoch H2D of scores/targets/gates (double-buffered on a copy
    stream), the operator epoch, and D2H of the readings, all inside the timed region."""
    names = ("q_scores", "k_scores", "target", "beta", "log_decay")
    host = {k: torch.empty(template[k].shape, dtype=template[k].dtype).pin_memory() for k in names}
    for k in names:
        host[k].copy_(template[k])
    slots = [{k: torch.empty_like(template[k]) for k in names} for _ in range(2)]
    readings_host = torch.empty((*template["beta"].shape, w.dim), dtype=torch.float32).pin_memory()
    copy_stream = torch.cuda.Stream(dev)
    main = torch.cuda.current_stream(dev)
    ready = [torch.cuda.Event() for _ in range(2)]
    freed = [torch.cuda.Event() for _ in range(2)]

    def upload(i):
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(freed[i])
            for k in names:
                slots[i][k].copy_(host[k], non_blocking=True)
            ready[i].record(copy_stream)

    def step():
        for i in range(2):
            freed[i].record(main)
        upload(0)
        for e in range(w.epochs):
            cur = e % 2
            if e + 1 < w.epochs:
                upload((e + 1) % 2)
            main.wait_event(ready[cur])
            x = slots[cur]
            out = op.epoch(x["q_scores"], x["k_scores"], x["target"], x["beta"], x["log_decay"])
            freed[cur].record(main)
            readings_host.copy_(out, non_blocking=True)
        return readings_host

    steps = max(1, min(args.steps, args.e2e_steps))
    step()
    barrier(dist)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(steps):
        step()
    t1.record()
    barrier(dist)
    ms = max_over_ranks(dist, t0.elapsed_time(t1), dev) / steps
    h2d = sum(host[k].numel() * host[k].element_size() for k in names) * w.epochs * world
    d2h = readings_host.numel() * 4 * w.epochs * world
    return {"value": w.tokens_per_step / (ms / 1e3), "unit": "tokens/s", "ms_per_step": ms, "steps": steps,
            "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
            "note": "one epoch of pinned host inputs re-sent for each of the step's epochs; uploads overlap compute on a copy stream"}


def main():
    from gl_sdm_b200 import workloads
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c4", choices=sorted(workloads.WORKLOADS))
    ap.add_argument("--sequences", type=int, default=None, help="override the batch (sequences per step)")
    ap.add_argument("--seq-len", type=int, default=None)
    ap.add_argument("--cpu-sample-tokens", type=int, default=8192)
    ap.add_argument("--e2e-steps", type=int, default=2)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-input pass (profiling runs)")
    args = ap.parse_args()
    w = workloads.WORKLOADS[args.workload]
    if args.sequences or args.seq_len:
        w = w.scaled(args.sequences, args.seq_len)
    rank, world, local, dist = dist_setup(args)
    if args.impl == "reference":
        reference_arm(args, w, rank)
        return
    if w.sequences % world:
        raise SystemExit("sequences per step must divide over the ranks")
    ours(args, w, rank, world, local, dist)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
