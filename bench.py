"""Benchmark of the GL-SDM memory operator on B200: memory-op tokens/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c4] [--routing dense|pk]
                    [--impl ours|reference]

A step is one pass of the operator over one batch of synthetic input of the chosen
configuration. Default c4: bf16 bank of 16,777,216 slots (d_k 128, d_v 256), top-32, 64 x 8192
tokens = 16 commit epochs of 32,768 tokens, slot-sharded over the N GPUs. Per epoch: query
routing + read, write routing + prediction read + delta proposal, buffered commit.

  --routing dense  (default) scores = queries x slot keys on the tensor cores (tcgen05) fused
                   with the streaming top-k; sharded: query all-gather, per-GPU partial top-k,
                   K-candidate all-gather + merge, read reduce-scatter, write operands to the
                   owning shard at the commit clock.
  --routing pk     the reference's product-key factor scores [tokens, 2*4096] fp32 as input
                   (the drop-in operator contract); its single-GPU numbers are also attached to
                   the dense line under "product_key_scores".

Rank 0 prints one JSON line:
  value         device-resident throughput (inputs already in HBM), CUDA events, max over ranks
  e2e           the same through the operator with pinned HOST inputs: H2D of every epoch's
                inputs and D2H of its readings inside the timed region
  roofline      the dominant kernel against the measured peak of MEASURED_PEAKS.json
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

FALLBACK = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
NOMINAL_HBM_GBS = 8000.0
NOMINAL_BF16_TFLOPS = 2250.0


_RESULT_FD = None


def claim_stdout():
    """Keep standard output for the ONE JSON line: libraries loaded later (NCCL prints its
    version there) get standard error instead."""
    global _RESULT_FD
    if _RESULT_FD is None:
        sys.stdout.flush()
        _RESULT_FD = os.dup(1)
        os.dup2(2, 1)


def emit(text):
    sys.stdout.flush()
    os.write(_RESULT_FD if _RESULT_FD is not None else 1, (text + "\n").encode())


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            data = json.load(f)
        return {k: float(data[k]) for k in FALLBACK}, "measured"
    return dict(FALLBACK), "fallback"


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
        clocks, maxes, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                clocks.append(float(r[1])), maxes.append(float(r[2])), power.append(float(r[3]))
            except (ValueError, IndexError):
                continue
            for name, cell in zip(names, r[5:9]):
                if cell.lower().startswith("active"):
                    reasons.add(name)
        if not clocks:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        busy = sorted(clocks)[len(clocks) // 2:]  # upper half by clock: samples taken under load
        return {"sm_mhz": statistics.median(clocks), "sm_mhz_upper_half": statistics.median(busy),
                "sm_max_mhz": max(maxes), "power_w_max": max(power), "reasons": sorted(reasons), "samples": len(clocks)}


def dist_setup(args):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1 and args.impl != "reference":
        import torch.distributed as dist
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")   # keep stdout for the one JSON line
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


def bank_dtype_name(w):
    return str(w.bank_dtype).split(".")[-1]


def workload_config(w, args, world):
    routing = ("dense keys: queries [tokens, d_k] bf16 x keys [slots, d_k] bf16 on tcgen05, fused top-k"
               if args.routing == "dense" else "product-key factor scores [tokens, 2*half] fp32 -> fused top-k")
    return {"workload": f"{w.name}: {w.description}", "routing": routing, "slots": w.slots, "d_k": w.dk, "d_v": w.dim,
            "top_k": w.width, "tokens_per_step": w.tokens_per_step, "commit_epochs": w.epochs,
            "tokens_per_epoch": w.tokens_per_epoch, "bank_dtype": bank_dtype_name(w),
            "sharding": f"slots over {world} GPUs, tokens data-parallel" if world > 1 else "single GPU",
            "l2": "inputs larger than L2: every epoch streams the whole key shard (>= 0.5 GB) or >= 1 GB of factor scores"}


# ---- the reference on the host cores (cpu_baseline and --impl reference) ----------------------------

def staged_reference():
    """The unmodified reference package when it is staged beside the oracle (oracle/make_ref.py):
    (its gl_sdm.memory module, its runtime.dense.proposal_delta). None when it is not there; the
    CPU port of oracle/torch_port.py then stands in (kind "port")."""
    from oracle import make_ref
    path = make_ref.ref_path()
    if path is None:
        return None
    if path not in sys.path:
        sys.path.insert(0, path)
    import importlib
    try:
        memory = importlib.import_module("gl_sdm.memory")
        importlib.import_module("gl_sdm.memory.routing")
        dense = importlib.import_module("gl_sdm.runtime.dense")
    except Exception:   # noqa: BLE001 - an unusable staging falls back to the port
        return None
    return memory, dense.proposal_delta


def run_cpu_reference(w, routing, steps, warmup, sample_tokens, threads, budget_s=150.0):
    """Time the reference's own code on `sample_tokens` tokens of one epoch per step, on the
    full-size bank as the reference holds it: float32 values (gl_sdm/memory/state.py:14), the
    batch's tokens folded into one request's token axis (one shared bank), routed read
    (memory/routing.py:10-28), row gather and addresses (:31-42), proposal_delta
    (runtime/dense.py:11-14), keys (layers/global_layer.py:52-53), merge and the functional
    commit with its whole-bank copy (memory/transactions.py:62-97). With dense keys the scoring
    stage q x keys^T + top-k has no counterpart in the reference and is the port's
    (oracle/torch_port.py flat_routes); everything after it is the reference's. The whole-bank
    copy makes a step take seconds on the large banks, so at most `budget_s` seconds are spent:
    one warm-up step and then as many of the `steps` as fit (at least one). Returns
    (tokens/s, tokens, median seconds, steps timed) or None when the reference is not staged."""
    ref = staged_reference()
    if ref is None:
        return None
    memory, proposal_delta = ref
    import bench_workloads as workloads
    from oracle import torch_port as port
    torch.set_num_threads(threads)
    gen = "cuda" if torch.cuda.is_available() else "cpu"
    values = workloads.make_bank(w, gen, banks=1).cpu().float()
    keys = workloads.make_keys(w, gen).cpu() if routing == "dense" else None
    seqs = max(1, sample_tokens // w.chunk)
    tokens = min(w.chunk, sample_tokens)
    n = seqs * tokens
    times = []
    warmup = min(warmup, 1)
    begun = time.perf_counter()
    for i in range(warmup + steps):
        if times and time.perf_counter() - begun + times[-1] > budget_s:
            break
        view = memory.MemoryView(values)
        if routing == "dense":
            x = {k: v.cpu() for k, v in workloads.make_epoch_inputs_dense(w, gen, 7000 + i, seqs, tokens,
                                                                          keys=keys.to(gen)).items()}
            t0 = time.perf_counter()
            index, weights = port.flat_routes(x["q"].reshape(-1, w.dk), keys, w.width)
            index, weights = index.view(1, n, 1, -1), weights.view(1, n, 1, -1)
            rows = memory.routing.gather_rows(view.values, index)
            (rows * weights[..., None]).sum(-2)
            windex, wweights = port.flat_routes(x["kq"].reshape(-1, w.dk), keys, w.width)
            windex, wweights = windex.view(1, n, 1, -1), wweights.view(1, n, 1, -1)
            rows = memory.routing.gather_rows(view.values, windex)
            prediction = (rows * wweights[..., None]).sum(-2)
        else:
            x = {k: v.cpu() for k, v in workloads.make_epoch_inputs(w, gen, 7000 + i, seqs, tokens).items()}
            fold = lambda t: t.reshape(1, n, *t.shape[2:])   # noqa: E731
            t0 = time.perf_counter()
            memory.routing.torch_routed_read(view.values, fold(x["q_scores"]), w.width)
            prediction, windex, wweights = memory.routing.torch_routed_read(view.values, fold(x["k_scores"]), w.width)
            rows = memory.routing.gather_rows(view.values, windex)
        addresses = memory.routing.absolute_addresses(view.values, windex)
        shape = (1, n, w.heads)
        delta = proposal_delta(rows, wweights, prediction, x["target"].float().reshape(*shape, w.dim),
                               x["beta"].reshape(*shape, 1), x["log_decay"].reshape(*shape, 1), torch.ones(1, n))
        position = (torch.arange(n) % tokens).view(1, n, 1, 1)
        sort_keys = addresses * w.chunk + position
        proposal = memory.WriteProposal(view.version, addresses.flatten(), delta.flatten(0, 3), view.lineage,
                                        sort_keys.flatten())
        after = memory.commit(view, memory.merge(view, [proposal]))
        dt = time.perf_counter() - t0
        del after, delta, rows
        if i >= warmup:
            times.append(dt)
    return n / statistics.median(times), n, statistics.median(times), len(times)


def reference_sample_text(w, routing, n, sec):
    scoring = ("q x keys^T + top-k by torch ops (no counterpart in the reference), then " if routing == "dense" else "")
    return (f"{n} tokens of one commit epoch on the full {w.slots}-slot bank held as the reference holds it (float32, "
            f"one shared request), {sec:.2f} s per step: {scoring}the reference's own torch_routed_read / gather_rows / "
            "proposal_delta / merge / functional commit (whole-bank copy included), unmodified package staged under "
            "oracle/_ref")


# ---- CPU port (stands in when the reference is not staged) -------------------------------------------

def run_cpu_port(w, routing, steps, warmup, sample_tokens, threads):
    """Time the CPU port on `sample_tokens` tokens of one epoch per step. Returns (tokens/s, n, s)."""
    import bench_workloads as workloads
    from oracle import torch_port as port
    torch.set_num_threads(threads)
    gen = "cuda" if torch.cuda.is_available() else "cpu"
    bank = workloads.make_bank(w, gen, banks=1).cpu()
    seqs = max(1, sample_tokens // w.chunk)
    tokens = min(w.chunk, sample_tokens)
    keys = workloads.make_keys(w, gen).cpu() if routing == "dense" else None
    times = []
    for i in range(warmup + steps):
        if routing == "dense":
            x = {k: v.cpu() for k, v in workloads.make_epoch_inputs_dense(w, gen, 7000 + i, seqs, tokens,
                                                                          keys=keys.to(gen)).items()}
            t0 = time.perf_counter()
            port.dense_epoch(bank, keys, x["q"], x["kq"], w.width, x["target"].float(), x["beta"], x["log_decay"], w.chunk)
        else:
            x = {k: v.cpu() for k, v in workloads.make_epoch_inputs(w, gen, 7000 + i, seqs, tokens).items()}
            t0 = time.perf_counter()
            port.routed_read(bank, x["q_scores"], w.width)
            a, d, k = port.propose(bank, x["k_scores"], w.width, x["target"].float(), x["beta"], x["log_decay"], None,
                                   0, 0, w.chunk, 1)
            port.commit(bank, a, d, k, in_place=True)
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
    n = seqs * tokens
    return n / statistics.median(times), n, statistics.median(times)


def run_torch_on_gpu(w, dev, sequences=16):
    """The reference's own code on CUDA tensors of the same GPU: a second comparison beside the CPU
    baseline. Product-key scores in, `sequences` x chunk tokens of one epoch on the full bank
    held as the reference holds it (float32, tokens folded into one request): routed read,
    write proposal (routed read + gather_rows + proposal_delta), the functional commit of
    gl_sdm/memory/transactions.py (whole-bank copy) and the reference's Triton commit kernel
    (gl_sdm/memory/backends/commit.py). Uses the staged reference package; where it is not
    staged, the port's tensor-op sequence (oracle/torch_port.py). Returns per-stage milliseconds
    and tokens/s."""
    import bench_workloads as workloads
    from oracle import torch_port as port
    ref = staged_reference()
    x = workloads.make_epoch_inputs(w, dev, 9000, sequences, w.chunk)
    marks = {}
    n = sequences * w.chunk

    def timed(name, fn):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        out = fn()
        b.record()
        torch.cuda.synchronize(dev)
        marks[name] = a.elapsed_time(b)
        return out

    if ref is None:
        bank = workloads.make_bank(w, dev, banks=1)
        for attempt in range(2):   # the first round is the warm-up
            timed("read_ms", lambda: port.routed_read(bank, x["q_scores"], w.width))
            a, d, k = timed("proposal_ms", lambda: port.propose(bank, x["k_scores"], w.width, x["target"].float(),
                                                                 x["beta"], x["log_decay"], None, 0, 0, w.chunk, 1))
            out = timed("commit_copy_ms", lambda: port.commit(bank, a, d, k, in_place=False))
            del out
            timed("commit_in_place_ms", lambda: port.commit(bank, a, d, k, in_place=True))
            del a, d, k
        total = marks["read_ms"] + marks["proposal_ms"] + marks["commit_in_place_ms"]
        what = "PyTorch CUDA tensor ops of the reference path (port), in-place commit counted"
    else:
        memory, proposal_delta = ref
        values = workloads.make_bank(w, dev, banks=1).float()
        fold = lambda t: t.reshape(1, n, *t.shape[2:])   # noqa: E731
        shape = (1, n, w.heads)

        def propose():
            prediction, index, weights = memory.routing.torch_routed_read(values, fold(x["k_scores"]), w.width)
            rows = memory.routing.gather_rows(values, index)
            addresses = memory.routing.absolute_addresses(values, index)
            delta = proposal_delta(rows, weights, prediction, x["target"].float().reshape(*shape, w.dim),
                                   x["beta"].reshape(*shape, 1), x["log_decay"].reshape(*shape, 1),
                                   torch.ones(1, n, device=dev))
            position = (torch.arange(n, device=dev) % w.chunk).view(1, n, 1, 1)
            return addresses.flatten(), delta.flatten(0, 3), (addresses * w.chunk + position).flatten()

        for attempt in range(2):
            view = memory.MemoryView(values)
            timed("read_ms", lambda: memory.routing.torch_routed_read(values, fold(x["q_scores"]), w.width))
            a, d, k = timed("proposal_ms", propose)
            proposal = memory.WriteProposal(view.version, a, d, view.lineage, k)
            out = timed("commit_torch_ms", lambda: memory.commit(view, memory.merge(view, [proposal])))
            del out
            try:
                import importlib
                triton_commit = importlib.import_module("gl_sdm.memory.backends.commit").commit
                out = timed("commit_triton_ms", lambda: triton_commit(values, a, d, k))
                del out
            except Exception as exc:   # noqa: BLE001 - Triton missing or unable to compile here
                marks["commit_triton_error"] = f"{type(exc).__name__}: {exc}"[:200]
            del a, d, k, proposal
        total = marks["read_ms"] + marks["proposal_ms"] + marks["commit_torch_ms"]
        what = ("the reference's own functions (unmodified package staged under oracle/_ref) on CUDA tensors, float32 bank, "
                "functional commit counted; commit_triton_ms is its Triton commit kernel on the same entries")
    marks = {k: (round(v, 3) if isinstance(v, float) else v) for k, v in marks.items()}
    marks.update({"value": n / (total / 1e3), "unit": "tokens/s",
                  "sample": f"{n} tokens of one commit epoch, product-key scores in; {what}"})
    return marks


def cpu_sample_text(w, routing, n, sec):
    what = "flat-key scores + routes" if routing == "dense" else "product-key routes"
    return (f"{n} tokens of one commit epoch ({what}, read, proposal, in-place commit) on the full "
            f"{w.slots}-slot bank, {sec:.2f} s; PyTorch CPU port of the reference path")


def enough_host_memory(w):
    """The reference holds the bank in float32 and its commit returns a second copy: allow for
    three banks of head room before taking that path on this machine."""
    try:
        import psutil
        available = psutil.virtual_memory().available
    except Exception:   # noqa: BLE001
        return False
    return available > 3 * w.heads * w.slots * w.dim * 4 + (16 << 30)


def reference_arm(args, w, rank):
    if rank != 0:
        return
    if w.per_request_banks:
        cpu = per_request_cpu_port(w, seconds=10.0)
        ms = cpu.pop("ms_per_step")
        emit(json.dumps({
            "impl": "reference", "metric": "memory-op tokens/s", "value": cpu["value"], "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": per_request_config(w), "cpu_baseline": cpu,
            "e2e": {"value": cpu["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return
    threads = os.cpu_count() or 1
    tokens = args.cpu_sample_tokens or (256 if args.routing == "dense" else 8192)
    kind, measured = "reference", None
    if enough_host_memory(w):
        measured = run_cpu_reference(w, args.routing, args.steps, args.warmup, tokens, threads)
    if measured is None:
        kind, measured = "port", (*run_cpu_port(w, args.routing, args.steps, args.warmup, tokens, threads), args.steps)
    value, n, sec, timed = measured
    line = {
        "impl": "reference", "metric": "memory-op tokens/s", "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": timed, "warmup": args.warmup if kind == "port" else min(args.warmup, 1), "ms_per_step": sec * 1e3,
        "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(w, args, 1),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": kind,
                         "sample": (reference_sample_text if kind == "reference" else cpu_sample_text)(w, args.routing, n, sec)},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    emit(json.dumps(line))


# ---- per-request banks (c1 / c2) through the reference-shaped API ------------------------------------

def api_inputs(w, device, seed):
    """Factor scores and write operands of every (epoch, global layer) of one step; the same
    distributions as make_epoch_inputs, one bank per request."""
    import bench_workloads as workloads
    return [[workloads.make_epoch_inputs(w, device, seed + 100 * e + layer) for layer in range(w.global_layers)]
            for e in range(w.epochs)]


def api_step(w, values, inputs, memory):
    """One step the way the reference's stack drives the operator (gl_sdm/layers/stack.py:41-70,
    global_layer.py:22-54): per 512-token chunk every global layer reads, proposes against the
    chunk-start snapshot (delta formula of gl_sdm/runtime/dense.py:11-14, written here with
    tensor ops as the caller does), then one functional commit of all proposals."""
    view = memory.MemoryView(values)
    L, C = w.global_layers, w.chunk
    readings = None
    for layers in inputs:
        proposals = []
        for layer, x in enumerate(layers):
            readings, _, _ = memory.routing.torch_routed_read(view.values, x["q_scores"], w.width)
            prediction, index, weights = memory.routing.torch_routed_read(view.values, x["k_scores"], w.width)
            rows = memory.routing.gather_rows(view.values, index)
            addresses = memory.routing.absolute_addresses(view.values, index)
            decay = x["log_decay"].exp().unsqueeze(-1)
            error = x["beta"].unsqueeze(-1) * (x["target"].float() - decay * prediction)
            delta = (decay.unsqueeze(-1) - 1) * rows + weights.unsqueeze(-1) * error.unsqueeze(-2)
            position = torch.arange(index.shape[1], device=index.device).view(1, -1, 1, 1)
            keys = addresses * (C * L) + position * L + layer
            proposals.append(memory.WriteProposal(view.version, addresses.flatten(), delta.flatten(0, 3), view.lineage,
                                                  keys.flatten()))
        view = memory.commit(view, memory.merge(view, proposals))
    return readings, view


def api_step_fused(w, values, inputs, memory):
    """The same step with every layer's write side on the fused proposal kernel
    (glsdm_pk_propose, what gl_sdm_b200.layers.propose runs after the layer's projections): the
    proposals of a chunk are written side by side into one buffer, so the commit concatenates
    nothing. Reads and commits are the calls of api_step."""
    from gl_sdm_b200 import _native
    view = memory.MemoryView(values)
    L, C = w.global_layers, w.chunk
    readings = None
    for layers in inputs:
        entries = layers[0]["k_scores"].numel() // layers[0]["k_scores"].shape[-1] * w.width
        dev = values.device
        addresses = torch.empty(L * entries, dtype=torch.int64, device=dev)
        deltas = torch.empty((L * entries, w.dim), dtype=torch.float32, device=dev)
        keys = torch.empty(L * entries, dtype=torch.int64, device=dev)
        proposals = []
        for layer, x in enumerate(layers):
            readings, _, _ = memory.routing.torch_routed_read(view.values, x["q_scores"], w.width)
            piece = slice(layer * entries, (layer + 1) * entries)
            out = (addresses[piece], deltas[piece], keys[piece])
            _native.pk_propose(view.values, x["k_scores"], x["target"], x["beta"], x["log_decay"], None,
                               tokens=x["k_scores"].shape[1], width=w.width, chunk_offset=0, chunk_size=C,
                               num_layers=L, layer_index=layer, out=out)
            proposals.append(memory.WriteProposal(view.version, *out[:2], view.lineage, out[2]))
        view = memory.commit(view, memory.merge(view, proposals))
    return readings, view


class PortMemory:
    """The CPU port behind the same five names, so api_step can time it unchanged."""

    def __init__(self):
        from oracle import torch_port as port
        self.port = port
        self.routing = self

    class View:
        def __init__(self, values, version=0):
            self.values, self.version, self.lineage = values, version, None

    def MemoryView(self, values):
        return PortMemory.View(values)

    def WriteProposal(self, version, addresses, deltas, lineage, keys):
        return (addresses, deltas, keys)

    def torch_routed_read(self, values, scores, width):
        return self.port.routed_read(values, scores, width)

    def gather_rows(self, values, index):
        return values.flatten(0, 2)[self.port.flat_rows(values, index)]

    def absolute_addresses(self, values, index):
        return self.port.flat_rows(values, index)

    def merge(self, view, proposals):
        return proposals

    def commit(self, view, proposals):
        a, d, k = (torch.cat([p[i] for p in proposals]) for i in range(3))
        return PortMemory.View(self.port.commit(view.values, a, d, k), view.version + 1)


def per_request_config(w):
    bank_mb = w.sequences * w.heads * w.slots * w.dim * 4 >> 20
    return {"workload": f"{w.name}: {w.description}",
            "routing": "product-key factor scores through the memory API (routed_read, gather_rows, merge, functional "
                       "commit), one bank per request: replicas only",
            "slots": w.slots, "d_v": w.dim, "top_k": w.width, "tokens_per_step": w.tokens_per_step,
            "global_layers": w.global_layers, "commit_epochs": w.epochs,
            "l2": f"banks of {bank_mb} MB: " + ("L2-resident, so the HBM fraction understates nothing and bounds nothing; "
                                                  "the step is launch-bound" if bank_mb < 100 else
                                                  "larger than L2; every commit copies them (functional commit)")}


def per_request_cpu_port(w, seconds=5.0):
    """The CPU port through api_step on all host cores: c1 whole, c2 one request x one chunk
    (8 layers); repeated until `seconds` have passed, median step. Returns the cpu_baseline."""
    import bench_workloads as workloads
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    sample = w if w.name == "c1" else w.scaled(sequences=1, seq_len=w.chunk)
    values = workloads.make_bank(sample, "cpu")
    inputs = api_inputs(sample, "cpu", 1000)
    ref = staged_reference()
    port = PortMemory() if ref is None else ref[0]      # the reference's own gl_sdm.memory when it is staged
    api_step(sample, values, inputs, port)
    times, begun = [], time.perf_counter()
    while not times or (time.perf_counter() - begun < seconds and len(times) < 50):
        t = time.perf_counter()
        api_step(sample, values, inputs, port)
        times.append(time.perf_counter() - t)
    sec = statistics.median(times)
    what = ("PyTorch CPU port of the reference path" if ref is None else
            "the reference's own gl_sdm.memory (unmodified package staged under oracle/_ref)")
    return {"value": sample.tokens_per_step / sec, "unit": "tokens/s", "cores": threads,
            "kind": "port" if ref is None else "reference",
            "sample": f"{sample.sequences} x {sample.seq_len} tokens, {sample.global_layers} global layer(s), through the same "
                      f"call sequence (functional commit), median of {len(times)} steps of {sec:.2f} s; {what}",
            "ms_per_step": sec * 1e3}


# ---- c2 as the reference runs it: its own 16-layer stack, unmodified, on this package --------------

STACK_CONFIG = dict(arch_type="gl_sdm", vocab_size=32000, hidden_size=512, head_dim=64, num_hidden_layers=16,
                    intermediate_size=2048, dtype="bfloat16", gl_layer_pattern=["local", "global"], gl_local_window=256,
                    gl_chunk_size=512, gl_slots=16384, gl_reads=16, gl_writes=16, gl_memory_backend="torch")


def stack_model(device, shim):
    """The reference's create_model at the widths of configuration 2 (gl_sdm/model.py), every
    matrix re-drawn N(0, 0.02) from a fixed seed, the learned bank left at its own float32
    initialiser. With `shim` the reference's gl_sdm.memory is replaced by gl_sdm_b200.memory
    BEFORE the model modules are imported, which is all it takes (gl_sdm_b200/install.py)."""
    from oracle import make_ref
    path = make_ref.ref_path()
    if path is None:
        raise SystemExit("the reference package is not staged under oracle/_ref (python oracle/make_ref.py <checkout>)")
    if path not in sys.path:
        sys.path.insert(0, path)
    if shim:
        from gl_sdm_b200 import install
        install.install()
    import importlib
    torch.manual_seed(1234)
    model = importlib.import_module("gl_sdm.model").create_model(STACK_CONFIG)
    gen = torch.Generator().manual_seed(1234)
    with torch.no_grad():
        for name, p in model.named_parameters():
            if p.ndim >= 2 and name != "bank.memory":
                p.copy_((torch.randn(p.shape, generator=gen) * 0.02).to(p.dtype))
    return model.to(device).eval()


def stack_reference_arm(args, w, rank):
    """--impl reference --stack: the same model on the reference's own memory package (torch
    path) on the host cores, 1 x 1024 tokens per step (a reduced batch; the full one is 8 x 4096)."""
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    model = stack_model("cpu", shim=False)
    ids = torch.randint(STACK_CONFIG["vocab_size"], (1, 1024), generator=torch.Generator().manual_seed(7))
    times, begun = [], time.perf_counter()
    with torch.inference_mode():
        for i in range(1 + args.steps):
            if times and time.perf_counter() - begun + times[-1] > 150.0:
                break
            t0 = time.perf_counter()
            model.hidden(ids, model.new_cache(1))
            if i:
                times.append(time.perf_counter() - t0)
            else:
                first = time.perf_counter() - t0
    sec = statistics.median(times or [first])
    value = ids.numel() / sec
    emit(json.dumps({
        "impl": "reference", "metric": "stack forward tokens/s", "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": len(times), "warmup": 1, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16 weights, f32 banks", "data": "synthetic",
        "config": {"workload": "c2: the reference's 16-layer stack (8 local + 8 global layers, hidden 512, 16,384 slots, "
                               "top-16, 512-token chunks), forward with every chunk committed", "batch": "1 x 1024 (reduced)"},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "reference",
                         "sample": f"1 x 1024 tokens, the unmodified reference model on its own torch memory path, {sec:.2f} s per step"},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


def stack_training_step(model, dev, args):
    """--train: forward + backward of the same model (cross-entropy on random targets, 8 x 2048
    token ids, every parameter and the learned bank receive gradients), with the reference's
    own GlobalLayer.propose and with the fused one (forward glsdm_pk_propose, backward
    glsdm_pk_propose_backward). Milliseconds per step and the peak of allocated device memory."""
    import importlib
    from gl_sdm_b200.layers import install_fused_proposals
    B, T = 8, 2048
    gen = torch.Generator().manual_seed(11)
    ids = torch.randint(STACK_CONFIG["vocab_size"], (B, T), generator=gen).to(dev)
    targets = torch.randint(STACK_CONFIG["vocab_size"], (B, T), generator=gen).to(dev)
    model.train()

    def step():
        model.zero_grad(set_to_none=True)
        hidden, _, _ = model.hidden(ids)
        logits = model.head(hidden)
        loss = torch.nn.functional.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(), targets.flatten())
        loss.backward()
        return loss

    def measure():
        for _ in range(2):
            step()
        torch.cuda.synchronize(dev)
        torch.cuda.reset_peak_memory_stats(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            loss = step()
        e1.record()
        torch.cuda.synchronize(dev)
        ms = e0.elapsed_time(e1) / args.steps
        return {"ms_per_step": ms, "tokens_per_s": B * T / (ms / 1e3),
                "peak_allocated_GB": torch.cuda.max_memory_allocated(dev) / 1e9, "loss": loss.item()}

    out = {"batch": f"{B} x {T}", "reference_propose": measure()}
    undo = install_fused_proposals(importlib.import_module("gl_sdm.layers.global_layer"))
    try:
        out["fused_propose"] = measure()
    finally:
        undo()
        model.eval()
        model.zero_grad(set_to_none=True)
    return out


def stack_arm(args, w, rank):
    """--workload c2 --stack: the reference's own model, unmodified, on the CUDA operator.
    A step = Model.hidden over 8 x 4096 token ids with a fresh request cache (16 layers, 8
    commit epochs, 128 routed reads, 64 row gathers, 8 commits of 4,194,304 entries).
    `value` counts the WHOLE forward (dense surround included); the time inside the memory
    operator is measured on a separate pass with events around its calls."""
    if rank != 0:
        return
    from unittest.mock import patch
    from gl_sdm_b200 import _native
    import gl_sdm_b200.memory as memory
    import bench_workloads as workloads
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    lib = _native.library()
    peaks, peak_kind = measured_peaks()
    model = stack_model(dev, shim=True)
    import importlib
    stack = importlib.import_module("gl_sdm.layers.stack")
    assert stack.commit is memory.commit, "the reference stack is not bound to gl_sdm_b200.memory"
    B, T = w.sequences, w.seq_len
    host_ids = torch.randint(STACK_CONFIG["vocab_size"], (B, T), generator=torch.Generator().manual_seed(7)).pin_memory()
    ids = host_ids.to(dev)

    def forward(tokens):
        with torch.inference_mode():
            hidden, _, _ = model.hidden(tokens, model.new_cache(B))
        return hidden

    for _ in range(args.warmup):
        forward(ids)
    sampler = ClockSampler(0)
    sampler.start()
    launches0 = lib.glsdm_kernel_launches()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(dev)
    start.record()
    for _ in range(args.steps):
        forward(ids)
    stop.record()
    torch.cuda.synchronize(dev)
    ms = start.elapsed_time(stop) / args.steps
    launches = lib.glsdm_kernel_launches() - launches0
    clocks = sampler.stop()
    _native.raise_on_device_status(dev)

    # time inside the operator: events around every call the stack makes into the package
    spans = {"routed_read": [], "gather_rows": [], "commit": []}

    def timed(name, fn):
        def call(*a, **k):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            out = fn(*a, **k)
            e1.record()
            spans[name].append((e0, e1))
            return out
        return call

    with patch.object(memory.routing, "routed_read", timed("routed_read", memory.routing.routed_read)), \
            patch.object(memory.routing, "gather_rows", timed("gather_rows", memory.routing.gather_rows)), \
            patch.object(stack, "commit", timed("commit", stack.commit)):
        forward(ids)
    torch.cuda.synchronize(dev)
    inside = {k: sum(a.elapsed_time(b) for a, b in v) for k, v in spans.items()}
    calls = {k: len(v) for k, v in spans.items()}
    op_ms = sum(inside.values())

    e2e_steps = max(1, min(args.steps, 3))
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(dev)
    t0.record()
    for _ in range(e2e_steps):
        last = forward(host_ids.to(dev, non_blocking=True))[:, -1].float().cpu()
    t1.record()
    torch.cuda.synchronize(dev)
    e2e_ms = t0.elapsed_time(t1) / e2e_steps
    algo = workloads.algorithmic_bytes(w, w.tokens_per_step, 1.0)
    algo["bank_copy"] = w.epochs * 2 * B * w.heads * w.slots * w.dim * 4
    total = sum(algo.values())
    gbs = total / (op_ms / 1e3) / 1e9
    tokens = B * T

    # the same forward with GlobalLayer.propose served by the fused write proposal (one kernel
    # instead of routed read + row gather + the delta arithmetic in tensor ops)
    from gl_sdm_b200.layers import install_fused_proposals
    plain = forward(ids).float()
    undo = install_fused_proposals(importlib.import_module("gl_sdm.layers.global_layer"))
    try:
        for _ in range(max(1, args.warmup)):
            fused_out = forward(ids).float()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize(dev)
        f0.record()
        for _ in range(args.steps):
            forward(ids)
        f1.record()
        torch.cuda.synchronize(dev)
        fused_ms = f0.elapsed_time(f1) / args.steps
    finally:
        undo()
    fused = {"value": tokens / (fused_ms / 1e3), "unit": "tokens/s", "ms_per_step": fused_ms,
             "what": "gl_sdm_b200.install(fused_proposals=True): GlobalLayer.propose on glsdm_pk_propose",
             "hidden_relative_l2_vs_unfused": ((fused_out - plain).norm() / plain.norm().clamp_min(1e-12)).item()}
    _native.raise_on_device_status(dev)
    del plain, fused_out
    training = stack_training_step(model, dev, args) if args.train else None
    emit(json.dumps({
        "metric": "stack forward tokens/s", "value": tokens / (ms / 1e3), "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16 weights, f32 banks and memory arithmetic", "data": "synthetic",
        "config": {"workload": "c2: the reference's 16-layer stack (8 local + 8 global layers, hidden 512, 16,384 slots, "
                               "top-16, 512-token chunks), forward with every chunk committed, unmodified reference code "
                               "bound to gl_sdm_b200.memory", "batch": f"{B} x {T}",
                   "l2": "per-request banks of 256 MB in all and 4.2 GB of factor scores per layer call: larger than L2"},
        "memory_operator": {"ms_per_step": op_ms, "share_of_forward": op_ms / ms, "tokens_per_s": tokens / (op_ms / 1e3),
                            "ms_by_call": inside, "calls": calls},
        "fused_proposals": fused,
        "training_step": training,
        "roofline": {"bound": "hbm", "kernel": "memory operator inside the stack (pk_select_read, gather_rows, commit sort + "
                                                "reduce, whole-bank copy of the functional commit)",
                     "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"],
                     "peak_kind": f"of {peak_kind}", "traffic": None, "algorithmic_bytes_per_step": total},
        "cpu_baseline": None,
        "e2e": {"value": tokens / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms, "steps": e2e_steps,
                "h2d_bytes_per_step": host_ids.numel() * 8, "d2h_bytes_per_step": last.numel() * 4},
        "gpu_launches": int(launches), "clocks": clocks}))


def per_request_arm(args, w, rank):
    """c1 / c2: one fp32 bank per request, no sharding (replicas only): rank 0 measures one GPU."""
    if rank != 0:
        return
    import gl_sdm_b200.memory as memory
    from gl_sdm_b200 import _native
    import bench_workloads as workloads
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    lib = _native.library()
    peaks, peak_kind = measured_peaks()
    values = workloads.make_bank(w, dev)
    inputs = api_inputs(w, dev, 1000)
    for _ in range(args.warmup):
        api_step(w, values, inputs, memory)
    sampler = ClockSampler(0)
    sampler.start()
    launches0 = lib.glsdm_kernel_launches()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(dev)
    start.record()
    for _ in range(args.steps):
        api_step(w, values, inputs, memory)
    stop.record()
    torch.cuda.synchronize(dev)
    ms = start.elapsed_time(stop) / args.steps
    launches = lib.glsdm_kernel_launches() - launches0
    clocks = sampler.stop()
    _native.raise_on_device_status(dev)
    # host inputs: every chunk's scores and write operands come from pinned memory, the last readings go back
    host = [[{k: v.cpu().pin_memory() for k, v in x.items()} for x in layers] for layers in inputs]
    h2d = sum(v.numel() * v.element_size() for layers in host for x in layers for v in x.values())
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(dev)
    t0.record()
    moved = [[{k: v.to(dev, non_blocking=True) for k, v in x.items()} for x in layers] for layers in host]
    readings, _ = api_step(w, values, moved, memory)
    back = readings.cpu()
    t1.record()
    torch.cuda.synchronize(dev)
    e2e_ms = t0.elapsed_time(t1)
    # the same step with the write side fused (one kernel per layer instead of routed read +
    # row gather + tensor ops), checked against the unfused step's bank
    _, want_view = api_step(w, values, inputs, memory)
    for _ in range(max(1, args.warmup)):
        _, got_view = api_step_fused(w, values, inputs, memory)
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(dev)
    f0.record()
    for _ in range(args.steps):
        api_step_fused(w, values, inputs, memory)
    f1.record()
    torch.cuda.synchronize(dev)
    fused_ms = f0.elapsed_time(f1) / args.steps
    scale = want_view.values.abs().max().clamp_min(1e-30)
    fused = {"value": w.tokens_per_step / (fused_ms / 1e3), "unit": "tokens/s", "ms_per_step": fused_ms,
             "what": "write side of every layer on glsdm_pk_propose (gl_sdm_b200.layers.propose), proposals of a "
                     "chunk side by side in one buffer",
             "bank_max_rel_err_vs_unfused": ((got_view.values - want_view.values).abs().max() / scale).item()}
    del want_view, got_view
    _native.raise_on_device_status(dev)
    algo = workloads.algorithmic_bytes(w, w.tokens_per_step, 1.0)
    # the functional commit writes a new bank per epoch: one read and one write of every bank
    algo["bank_copy"] = w.epochs * 2 * values.numel() * values.element_size()
    total = sum(algo.values())
    gbs = total / (ms / 1e3) / 1e9
    cpu = None if args.no_cpu_baseline else per_request_cpu_port(w)
    line = {
        "metric": "memory-op tokens/s", "value": w.tokens_per_step / (ms / 1e3), "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": per_request_config(w),
        "roofline": {"bound": "hbm", "kernel": "whole step (pk_select_read, gather_rows, commit sort + reduce; delta by tensor ops)",
                     "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"],
                     "peak_kind": f"of {peak_kind}", "traffic": None, "algorithmic_bytes_per_step": total,
                     "algorithmic_bytes_by_stage": {k: int(v) for k, v in algo.items()}},
        "cpu_baseline": cpu,
        "fused_proposals": {**fused, "frac_of_hbm_peak": total / (fused_ms / 1e3) / 1e9 / peaks["hbm_gbs"]},
        "e2e": {"value": w.tokens_per_step / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms, "steps": 1,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": back.numel() * 4},
        "gpu_launches": int(launches), "clocks": clocks,
    }
    emit(json.dumps(line))


# ---- correctness of the multi-GPU path, recorded with every number ---------------------------------

def parity_check(routing, rank, world, dist, dev):
    """One small commit epoch through the same ShardedBankOperator the timed run uses (same
    collectives, same kernels, `world` ranks), checked on rank 0 against the CPU port of the
    reference path (the checker, outside any timed region): 2 sequences x 512 tokens per rank
    on a bf16 bank of 65,536 slots, d_v 128, top-16. Returns the `parity` object of the JSON
    line: how many routing rows have the oracle's routes, how many differ only at a documented
    near tie of the tensor-core scores (dense keys; product-key routes admit none), how many
    are wrong; the largest error of the readings and of the committed bank relative to their
    largest value; and whether all ranks hold the same routes."""
    import bench_workloads as workloads
    from gl_sdm_b200.sharded import ShardedBankOperator
    w = workloads.Workload("parity", "one epoch of 2 x 512 tokens per rank, 65,536 slots, d_v 128, top-16", 1, 256, 128,
                           128, 16, 2 * world, 512, torch.bfloat16)
    bank = workloads.make_bank(w, dev)
    mine = slice(2 * rank, 2 * rank + 2)
    if routing == "dense":
        keys = workloads.make_keys(w, dev)
        x = workloads.make_epoch_inputs_dense(w, dev, 4242)
        op = ShardedBankOperator(bank.clone(), w.width, w.width, dist, chunk_size=w.chunk, keys=keys)
        readings = op.epoch_dense(*[x[k][mine].contiguous() for k in ("q", "kq", "target", "beta", "log_decay")])
    else:
        keys = None
        x = workloads.make_epoch_inputs(w, dev, 4242)
        op = ShardedBankOperator(bank.clone(), w.width, w.width, dist, chunk_size=w.chunk)
        readings = op.epoch(*[x[k][mine].contiguous() for k in ("q_scores", "k_scores", "target", "beta", "log_decay")])
    read_slots, read_weights, write_slots, _ = op.last_routes()
    digest = torch.stack([(read_slots.long() * 1000003 % 2147483629).sum(), (write_slots.long() * 999983 % 2147483629).sum(),
                          (read_weights.double().sum() * 1e6).long()]).view(1, 3)
    every_digest = torch.empty(world, 3, dtype=torch.long, device=dev)
    every_reading = torch.empty(world, *readings.shape, dtype=readings.dtype, device=dev)
    if dist is not None:
        dist.all_gather_into_tensor(every_digest, digest)
        dist.all_gather_into_tensor(every_reading, readings.contiguous())
    else:
        every_digest.copy_(digest)
        every_reading[0].copy_(readings)
    after = op.gather_bank()
    from gl_sdm_b200 import _native
    _native.raise_on_device_status(dev)
    if rank != 0:
        return None
    from oracle import torch_port as port
    torch.set_num_threads(os.cpu_count() or 1)
    cpu = {k: v.cpu() for k, v in x.items()}
    got_reads = every_reading.flatten(0, 1).cpu().reshape(-1, w.dim)
    got = {"read": read_slots.cpu().long(), "write": write_slots.cpu().long()}
    rows = got["read"].shape[0]
    exempt = {"read": torch.zeros(rows, dtype=torch.bool), "write": torch.zeros(rows, dtype=torch.bool)}
    wrong = 0
    if routing == "dense":
        host_keys = keys.cpu().float()
        sides = {"read": cpu["q"].float().reshape(-1, w.dk), "write": cpu["kq"].float().reshape(-1, w.dk)}
        for side, q in sides.items():
            scores = q @ host_keys.T
            want, _ = port.flat_routes(q, host_keys, w.width)
            differs = (want != got[side]).any(-1)
            for r in torch.nonzero(differs).flatten().tolist():
                kth = scores[r, want[r]].min()
                only = set(want[r].tolist()) ^ set(got[side][r].tolist())
                if all(abs(float(scores[r, s] - kth)) <= 8e-6 for s in only):
                    exempt[side][r] = True
                else:
                    wrong += 1
        want_reads, want_bank = port.dense_epoch(bank.cpu().clone(), host_keys, cpu["q"].float(), cpu["kq"].float(), w.width,
                                                 cpu["target"].float(), cpu["beta"], cpu["log_decay"], w.chunk)
    else:
        for side, name in (("read", "q_scores"), ("write", "k_scores")):
            want, _ = port.select_routes(cpu[name].reshape(-1, cpu[name].shape[-1]), w.width)
            wrong += int((want != got[side]).any(-1).sum())
        host_bank = bank.cpu().clone()
        want_reads, _, _ = port.routed_read(host_bank, cpu["q_scores"], w.width)
        a, d, k = port.propose(host_bank, cpu["k_scores"], w.width, cpu["target"].float(), cpu["beta"], cpu["log_decay"],
                               None, 0, 0, w.chunk, 1)
        want_bank = port.commit(host_bank, a, d, k, in_place=True)
    want_reads = want_reads.reshape(-1, w.dim)
    keep = ~exempt["read"]
    read_err = float((got_reads[keep] - want_reads[keep]).abs().max() / want_reads.abs().max())
    loose = torch.zeros(w.slots, dtype=torch.bool)
    if exempt["write"].any():
        loose[got["write"][exempt["write"]].flatten()] = True     # rows a differently routed write may touch
        loose[port.flat_routes(sides["write"][exempt["write"]], host_keys, w.width)[0].flatten()] = True
    got_bank, want_bank = after.cpu().float().view(-1, w.dim), want_bank.float().view(-1, w.dim)
    bank_err = float((got_bank[~loose] - want_bank[~loose]).abs().max() / want_bank.abs().max())
    near = int(exempt["read"].sum() + exempt["write"].sum())
    agree = bool((every_digest == every_digest[0]).all())
    return {"workload": w.description + f", {world} rank(s), routing {routing}", "routing_rows": 2 * rows,
            "routes_identical": 2 * rows - near - wrong, "near_tie_exempt": near, "wrong": wrong,
            "ranks_agree_on_routes": agree, "readings_max_rel_err": read_err, "bank_max_rel_err": bank_err,
            "tolerance": 2e-2, "ok": wrong == 0 and agree and read_err <= 2e-2 and bank_err <= 2e-2,
            "checker": "oracle/torch_port.py on rank 0, outside the timed region"}


# ---- our arm ---------------------------------------------------------------------------------------

class Runner:
    """Binds a workload to the operator for one routing mode: device inputs and one epoch call."""

    def __init__(self, w, routing, dev, rank, world, dist, factored=True):
        import bench_workloads as workloads
        from gl_sdm_b200.operator import SharedBankOperator
        from gl_sdm_b200.sharded import ShardedBankOperator
        self.w, self.routing, self.dev, self.world = w, routing, dev, world
        seqs_local = w.sequences // world
        bank = workloads.make_bank(w, dev)
        if routing == "dense":
            keys = workloads.make_keys(w, dev)
            self.op = ShardedBankOperator(bank, w.width, w.width, dist, chunk_size=w.chunk, keys=keys, factored=factored)
            self.names = ("q", "kq", "target", "beta", "log_decay")
            self.epochs = [workloads.make_epoch_inputs_dense(w, dev, 1000 * (rank + 1) + e, seqs_local, keys=keys)
                           for e in range(w.epochs)]
            del keys
        else:
            self.op = (ShardedBankOperator(bank, w.width, w.width, dist, chunk_size=w.chunk, factored=factored)
                       if world > 1 else SharedBankOperator(bank, w.width, w.width, chunk_size=w.chunk, factored=factored))
            self.names = ("q_scores", "k_scores", "target", "beta", "log_decay")
            self.epochs = [workloads.make_epoch_inputs(w, dev, 1000 * (rank + 1) + e, seqs_local)
                           for e in range(w.epochs)]
        del bank

    def epoch(self, x):
        a = [x[n] for n in self.names]
        if self.routing == "dense":
            return self.op.epoch_dense(*a)
        return self.op.epoch(*a)

    def step(self):
        out = None
        for x in self.epochs:
            out = self.epoch(x)
        return out


def timed_steps(runner, steps, warmup, dist, dev):
    for _ in range(warmup):
        runner.step()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier(dist)
    start.record()
    for _ in range(steps):
        runner.step()
    stop.record()
    barrier(dist)
    return max_over_ranks(dist, start.elapsed_time(stop), dev) / steps


def phase_times_marks(runner):
    """Device time of every stage of one step (events recorded inside the sharded operator)."""
    op = runner.op
    op.marks = []
    runner.step()
    torch.cuda.synchronize()
    marks, op.marks = op.marks, None
    total = {}
    for (name, ev), (_, nxt) in zip(marks, marks[1:]):
        if name != "end":
            total[name] = total.get(name, 0.0) + ev.elapsed_time(nxt)
    return {k: v / len(runner.epochs) for k, v in total.items()}


def phase_times_pk(runner):
    op = runner.op
    phase = {"read": 0.0, "propose": 0.0, "commit": 0.0}
    marks, prop = [], None
    for x in runner.epochs:
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        ev[0].record()
        op.read(x["q_scores"])
        ev[1].record()
        if op.factored:
            prop = op.write_operands(x["k_scores"], x["target"], x["beta"], x["log_decay"])
            ev[2].record()
            op.commit_operands(*prop)
        else:
            prop = op.propose(x["k_scores"], x["target"], x["beta"], x["log_decay"])
            ev[2].record()
            op.commit(*prop)
        ev[3].record()
        marks.append(ev)
    torch.cuda.synchronize()
    for ev in marks:
        for i, name in enumerate(("read", "propose", "commit")):
            phase[name] += ev[i].elapsed_time(ev[i + 1])
    touched = prop[0].long().flatten() if op.factored else prop[0]   # one shared single-head-per-row address space
    if op.factored and op.heads > 1:
        touched = touched.view(-1, op.heads, prop[0].shape[-1]) + torch.arange(op.heads, device=touched.device).view(1, -1, 1) * op.slots
    unique = float(torch.unique(touched).numel()) / max(1, touched.numel())
    phase_times_pk.popularity = slot_popularity(touched)
    return {k: v / len(marks) for k, v in phase.items()}, unique


def slot_popularity(slots):
    """How the write routes of one epoch pile up on slots (the skewed configuration plants a
    Zipf popularity): entries, unique touched rows and their fraction u, the longest segment one
    address receives, the share of the entries that go to the 1 / 10 / 100 / 1000 most written
    slots, and the deciles of the per-slot entry counts over the touched slots."""
    flat = slots.reshape(-1).long()
    flat = flat[flat >= 0]
    counts = torch.bincount(flat).float()
    counts = counts[counts > 0].sort(descending=True).values
    entries = float(counts.sum())
    deciles = torch.quantile(counts, torch.linspace(0.1, 0.9, 9, device=counts.device)).tolist()
    share = {f"top_{k}": float(counts[:k].sum()) / entries for k in (1, 10, 100, 1000)}
    return {"entries": int(entries), "unique_rows": int(counts.numel()), "unique_row_fraction": counts.numel() / entries,
            "longest_segment": int(counts[0]), "share_of_entries": share,
            "deciles_of_entries_per_touched_slot": [round(d, 2) for d in deciles]}


def dense_roofline(w, runner, world, peaks, peak_kind):
    """score_topk against the measured bf16 tensor peak; the HBM-bound stages alongside."""
    phases = phase_times_marks(runner)
    tokens = w.tokens_per_epoch            # every rank scores ALL tokens of the epoch (both sides) ...
    shard_slots = w.slots // world         # ... against its own shard of the keys
    flops = 2.0 * (2 * tokens) * shard_slots * w.dk
    ms = phases["score_topk"]
    achieved = flops / (ms / 1e3) / 1e12
    e = 2 if w.bank_dtype == torch.bfloat16 else 4
    rows = 2 * tokens
    entries = getattr(runner.op, "last_entries", tokens * w.width // world)
    hbm = {
        "read": rows * (w.width * 8 + 4 * w.dim) + rows * w.width * w.dim * e / world,
        "propose": tokens * (w.dim + 1) * 4 + entries * (w.dim * e + 4 * w.dim + 16) + tokens * w.width * 8,
        "commit": entries * (4 * w.dim + 16) + entries * 2 * w.dim * e,
    }
    if getattr(runner.op, "factored", False):
        # no delta rows: the proposal stage only forms the error vectors (prediction in, errors out);
        # the commit reads a route per entry and an error vector per token, and updates each row once
        hbm["propose"] = tokens * ((w.dim + 1) * 4 + w.dim * 4 + w.dim * e + 8)
        hbm["commit"] = entries * 8 + tokens * (w.dim + 1) * 4 + entries * 2 * w.dim * e
    two_step_commit = entries * (4 * w.dim + 16) + entries * 2 * w.dim * e
    out = {"bound": "tensor", "kernel": "score_topk_wide_kernel (tcgen05 128x256x16 + TMEM + TMA, fused top-k)", "achieved": achieved,
           "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s", "frac": achieved / peaks["bf16_tflops_sustained"],
           "peak_kind": f"of {peak_kind} sustained cuBLAS bf16 (the kernel runs for >0.1 s inside a multi-second step)",
           "frac_of_burst_peak": achieved / peaks["bf16_tflops"], "frac_of_nominal_2250": achieved / NOMINAL_BF16_TFLOPS,
           "traffic": load_traffic("score_topk", w), "algorithmic_flops_per_launch": flops, "ms_per_launch": ms,
           "phases": {k: {"ms_per_epoch": v} for k, v in phases.items()}}
    if hasattr(runner.op, "last_routes"):
        out["slot_popularity"] = slot_popularity(runner.op.last_routes()[2])
    for name, nbytes in hbm.items():
        if name in phases and phases[name] > 0:
            gbs = nbytes / (phases[name] / 1e3) / 1e9
            out["phases"][name].update({"algorithmic_GBs": gbs, "frac_of_hbm_peak": gbs / peaks["hbm_gbs"]})
    if getattr(runner.op, "factored", False) and phases.get("commit", 0) > 0:
        # the same milliseconds against the bytes of a commit that reads materialised delta rows
        gbs = two_step_commit / (phases["commit"] / 1e3) / 1e9
        out["phases"]["commit"]["not_a_roofline"] = {
            "what": "the same milliseconds against the bytes a commit of materialised delta rows would move; the kernel "
                    "does not move them, so this is a comparison with the two-step design, not a roofline fraction",
            "delta_row_commit_equivalent_GBs": gbs, "delta_row_commit_equivalent_frac": gbs / peaks["hbm_gbs"]}
    return out


def pk_roofline(w, runner, world, peaks, peak_kind):
    import bench_workloads as workloads
    if world > 1:
        return pk_sharded_roofline(w, runner, world, peaks, peak_kind)
    phase, unique = phase_times_pk(runner)
    algo = workloads.algorithmic_bytes(w, w.tokens_per_epoch // world, unique, layers=1, factored=runner.op.factored)
    dominant = max(phase, key=phase.get)
    achieved = algo[dominant] / (phase[dominant] / 1e3) / 1e9
    extra = {}
    if runner.op.factored:
        plain = workloads.algorithmic_bytes(w, w.tokens_per_epoch // world, unique, layers=1, factored=False)
        gbs = plain["commit"] / (phase["commit"] / 1e3) / 1e9
        extra = {"not_a_roofline": {
            "what": "the same milliseconds against the bytes a commit of materialised delta rows would move; the kernel "
                    "does not move them, so this is a comparison with the two-step design, not a roofline fraction",
            "delta_row_commit_equivalent_GBs": gbs, "delta_row_commit_equivalent_frac": gbs / peaks["hbm_gbs"]}}
    names = ({"read": "pk_select_read_kernel", "propose": "pk_select_read_kernel + write_error_kernel",
              "commit": "factored commit (apply_split_kernel: single-writer rows straight from the routes, shared addresses from a sorted list)"} if runner.op.factored else
             {"read": "pk_select_read_kernel", "propose": "pk_propose_kernel", "commit": "commit (radix sort + reduce_kernel)"})
    return {"bound": "hbm", "kernel": names[dominant], "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
            "frac": achieved / peaks["hbm_gbs"], "peak_kind": f"of {peak_kind}",
            "frac_of_nominal_8TBs": achieved / NOMINAL_HBM_GBS, "traffic": load_traffic(dominant, w),
            "algorithmic_bytes_per_launch": algo[dominant], "ms_per_launch": phase[dominant],
            "phases": {k: {"ms_per_epoch": phase[k], "algorithmic_GBs": algo[k] / (phase[k] / 1e3) / 1e9,
                           "frac_of_hbm_peak": algo[k] / (phase[k] / 1e3) / 1e9 / peaks["hbm_gbs"],
                           **(extra if k == "commit" else {})} for k in phase},
            "unique_row_fraction": unique, "slot_popularity": getattr(phase_times_pk, "popularity", None)}


def pk_sharded_roofline(w, runner, world, peaks, peak_kind):
    """Sharded product-key mode: local routing of the rank's own tokens, then the shared
    read / proposal / commit stages over the rank's slots."""
    phases = phase_times_marks(runner)
    e = 2 if w.bank_dtype == torch.bfloat16 else 4
    local_rows = 2 * w.tokens_per_epoch * w.heads // world
    rows = 2 * w.tokens_per_epoch * w.heads
    entries = getattr(runner.op, "last_entries", w.tokens_per_epoch * w.width // world)
    algo = {
        "route": local_rows * (8 * w.half + 8 * w.width),
        "read": rows * (w.width * 8 + 4 * w.dim) + rows * w.width * w.dim * e / world,
        "propose": w.tokens_per_epoch * (w.dim + 1) * 4 + entries * (w.dim * e + 4 * w.dim + 16),
        "commit": entries * (4 * w.dim + 16) + entries * 2 * w.dim * e,
    }
    if getattr(runner.op, "factored", False):
        th = w.tokens_per_epoch * w.heads
        algo["propose"] = th * ((w.dim + 1) * 4 + w.dim * 4 + w.dim * e + 8) // world
        algo["commit"] = entries * 8 + th * (w.dim + 1) * 4 + entries * 2 * w.dim * e
    dominant = max((k for k in algo if k in phases), key=lambda k: phases[k])
    achieved = algo[dominant] / (phases[dominant] / 1e3) / 1e9
    return {"bound": "hbm", "kernel": {"route": "pk_select_kernel", "read": "snapshot_read_kernel (shard)",
                                       "propose": "shard_propose_kernel", "commit": "commit (radix sort + reduce_kernel)"}[dominant],
            "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
            "peak_kind": f"of {peak_kind}", "frac_of_nominal_8TBs": achieved / NOMINAL_HBM_GBS, "traffic": None,
            "algorithmic_bytes_per_launch": algo[dominant], "ms_per_launch": phases[dominant],
            "phases": {k: {"ms_per_epoch": v, **({"algorithmic_GBs": algo[k] / (v / 1e3) / 1e9,
                                                   "frac_of_hbm_peak": algo[k] / (v / 1e3) / 1e9 / peaks["hbm_gbs"]}
                                                  if k in algo and v > 0 else {})} for k, v in phases.items()}}


def load_traffic(kernel, w):
    """DRAM bytes per launch of a kernel from the committed ncu summary (profiles/traffic.json)."""
    path = os.path.join(ROOT, "profiles", "traffic.json")
    if not os.path.exists(path):
        return None
    with open(path) as f:
        table = json.load(f)
    entry = table.get(f"{w.name}:{kernel}")
    return None if entry is None else entry.get("dram_bytes_per_launch")


def end_to_end(args, w, runner, dev, dist, world):
    """Host-resident inputs: per epoch H2D of the operator inputs (double-buffered on a copy
    stream), the operator epoch, and D2H of the readings, all inside the timed region."""
    names, template = runner.names, runner.epochs[0]
    host = {k: torch.empty(template[k].shape, dtype=template[k].dtype).pin_memory() for k in names}
    for k in names:
        host[k].copy_(template[k])
    slots = [{k: torch.empty_like(template[k]) for k in names} for _ in range(2)]
    readings_host = torch.empty((*template["beta"].shape[:2], w.heads, w.dim), dtype=torch.float32).pin_memory()
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
            out = runner.epoch(slots[cur])
            freed[cur].record(main)
            readings_host.copy_(out.view(readings_host.shape), non_blocking=True)
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


def ours(args, w, rank, world, local, dist):
    from gl_sdm_b200 import _native
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    lib = _native.library()
    peaks, peak_kind = measured_peaks()
    parity = None if args.no_parity else parity_check(args.routing, rank, world, dist, dev)
    runner = Runner(w, args.routing, dev, rank, world, dist, not args.delta_rows)
    for _ in range(args.warmup):
        runner.step()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = lib.glsdm_kernel_launches()
    ms_per_step = timed_steps(runner, args.steps, 0, dist, dev)
    launches = lib.glsdm_kernel_launches() - launches0
    clocks = sampler.stop() if rank == 0 else None
    _native.raise_on_device_status(dev)
    value = w.tokens_per_step / (ms_per_step / 1e3)
    roofline = (dense_roofline if args.routing == "dense" else pk_roofline)(w, runner, world, peaks, peak_kind)
    e2e = None if args.no_e2e else end_to_end(args, w, runner, dev, dist, world)

    extra = None
    if args.routing == "dense" and not args.no_pk_block:
        del runner
        torch.cuda.empty_cache()
        pk = Runner(w, "pk", dev, rank, world, dist, not args.delta_rows)
        pk_ms = timed_steps(pk, args.steps, args.warmup, dist, dev)
        extra = {"note": "same workload with the reference's operator contract: factor scores [tokens, 2*half] fp32 in",
                 "value": w.tokens_per_step / (pk_ms / 1e3), "unit": "tokens/s", "ms_per_step": pk_ms,
                 "roofline": pk_roofline(w, pk, world, peaks, peak_kind),
                 "parity": None if args.no_parity else parity_check("pk", rank, world, dist, dev)}
        del pk
        torch.cuda.empty_cache()
        if world == 1 and not args.no_cpu_baseline:
            extra["torch_on_gpu"] = run_torch_on_gpu(w, dev)
            torch.cuda.empty_cache()

    if rank != 0:
        return
    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        tokens = args.cpu_sample_tokens or (256 if args.routing == "dense" else 8192)
        kind, measured = "reference", None
        if enough_host_memory(w):
            measured = run_cpu_reference(w, args.routing, 1, 1, tokens, threads)
        if measured is None:
            kind, measured = "port", (*run_cpu_port(w, args.routing, 1, 1, tokens, threads), 1)
        cv, n, sec, _ = measured
        cpu = {"value": cv, "unit": "tokens/s", "cores": threads, "kind": kind,
               "sample": (reference_sample_text if kind == "reference" else cpu_sample_text)(w, args.routing, n, sec)}
    line = {
        "metric": "memory-op tokens/s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None,
        "dtype": ("bf16 tensor-core scores, " if args.routing == "dense" else "") + "f32 accumulate over %s bank" % bank_dtype_name(w),
        "data": "synthetic", "config": workload_config(w, args, world), "roofline": roofline, "cpu_baseline": cpu,
        "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks, "parity": parity,
    }
    if extra is not None:
        line["product_key_scores"] = extra
    emit(json.dumps(line))


def main():
    import bench_workloads as workloads
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c4", choices=sorted(workloads.WORKLOADS))
    ap.add_argument("--routing", default="dense", choices=["dense", "pk"])
    ap.add_argument("--sequences", type=int, default=None, help="override the batch (sequences per step)")
    ap.add_argument("--seq-len", type=int, default=None)
    ap.add_argument("--cpu-sample-tokens", type=int, default=0, help="0 = 256 (dense) / 8192 (pk)")
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-input pass (profiling runs)")
    ap.add_argument("--delta-rows", action="store_true",
                    help="write the proposal's delta rows to memory and commit them (the two-step path) instead of the "
                         "factored commit")
    ap.add_argument("--no-pk-block", action="store_true", help="skip the attached product-key-scores measurement")
    ap.add_argument("--stack", action="store_true",
                    help="with --workload c2: drive the reference's own 16-layer model (staged under oracle/_ref), "
                         "unmodified, over this package instead of the memory API alone")
    ap.add_argument("--train", action="store_true",
                    help="with --stack: also time a forward + backward step (8 x 2048 tokens)")
    ap.add_argument("--no-parity", action="store_true", help="skip the small checked epoch that precedes the timing")
    args = ap.parse_args()
    claim_stdout()
    w = workloads.WORKLOADS[args.workload]
    if args.sequences or args.seq_len:
        w = w.scaled(args.sequences, args.seq_len)
    rank, world, local, dist = dist_setup(args)
    if args.stack:
        if args.workload != "c2":
            raise SystemExit("--stack runs configuration c2 (the reference's own model)")
        (stack_reference_arm if args.impl == "reference" else stack_arm)(args, w, rank)
        if dist is not None:
            dist.destroy_process_group()
        return
    if args.impl == "reference":
        reference_arm(args, w, rank)
        return
    if w.per_request_banks:
        per_request_arm(args, w, rank)
        if dist is not None:
            dist.destroy_process_group()
        return
    if w.sequences % world:
        raise SystemExit("sequences per step must divide over the ranks")
    ours(args, w, rank, world, local, dist)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
