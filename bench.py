#!/usr/bin/env python
"""Benchmark of the decode-attention hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload c1|c2|c3|c4|c5|ref_b1|...] [--scaling weak|strong]

One "step" is one decode-attention call over one batch of synthetic KV cache.
The default workload is benchmark configuration 2 (Llama-3-8B-shaped GQA
decode: batch 32, 32 query / 8 kv heads, head dim 128, 4096 cache rows, bf16,
K and V ~ 0.5 * N(0,1)). Prints ONE JSON line.

metric / value : algorithmic KV-read bandwidth, GB/s, whole job, inputs
                 resident in HBM: bytes = sum_b len_b*Hkv*D*2*sizeof + 2*B*Hq*D*sizeof
                 per step, divided by the CUDA-event time of the timed steps
                 (max over ranks). The region of `--steps` back-to-back steps is
                 timed `--rounds` times (default 5); `value` is the median round
                 and `rounds_ms_per_step` lists them all.
kv_split,
c2_strong      : (N > 1, default workload) two more measurements in the same
                 line: configuration 4 with the KV length split over the N GPUs
                 (the one path with an exchange between GPUs) and configuration
                 2 with its batch of 32 divided over the N GPUs.
e2e            : the same metric through the public Python operator with the
                 step's inputs (q, lens) copied from pinned host memory and the
                 result copied back and read, every step. The KV cache is decode
                 STATE (it persists on the device between steps), not a step
                 input; `e2e_staged` additionally reports the staged entry point
                 that copies the whole cache from host memory each call.
e2e_graph      : (N=1) the same end-to-end step captured once and replayed as a
                 CUDA graph; information beside `e2e`, never instead of it.
roofline       : HBM bound; achieved = algorithmic bytes / step time (partial
                 kernel incl. its in-kernel merge, plus the launch gap between
                 steps); peak = measured copy bandwidth; `read_only_stream`
                 (N=1) = a read-only pass of the library's own streaming kernel,
                 measured live, and the fraction of it that was achieved.
decode_step    : (N=1, contiguous) the whole step on the device: rope of q and k_new +
                 cache write (one launch) followed by the attention kernel.
cpu_baseline   : the reference's own CPU implementation (built from the
                 reference sources) or, where that build is absent, the C
                 restatement, on the host cores, on a bounded sample.

`--impl reference` times that CPU implementation alone, on all host cores.
"""

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

L2_BYTES = 126 * 1024 * 1024
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the decode
# kernel on a workload, from an ncu capture of that kernel on that workload
# (profiles/: not re-measured by this script, a profiler cannot run inside a
# timed benchmark). Workloads without a capture report null.
NCU_TRAFFIC_BYTES = {"c2": 541281280, "c3": 1118520704, "c2_f32": 1078616368}

WORKLOADS = {
    # name: (batch, q heads, kv heads, dim, rows, dtype, paged, description)
    "c2": dict(B=32, Hq=32, Hkv=8, D=128, T=4096, dtype="bf16", paged=False, kv_scale=0.5,
               desc="config 2: Llama-3-8B GQA decode, contiguous cache"),
    "c3": dict(B=64, Hq=32, Hkv=8, D=128, T=8192, dtype="fp16", paged=True, kv_scale=1.0, lens="uniform",
               desc="config 3: paged, ragged lengths U[128,8192], page 16"),
    "c4": dict(B=4, Hq=64, Hkv=8, D=128, T=131072, dtype="bf16", paged=False, kv_scale=1.0,
               desc="config 4: long-context split-KV (KV length split across GPUs when N>1)"),
    "c5": dict(B=256, Hq=40, Hkv=8, D=128, T=32768, dtype="bf16", paged=True, kv_scale=1.0, lens="loguniform",
               desc="config 5: serving mix, paged, lengths log-uniform [1024,32768], graph replay"),
    "c1": dict(B=1, Hq=8, Hkv=8, D=64, T=512, dtype="f32", paged=False, kv_scale=1.0,
               desc="config 1: single sequence, MHA, fp32 (2 MB: launch-bound, L2-resident without rotation)"),
    "ref_b1_f32": dict(B=1, Hq=32, Hkv=8, D=128, T=16384, dtype="f32", paged=False, kv_scale=1.0,
                       desc="the reference's own benchmark shape in float32 (batch 1, T=16384)"),
    "c2_f32": dict(B=32, Hq=32, Hkv=8, D=128, T=4096, dtype="f32", paged=False, kv_scale=0.5,
                   desc="config 2's shape with a float32 cache (CUDA-core kernel)"),
    "ref_b1": dict(B=1, Hq=32, Hkv=8, D=128, T=16384, dtype="bf16", paged=False, kv_scale=1.0,
                   desc="the reference's own benchmark shape (batch 1, T=16384)"),
}


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def read_only_stream_gbs(torch, device):
    """Bandwidth of a read-only pass over a buffer far larger than L2 (the library's read_stream kernel),
    or None if this build of the library lacks it."""
    from fusedtok_b200 import _fusedtok
    fn = getattr(_fusedtok._lib, "fusedtok_debug_read_stream", None)
    if fn is None:
        return None
    nbytes = 2 << 30
    buf = torch.empty(nbytes, dtype=torch.uint8, device=device)
    buf.zero_()
    stream = torch.cuda.current_stream().cuda_stream
    for _ in range(3):
        if fn(buf.data_ptr(), nbytes, stream) != 0:
            return None
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(10):
        fn(buf.data_ptr(), nbytes, stream)
    e1.record()
    torch.cuda.synchronize()
    del buf
    return nbytes * 10 / (e0.elapsed_time(e1) * 1e-3) / 1e9


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed
    region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.QUERY,
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [x.strip() for x in ln.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ---------------------------------------------------------------------------
# workload construction
# ---------------------------------------------------------------------------

def make_lens(w, batch):
    import numpy as np
    import cases
    kind = w.get("lens")
    if kind == "uniform":
        return cases.config3_lens(batch)
    if kind == "loguniform":
        return cases.config5_lens(batch)
    if kind == "full" or (kind is None and w["paged"]):
        return np.full(batch, w["T"], np.int32)
    return None


def algorithmic_bytes(w, lens, batch):
    es = 4 if w["dtype"] == "f32" else 2
    rows = int(lens.sum()) if lens is not None else batch * w["T"]
    return rows * w["Hkv"] * w["D"] * 2 * es + 2 * batch * w["Hq"] * w["D"] * es


def build_inputs(w, batch, device, seed, n_sets):
    """Device-resident q, K/V (n_sets independent copies to defeat L2 where one
    copy would fit in it), lens / block table."""
    import numpy as np
    import torch
    import cases
    dt = {"bf16": torch.bfloat16, "fp16": torch.float16, "f32": torch.float32}[w["dtype"]]
    g = torch.Generator(device=device).manual_seed(seed)
    lens = make_lens(w, batch)
    q = torch.randn(batch, w["Hq"], w["D"], device=device, generator=g).to(dt)
    sets = []
    table = None
    if w["paged"]:
        table_np, nb, width = cases.paged_layout(lens)
        table = torch.from_numpy(table_np).to(device)
        shape = (nb, w["Hkv"], 16, w["D"])
    else:
        shape = (batch, w["Hkv"], w["T"], w["D"])
    for _ in range(n_sets):
        k = torch.empty(shape, device=device, dtype=dt)
        v = torch.empty(shape, device=device, dtype=dt)
        # fill in slabs to bound the fp32 temporaries
        for t, in ((k,), (v,)):
            flat = t.view(-1)
            step = 1 << 26
            for o in range(0, flat.numel(), step):
                n = min(step, flat.numel() - o)
                flat[o:o + n] = (torch.randn(n, device=device, generator=g) * w["kv_scale"]).to(dt)
        sets.append((k, v))
    lens_t = torch.from_numpy(lens).to(device) if lens is not None else None
    return q, sets, lens_t, table, lens


# ---------------------------------------------------------------------------
# CPU baseline (reference implementation on the host cores)
# ---------------------------------------------------------------------------

def cpu_baseline(w, target_seconds, threads):
    """Times the reference's CPU decode attention on `threads` host threads,
    each looping over single-sequence calls of the workload's shape (float32
    values; the CPU path is float32 only). Returns (GB/s of the workload's
    algorithmic bytes, description)."""
    import numpy as np
    import oracle
    kind = "reference" if oracle.ref_available() else "port"
    fn = oracle.ref_decode if kind == "reference" else oracle.decode
    if kind == "port":
        oracle.decode(np.zeros((1, 1, 4), np.float32), np.zeros((1, 1, 1, 4), np.float32),
                      np.zeros((1, 1, 1, 4), np.float32))
    t_rows = min(w["T"], 4096)
    rng = np.random.default_rng(0)
    q = rng.standard_normal((1, w["Hq"], w["D"])).astype(np.float32)
    data = []
    for _ in range(threads):
        k = (rng.standard_normal((1, w["Hkv"], t_rows, w["D"])) * w["kv_scale"]).astype(np.float32)
        data.append((k, k.copy()))
    t0 = time.perf_counter()
    fn(q, data[0][0], data[0][1])
    one = time.perf_counter() - t0
    reps = max(1, int(target_seconds / max(one, 1e-4)))

    def work(i):
        for _ in range(reps):
            fn(q, data[i][0], data[i][1])

    ths = [threading.Thread(target=work, args=(i,)) for i in range(threads)]
    t0 = time.perf_counter()
    for t in ths:
        t.start()
    for t in ths:
        t.join()
    dt = time.perf_counter() - t0
    es = 4 if w["dtype"] == "f32" else 2
    bytes_per_seq = t_rows * w["Hkv"] * w["D"] * 2 * es + 2 * w["Hq"] * w["D"] * es
    seqs = threads * reps
    gbs = seqs * bytes_per_seq / dt / 1e9
    sample = ("%d single-sequence calls (%d threads x %d) of shape Hq=%d Hkv=%d D=%d T=%d, float32 values, "
              "%.1f s; bytes counted at the workload's storage width"
              % (seqs, threads, reps, w["Hq"], w["Hkv"], w["D"], t_rows, dt))
    return gbs, seqs / dt, kind, sample, dt


def run_reference_arm(args, w, rank):
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    per_step = min(8.0, max(0.3, 60.0 / args.steps))
    for _ in range(args.warmup):
        cpu_baseline(w, 0.2, threads)
    vals, seqs, total_t = [], [], 0.0
    kind = sample = None
    for _ in range(args.steps):
        gbs, sps, kind, sample, dt = cpu_baseline(w, per_step, threads)
        vals.append(gbs)
        seqs.append(sps)
        total_t += dt
    value = sum(vals) / len(vals)
    line = {
        "impl": "reference", "metric": "decode_attn_kv_read_GBps", "value": value, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": total_t / args.steps * 1e3, "higher_is_better": True, "scaling": args.scaling,
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "seq_steps_per_s": sum(seqs) / len(seqs),
        "config": {"workload": args.workload + ": " + w["desc"] + " (CPU sample, see cpu_baseline.sample)"},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------

def multi_gpu_extras(args, torch, dist, device, rank, world, c2_weak_ms_step, barrier):
    """Two more measurements for the N > 1 line (every rank calls this; the returned dict matters on rank 0):

    kv_split  - configuration 4 (batch 4, 64/8 heads, 131072 rows, bf16) with the KV length split over the
                `world` GPUs: per step every rank streams its 1/N of the rows, the ranks exchange the raw
                (m, l, acc) triples over NVLink and every rank folds them. Beside it, measured in the same
                process: one rank's 1/N share WITHOUT the exchange (what the split can at best reach) and
                the whole configuration on ONE GPU (what it is a speed-up over).
    c2_strong - configuration 2 with its batch of 32 divided over the GPUs (no communication); the
                single-GPU time it is compared with is this run's own headline (same per-GPU work)."""
    from fusedtok_b200 import _fusedtok
    steps, rounds = args.steps, max(3, min(args.rounds, 5))
    out = {}

    def measure(case):
        for i in range(5):
            case.step(i)
        torch.cuda.synchronize()
        r = timed_rounds(torch, case.step, steps, rounds, barrier)
        r = max_over_ranks(torch, dist, device, r)
        return statistics.median(r) / steps, [x / steps for x in r]

    # ---- configuration 4, KV length split
    w4 = dict(WORKLOADS["c4"])
    if w4["T"] % world == 0:
        split = Case(w4, w4["B"], device, seed=100 + rank, mode="split", world=world, group=dist.group.WORLD,
                     exchange=args.exchange, dist=dist)
        ms_split, split_rounds = measure(split)
        status = _fusedtok.attention_device_status()
        st = torch.tensor([float(status)], device=device, dtype=torch.float64)
        dist.all_reduce(st, op=dist.ReduceOp.MAX)
        # the same per-rank rows through the ordinary operator: no exchange, no merge across GPUs
        local = Case(split.wl, w4["B"], device, seed=100 + rank)
        local.sets, local.n_sets = split.sets, split.n_sets          # same tensors
        ms_local, _ = measure(local)
        bytes_total = algorithmic_bytes(w4, None, w4["B"])
        split.close()
        del split, local
        torch.cuda.empty_cache()
        # the whole configuration on one GPU, timed on rank 0 while the others wait at the barrier
        ms_full = 0.0
        if rank == 0:
            full = Case(w4, w4["B"], device, seed=100)
            for i in range(5):
                full.step(i)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            vals = []
            for _ in range(3):
                e0.record()
                for i in range(steps):
                    full.step(i)
                e1.record()
                torch.cuda.synchronize()
                vals.append(e0.elapsed_time(e1) / steps)
            ms_full = statistics.median(vals)
            full.close()
            del full
            torch.cuda.empty_cache()
        barrier()
        out["kv_split"] = {
            "workload": "c4: " + w4["desc"], "n_gpus": world, "exchange": args.exchange,
            "launches_per_step_per_gpu": 1 if args.exchange == "p2p" else 3,
            "ms_per_step": ms_split, "rounds_ms_per_step": split_rounds,
            "GBps": bytes_total / (ms_split * 1e-3) / 1e9, "seq_steps_per_s": w4["B"] / (ms_split * 1e-3),
            "single_gpu_ms_per_step": ms_full,
            "speedup_vs_single_gpu": (ms_full / ms_split) if ms_full else None,
            "local_share_ms_per_step": ms_local,
            "speedup_bound_from_local_share": (ms_full / ms_local) if ms_full else None,
            "exchange_and_sync_ms_per_step": ms_split - ms_local,
            "device_status": int(st.item()),
            "note": "KV length 131072 split over the GPUs; (m, l, acc) of every finished unit stored into every "
                    "rank's buffer over NVLink and folded at the end of the same kernel; times are the max over "
                    "ranks per round, median round; single_gpu = the whole configuration on rank 0's GPU",
        }
    # ---- configuration 2, batch divided over the GPUs
    w2 = dict(WORKLOADS["c2"])
    if w2["B"] % world == 0:
        strong = Case(w2, w2["B"] // world, device, seed=200 + rank)
        ms_strong, strong_rounds = measure(strong)
        bytes_total = algorithmic_bytes(w2, None, w2["B"])
        n_sets = strong.n_sets
        strong.close()
        del strong
        torch.cuda.empty_cache()
        out["c2_strong"] = {
            "workload": "c2: " + w2["desc"], "n_gpus": world, "batch_per_gpu": w2["B"] // world,
            "ms_per_step": ms_strong, "rounds_ms_per_step": strong_rounds,
            "GBps": bytes_total / (ms_strong * 1e-3) / 1e9, "seq_steps_per_s": w2["B"] / (ms_strong * 1e-3),
            "single_gpu_ms_per_step": c2_weak_ms_step,
            "speedup_vs_single_gpu": c2_weak_ms_step / ms_strong,
            "l2": "rotating over %d independent K/V sets so reads come from HBM" % n_sets,
            "note": "batch 32 divided over the GPUs, no communication; single_gpu = this line's own ms_per_step "
                    "(batch 32 on every GPU)",
        }
    return out


class Case:
    """One workload as one rank runs it: inputs resident on the device, one `step(i)` call per decode step.

    mode "plain": the ordinary operator on this rank's batch; "split": configuration-4 style KV-length split
    (this rank holds rows/world of every sequence, partials exchanged between the GPUs)."""

    def __init__(self, w, batch, device, seed, mode="plain", world=1, group=None, exchange="p2p", dist=None):
        import torch
        from fusedtok_b200 import _fusedtok
        self.w = w
        self.batch = batch
        self.mode = mode
        self.wl = dict(w)
        if mode == "split":
            assert w["T"] % world == 0
            self.wl["T"] = w["T"] // world            # this rank's slice of the cache rows
        es = 4 if w["dtype"] == "f32" else 2
        self.kv_bytes = 2 * batch * w["Hkv"] * self.wl["T"] * w["D"] * es
        self.n_sets = 1 if self.kv_bytes >= 3 * L2_BYTES else int(math.ceil(3 * L2_BYTES / self.kv_bytes))
        self.q, self.sets, self.lens_t, self.table, self.lens_np = build_inputs(self.wl, batch, device, seed,
                                                                                self.n_sets)
        self.bytes_step = algorithmic_bytes(self.wl, self.lens_np, batch)
        self.out = torch.empty_like(self.q)
        self.sfx = {"f32": "", "bf16": "_bf16", "fp16": "_fp16"}[w["dtype"]]
        self.lens_ptr = self.lens_t.data_ptr() if self.lens_t is not None else 0
        self.dec = None
        self.exchange = exchange
        if mode == "split":
            from fusedtok_b200 import sharded
            cls = sharded.PeerSplitKVDecoder if exchange == "p2p" else sharded.SplitKVDecoder
            self.dec = cls(batch, w["Hq"], w["Hkv"], w["D"], self.q.dtype, device, group)
        self._ft = _fusedtok
        self._torch = torch

    def step(self, i):
        w, wl = self.w, self.wl
        k, v = self.sets[i % self.n_sets]
        stream = self._torch.cuda.current_stream()      # the capture stream while a graph is being recorded
        if self.dec is not None:
            self.dec.decode(self.q, k, v, None, self.out)
        elif w["paged"]:
            getattr(self._ft, "attention_decode_paged_launch" + self.sfx)(
                self.q.data_ptr(), k.data_ptr(), v.data_ptr(), self.table.data_ptr(), self.lens_ptr,
                self.out.data_ptr(), self.batch, w["Hq"], w["Hkv"], 16, self.table.shape[1], w["D"],
                stream.cuda_stream)
        else:
            getattr(self._ft, "attention_decode_launch" + self.sfx)(
                self.q.data_ptr(), k.data_ptr(), v.data_ptr(), self.lens_ptr, self.out.data_ptr(),
                self.batch, w["Hq"], w["Hkv"], wl["T"], w["D"], stream.cuda_stream)

    def launches_per_step(self):
        if self.dec is None or self.exchange == "p2p":
            return 1
        return 3            # partial kernel, NCCL all-gather, merge kernel

    def close(self):
        if self.dec is not None and hasattr(self.dec, "close"):
            self._torch.cuda.synchronize()
            self.dec.close()
        self.sets = None


def timed_rounds(torch, run, steps, rounds, barrier):
    """`rounds` regions of exactly `steps` back-to-back calls of run(i), each bracketed by a barrier and a
    device synchronize on both sides and timed with CUDA events on the launching stream. Returns the
    per-round times in ms."""
    out = []
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    n = 0
    for _ in range(rounds):
        barrier()
        e0.record()
        for _ in range(steps):
            run(n)
            n += 1
        e1.record()
        barrier()
        out.append(e0.elapsed_time(e1))
    return out


def max_over_ranks(torch, dist, device, values):
    """Element-wise maximum of a list of floats over the ranks (identity on one GPU)."""
    if dist is None:
        return list(values)
    t = torch.tensor(list(values), device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(x) for x in t]


def run_ours(args, w, rank, world, local_rank):
    import numpy as np
    import torch
    import fusedtok_b200 as ft
    from fusedtok_b200 import _fusedtok

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU path")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=device)

    split_kv = args.workload == "c4" and world > 1
    # work per rank
    if args.scaling == "weak" or world == 1 or split_kv:
        batch = w["B"]
    else:
        assert w["B"] % world == 0, "strong scaling shards the batch evenly"
        batch = w["B"] // world
    case = Case(w, batch, device, seed=rank, mode="split" if split_kv else "plain", world=world,
                group=dist.group.WORLD if dist else None, exchange=args.exchange, dist=dist)
    wl, n_sets, bytes_step, kv_bytes = case.wl, case.n_sets, case.bytes_step, case.kv_bytes
    q, sets, lens_t, table, out = case.q, case.sets, case.lens_t, case.table, case.out
    sfx, lens_ptr, dec = case.sfx, case.lens_ptr, case.dec
    stream = torch.cuda.current_stream()
    dt_code = {"f32": 0, "bf16": 1, "fp16": 2}[w["dtype"]]
    step = case.step

    use_graph = args.graph or args.workload == "c5"
    graphs = None
    for i in range(max(args.warmup, 3)):
        step(i)
    torch.cuda.synchronize()
    if use_graph and not (split_kv and args.exchange == "nccl"):      # (capturing the collective is left to the caller)
        graphs = []
        for i in range(n_sets):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                step(i)
            graphs.append(g)
        for g in graphs:
            g.replay()
        torch.cuda.synchronize()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def run(i):
        if graphs:
            graphs[i % n_sets].replay()
        else:
            step(i)

    # ---- device-timed regions: `rounds` x exactly K steps, inputs resident
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    _fusedtok.attention_launch_count(reset=True)
    round_ms = timed_rounds(torch, run, args.steps, 1 if args.profile else args.rounds, barrier)
    launches = (_fusedtok.attention_launch_count() if not graphs else len(round_ms) * args.steps) // len(round_ms)
    if dec is not None and args.exchange == "nccl":
        launches = args.steps * case.launches_per_step()
    ms = statistics.median(round_ms)
    if args.profile:
        print(json.dumps({"profile_run": True, "ms_per_step": ms / args.steps, "workload": args.workload,
                          "GBps": bytes_step / (ms / args.steps * 1e-3) / 1e9}), flush=True)
        if rank == 0:
            sampler.stop()
        return
    # a few more steps keep the clock sampler busy long enough to see the load
    t_end = time.perf_counter() + 1.0
    j = 0
    while time.perf_counter() < t_end:
        for _ in range(50):
            run(j)
            j += 1
        torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None
    status = _fusedtok.attention_device_status()

    # ---- end-to-end region through the public operator: q, lens from pinned host memory
    q_host = q.cpu().pin_memory()
    out_host = torch.empty_like(q_host).pin_memory()
    lens_host = lens_t.cpu().pin_memory() if lens_t is not None else None
    q_dev = torch.empty_like(q)
    lens_dev = torch.empty_like(lens_t) if lens_t is not None else None

    def e2e_step(i):
        k, v = sets[i % n_sets]
        q_dev.copy_(q_host, non_blocking=True)
        if lens_dev is not None:
            lens_dev.copy_(lens_host, non_blocking=True)
        if split_kv:
            o = torch.empty_like(q_dev)
            dec.decode(q_dev, k, v, None, o)
        elif w["paged"]:
            if w["Hq"] // w["Hkv"] in (1, 2, 4, 8, 16):
                o = ft.attention_decode_paged(q_dev, k, v, table, lens_dev)
            else:   # the wrapper keeps the reference's group rule; the launcher is the public entry for other groups
                o = torch.empty_like(q_dev)
                getattr(_fusedtok, "attention_decode_paged_launch" + sfx)(
                    q_dev.data_ptr(), k.data_ptr(), v.data_ptr(), table.data_ptr(), lens_dev.data_ptr(),
                    o.data_ptr(), batch, w["Hq"], w["Hkv"], 16, table.shape[1], w["D"], stream.cuda_stream)
        else:
            o = ft.attention_decode(q_dev, k, v, lens_dev)
        out_host.copy_(o, non_blocking=True)
        torch.cuda.synchronize()
        return float(out_host[0, 0, 0])     # the host reads the result

    for i in range(3):
        e2e_step(i)
    e2e_rounds = []
    for _ in range(3):
        barrier()
        t0 = time.perf_counter()
        for i in range(args.steps):
            e2e_step(i)
        barrier()
        e2e_rounds.append(time.perf_counter() - t0)
    h2d = q_host.numel() * q_host.element_size() + (lens_host.numel() * 4 if lens_host is not None else 0)
    d2h = out_host.numel() * out_host.element_size()

    # ---- the same end-to-end step replayed from a CUDA graph (one graph per K/V set: copy in, decode, copy
    # out), as a latency-conscious caller of the capturable launchers would run it. Reported beside `e2e`,
    # never instead of it. Single GPU, plain batch-sharded workloads only.
    e2e_graph_s = None
    if dist is None and not split_kv and not args.profile and (not w["paged"] or w["Hq"] // w["Hkv"] in (1, 2, 4, 8, 16)):
        try:
            side = torch.cuda.Stream()
            step_graphs = []
            with torch.cuda.stream(side):
                for si in range(n_sets):
                    k, v = sets[si]
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=side):
                        q_dev.copy_(q_host, non_blocking=True)
                        if lens_dev is not None:
                            lens_dev.copy_(lens_host, non_blocking=True)
                        o = (ft.attention_decode_paged(q_dev, k, v, table, lens_dev) if w["paged"]
                             else ft.attention_decode(q_dev, k, v, lens_dev))
                        out_host.copy_(o, non_blocking=True)
                    step_graphs.append(g)
            torch.cuda.synchronize()

            def e2e_graph_step(i):
                step_graphs[i % n_sets].replay()
                torch.cuda.synchronize()
                return float(out_host[0, 0, 0])

            for i in range(3):
                e2e_graph_step(i)
            rounds_g = []
            for _ in range(3):
                t0 = time.perf_counter()
                for i in range(args.steps):
                    e2e_graph_step(i)
                rounds_g.append(time.perf_counter() - t0)
            e2e_graph_s = statistics.median(rounds_g)
            del step_graphs
        except Exception as exc:      # capture refused by this torch build: the plain figure stands alone
            print("e2e graph variant skipped: %r" % (exc,), file=sys.stderr)

    # ---- max over ranks (round by round), then the median round
    round_ms = max_over_ranks(torch, dist, device, round_ms)
    e2e_rounds = max_over_ranks(torch, dist, device, e2e_rounds)
    ms = statistics.median(round_ms)
    e2e_s = statistics.median(e2e_rounds)
    if dist is not None:
        tot = torch.tensor([float(bytes_step), float(batch)], device=device, dtype=torch.float64)
        dist.all_reduce(tot, op=dist.ReduceOp.SUM)
        job_bytes, job_seqs = float(tot[0]), float(tot[1])
        if split_kv:
            job_seqs = float(batch)            # every rank works on the same sequences
    else:
        job_bytes, job_seqs = float(bytes_step), float(batch)

    # ---- N > 1, default workload: the multi-GPU paths the headline does not cover
    extra = {}
    if dist is not None and args.workload == "c2" and not args.no_multi_extras:
        case.close()
        del sets, case
        torch.cuda.empty_cache()
        extra = multi_gpu_extras(args, torch, dist, device, rank, world, ms / args.steps, barrier)

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    ms_step = ms / args.steps
    value = job_bytes / (ms_step * 1e-3) / 1e9
    e2e_value = job_bytes / (e2e_s / args.steps) / 1e9
    peak, peak_kind = measured_peak()
    per_gpu = bytes_step / (ms_step * 1e-3) / 1e9
    line = {
        "metric": "decode_attn_kv_read_GBps", "value": value, "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
        "rounds": len(round_ms), "rounds_ms_per_step": [r / args.steps for r in round_ms],
        "higher_is_better": True, "scaling": "strong" if split_kv else args.scaling,
        "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic",
        "seq_steps_per_s": job_seqs / (ms_step * 1e-3),
        "pct_of_8TBs_per_gpu": 100.0 * per_gpu / NOMINAL_HBM_GBS,
        "config": {
            "workload": args.workload + ": " + w["desc"],
            "batch_per_gpu": batch, "q_heads": w["Hq"], "kv_heads": w["Hkv"], "head_dim": w["D"],
            "cache_rows": wl["T"], "paged": w["paged"], "page": 16 if w["paged"] else None,
            "algorithmic_bytes_per_step_per_gpu": bytes_step,
            "l2": ("inputs larger than L2 (%.0f MB of K/V per step)" % (kv_bytes / 1e6)) if n_sets == 1 else
                  ("rotating over %d independent K/V sets (%.0f MB each) so reads come from HBM" % (n_sets, kv_bytes / 1e6)),
            "parallelism": ("kv-length split x%d, %s exchange of (m,l,acc) + merge" % (world, args.exchange)) if split_kv else
                           ("batch-sharded x%d, no communication" % world),
            "cuda_graph": bool(graphs),
            "timing": "%d rounds of %d back-to-back steps, CUDA events, max over ranks per round, median round"
                      % (len(round_ms), args.steps),
        },
        "roofline": {"bound": "hbm", "achieved": per_gpu, "peak": peak, "unit": "GB/s",
                     "frac": per_gpu / peak, "peak_kind": "of " + peak_kind,
                     "traffic": NCU_TRAFFIC_BYTES.get(args.workload),
                     "traffic_source": "ncu capture of one launch of this kernel on this workload, taken separately",
                     "note": "achieved = algorithmic bytes / whole step time (one kernel per step, launch gaps included); "
                             "the peak is a copy (read + write) bandwidth while this kernel almost only reads, so "
                             "a fraction slightly above 1 is possible"},
        "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_s / args.steps * 1e3,
                "rounds_ms_per_step": [r / args.steps * 1e3 for r in e2e_rounds],
                "note": "public operator; q/lens H2D from pinned memory and result D2H + host read every step; "
                        "KV cache is device-resident decode state"},
        "gpu_launches": launches,
        "device_status": status,
        "clocks": clocks,
    }
    if e2e_graph_s is not None:
        line["e2e_graph"] = {"value": job_bytes / (e2e_graph_s / args.steps) / 1e9, "unit": "GB/s",
                             "ms_per_step": e2e_graph_s / args.steps * 1e3,
                             "note": "the e2e step (H2D of q/lens from pinned memory, decode, D2H of the result) "
                                     "captured once per K/V set and replayed as a CUDA graph, then synchronised and "
                                     "read on the host every step"}
    if world == 1 and not args.profile:
        rs = read_only_stream_gbs(torch, device)
        if rs:
            line["roofline"]["read_only_stream"] = {
                "GBps": rs, "frac": per_gpu / rs,
                "note": "this library's plain-load kernel reading a 2 GiB buffer once (CUDA events, 10 launches "
                        "after 3 warm-ups), measured live after the timed region: the read-only counterpart of the "
                        "copy bandwidth in `peak`"}
    line.update(extra)
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)

    if world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        gbs, sps, kind, sample, _ = cpu_baseline(w, 12.0, threads)
        line["cpu_baseline"] = {"value": gbs, "unit": "GB/s", "cores": threads, "kind": kind,
                                "sample": sample, "seq_steps_per_s": sps}
    if world == 1 and not w["paged"] and not args.no_cpu_baseline:
        # the staged C-ABI entry point: every operand in HOST memory (float32, as in the reference's staged
        # binding), whole cache copied to the device inside the call, result copied back; bytes counted at fp32
        try:
            from fusedtok_b200 import _fusedtok as _ft
            k0, v0 = sets[0]
            hq_, hk_, hv_ = q.float().cpu().numpy(), k0.float().cpu().numpy(), v0.float().cpu().numpy()
            hl_ = None if lens_t is None else lens_t.cpu().numpy()
            _ft.attention_decode(hq_, hk_, hv_, hl_, batch, w["Hq"], w["Hkv"], wl["T"], w["D"])
            t0 = time.perf_counter()
            n_st = 2
            for _ in range(n_st):
                ys = _ft.attention_decode(hq_, hk_, hv_, hl_, batch, w["Hq"], w["Hkv"], wl["T"], w["D"])
            st_s = (time.perf_counter() - t0) / n_st
            fp32_bytes = bytes_step * 4 // (4 if w["dtype"] == "f32" else 2)
            line["e2e_staged"] = {"value": fp32_bytes / st_s / 1e9, "unit": "GB/s", "ms_per_step": st_s * 1e3,
                                  "h2d_bytes_per_step": int(hq_.nbytes + hk_.nbytes + hv_.nbytes),
                                  "d2h_bytes_per_step": int(ys.nbytes), "steps": n_st,
                                  "note": "fusedtok_attention_decode: all operands in pageable host memory, float32; "
                                          "dominated by the host-to-device copy of the whole cache"}
            del hq_, hk_, hv_
        except Exception as exc:   # informational only
            line["e2e_staged"] = {"error": str(exc)[:200]}
    if world == 1 and not w["paged"]:
        # the whole decode step on the device: rope of q / k_new at position T-1 + cache write (one launch) followed
        # by the attention kernel, direct launches chained by programmatic stream serialization (informational)
        try:
            g2 = torch.Generator(device=device).manual_seed(7)
            k_new = torch.randn(batch, w["Hkv"], w["D"], device=device, generator=g2).to(q.dtype)
            v_new = torch.randn(batch, w["Hkv"], w["D"], device=device, generator=g2).to(q.dtype)
            q_rot = torch.empty_like(q)
            pos = torch.full((batch,), wl["T"] - 1, dtype=torch.int32, device=device)

            def full_step(i):
                k, v = sets[i % n_sets]
                _fusedtok.rope_kv_append_launch(dt_code, True, q.data_ptr(), q_rot.data_ptr(), k_new.data_ptr(),
                                                v_new.data_ptr(), pos.data_ptr(), k.data_ptr(), v.data_ptr(), batch,
                                                w["Hq"], w["Hkv"], w["D"], wl["T"], 10000.0, 0, stream.cuda_stream)
                getattr(_fusedtok, "attention_decode_launch" + sfx)(
                    q_rot.data_ptr(), k.data_ptr(), v.data_ptr(), lens_ptr, out.data_ptr(),
                    batch, w["Hq"], w["Hkv"], wl["T"], w["D"], stream.cuda_stream)

            for i in range(5):
                full_step(i)
            torch.cuda.synchronize()
            e0.record()
            for i in range(args.steps):
                full_step(i)
            e1.record()
            torch.cuda.synchronize()
            fs_ms = e0.elapsed_time(e1) / args.steps
            line["decode_step"] = {"ms_per_step": fs_ms, "attention_only_ms_per_step": ms_step,
                                   "launches_per_step": 2,
                                   "note": "rope_kv_append (rope of q and k_new + cache write, one launch) + "
                                           "attention_decode, back to back on one stream"}
        except Exception as exc:   # informational only
            line["decode_step"] = {"error": str(exc)[:200]}
    if world == 1:
        # the reference's own GPU kernels on the same inputs (informational)
        try:
            import oracle
            if oracle.ref_available() and not w["paged"]:
                k, v = sets[0]
                yr = torch.empty_like(q)
                for _ in range(3):
                    oracle.ref_gpu_decode_launch(dt_code, q.data_ptr(), k.data_ptr(), v.data_ptr(), lens_ptr,
                                                 yr.data_ptr(), batch, w["Hq"], w["Hkv"], wl["T"], w["D"],
                                                 stream.cuda_stream)
                torch.cuda.synchronize()
                e0.record()
                for i in range(10):
                    k, v = sets[i % n_sets]
                    oracle.ref_gpu_decode_launch(dt_code, q.data_ptr(), k.data_ptr(), v.data_ptr(), lens_ptr,
                                                 yr.data_ptr(), batch, w["Hq"], w["Hkv"], wl["T"], w["D"],
                                                 stream.cuda_stream)
                e1.record()
                torch.cuda.synchronize()
                rms = e0.elapsed_time(e1) / 10
                line["reference_gpu_kernel"] = {"ms_per_step": rms, "GBps": bytes_step / (rms * 1e-3) / 1e9,
                                                "note": "the reference's CUDA kernels compiled for sm_100a, same inputs"}
        except Exception as exc:   # informational only
            line["reference_gpu_kernel"] = {"error": str(exc)[:200]}
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


PREFILL_WORKLOADS = {
    # the reference's own prefill benchmark shape (benchmarks/bench.py:518-541)
    "pf_ref": dict(desc="prefill, reference benchmark shape: batch 1, 32/8 heads, D=128, S=1024, causal, bf16",
                   B=1, Hq=32, Hkv=8, D=128, S=1024, dtype="bf16", causal=True),
    # a long-prompt batch where the operator is compute-bound
    "pf_long": dict(desc="prefill, batch 2, 32/8 heads, D=128, S=8192, causal, bf16",
                    B=2, Hq=32, Hkv=8, D=128, S=8192, dtype="bf16", causal=True),
    "pf_long_f32": dict(desc="prefill, batch 1, 32/8 heads, D=128, S=4096, causal, float32 (CUDA-core kernel)",
                        B=1, Hq=32, Hkv=8, D=128, S=4096, dtype="f32", causal=True),
}


def prefill_cpu_sample(w, target_seconds, threads):
    """The reference's CPU prefill (oracle/_ref, else the C restatement) on `threads` host threads, each on
    one (head group, short sequence) problem of the workload's head shape; returns TFLOP/s."""
    import numpy as np
    import oracle
    kind = "reference" if oracle.ref_available() else "port"
    fn = oracle.ref_prefill if kind == "reference" else oracle.prefill
    s_len = min(w["S"], 256)
    rng = np.random.default_rng(0)
    g = w["Hq"] // w["Hkv"]
    q = rng.standard_normal((1, g, s_len, w["D"])).astype(np.float32)
    k = rng.standard_normal((1, 1, s_len, w["D"])).astype(np.float32)
    t0 = time.perf_counter()
    fn(q, k, k, w["causal"])
    one = time.perf_counter() - t0
    reps = max(1, int(target_seconds / max(one, 1e-4)))

    def work():
        for _ in range(reps):
            fn(q, k, k, w["causal"])

    ths = [threading.Thread(target=work) for _ in range(threads)]
    t0 = time.perf_counter()
    for t in ths:
        t.start()
    for t in ths:
        t.join()
    dt = time.perf_counter() - t0
    flops = 4.0 * s_len * s_len * w["D"] * g / (2 if w["causal"] else 1)
    sample = ("%d calls (%d threads x %d) of one kv head's group (%d query heads), S=%d, D=%d, float32, %.1f s"
              % (threads * reps, threads, reps, g, s_len, w["D"], dt))
    return threads * reps * flops / dt / 1e12, kind, sample, dt


def run_prefill(args, rank, world, local_rank):
    """Prefill workloads: one step = one attention_prefill call over the whole batch. value = TFLOP/s with the
    operands resident (FLOPs = 4*S*S*D*Hq*B, halved when causal); roofline against the measured dense bf16
    GEMM rate (fp32: no tensor peak applies, reported against the same number for scale)."""
    import torch
    import torch.distributed as dist
    import fusedtok_b200 as ft
    from fusedtok_b200 import _fusedtok
    w = dict(PREFILL_WORKLOADS[args.workload])
    for kv in args.set:
        key, val = kv.split("=", 1)
        w[key] = type(w[key])(val) if not isinstance(w[key], bool) else val in ("1", "true", "True")
    if args.impl == "reference":
        if rank == 0:
            threads = os.cpu_count() or 1
            per_step = min(8.0, max(0.3, 60.0 / args.steps))
            for _ in range(args.warmup):
                prefill_cpu_sample(w, 0.2, threads)
            vals, total_t = [], 0.0
            for _ in range(args.steps):
                v, kind, sample, dt = prefill_cpu_sample(w, per_step, threads)
                vals.append(v)
                total_t += dt
            value = sum(vals) / len(vals)
            print(json.dumps({
                "impl": "reference", "metric": "prefill_attn_TFLOPs", "value": value, "unit": "TFLOP/s",
                "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": total_t / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": args.workload + ": " + w["desc"] + " (CPU sample, see cpu_baseline.sample)"},
                "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": threads, "kind": kind, "sample": sample},
                "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0}), flush=True)
        return
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dt = torch.bfloat16 if w["dtype"] == "bf16" else (torch.float16 if w["dtype"] == "f16" else torch.float32)
    gen = torch.Generator(device=dev).manual_seed(1234 + rank)
    shape_q = (w["B"], w["Hq"], w["S"], w["D"])
    shape_kv = (w["B"], w["Hkv"], w["S"], w["D"])
    q = torch.randn(shape_q, device=dev, generator=gen).to(dt)
    k = torch.randn(shape_kv, device=dev, generator=gen).to(dt)
    v = torch.randn(shape_kv, device=dev, generator=gen).to(dt)
    flops = 4.0 * w["S"] * w["S"] * w["D"] * w["Hq"] * w["B"] / (2 if w["causal"] else 1)
    flush = torch.empty(160 << 20, dtype=torch.uint8, device=dev)        # larger than L2 (126 MB)
    small = q.numel() * q.element_size() * 2 + k.numel() * k.element_size() * 2 < (126 << 20)

    def step():
        return ft.attention_prefill(q, k, v, causal=w["causal"])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if args.profile:
        for _ in range(args.warmup):
            step()
        for _ in range(args.steps):
            step()
        torch.cuda.synchronize()
        print(json.dumps({"profile_run": True, "workload": args.workload}), flush=True)
        return
    for _ in range(max(3, args.warmup)):
        step()
    barrier()
    n0 = _fusedtok.attention_launch_count()
    sampler = ClockSampler(local_rank)
    sampler.start()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    barrier()
    for a, b in ev:
        if small:
            flush.fill_(1)                     # operands fit L2: evict them between timed steps
        a.record()
        step()
        b.record()
    barrier()
    clocks = sampler.stop()
    launches = _fusedtok.attention_launch_count() - n0
    ms = sum(a.elapsed_time(b) for a, b in ev) / args.steps
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    value = world * flops / (ms * 1e-3) / 1e12

    # end to end: operands from pinned host memory, result read back, every step
    hq, hk, hv = (x.cpu().pin_memory() for x in (q, k, v))
    hout = torch.empty(shape_q, dtype=dt).pin_memory()
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)

    def e2e_step():
        dq.copy_(hq, non_blocking=True)
        dk.copy_(hk, non_blocking=True)
        dv.copy_(hv, non_blocking=True)
        hout.copy_(ft.attention_prefill(dq, dk, dv, causal=w["causal"]), non_blocking=True)
        torch.cuda.synchronize()
        return float(hout[0, 0, 0, 0])

    for _ in range(3):
        e2e_step()
    n_e2e = max(3, min(args.steps, 20))
    barrier()
    t0 = time.perf_counter()
    for _ in range(n_e2e):
        e2e_step()
    e2e_ms = (time.perf_counter() - t0) / n_e2e * 1e3
    t = torch.tensor([e2e_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t.item())
    if rank != 0:
        return
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            peak, peak_kind = float(json.load(f)["bf16_tflops"]), "of measured (cuBLAS bf16 burst)"
    except Exception:
        peak, peak_kind = 1590.0, "of fallback"
    line = {
        "metric": "prefill_attn_TFLOPs", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic",
        "config": {"workload": args.workload + ": " + w["desc"], "batch_per_gpu": w["B"], "q_heads": w["Hq"],
                   "kv_heads": w["Hkv"], "head_dim": w["D"], "seq": w["S"], "causal": w["causal"],
                   "flops_per_step_per_gpu": flops,
                   "l2": ("L2 flushed between timed steps (160 MB fill)" if small else "operands larger than L2"),
                   "parallelism": "batch-sharded x%d, no communication" % world},
        "roofline": {"bound": "tensor", "achieved": value / world, "peak": peak, "unit": "TFLOP/s",
                     "frac": value / world / peak, "peak_kind": peak_kind, "traffic": None,
                     "note": ("float32 runs on CUDA cores: the tensor peak is shown for scale only"
                              if w["dtype"] == "f32" else "one kernel per step")},
        "e2e": {"value": world * flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": sum(x.numel() * x.element_size() for x in (q, k, v)),
                "d2h_bytes_per_step": q.numel() * q.element_size()},
        "gpu_launches": int(launches), "device_status": _fusedtok.attention_device_status(), "clocks": clocks,
    }
    if not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        v_cpu, kind, sample, _ = prefill_cpu_sample(w, 10.0, threads)
        line["cpu_baseline"] = {"value": v_cpu, "unit": "TFLOP/s", "cores": threads, "kind": kind, "sample": sample}
    print(json.dumps(line), flush=True)


def run_reference_rows(args):
    """The reference's own attention-decode benchmark rows (benchmarks/bench.py:468-516) on this
    GPU: batch 1, 32/8 heads, head dim 128, T in {4096, 16384}, fp32 and bf16, plus the paged fp32
    row (page 16), each through the public operator, beside torch SDPA with pre-expanded heads
    (the reference's comparison) and the reference's own kernels compiled for sm_100a. Protocol as
    in the reference: 3 rounds, each with its own warm-up, CUDA events, mean; the same tensors every
    iteration (at these sizes they can stay L2-resident: this is the reference's protocol, not the
    HBM-roofline one used for `value` elsewhere). GB/s counts (2*K.numel + 2*q.numel)*sizeof."""
    import numpy as np
    import torch
    import fusedtok_b200 as ft
    import oracle

    torch.cuda.set_device(0)

    def timeit(fn, iters):
        vals = []
        for _ in range(3):
            for _ in range(5):
                fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(iters):
                fn()
            e1.record()
            torch.cuda.synchronize()
            vals.append(e0.elapsed_time(e1) / iters * 1e3)
        return sum(vals) / len(vals)

    rows = []
    have_ref = oracle.ref_available()
    b, hq, hkv, d = 1, 32, 8, 128
    for t_rows in (4096, 16384):
        q = torch.randn(b, hq, d, device="cuda")
        k = torch.randn(b, hkv, t_rows, d, device="cuda")
        v = torch.randn(b, hkv, t_rows, d, device="cuda")
        for dt, code, name in ((torch.float32, 0, "attn decode"), (torch.bfloat16, 1, "attn decode bf16")):
            qd, kd, vd = q.to(dt), k.to(dt), v.to(dt)
            kk = kd.repeat_interleave(hq // hkv, dim=1)
            vv = vd.repeat_interleave(hq // hkv, dim=1)
            nbytes = (2 * kd.numel() + 2 * qd.numel()) * kd.element_size()
            ours = timeit(lambda: ft.attention_decode(qd, kd, vd), args.steps)
            sdpa = timeit(lambda: torch.nn.functional.scaled_dot_product_attention(qd.unsqueeze(2), kk, vv).squeeze(2),
                          args.steps)
            row = {"op": name, "shape": "T=%d" % t_rows, "us": ours, "GBps": nbytes / ours / 1e3,
                   "sdpa_us": sdpa, "speedup_vs_sdpa": sdpa / ours}
            if have_ref:
                out = torch.empty_like(qd)
                st = torch.cuda.current_stream().cuda_stream
                ref = timeit(lambda: oracle.ref_gpu_decode_launch(code, qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), 0,
                                                                  out.data_ptr(), b, hq, hkv, t_rows, d, st), args.steps)
                row["reference_kernel_us"] = ref
                row["speedup_vs_reference_kernel"] = ref / ours
            rows.append(row)
        if t_rows == 16384:
            page = 16
            nblk = t_rows // page
            perm = torch.randperm(nblk, device="cuda").to(torch.int32)
            kp = k.view(b, hkv, nblk, page, d)[0].permute(1, 0, 2, 3).contiguous()[perm.argsort().long()]
            vp = v.view(b, hkv, nblk, page, d)[0].permute(1, 0, 2, 3).contiguous()[perm.argsort().long()]
            table = perm.argsort().argsort().to(torch.int32).view(1, nblk).contiguous()
            ours = timeit(lambda: ft.attention_decode_paged(q, kp, vp, table), args.steps)
            kk = k.repeat_interleave(hq // hkv, dim=1)
            vv = v.repeat_interleave(hq // hkv, dim=1)
            sdpa = timeit(lambda: torch.nn.functional.scaled_dot_product_attention(q.unsqueeze(2), kk, vv).squeeze(2),
                          args.steps)
            nbytes = (2 * k.numel() + 2 * q.numel()) * 4
            err = (ft.attention_decode_paged(q, kp, vp, table) - ft.attention_decode(q, k, v)).abs().max().item()
            row = {"op": "attn decode paged", "shape": "T=16384 P=16", "us": ours, "GBps": nbytes / ours / 1e3,
                   "sdpa_us": sdpa, "speedup_vs_sdpa": sdpa / ours, "max_abs_vs_contiguous": err}
            if have_ref:
                out = torch.empty_like(q)
                st = torch.cuda.current_stream().cuda_stream
                ref = timeit(lambda: oracle.ref_gpu_decode_paged_launch(0, q.data_ptr(), kp.data_ptr(), vp.data_ptr(),
                                                                        table.data_ptr(), 0, out.data_ptr(), b, hq, hkv,
                                                                        page, nblk, d, st), args.steps)
                row["reference_kernel_us"] = ref
                row["speedup_vs_reference_kernel"] = ref / ours
            rows.append(row)
    # prefill rows (benchmarks/bench.py:518-541: batch 1, 32/8 heads, D=128, S=1024, causal), plus longer
    # sequences where the operator is compute-bound; FLOPs = 4*S*S*D*Hq/2 (causal half)
    for s_len, batch in ((1024, 1), (4096, 1), (8192, 2)):
        for dt, code, name in ((torch.float32, 0, "attn prefill"), (torch.bfloat16, 1, "attn prefill bf16")):
            if dt is torch.float32 and s_len > 4096:
                continue
            qp = torch.randn(batch, hq, s_len, d, device="cuda").to(dt)
            kp_ = torch.randn(batch, hkv, s_len, d, device="cuda").to(dt)
            vp_ = torch.randn(batch, hkv, s_len, d, device="cuda").to(dt)
            kk = kp_.repeat_interleave(hq // hkv, dim=1)
            vv = vp_.repeat_interleave(hq // hkv, dim=1)
            iters = max(3, args.steps // 8) if s_len <= 1024 else 3
            flops = 4.0 * s_len * s_len * d * hq * batch / 2
            ours = timeit(lambda: ft.attention_prefill(qp, kp_, vp_, causal=True), iters)
            sdpa = timeit(lambda: torch.nn.functional.scaled_dot_product_attention(qp, kk, vv, is_causal=True), iters)
            row = {"op": name, "shape": "B=%d S=%d" % (batch, s_len), "us": ours, "TFLOPs": flops / ours / 1e6,
                   "sdpa_us": sdpa, "speedup_vs_sdpa": sdpa / ours}
            if have_ref:
                out = torch.empty_like(qp)
                st = torch.cuda.current_stream().cuda_stream
                ref = timeit(lambda: oracle.ref_gpu_prefill_launch(code, qp.data_ptr(), kp_.data_ptr(), vp_.data_ptr(),
                                                                   out.data_ptr(), batch, hq, hkv, s_len, d, True, st),
                             iters)
                row["reference_kernel_us"] = ref
                row["speedup_vs_reference_kernel"] = ref / ours
                row["max_abs_vs_reference_kernel"] = (out.float() - ft.attention_prefill(qp, kp_, vp_).float()).abs().max().item()
            rows.append(row)
            del qp, kp_, vp_, kk, vv
    print(json.dumps({"benchmark": "reference attention decode / prefill rows on this GPU", "protocol":
                      "3 rounds x own warm-up, CUDA events, mean; public Python operator; same tensors every iteration",
                      "gpu": torch.cuda.get_device_name(0), "rows": rows}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS) + sorted(PREFILL_WORKLOADS) + ["refrows"])
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"])
    ap.add_argument("--graph", action="store_true", help="replay the step as a CUDA graph")
    ap.add_argument("--exchange", default="p2p", choices=["p2p", "nccl"],
                    help="KV-length split (c4, N>1): the library's own peer exchange or an NCCL all-gather")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--rounds", type=int, default=5, help="timed regions of --steps steps each; the median is reported")
    ap.add_argument("--no-multi-extras", action="store_true",
                    help="N > 1: skip the kv_split and c2_strong measurements that ride on the default line")
    ap.add_argument("--set", action="append", default=[], metavar="KEY=VALUE",
                    help="override a field of the workload (e.g. --set T=32768), for experiments")
    ap.add_argument("--profile", action="store_true",
                    help="profiler run: warm-up and timed steps only (no clock sampling, no end-to-end or CPU legs)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    # (NCCL_DEBUG and NCCL_DEBUG_FILE are left as the caller set them: whatever NCCL logs goes where the caller
    # sent it; the result is the one line of stdout that starts with '{')
    if args.workload == "refrows":
        if rank == 0:
            run_reference_rows(args)
        return
    if args.gpus > 1 and "RANK" not in os.environ and args.impl != "reference":
        # not under a launcher yet: start one rank per GPU
        import socket
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            port = s.getsockname()[1]
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(args.gpus),
               "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.abspath(__file__)] + sys.argv[1:]
        raise SystemExit(subprocess.call(cmd))
    if args.workload in PREFILL_WORKLOADS:
        if world > 1:
            import torch.distributed as dist
            if args.impl == "reference":
                if rank == 0:
                    run_prefill(args, rank, world, local_rank)
                return
            dist.init_process_group("nccl", device_id=__import__("torch").device("cuda", local_rank))
            try:
                run_prefill(args, rank, world, local_rank)
            finally:
                dist.destroy_process_group()
            return
        run_prefill(args, rank, world, local_rank)
        return
    w = dict(WORKLOADS[args.workload])
    for kv in args.set:
        key, val = kv.split("=", 1)
        w[key] = int(val) if val.lstrip("-").isdigit() else val
        w["desc"] += " [%s]" % kv
    if args.impl == "reference":
        run_reference_arm(args, w, rank)
        return
    run_ours(args, w, rank, world, local_rank)


if __name__ == "__main__":
    main()
