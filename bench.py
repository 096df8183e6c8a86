"""Benchmark of the decode / prefill path: one JSON line on stdout.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config NAME]

A step is one request in the shape of the reference's own benchmark (crates/bobcat-bench/src/bin/
bobcat_bench.rs:125-147): reset, prefill a 512-token prompt in one call, then decode 128 tokens
greedily in one pipelined call. The model is the LFM2.5-2.6B-shaped synthetic Q4_0 file
(``bobcat_b200.synth``), written to a scratch directory on first use. ``value`` is decode tokens
per second from CUDA events; prefill tokens per second rides along under ``prefill``.

With N > 1 (launched under torchrun, one rank per GPU) every rank serves its own request replica
with a distinct prompt; there is no collective on the data path.

``--impl reference`` times the CPU restatement of the reference's scalar path (``oracle/``, all
host threads) on a bounded sample of the same workload; no GPU work happens on that arm.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

PROMPT_TOKENS, DECODE_TOKENS, PREFILL_CHUNK = 512, 128, 512
# The reference's headline metric; `value` is its decode half, the prefill half rides along under "prefill".
METRIC = "decode & prefill tok/s, Q4 LFM2.5-2.6B-shape, batch 1; % of HBM roofline"

# Request shape per configuration: (prompt tokens, decode tokens, prefill chunk). The headline shape
# follows the reference benchmark (512 + 128, one prefill call); the others follow the run each
# configuration is specified with.
PROTOCOLS = {
    "lfm2-350m": (128, 64, 128),
    "lfm2-2.6b": (512, 128, 512),
    "qwen35-2b": (2048, 256, 64),
    "lfm2moe-8b-a1b": (256, 128, 256),
    "qwen35-9b": (2048, 256, 512),
}


def recorded_traffic(kernel_key: str):
    """DRAM bytes per launch of `kernel_key` ("name ROWSxCOLS") from the profiler summaries under
    profiles/: lines of the form `traffic <name> <rows>x<cols> <bytes>`. None when no summary
    records that kernel and shape."""
    import glob
    import re
    for path in sorted(glob.glob(os.path.join(ROOT, "profiles", "*.md")) + glob.glob(os.path.join(ROOT, "profiles", "*.txt"))):
        for line in open(path, errors="replace"):
            m = re.match(r"^\s*traffic\s+(\S+)\s+(\d+x\d+)\s+(\d+)\s*$", line)
            if m and "%s %s" % (m.group(1), m.group(2)) == kernel_key:
                return int(m.group(3))
    return None


def measured_peaks() -> tuple[float, float, str]:
    """(HBM GB/s, sustained dense bf16 TFLOP/s) to divide by: measured on this pool, else the stated fallback."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            peaks = json.load(open(path))
            return float(peaks["hbm_gbs"]), float(peaks["bf16_tflops_sustained"]), "measured"
        except Exception:
            pass
    return 6650.0, 1400.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device: int):
        self.device = device
        self.rows: list[list[str]] = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.device), "--query-gpu=" + self.QUERY, "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 9:
                self.rows.append(parts)

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        clocks = [float(r[1]) for r in self.rows if r[1].replace(".", "").isdigit()]
        max_clock = [float(r[2]) for r in self.rows if r[2].replace(".", "").isdigit()]
        reasons = set()
        for r in self.rows:
            for name, value in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(clocks)) if clocks else None, "sm_max_mhz": max(max_clock) if max_clock else None,
                "reasons": sorted(reasons), "samples": len(clocks)}


def rank_info():
    return int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))


def prompt_for(n_vocab: int, seed: int) -> np.ndarray:
    return np.random.default_rng(seed).integers(0, n_vocab, size=PROMPT_TOKENS).astype(np.uint32)


def model_file(config: str) -> str:
    from bobcat_b200 import synth
    return synth.cached_model(config, seed=0, directory=os.environ.get("BOBCAT_SYNTH_DIR", os.path.join(tempfile.gettempdir(), "bobcat_synth")))


def cpu_sample(path: str, threads: int, n_prompt: int, n_decode: int) -> tuple[float, float]:
    """Run the CPU restatement on a short request. Returns (decode tok/s, seconds)."""
    from oracle import oracle
    model = oracle.Model(path, threads=threads)
    state = model.state(n_prompt + n_decode + 1)
    prompt = prompt_for(model.n_vocab, 1)[:n_prompt]
    logits = None
    for i, tok in enumerate(prompt):
        logits = state.step(int(tok), want_logits=(i == n_prompt - 1)).get("logits")
    start = time.perf_counter()
    for _ in range(n_decode):
        logits = state.step(int(np.argmax(logits)))["logits"]
    seconds = time.perf_counter() - start
    return n_decode / seconds, seconds


def run_reference(args) -> None:
    rank, _, world = rank_info()
    if rank != 0:
        return
    # This arm runs the CPU restatement only: it neither loads the CUDA library nor touches a GPU.
    path = model_file(args.config)
    threads = len(os.sched_getaffinity(0))
    n_prompt, n_decode = 4, 4
    times = []
    for i in range(args.warmup + args.steps):
        rate, seconds = cpu_sample(path, threads, n_prompt, n_decode)
        if i >= args.warmup:
            times.append(seconds)
    ms_per_step = 1e3 * float(np.mean(times))
    value = n_decode / (ms_per_step * 1e-3)
    sample = "%d-token prompt then %d greedy decode steps of the scalar restatement per step, %d threads over matrix rows" % (n_prompt, n_decode, threads)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32 (f64 sums)", "data": "synthetic",
        "config": {"workload": "%s Q4_0, batch 1, decode after a short prompt (bounded sample of the %d+%d request)" % (args.config, PROMPT_TOKENS, DECODE_TOKENS)},
        "cpu_baseline": {"value": value, "unit": "tok/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def dominant_kernel(cuda, seq, prompt) -> dict:
    """Time every launch of one more decode pass with CUDA events (profiling mode serialises the
    launches) and report the kernel with the largest share of the time."""
    def rows_of(entries, count):
        total = sum(e["seconds"] for e in entries) or 1.0
        return [{"kernel": e["name"], "rows": e["n_rows"], "cols": e["n_cols"], "calls": e["calls"], "us": 1e6 * e["seconds"] / e["calls"],
                 "bytes_per_launch": e["bytes"] / e["calls"],
                 "gbs": (e["bytes"] / e["seconds"] / 1e9) if e["seconds"] else 0.0, "share": e["seconds"] / total}
                for e in sorted(entries, key=lambda e: -e["seconds"])[:count]]

    seq.reset()
    cuda.set_profiling(True)
    seq.prefill(prompt)
    cuda.set_profiling(False)
    prefill_table = rows_of(cuda.profile(), 10)
    cuda.set_profiling(True)
    seq.generate(min(16, DECODE_TOKENS))
    cuda.set_profiling(False)
    entries = cuda.profile()
    total = sum(e["seconds"] for e in entries) or 1.0
    top = max(entries, key=lambda e: e["seconds"])
    per_launch_s = top["seconds"] / top["calls"]
    per_launch_bytes = top["bytes"] / top["calls"]
    return {"top": top, "share": top["seconds"] / total, "seconds": per_launch_s, "bytes": per_launch_bytes,
            "table": rows_of(entries, 8), "all": rows_of(entries, len(entries)), "prefill_table": prefill_table}


def in_graph_costs(seq, prompt, table, every) -> list[dict]:
    """What each kind of launch costs inside the replayed decode step, where launches overlap their
    neighbours: the step is re-captured with that kind left out and the difference in time per token
    is divided by its launches per token. (The per-launch event timing of `dominant_kernel`
    serialises launches, so it over-states kernels that normally start under their predecessor.)"""
    per_token = DECODE_TOKENS

    def decode_seconds():
        seq.reset()
        seq.prefill(prompt)
        seq.generate(per_token)
        return seq.last_gpu_seconds() / per_token

    out = []
    steps = min(16, DECODE_TOKENS)
    try:
        full = decode_seconds()
        seen = set()
        for row in table:
            # Attention launches are recorded with their position as the column count, which the
            # replayed step does not carry: leave every launch of that name out together.
            by_name = row["kernel"].startswith("attention")
            key = (row["kernel"],) if by_name else (row["kernel"], row["rows"], row["cols"])
            if key in seen:
                continue
            seen.add(key)
            seq.set_skip(row["kernel"], 0 if by_name else row["rows"], 0 if by_name else row["cols"])
            without = decode_seconds()
            calls_per_token = sum(r["calls"] for r in every if r["kernel"] == row["kernel"]) / steps if by_name else row["calls"] / steps
            out.append({"kernel": row["kernel"], "rows": row["rows"], "cols": row["cols"], "calls_per_token": calls_per_token,
                        "us": 1e6 * (full - without) / calls_per_token if calls_per_token else None})
    finally:
        seq.set_skip(None)
    return out


def run_batch(args) -> None:
    """--seqs B > 1: B concurrent sequences of one model per GPU (the multi-sequence decode), every
    weight read once per pass for all of them. `value` is aggregate decode tokens per second."""
    import torch
    import torch.distributed as dist

    from bobcat_b200 import BatchCuda, Cuda, Model, replicas

    rank, local_rank, world = rank_info()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU path")
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    if rank == 0:
        model_file(args.config)
    if world > 1:
        dist.barrier()
    path = model_file(args.config)
    model = Model.load(path)
    hp = model.hyperparameters()
    torch.cuda.set_stream(torch.cuda.Stream())
    cuda = Cuda.open(local_rank, torch.cuda.current_stream().cuda_stream)
    n_seqs = args.seqs
    batch = BatchCuda(model, cuda, n_seqs, PROMPT_TOKENS + DECODE_TOKENS, kv_half=True)
    # Every sequence of every rank has its own prompt.
    prompts = [torch.from_numpy(prompt_for(hp.n_vocab, 1 + rank * n_seqs + i).view(np.int32).copy()).pin_memory() for i in range(n_seqs)]

    def request():
        t0 = time.perf_counter()
        prefill_gpu = 0.0
        for i in range(n_seqs):
            seq = batch.seq(i)
            seq.reset()
            ids = prompts[i].numpy().view(np.uint32)
            for first in range(0, PROMPT_TOKENS, PREFILL_CHUNK):
                seq.prefill(ids[first:first + PREFILL_CHUNK])
                prefill_gpu += seq.last_gpu_seconds()
        t1 = time.perf_counter()
        tokens = batch.generate(DECODE_TOKENS)
        t2 = time.perf_counter()
        return prefill_gpu, batch.last_gpu_seconds(), t1 - t0, t2 - t1, tokens

    for _ in range(args.warmup):
        request()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    launches_before = batch.launches()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    rows = [request() for _ in range(args.steps)]
    end.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    clocks = sampler.stop() if rank == 0 else None
    prefill_gpu, decode_gpu, prefill_wall, decode_wall, ms_per_step = replicas.max_over_ranks(
        [float(np.mean([r[0] for r in rows])), float(np.mean([r[1] for r in rows])), float(np.mean([r[2] for r in rows])),
         float(np.mean([r[3] for r in rows])), start.elapsed_time(end) / args.steps], device="cuda")
    launches = replicas.sum_over_ranks([batch.launches() - launches_before], device="cuda")[0]
    if rank == 0:
        peak, tensor_peak, peak_kind = measured_peaks()
        # A pass of many sequences touches (nearly) every expert, so its bytes are every weight
        # once (each distinct expert counted once), plus every sequence's KV rows.
        import gguf
        reader = gguf.GGUFReader(path)
        all_weight_bytes = int(sum(int(t.n_bytes) for t in reader.tensors)) - hp.n_vocab * hp.n_embd * 4 + hp.n_vocab * hp.n_embd * 4
        kv_bytes = n_seqs * hp.n_attention_layers * 2 * hp.n_kv_heads * hp.head_dim * 2 * (PROMPT_TOKENS + DECODE_TOKENS / 2)
        step_bytes = all_weight_bytes + kv_bytes
        tok_s = world * n_seqs * DECODE_TOKENS / decode_gpu
        line = {
            "metric": METRIC, "value": tok_s, "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32 activations (half-precision operands in the batched products), Q4_0 weights, f16 KV",
            "data": "synthetic",
            "config": {"workload": "%s Q4_0 (random init N(0,0.02), seed 0), %d concurrent sequences per GPU, each a %d-token uniform-random prompt then %d greedy tokens; "
                                   "%d replica(s) of that batch, one per GPU" % (args.config, n_seqs, PROMPT_TOKENS, DECODE_TOKENS, world),
                       "l2": "every pass streams %.2f GB of weights, far larger than the 126 MB L2" % (all_weight_bytes / 1e9), "kv_cache": "f16"},
            "decode": {"tok_s": tok_s, "passes_per_s": world * DECODE_TOKENS / decode_gpu, "ms_per_pass": 1e3 * decode_gpu / DECODE_TOKENS,
                       "bytes_per_pass": step_bytes, "hbm_gbs": step_bytes * DECODE_TOKENS / decode_gpu / 1e9,
                       "hbm_frac": step_bytes * DECODE_TOKENS / decode_gpu / 1e9 / peak, "token_hash": replicas.token_hash(rows[-1][4].ravel().tolist())},
            "prefill": {"tok_s": world * n_seqs * PROMPT_TOKENS / prefill_gpu},
            "roofline": {"bound": "hbm", "kernel": "whole multi-sequence pass", "achieved": step_bytes * DECODE_TOKENS / decode_gpu / 1e9, "peak": peak,
                         "peak_kind": peak_kind, "unit": "GB/s", "frac": step_bytes * DECODE_TOKENS / decode_gpu / 1e9 / peak, "traffic": None},
            "e2e": {"value": world * n_seqs * DECODE_TOKENS / decode_wall, "unit": "tok/s", "h2d_bytes_per_step": n_seqs * PROMPT_TOKENS * 4,
                    "d2h_bytes_per_step": n_seqs * DECODE_TOKENS * 4},
            "gpu_launches": launches, "clocks": clocks,
        }
        print(json.dumps(line))
    batch.close()
    if world > 1:
        dist.destroy_process_group()


def sharded_blocks(args, cuda, rank, local_rank, world) -> dict:
    """The two sharded configurations on the same ranks, each as a block beside the replica headline:
    `ep` - 32 concurrent sequences of the LFM2.5-8B-A1B shape, experts sharded over the ranks
    (256-token prompts, 128 greedy tokens each); `tp` - one Qwen3.5-9B-shaped sequence tensor-
    parallel over the ranks (a 2048-token prompt in 512-token chunks, 128 greedy tokens; the
    60 000-token protocol of that configuration is `--mode prefix`). Both are strong scaling: the
    work is fixed and the ranks split it. At one GPU the same code runs unsharded, which gives the
    efficiency its denominator."""
    import torch
    import torch.distributed as dist

    from bobcat_b200 import BatchCuda, Model, Qwen35Cuda, replicas
    from bobcat_b200.sharding import COMM_ID_BYTES, Comm

    def comm_for():
        if world == 1:
            return None
        raw = torch.zeros(COMM_ID_BYTES, dtype=torch.uint8, device="cuda")
        if rank == 0:
            raw = torch.tensor(list(Comm.unique_id()), dtype=torch.uint8, device="cuda")
        dist.broadcast(raw, 0)
        return Comm(cuda, bytes(raw.cpu().tolist()), rank, world)

    def shared_file(config):
        if rank == 0:
            model_file(config)
        if world > 1:
            dist.barrier()
        return model_file(config)

    def timed(fn, reps):
        fn()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        return [fn() for _ in range(reps)]

    blocks = {}
    # ---- expert parallel
    try:
        n_total, n_prompt, n_decode = 32, 256, 128
        if n_total % world == 0:
            model = Model.load(shared_file("lfm2moe-8b-a1b"))
            hp = model.hyperparameters()
            comm = comm_for()
            n_local = n_total // world
            batch = BatchCuda(model, cuda, n_local, max(n_prompt + n_decode, n_total), True, comm=comm)
            prompts = [np.random.default_rng(100 + rank * n_local + i).integers(0, hp.n_vocab, n_prompt).astype(np.uint32) for i in range(n_local)]

            def ep_request():
                for i in range(n_local):
                    batch.seq(i).reset()
                    batch.seq(i).prefill(prompts[i])
                tokens = batch.generate(n_decode)
                return batch.last_gpu_seconds(), tokens

            rows = timed(ep_request, 2)
            seconds = replicas.max_over_ranks([float(np.mean([r[0] for r in rows]))], device="cuda")[0]
            blocks["ep"] = {"config": "lfm2moe-8b-a1b, %d concurrent sequences in all (%d per rank), %d-token prompts, %d greedy tokens each, experts %d per rank" %
                                      (n_total, n_local, n_prompt, n_decode, hp.n_experts // world),
                            "scaling": "strong", "n_gpus": world, "tok_s": n_total * n_decode / seconds, "ms_per_pass": 1e3 * seconds / n_decode,
                            "collectives_per_pass": (comm.collectives() // (3 * n_decode)) if comm else 0,
                            "token_hash_rank0": replicas.token_hash(rows[-1][1].ravel().tolist())}
            batch.close()
            if comm:
                comm.close()
            model.close()
    except Exception as e:  # a block that cannot run must not take the headline with it
        blocks["ep"] = {"error": "%s: %s" % (type(e).__name__, e)}
    # ---- tensor parallel
    try:
        n_prompt, n_decode, chunk = 2048, 128, 512
        model = Model.load(shared_file("qwen35-9b"))
        hp = model.hyperparameters()
        comm = comm_for()
        seq = Qwen35Cuda(model, cuda, n_prompt + n_decode, True, comm=comm)
        prompt = np.random.default_rng(200).integers(0, hp.n_vocab, n_prompt).astype(np.uint32)

        def tp_request():
            seq.reset()
            prefill = 0.0
            for first in range(0, n_prompt, chunk):
                seq.prefill(prompt[first:first + chunk])
                prefill += seq.last_gpu_seconds()
            tokens = seq.generate(n_decode)
            return prefill, seq.last_gpu_seconds(), tokens

        rows = timed(tp_request, 2)
        prefill_s, decode_s = replicas.max_over_ranks([float(np.mean([r[0] for r in rows])), float(np.mean([r[1] for r in rows]))], device="cuda")
        blocks["tp"] = {"config": "qwen35-9b, one sequence, %d-token prompt in chunks of %d, %d greedy tokens" % (n_prompt, chunk, n_decode),
                        "scaling": "strong", "n_gpus": world, "decode_tok_s": n_decode / decode_s, "prefill_tok_s": n_prompt / prefill_s,
                        "ms_per_token": 1e3 * decode_s / n_decode, "token_hash_rank0": replicas.token_hash(rows[-1][2].tolist())}
        seq.close()
        if comm:
            comm.close()
        model.close()
    except Exception as e:
        blocks["tp"] = {"error": "%s: %s" % (type(e).__name__, e)}
    return blocks


def run_prefix(args) -> None:
    """--mode prefix: the long-context protocol with a cached prefix. One shared prefix is prefilled
    in 512-token chunks and cached; then 8 requests each load it, append their own suffix and decode.
    Defaults are the Qwen3.5-9B configuration's (60 000 + 8 x (4096 + 256)); --prefix-tokens,
    --prompt-tokens (the suffix) and --decode-tokens scale it down. One GPU: paged caches, the
    prefix's full pages mapped, not copied. Several GPUs: the sequence is tensor-parallel and every
    rank caches its own share. `value` is decode tokens per second over the 8 requests."""
    import torch
    import torch.distributed as dist

    from bobcat_b200 import Cuda, Model, Qwen35Cuda, replicas
    from bobcat_b200.sharding import COMM_ID_BYTES, Comm

    rank, local_rank, world = rank_info()
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    config = args.config if args.config.startswith("qwen") else "qwen35-9b"
    if rank == 0:
        model_file(config)
    if world > 1:
        dist.barrier()
    model = Model.load(model_file(config))
    hp = model.hyperparameters()
    torch.cuda.set_stream(torch.cuda.Stream())
    cuda = Cuda.open(local_rank, torch.cuda.current_stream().cuda_stream)
    comm = None
    if world > 1:
        raw = torch.zeros(COMM_ID_BYTES, dtype=torch.uint8, device="cuda")
        if rank == 0:
            raw = torch.tensor(list(Comm.unique_id()), dtype=torch.uint8, device="cuda")
        dist.broadcast(raw, 0)
        comm = Comm(cuda, bytes(raw.cpu().tolist()), rank, world)
    n_prefix, n_suffix, n_decode, n_requests, chunk = args.prefix_tokens, args.prompt_tokens or 4096, args.decode_tokens or 256, 8, 512
    n_ctx = n_prefix + n_suffix + n_decode
    rng = np.random.default_rng(1)
    prefix_tokens = rng.integers(0, hp.n_vocab, n_prefix).astype(np.uint32)
    suffixes = [np.random.default_rng(10 + i).integers(0, hp.n_vocab, n_suffix).astype(np.uint32) for i in range(n_requests)]

    def new_seq():
        return Qwen35Cuda(model, cuda, n_ctx, True, comm=comm, paged=comm is None)

    def prefill(seq, tokens):
        seconds = 0.0
        for first in range(0, len(tokens), chunk):
            seq.prefill(tokens[first:first + chunk])
            seconds += seq.last_gpu_seconds()
        return seconds

    source = new_seq()
    t0 = time.perf_counter()
    prefix_seconds = prefill(source, prefix_tokens)
    prefix = source.save_prefix()
    source.close()
    seq = new_seq()
    suffix_seconds = decode_seconds = load_seconds = 0.0
    hashes = []
    shared = 0
    for suffix in suffixes:
        t1 = time.perf_counter()
        seq.load_prefix(prefix)
        load_seconds += time.perf_counter() - t1
        shared = seq.kv_pages()[2]
        suffix_seconds += prefill(seq, suffix)
        tokens = seq.generate(n_decode)
        decode_seconds += seq.last_gpu_seconds()
        hashes.append(replicas.token_hash(tokens.tolist()))
    wall = time.perf_counter() - t0
    prefix_seconds, suffix_seconds, decode_seconds = replicas.max_over_ranks([prefix_seconds, suffix_seconds, decode_seconds], device="cuda")
    if rank == 0:
        peak, _, peak_kind = measured_peaks()
        value = n_requests * n_decode / decode_seconds
        kv_row_bytes = hp.n_attention_layers * 2 * hp.n_kv_heads * hp.head_dim * 2
        token_bytes = model.decode_bytes() + kv_row_bytes * (n_prefix + n_suffix + n_decode / 2) + hp.n_delta_layers * hp.n_v_heads * hp.k_head_dim * hp.v_head_dim * 8
        line = {
            "metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": world, "steps": 1, "warmup": 0, "ms_per_step": 1e3 * wall, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32 activations, Q4_0 weights, f16 KV", "data": "synthetic",
            "config": {"workload": "%s Q4_0, one %d-token shared prefix prefilled in %d-token chunks and cached, then %d requests of a %d-token suffix and %d greedy "
                                   "tokens each from the cached prefix; %s" % (config, n_prefix, chunk, n_requests, n_suffix, n_decode,
                                   "tensor-parallel over %d GPUs" % world if world > 1 else "one GPU, paged KV caches"),
                       "kv_cache": "f16"},
            "prefix": {"prefill_tok_s": n_prefix / prefix_seconds, "suffix_prefill_tok_s": n_requests * n_suffix / suffix_seconds, "load_ms_per_request": 1e3 * load_seconds / n_requests,
                       "kv_pages_shared_per_request": shared, "token_hashes": hashes},
            "decode": {"tok_s": value, "ms_per_token": 1e3 * decode_seconds / (n_requests * n_decode), "bytes_per_token": token_bytes / world,
                       "hbm_frac_per_gpu": token_bytes / world * n_requests * n_decode / decode_seconds / 1e9 / peak},
            "roofline": {"bound": "hbm", "kernel": "whole decode step at the long context", "achieved": token_bytes / world * n_requests * n_decode / decode_seconds / 1e9,
                         "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": token_bytes / world * n_requests * n_decode / decode_seconds / 1e9 / peak, "traffic": None},
            "e2e": {"value": n_requests * n_decode / (wall - 0.0), "unit": "tok/s (decode tokens over the whole job's wall time)", "h2d_bytes_per_step": (n_prefix + n_requests * n_suffix) * 4,
                    "d2h_bytes_per_step": n_requests * n_decode * 4},
            "gpu_launches": seq.launches(),
        }
        print(json.dumps(line))
    seq.close()
    if comm:
        comm.close()
    if world > 1:
        dist.destroy_process_group()


def run_ours(args) -> None:
    import torch
    import torch.distributed as dist

    from bobcat_b200 import Cuda, Lfm2Cuda, Model

    rank, local_rank, world = rank_info()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU path")
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    # Rank 0 writes the model file; the others wait for it.
    if rank == 0:
        path = model_file(args.config)
    if world > 1:
        dist.barrier()
    path = model_file(args.config)

    model = Model.load(path)
    hp = model.hyperparameters()
    # Launch on torch's current stream so torch's events and barriers order with our kernels.
    torch.cuda.set_stream(torch.cuda.Stream())
    stream = torch.cuda.current_stream().cuda_stream
    cuda = Cuda.open(local_rank, stream)
    n_ctx = PROMPT_TOKENS + DECODE_TOKENS
    seq = Lfm2Cuda(model, cuda, n_ctx, kv_half=True)
    # Request replicas: timed step i of rank r serves request r + i * world, each with its own prompt.
    from bobcat_b200 import replicas
    mine = replicas.requests_of(rank, world, world * args.steps)
    prompts = [torch.from_numpy(prompt_for(hp.n_vocab, replicas.prompt_seed(r)).view(np.int32).copy()).pin_memory() for r in mine]
    prompt = prompts[0].numpy().view(np.uint32)

    def request(i=0):
        """One request through the public API with host buffers (pinned prompt ids in, token ids out).
        Returns device and wall seconds."""
        seq.reset()
        ids = prompts[i % len(prompts)].numpy().view(np.uint32)
        t0 = time.perf_counter()
        prefill_gpu = 0.0
        for first in range(0, PROMPT_TOKENS, PREFILL_CHUNK):
            seq.prefill(ids[first:first + PREFILL_CHUNK])
            prefill_gpu += seq.last_gpu_seconds()
        t1 = time.perf_counter()
        tokens = seq.generate(DECODE_TOKENS)
        t2 = time.perf_counter()
        return prefill_gpu, seq.last_gpu_seconds(), t1 - t0, t2 - t1, tokens

    for _ in range(args.warmup):
        request()

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    launches_before = seq.launches()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    sync_all()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    rows = [request(i) for i in range(args.steps)]
    end.record()
    sync_all()
    clocks = sampler.stop() if rank == 0 else None
    launches = seq.launches() - launches_before
    total_ms = start.elapsed_time(end)

    prefill_gpu = float(np.mean([r[0] for r in rows]))
    decode_gpu = float(np.mean([r[1] for r in rows]))
    prefill_wall = float(np.mean([r[2] for r in rows]))
    decode_wall = float(np.mean([r[3] for r in rows]))
    # The slowest rank sets the job's time; launches add up.
    decode_gpu, prefill_gpu, decode_wall, prefill_wall, ms_per_step = replicas.max_over_ranks(
        [decode_gpu, prefill_gpu, decode_wall, prefill_wall, total_ms / args.steps], device="cuda")
    launches = replicas.sum_over_ranks([launches], device="cuda")[0]

    # Replicas must not change results: every rank also serves request 0, and the token hashes must agree.
    replica_check = None
    if world > 1:
        seq.reset()
        seq.prefill(prompt_for(hp.n_vocab, replicas.prompt_seed(0)))
        mine_hash = replicas.token_hash(seq.generate(DECODE_TOKENS).tolist()) & 0x7FFFFFFFFFFFFFFF
        lo, hi = replicas.max_over_ranks([-float(mine_hash >> 32), float(mine_hash >> 32)], device="cuda")
        lo2, hi2 = replicas.max_over_ranks([-float(mine_hash & 0xFFFFFFFF), float(mine_hash & 0xFFFFFFFF)], device="cuda")
        replica_check = {"request": 0, "token_hash": mine_hash, "identical_on_all_ranks": (-lo == hi) and (-lo2 == hi2)}
        if not replica_check["identical_on_all_ranks"]:
            raise SystemExit("request 0 decoded to different tokens on different ranks")

    # The sharded configurations ride along as blocks (every rank takes part; rank 0 reports).
    sharded = {} if args.no_sharded else sharded_blocks(args, cuda, rank, local_rank, world)

    if rank == 0:
        peak, tensor_peak, peak_kind = measured_peaks()
        weight_bytes = model.decode_bytes()
        # KV traffic: f16 K and V rows of every attention layer at the mean decode position.
        kv_bytes = hp.n_attention_layers * 2 * hp.n_kv_heads * hp.head_dim * 2 * (PROMPT_TOKENS + DECODE_TOKENS / 2)
        token_bytes = weight_bytes + kv_bytes
        decode_tok_s = world * DECODE_TOKENS / decode_gpu
        prefill_tok_s = world * PROMPT_TOKENS / prefill_gpu
        decode_rates = [DECODE_TOKENS / r[1] for r in rows]
        # Flops of a prefilled token: two per weight of the quantised linears (the F32 output
        # matrix runs once per prompt, for the last token only).
        linear_weights = (weight_bytes - hp.n_vocab * hp.n_embd * 4) * 32 / 18
        prefill_tflops = 2 * linear_weights * PROMPT_TOKENS / prefill_gpu / 1e12
        token_hash = 0
        for tok in rows[-1][4].tolist():
            token_hash = (token_hash * 1000003 + tok) & 0xFFFFFFFFFFFFFFFF
        dom = dominant_kernel(cuda, seq, prompt)
        in_graph = in_graph_costs(seq, prompt, dom["table"], dom["all"])
        # The dominant kernel is the one with the largest share of the replayed step, and its
        # duration is what a launch of it costs there (launches overlap their neighbours, which a
        # serialised per-launch timing cannot see); the serialised figure rides along.
        costed = [r for r in in_graph if r["us"] and r["us"] > 0]
        top_row = max(costed, key=lambda r: r["us"] * r["calls_per_token"]) if costed else None
        serial = next((r for r in dom["all"] if top_row and (r["kernel"], r["rows"], r["cols"]) == (top_row["kernel"], top_row["rows"], top_row["cols"])), None)
        if top_row and serial and serial["bytes_per_launch"]:
            top_key = "%s %dx%d" % (top_row["kernel"], top_row["rows"], top_row["cols"])
            launch_bytes, launch_us, serial_us = serial["bytes_per_launch"], top_row["us"], serial["us"]
            share = top_row["us"] * top_row["calls_per_token"] / sum(r["us"] * r["calls_per_token"] for r in costed)
        else:
            top_key = "%s %dx%d" % (dom["top"]["name"], dom["top"]["n_rows"], dom["top"]["n_cols"])
            launch_bytes, launch_us, serial_us, share = dom["bytes"], 1e6 * dom["seconds"], 1e6 * dom["seconds"], dom["share"]
        achieved = launch_bytes / (launch_us * 1e-6) / 1e9
        cpu_rate, cpu_seconds = cpu_sample(path, 1, 2, 4) if world == 1 and not args.no_cpu_baseline else (None, None)
        line = {
            "metric": METRIC, "value": decode_tok_s, "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32 activations, Q4_0 weights, f16 KV",
            "data": "synthetic",
            "config": {"workload": "%s Q4_0 (random init N(0,0.02), seed 0), batch 1 per GPU, %d-token uniform-random prompt prefilled in chunks of %d then %d greedy tokens; "
                                   "%d request replica(s), one per GPU, %d requests with distinct prompts" % (args.config, PROMPT_TOKENS, PREFILL_CHUNK, DECODE_TOKENS, world, world * args.steps),
                       "l2": "every token streams %.2f GB of weights, far larger than the 126 MB L2" % (weight_bytes / 1e9),
                       "n_ctx": n_ctx, "kv_cache": "f16"},
            "decode": {"tok_s": decode_tok_s, "tpot_ms": 1e3 * decode_gpu / DECODE_TOKENS, "bytes_per_token": token_bytes,
                       "hbm_gbs": token_bytes * DECODE_TOKENS / decode_gpu / 1e9, "hbm_frac": token_bytes * DECODE_TOKENS / decode_gpu / 1e9 / peak,
                       "hbm_frac_of_nominal_8tbs": token_bytes * DECODE_TOKENS / decode_gpu / 8e12, "token_hash": token_hash,
                       "tok_s_sd_rank0": float(np.std(decode_rates))},
            "prefill": {"tok_s": prefill_tok_s, "ttft_ms": 1e3 * prefill_gpu, "tokens": PROMPT_TOKENS, "tflops": prefill_tflops,
                        "tensor_peak_tflops": tensor_peak, "tensor_frac": prefill_tflops / tensor_peak,
                        "weights_pass_ms": 1e3 * (weight_bytes - hp.n_vocab * hp.n_embd * 4) / (peak * 1e9), "kernels": dom["prefill_table"]},
            "roofline": {"bound": "hbm", "kernel": top_key,
                         "achieved": achieved, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak,
                         "timing": "duration of one launch inside the replayed decode step: the step re-captured without this kernel, difference in CUDA-event time per token over its launches per token",
                         "traffic": recorded_traffic(top_key), "traffic_source": "ncu summary under profiles/ (recorded, not captured in this run)",
                         "share_of_decode": share, "launch_us": launch_us, "bytes_per_launch": launch_bytes,
                         "launch_us_serialised": serial_us, "frac_serialised": launch_bytes / (serial_us * 1e-6) / 1e9 / peak,
                         "kernels": dom["table"], "in_graph_us": in_graph},
            "e2e": {"value": world * DECODE_TOKENS / decode_wall, "unit": "tok/s", "h2d_bytes_per_step": PROMPT_TOKENS * 4,
                    "d2h_bytes_per_step": DECODE_TOKENS * 4, "prefill_tok_s": world * PROMPT_TOKENS / prefill_wall},
            "gpu_launches": launches,
            "clocks": clocks,
        }
        if replica_check is not None:
            line["replica_check"] = replica_check
        line.update(sharded)
        if cpu_rate is not None:
            line["cpu_baseline"] = {"value": cpu_rate, "unit": "tok/s", "cores": 1, "kind": "port",
                                    "sample": "2-token prompt then 4 greedy decode steps of the scalar restatement, single thread (%.1f s)" % cpu_seconds}
        print(json.dumps(line))
    seq.close()
    if world > 1:
        dist.destroy_process_group()


def main() -> None:
    global PROMPT_TOKENS, DECODE_TOKENS, PREFILL_CHUNK
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=5)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--config", default="lfm2-2.6b")
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-sharded", action="store_true", help="leave out the expert-parallel and tensor-parallel blocks")
    parser.add_argument("--prompt-tokens", type=int, default=0, help="shorter requests, for profiler captures only (0: the configuration's own)")
    parser.add_argument("--decode-tokens", type=int, default=0)
    parser.add_argument("--prefill-chunk", type=int, default=0)
    parser.add_argument("--mode", default="request", choices=["request", "prefix"], help="prefix: the long-context protocol with a cached prefix")
    parser.add_argument("--prefix-tokens", type=int, default=60000)
    parser.add_argument("--seqs", type=int, default=1, help="concurrent sequences per GPU (the multi-sequence decode when > 1)")
    args = parser.parse_args()
    protocol = PROTOCOLS.get(args.config, (512, 128, 512))
    PROMPT_TOKENS = args.prompt_tokens or protocol[0]
    DECODE_TOKENS = args.decode_tokens or protocol[1]
    PREFILL_CHUNK = args.prefill_chunk or min(protocol[2], PROMPT_TOKENS)
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    elif args.mode == "prefix":
        run_prefix(args)
    elif args.seqs > 1:
        run_batch(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
