#!/usr/bin/env python
"""Decode benchmark: tokens/s of the greedy decode step on a synthetic Llama-3-8B-shaped
Q4_K_M model (benchmark configuration 4, batch 1), with the HBM roofline of the dominant kernel and
the CPU checker timed beside it.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

A step is one decode step of the whole model (one generated token per sequence).  Weights
are seeded N(0, 0.02) generated and quantised on the device; the prompt is uniform-random ids;
`value` is device-timed (CUDA events on the engine's stream) with everything resident in HBM;
`e2e` is the same metric through the reference-facing per-token call with host buffers
(embedding + RoPE rows up, token id down, every step).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

SEED = 20261125
WORKLOADS = {
    # name: (shape, mix, prompt tokens, context limit)
    "llama-8b-q4_k_m": ("llama-8b", "q4_k_m", 1024, 8192),
    "llama-3b-q4_k_m": ("llama-3b", "q4_k_m", 512, 4096),
    "llama-1b-q8_0": ("llama-1b", "q8_0", 32, 512),
    "mixtral-8x7b-q4_k_m": ("mixtral-8x7b", "q4_k_m", 512, 4096),
    "tiny-q4_k_m": ("tiny", "q4_k_m", 16, 512),
}


# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the staged matvec, from an ncu
# capture of this kernel at this shape (weights 33.03 MB on the wire).
NCU_DRAM_BYTES_PER_LAUNCH = {("Q4_K", 14336, 4096): 33118208}

ENGINE_MODES = {
    0: "default: reference-order f32 sums in the staged kernels (bit-identical to the CPU path)",
    16: "plain reference-order kernels (one lane per sum)",
    128: "fast order: lane-parallel f32 sums (opt-in, not bit-identical)",
}


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class NvmlSampler:
    """Polls SM clock and clock-event reasons through NVML (read-only) every few milliseconds while the
    timed region runs; a 20-step region lasts tens of milliseconds, too short for nvidia-smi's loop."""

    def __init__(self, device_index: int):
        import pynvml

        self.nv = pynvml
        pynvml.nvmlInit()
        self.h = pynvml.nvmlDeviceGetHandleByIndex(device_index)
        self.sm, self.reasons, self.run = [], set(), False
        self.max = float(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))

    def _poll(self):
        nv = self.nv
        names = (("hw_slowdown", nv.nvmlClocksEventReasonHwSlowdown), ("hw_thermal_slowdown", nv.nvmlClocksEventReasonHwThermalSlowdown),
                 ("sw_thermal_slowdown", nv.nvmlClocksEventReasonSwThermalSlowdown), ("sw_power_cap", nv.nvmlClocksEventReasonSwPowerCap))
        while self.run:
            try:
                self.sm.append(float(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                for name, bit in names:
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.004)

    def start(self):
        self.run = True
        self.t = threading.Thread(target=self._poll, daemon=True)
        self.t.start()

    def stop(self) -> dict:
        self.run = False
        self.t.join(timeout=2)
        return {"sm_mhz": statistics.median(self.sm) if self.sm else None, "sm_max_mhz": self.max, "reasons": sorted(self.reasons),
                "samples": len(self.sm), "source": "nvml"}


def clock_sampler(device_index: int):
    # CUDA_VISIBLE_DEVICES renumbers CUDA devices but not NVML's
    vis = os.environ.get("CUDA_VISIBLE_DEVICES", "")
    phys = device_index
    if vis:
        try:
            phys = int(vis.split(",")[device_index])
        except Exception:
            phys = device_index
    try:
        return NvmlSampler(phys)
    except Exception:
        return ClockSampler(phys)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.idx = device_index
        self.proc = None
        self.lines: list[str] = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def host_threads() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


def build_reference_model(workload: str, n_layers: int | None = None, max_pos: int = 64):
    """The workload's model in the CPU checker, generated by the checker itself."""
    from camelid_b200 import synth  # shapes and tensor plan only; no GPU work
    from oracle import oracle as orc

    shape, mix, _, ctx = WORKLOADS[workload]
    cfg = synth.engine_config(shape, max_pos=max_pos, n_layers=n_layers)
    plan = synth.quant_plan(mix)
    shapes = synth.proj_shapes(cfg)
    m = orc.OracleModel(cfg.oracle_dict())
    ones = np.ones(cfg.hidden, np.float32)
    for layer in range(cfg.n_layers):
        projs = {}
        for slot, name in enumerate(synth.SLOTS):
            rows, cols = shapes[name]
            if cfg.n_experts > 0 and slot >= 4:
                projs[name] = (8, np.zeros(4, np.uint8))
                continue
            projs[name] = (plan[name], orc.synth_tensor(plan[name], SEED, synth.stream_of(layer, slot), rows, cols, 0.02))
        m.set_layer(layer, projs, ones, ones)
        if cfg.n_experts > 0:
            router = orc.synth_tensor(0, SEED, synth.stream_of(layer, 12), cfg.n_experts, cfg.hidden, 0.1).view(np.float32)
            exps = []
            for i, name in enumerate(("gate", "up", "down")):
                rows, cols = shapes[name]
                qt = plan[name] if name != "down" else 12
                exps.append((qt, orc.synth_tensor(qt, SEED, synth.stream_of(layer, 8 + i), cfg.n_experts * rows, cols, 0.02)))
            m.set_moe(layer, router, *exps)
    m.set_output(ones, plan["output"], orc.synth_tensor(plan["output"], SEED, synth.STREAM_OUTPUT, cfg.vocab, cfg.hidden, 0.02))
    m.set_token_embd(plan["token_embd"], orc.synth_tensor(plan["token_embd"], SEED, synth.STREAM_EMBD, cfg.vocab, cfg.hidden, 0.02))
    return m, cfg


def seed_cpu_kv(model, cfg, n_positions: int):
    """Positions 0..n-1 of every layer of the CPU model's KV cache take seeded N(0, 1) values (f16-rounded),
    so that its timed tokens attend over the benchmark's context without a CPU prompt ingestion."""
    from oracle import oracle as orc

    n = cfg.n_kv_heads * n_positions * cfg.head_dim
    for layer in range(cfg.n_layers):
        ck = orc.synth_normal(SEED, 7_000_000 + 2 * layer, 0, n, 1.0).reshape(cfg.n_kv_heads, n_positions, cfg.head_dim)
        cv = orc.synth_normal(SEED, 7_000_001 + 2 * layer, 0, n, 1.0).reshape(cfg.n_kv_heads, n_positions, cfg.head_dim)
        model.write_kv_layer(layer, ck, cv)


def time_cpu_decode(model, cfg, n_tokens: int, warmup: int, start_pos: int, first_token: int):
    """Greedy decode on the CPU checker from `first_token` at `start_pos` (the KV prefix is already in
    its cache): seconds per timed token, all tokens produced (warm-up ones included), next position."""
    from oracle import oracle as orc

    tok, pos, toks = int(first_token), start_pos, []
    t0 = time.perf_counter()
    for i in range(warmup + n_tokens):
        if i == warmup:
            t0 = time.perf_counter()
        logits, _, _ = model.forward(model.embedding(tok), pos)
        tok = int(orc.argmax(logits))
        toks.append(tok)
        pos += 1
    return (time.perf_counter() - t0) / max(1, n_tokens), toks, pos


def run_reference(args):
    """--impl reference: the reference's CPU decode path (its Rust cannot be built here, so the
    C restatement in oracle/ stands in) on all host threads, same workload, context and metric."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle as orc

    try:
        orc.build(march="native", out=str(ROOT / "oracle" / "libcamelid_oracle_native.so"))
        orc._lib = None
        orc._LIB_PATH = ROOT / "oracle" / "libcamelid_oracle_native.so"
    except Exception:
        pass
    threads = host_threads()
    orc.lib().orc_set_num_threads(threads)
    shape, mix, n_prompt, ctx = WORKLOADS[args.workload]
    n_prompt = args.prompt or n_prompt
    t_build = time.perf_counter()
    model, cfg = build_reference_model(args.workload, max_pos=n_prompt + args.steps + args.warmup + 8)
    seed_cpu_kv(model, cfg, n_prompt)
    build_s = time.perf_counter() - t_build
    # keep the whole run within a few minutes: cap the timed and the warm-up tokens by a one-token probe
    probe, toks, pos = time_cpu_decode(model, cfg, 1, 0, n_prompt, 1)
    steps = max(1, min(args.steps, int(120.0 / max(probe, 1e-3))))
    warm = max(0, min(args.warmup, int(60.0 / max(probe, 1e-3))))
    sec, _, pos = time_cpu_decode(model, cfg, steps, warm, pos, toks[-1])
    value = 1.0 / sec
    line = {
        "impl": "reference", "metric": "decode tokens/s", "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": warm, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int8 x int8 -> f32", "data": "synthetic",
        "config": {"workload": args.workload, "batch": 1, "prompt_tokens": n_prompt,
                   "context": f"positions {n_prompt + 1 + warm}..{pos - 1} over a seeded KV prefix of {n_prompt} positions",
                   "threads": threads, "model_build_s": round(build_s, 1)},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port",
                         "sample": f"{steps} decode tokens of the full model at context {n_prompt + 1 + warm}..{pos - 1} "
                                   f"(C restatement of Camelid's CPU path, OpenMP over rows, {threads} threads)"},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def gemv_roofline(cm, qt_name: str, rows: int, cols: int, batch: int = 1):
    """Times the dominant kernel alone: the quantised matvec at the model's largest layer shape,
    cycling through enough distinct weight copies to exceed the L2 (126 MB)."""
    from camelid_b200._lib import check
    from camelid_b200.engine import DeviceBuffer, QT_NAMES, quantize_activation
    import ctypes as C

    qt = QT_NAMES[qt_name]
    bpw = {8: 34 / 32, 12: 144 / 256, 14: 210 / 256}[qt]
    wbytes = rows * cols * bpw
    n_copies = max(2, int(np.ceil(400e6 / wbytes)))
    copies = [cm.Weight.synth(qt, SEED, 5000 + i, rows, cols, 0.02) for i in range(n_copies)]
    x = np.random.default_rng(0).standard_normal((batch, cols)).astype(np.float32)
    act = quantize_activation(cm.ACT_Q8_0 if qt == 8 else cm.ACT_Q8_K, x)
    y = DeviceBuffer(batch * rows * 4)
    arr = (C.c_void_p * n_copies)(*[w._h for w in copies])
    ms = C.c_float(0)
    check(cm.lib().cmld_gemv_select_kernel(2))  # launches chained by programmatic dependent launch, as inside the engine's step
    check(cm.lib().cmld_gemv_time(arr, n_copies, act.ptr, batch, y.ptr, 20, 200, C.byref(ms)))
    check(cm.lib().cmld_gemv_select_kernel(0))
    alg_bytes = wbytes + cols * batch + rows * 4 * batch  # weights + int8 activation codes + f32 outputs
    return alg_bytes, ms.value * 1e-3


def prompt_tokens(vocab: int, n: int, stream: int) -> np.ndarray:
    return np.random.default_rng(SEED + stream).integers(0, vocab, n).astype(np.int32)


def decode_run(eng, cfg, batch: int, n_prompt: int, steps: int, warmup: int, salt: int, dist, local_rank: int, skip_prefill: bool = False):
    """Prompt ingestion, W untimed steps, then exactly K device-timed steps of `batch` sequences (max over
    ranks).  Returns the timing and every token produced, so callers can compare runs."""
    prefill_ms = None
    if skip_prefill:
        firsts = [int(prompt_tokens(cfg.vocab, n_prompt, s + salt)[0]) for s in range(batch)]
    else:
        firsts, prefill_ms = [], 0.0
        for s in range(batch):
            firsts.append(eng.prefill_tokens(s, prompt_tokens(cfg.vocab, n_prompt, s + salt), 0))
            prefill_ms += eng.last_timing()[0]  # device time of this prompt's ingestion (CUDA events in the engine)
    seqs = list(range(batch))
    pos = [n_prompt] * batch
    warm = eng.decode_greedy(seqs, firsts, pos, warmup)
    cur = [int(t) for t in warm[-1]]
    pos = [p + warm.shape[0] for p in pos]
    if dist:
        dist.barrier()
    sampler = clock_sampler(local_rank)
    sampler.start()
    out = eng.decode_greedy(seqs, cur, pos, steps)
    ms, launches = eng.last_timing()
    clocks = sampler.stop()
    if dist:
        import torch

        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return {"ms": ms, "launches": int(launches), "clocks": clocks, "firsts": firsts, "warm": warm, "out": out, "cur": cur, "pos": pos,
            "prefill_ms": prefill_ms}


def shard_of(cfg, rank: int, world: int, sharded: bool):
    if not sharded:
        return cfg
    from camelid_b200 import shard

    return shard.rank_config(cfg, rank, world)


def join_ranks(eng, dist, rank: int, world: int):
    """Hands every rank of a sharded engine the same communicator id (broadcast over torch.distributed)."""
    import torch

    idt = torch.zeros(128, dtype=torch.uint8, device="cuda")
    if rank == 0:
        idt.copy_(torch.frombuffer(bytearray(eng.comm_unique_id()), dtype=torch.uint8))
    dist.broadcast(idt, src=0)
    eng.comm_init(bytes(idt.cpu().numpy().tobytes()), rank, world)


def extra_run(cm, synth, workload: str, batch: int, n_prompt: int, steps: int, args, rank, world, local_rank, dist, sharded):
    """A second, shorter measurement kept as an extra key of the line (batch 32; the Mixtral shape)."""
    shape, mix, _, _ = WORKLOADS[workload]
    warmup = 3
    cfg = synth.engine_config(shape, max_pos=n_prompt + steps + warmup + 8, max_seqs=batch, device=local_rank, flags=args.engine_flags)
    cfg = shard_of(cfg, rank, world, sharded)
    eng = synth.build_engine(cfg, mix, SEED)
    if sharded:
        join_ranks(eng, dist, rank, world)
    r = decode_run(eng, cfg, batch, n_prompt, steps, warmup, 0 if sharded else 1000 * rank, dist, local_rank)
    eng.close()
    tokens = steps * batch * (1 if sharded else world)
    out = {"workload": workload, "batch": batch, "prompt_tokens": n_prompt, "steps": steps, "warmup": warmup,
           "value": tokens / (r["ms"] * 1e-3), "unit": "tokens/s", "ms_per_step": r["ms"] / steps, "gpu_launches": r["launches"],
           "parallelism": "single" if world == 1 else "replicas" if not sharded else (f"ep{world}" if cfg.n_experts > 0 else f"tp{world}")}
    if r["prefill_ms"]:
        out["prefill_tokens_per_s"] = n_prompt * batch / (r["prefill_ms"] * 1e-3)
    return out


def run_ours(args):
    import camelid_b200 as cm
    from camelid_b200 import synth

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist

        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    if cm.device_count() < 1:
        raise SystemExit("bench.py needs a CUDA device: the engine has no CPU path")

    shape, mix, n_prompt, ctx = WORKLOADS[args.workload]
    n_prompt = args.prompt or n_prompt
    batch = args.batch
    warmup = max(args.warmup, 3)
    full_cfg = synth.engine_config(shape, max_pos=ctx, max_seqs=batch, device=local_rank, flags=args.engine_flags)
    # N > 1: ONE model over the N GPUs (tensor-parallel for dense shapes, expert-parallel for Mixtral
    # shapes), total work fixed; --parallel replicas runs N independent copies instead.
    sharded = world > 1 and args.parallel != "replicas"
    cfg = shard_of(full_cfg, rank, world, sharded)
    want_cpu = rank == 0 and world == 1 and batch == 1 and not args.no_cpu_baseline
    cpu_model = None
    if want_cpu:
        from oracle import oracle as orc

        cpu_cfg = synth.engine_config(shape, max_pos=n_prompt + 96, max_seqs=1)
        cpu_model = orc.OracleModel(cpu_cfg.oracle_dict())
        layer_projs: dict[int, dict] = {}
        moe: dict[int, dict] = {}

        def tap(role, layer, w):
            wire = w.export_wire()
            if role in synth.SLOTS:
                layer_projs.setdefault(layer, {})[role] = (w.qt, wire)
            elif role == "output":
                cpu_model.set_output(np.ones(cfg.hidden, np.float32), w.qt, wire)
            elif role == "token_embd":
                cpu_model.set_token_embd(w.qt, wire)
            else:
                moe.setdefault(layer, {})[role] = (w.qt, wire)
    else:
        tap = None

    t0 = time.perf_counter()
    eng = synth.build_engine(cfg, mix, SEED, tap=tap)
    build_s = time.perf_counter() - t0
    if sharded:
        join_ranks(eng, dist, rank, world)
    if want_cpu:
        ones = np.ones(cfg.hidden, np.float32)
        for layer in range(cfg.n_layers):
            projs = layer_projs.get(layer, {})
            for name in ("gate", "up", "down"):
                projs.setdefault(name, (8, np.zeros(4, np.uint8)))
            cpu_model.set_layer(layer, projs, ones, ones)
            if layer in moe:
                mm = moe[layer]
                cpu_model.set_moe(layer, mm["router"][1].view(np.float32), mm["gate_exps"], mm["up_exps"], mm["down_exps"])

    salt = 0 if sharded else 1000 * rank  # ranks of one sharded model must feed identical rows
    r = decode_run(eng, cfg, batch, n_prompt, args.steps, warmup, salt, dist, local_rank, args.skip_prefill)
    ms, pos, cur, out = r["ms"], r["pos"], r["cur"], r["out"]
    tokens_total = args.steps * batch * (1 if sharded else world)
    value = tokens_total / (ms * 1e-3)
    device_tokens = np.concatenate([r["warm"][:, 0], out[:, 0]]).astype(np.int64)  # sequence 0, from the first decode step

    # end to end through the reference-facing call: host embedding + RoPE rows in, token id out
    e2e = None
    if batch == 1:
        e2e = run_e2e(cm, eng, cfg, synth, mix, cur, pos, out[:, 0], min(args.steps, 128))

    hbm_peak, peak_kind = measured_peaks()
    wbytes = synth.weight_bytes_per_token(full_cfg, mix)
    kvb = synth.kv_bytes_per_position(full_cfg)
    mean_ctx = pos[0] + args.steps / 2
    step_bytes = wbytes + batch * kvb * mean_ctx  # whole model, whichever way it is spread
    peaks = world  # the roofline of N GPUs is N times one GPU's bandwidth
    gbs = step_bytes / (ms / args.steps * 1e-3) / 1e9
    par = "single" if world == 1 else "replicas" if not sharded else (f"ep{world}" if cfg.n_experts > 0 else f"tp{world}")
    line = {
        "metric": "decode tokens/s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
        "scaling": "weak" if (world > 1 and not sharded) else "strong",
        "vs_baseline": None, "dtype": "int8 x int8 -> f32", "data": "synthetic",
        "config": {"workload": args.workload, "batch": batch, "prompt_tokens": n_prompt, "ctx_limit": ctx,
                   "context": f"positions {pos[0]}..{pos[0] + args.steps - 1} over a KV cache the engine filled from the prompt",
                   "parallelism": par, "engine_flags": args.engine_flags,
                   "engine_mode": ENGINE_MODES.get(args.engine_flags & (16 | 128), f"flags {args.engine_flags}"),
                   "l2": "inputs larger than L2: every step streams the model's weights (>= 1.3 GB) from HBM",
                   "model_build_s": round(build_s, 1)},
        "clocks": r["clocks"], "gpu_launches": r["launches"],
        "step_roofline": {"bytes_per_step": step_bytes, "achieved_gbs": gbs,
                          "frac_of_measured_copy_peak": gbs / (hbm_peak * peaks), "frac_of_8tbs_nominal": gbs / (8000.0 * peaks)},
    }
    if r["prefill_ms"] is not None:
        # not part of the metric: the prompts are ingested 32 rows at a time through the batched matvec
        line["prefill"] = {"prompt_tokens": n_prompt * batch, "ms": r["prefill_ms"], "tokens_per_s": n_prompt * batch / (r["prefill_ms"] * 1e-3)}
    if e2e:
        line["e2e"] = e2e

    if cpu_model is not None and not args.skip_prefill:
        # The CPU checker continues from the very KV prefix the engine built: its tokens are the parity
        # check of this run (the engine's default mode reproduces the CPU path bit for bit, so every
        # token must be equal), and its speed at this context is the CPU baseline.
        from oracle import oracle as orc

        threads = host_threads()
        orc.lib().orc_set_num_threads(threads)
        for layer in range(cfg.n_layers):
            ck, cv = eng.read_kv_layer(layer, n_prompt)
            cpu_model.write_kv_layer(layer, ck, cv)
        probe, toks, p = time_cpu_decode(cpu_model, cfg, 1, 0, n_prompt, r["firsts"][0])
        n = max(2, min(32, len(device_tokens) - 1, int(20.0 / max(probe, 1e-3))))
        sec_tok, more, p = time_cpu_decode(cpu_model, cfg, n, 0, p, toks[-1])
        cpu_tokens = np.array(toks + more, np.int64)
        same = int(np.sum(cpu_tokens == device_tokens[: cpu_tokens.size]))
        line["parity"] = {"tokens_equal_to_cpu_checker": f"{same}/{cpu_tokens.size}",
                          "what": f"greedy tokens at positions {n_prompt}..{p - 1}: this engine (timed mode, same weights, same KV prefix) "
                                  "against the CPU restatement of the reference"}
        line["cpu_baseline"] = {"value": 1.0 / sec_tok, "unit": "tokens/s", "cores": threads, "kind": "port",
                                "sample": f"{n} decode tokens of the same model (byte-identical weights) at context {n_prompt + 2}..{p}, "
                                          f"{threads} threads"}
    eng.close()  # before the process group goes: the engine's communicator is torn down on every rank here

    if sharded and not args.no_single_gpu_check:
        # The round-end tests run on one GPU: this key compares the sharded model's greedy tokens with a
        # single-GPU engine holding the whole model, on the same prompt (rank 0; the others wait).
        if rank == 0:
            n_cmp = int(min(32, device_tokens.size))
            one_cfg = synth.engine_config(shape, max_pos=n_prompt + n_cmp + 8, max_seqs=1, device=local_rank, flags=args.engine_flags)
            one = synth.build_engine(one_cfg, mix, SEED)
            first = one.prefill_tokens(0, prompt_tokens(cfg.vocab, n_prompt, 0), 0)
            # teacher forcing: the single-GPU engine is fed the sharded run's own tokens, so every position is an
            # independent comparison (a free-running pair parts for good at the first near tie of these random weights)
            same, tok_in, first_diff = 0, int(r["firsts"][0]), None
            for i in range(n_cmp):
                nxt = int(one.step_batch([0], [tok_in], [n_prompt + i])[0][0])
                if nxt == int(device_tokens[i]):
                    same += 1
                elif first_diff is None:
                    first_diff = i
                tok_in = int(device_tokens[i])
            one.close()
            line["multi_gpu_check"] = {"next_token_equal_to_single_gpu": f"{same}/{n_cmp}", "first_token_equal": bool(first == r["firsts"][0]),
                                       "first_difference_at_step": first_diff,
                                       "what": "rank 0's single-GPU engine (whole model, same prompt) fed the sharded run's tokens: positions where it "
                                               "predicts the sharded run's next token",
                                       "note": "sums over ranks are taken in another order than one GPU's, so a near tie can fall the other way"}
        dist.barrier()

    extras = [e for e in args.extras.split(",") if e] if (batch == 1 and args.workload == "llama-8b-q4_k_m" and not args.skip_prefill) else []
    for e in extras:
        if e == "batch32":
            x = extra_run(cm, synth, "llama-8b-q4_k_m", 32, 1024, min(args.steps, 32), args, rank, world, local_rank, dist, sharded)
        elif e == "mixtral":
            x = extra_run(cm, synth, "mixtral-8x7b-q4_k_m", 1, 512, min(args.steps, 32), args, rank, world, local_rank, dist, sharded)
        else:
            continue
        line[e] = x

    if rank == 0:
        # dominant kernel alone, at the model's largest layer shape
        qname = "Q8_0" if mix == "q8_0" else "Q4_K"
        alg, sec = gemv_roofline(cm, qname, full_cfg.ffn_dim, full_cfg.hidden, 1)
        line["roofline"] = {"bound": "hbm", "kernel": f"gemv_pipe_kernel<1> {qname} {full_cfg.ffn_dim}x{full_cfg.hidden}", "achieved": alg / sec / 1e9,
                            "peak": hbm_peak, "peak_kind": peak_kind + " copy bandwidth (burst: the kernel is timed alone)",
                            "unit": "GB/s", "frac": alg / sec / 1e9 / hbm_peak,
                            "traffic": NCU_DRAM_BYTES_PER_LAUNCH.get((qname, full_cfg.ffn_dim, full_cfg.hidden)),
                            "algorithmic_bytes": alg, "launch_us": sec * 1e6,
                            "timing": "CUDA events around one graph replay of 200 launches over rotating weight copies (> L2), "
                                      "chained by programmatic dependent launch like the engine's own step"}
        print(json.dumps(line), flush=True)
    if dist:
        dist.barrier()
        dist.destroy_process_group()


def run_e2e(cm, eng, cfg, synth, mix, cur, pos, device_tokens, n_steps):
    """K steps through cmld_engine_forward_token with host buffers, timed on the host clock
    (each call ends with the device-to-host read of the token)."""
    plan = synth.quant_plan(mix)
    emb_w = cm.Weight.synth(plan["token_embd"], SEED, synth.STREAM_EMBD, cfg.vocab, cfg.hidden, 0.02)
    toks = [cur[0]] + [int(t) for t in device_tokens[: n_steps - 1]]
    rows = np.stack([emb_w.dequant(t, 1)[0] for t in toks])
    emb_w.free()
    half = cfg.rope_dim // 2
    scale = float(np.float32(1.0) / np.sqrt(np.float32(cfg.head_dim)))
    # rewind: the same positions again (the KV rows are rewritten with the same values)
    ropes = [eng.rope_row(pos[0] + i) for i in range(n_steps)]  # the host-side table a Camelid caller computes per token
    got = []
    t0 = time.perf_counter()
    for i in range(n_steps):
        p = pos[0] + i
        c, sn = ropes[i]
        got.append(eng.forward_token(rows[i], c, sn, p, scale, True))
    dt = time.perf_counter() - t0
    same = int(np.sum(np.array(got[:-1]) == np.array(toks[1:])))
    return {"value": n_steps / dt, "unit": "tokens/s", "h2d_bytes_per_step": cfg.hidden * 4 + 2 * half * 4 + 8,
            "d2h_bytes_per_step": 4, "steps": n_steps, "tokens_equal_to_device_loop": f"{same}/{n_steps - 1}"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="llama-8b-q4_k_m", choices=sorted(WORKLOADS))
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--parallel", default="shard", choices=["shard", "replicas"],
                    help="N > 1: one model tensor-/expert-parallel over the GPUs (default), or N independent copies")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-single-gpu-check", action="store_true", help="N > 1: skip rank 0's comparison against a single-GPU engine")
    ap.add_argument("--extras", default="batch32,mixtral",
                    help="extra measurements kept as keys of the default line: batch32 (32 sequences) and mixtral (8x7B shape); '' for none")
    ap.add_argument("--skip-prefill", action="store_true",
                    help="profiling runs only: start decoding at the prompt length over an all-zero KV cache instead of ingesting a prompt")
    ap.add_argument("--prompt", type=int, default=0, help="override the workload's prompt length (profiling runs)")
    ap.add_argument("--engine-flags", type=int, default=0, help="CMLD_FLAG_* bits: 1 no CUDA graph, 2 direct-load matvec, 4 no PDL, 8 separate prep kernels, 16 plain reference-order kernels, 32 NCCL-only sums, 64 tensor-core matvec from 5 rows, 128 lane-parallel f32 sums")
    ap.add_argument("--watchdog", type=int, default=-1,
                    help="seconds after which a stuck run dumps its Python stacks and exits (default: 1500 when N > 1, off at N = 1)")
    args = ap.parse_args()
    wd = args.watchdog if args.watchdog >= 0 else (1500 if int(os.environ.get("WORLD_SIZE", "1")) > 1 else 0)
    if wd:
        import faulthandler

        faulthandler.dump_traceback_later(wd, exit=True)  # a rank waiting for a peer that died must not wait for ever
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
