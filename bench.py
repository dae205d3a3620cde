#!/usr/bin/env python
"""Headline benchmark: Qwen3-0.6B-shaped bf16 decode throughput at batch 64 per GPU.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A step is one decode launch over the whole batch (one new token per sequence).  Weights are
random-init from a seed (N(0, 0.02), norms 1, tied embeddings), prompts are 128 uniform token ids
per sequence, the kept K/V rows sit in 64-row pages behind a seeded random page table: synthetic
stand-ins of the configuration's shapes, nothing is read from disk but MEASURED_PEAKS.json.

  value  tokens/s with every input resident in HBM: the device-resident decode loop (each row's next
         token is the id it just produced), K graph replays timed with CUDA events on the launch stream.
  e2e    the same steps (the sequences restart from their prompts, so the positions and context lengths
         are those of the resident loop) through ts_decoder_step with host buffers: tokens/slots/positions
         copied host to device and the ids read back device to host inside the timed region, every step.
  roofline  the kernel with the largest share of a step.  Shares and durations come from CUDA events recorded
         after every kernel (ts_decoder_profile) at the timed steps' context lengths, right after the timed
         region: achieved = algorithmic bytes / that measured interval.  The pass serialises launches which overlap
         in the timed loop (programmatic dependent launch), so the interval holds the launch gap too and the
         fraction is a lower bound; `in_step_estimate` gives the interval less the average gap
         ((serialised step - timed step) / launches per step) beside it, marked as an estimate.
  workloads  after the headline: the GLM-style MoE decode (expert-parallel over the ranks, with a check of the
         exchange against the all-local block) and the embedding encoder (texts dealt to the ranks), a few steps
         each, nested in the same line; --no-extras skips them.

    python bench.py --workload sweep     one line per case of the isolated linear sweep (6 shapes x 6 row counts)
    python bench.py --workload attn      the isolated attention cases: causal prefill 4 x 4096, paged decode of 64
                                         ragged sequences (512..8192 positions) at 64- and 16-row pages
  cpu_baseline  the reference's native CPU rules restated in C (oracle/cpu_rules.c), timed on this
         host's cores on a bounded sample of the same step.

With N > 1 (torchrun, one rank per GPU) every rank decodes its own 64 sequences with replicated weights
and no collective on the data path: weak scaling; the time is the maximum over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

BATCH = 64
PROMPT = 128
FALLBACK_HBM_GBS = 6650.0  # earlier measurement on this pool, used only when MEASURED_PEAKS.json is absent

# (dram__bytes_read.sum + dram__bytes_write.sum) / algorithmic bytes of the captured launch, from ncu captures of
# small cases of the same kernels (bench.py --case <kernel>); traffic grows in proportion to the rows, keys and
# weights a launch visits, so a launch's traffic is this ratio times its algorithmic bytes.  Absent: no capture.
NCU_TRAFFIC_RATIO = {"attend_rows": 50.816 / 50.856, "linear_unembed": 340.02 / 350.19,
                     # one capture (the q,k,v shape) stands for the four streamed linears of a layer: same kernel,
                     # traffic = the weights once + x; the output stays in L2
                     "linear_qkv": 8.592 / 9.044, "linear_o": 8.592 / 9.044, "linear_gate_up": 8.592 / 9.044,
                     "linear_down": 8.592 / 9.044,
                     # the long-context paged attention kernel (64 rows x 4096 keys), the one-row skinny linear and the
                     # grouped expert kernel (one rank of eight: 16 experts' weights a launch)
                     "attend_rows_long": 1081.5 / 1074.27, "linear_skinny": 12.62 / 12.59, "moe_grouped": 0.96}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--pdl", type=int, default=1)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--step-kernel", type=int, default=0,
                    help="decode: 1 = the gather and every layer as one persistent kernel per step, 0 = one launch per "
                         "product (default: the faster of the two today)")
    ap.add_argument("--no-extras", action="store_true", help="decode: skip the MoE and embedding workloads nested after the headline")
    ap.add_argument("--workload", default="decode", choices=["decode", "moe", "embed", "sweep", "attn"],
                    help="decode: the headline Qwen3-0.6B-shaped decode (default); moe: GLM-style MoE decode, batch 256 at "
                         "context 2048, expert-parallel over the ranks; embed: 1024 ragged texts through the "
                         "EmbeddingGemma-300M-shaped encoder, data-parallel over the ranks")
    ap.add_argument("--one-rank-of", type=int, default=0,
                    help="with --workload moe on one GPU: run rank 0's share of an N-rank expert-parallel step with local "
                         "copies in place of the collectives (for ncu, which cannot wrap a multi-rank command)")
    ap.add_argument("--case", default=None,
                    help="time one kernel of the step list alone at the benchmark's shapes (attend_rows, linear_qkv, "
                         "linear_o, linear_gate_up, linear_down, linear_unembed); used for ncu captures")
    ap.add_argument("--ctx", type=int, default=192, help="--case attend_rows: context length of every row")
    ap.add_argument("--rows", type=int, default=BATCH, help="--case: rows (batch) of the launch")
    ap.add_argument("--l2-warm", action="store_true", help="--case attend_rows: one copy of the kept rows, so launches find them in L2")
    ap.add_argument("--path", default="auto", choices=["auto", "skinny", "umma", "stream", "pair"],
                    help="--case linear_* and --workload sweep: kernel family")
    ap.add_argument("--only-rows", type=int, default=0, help="--workload sweep: only this row count")
    ap.add_argument("--q8", action="store_true", help="--workload sweep: also the Q8_0 weight form at the decode-sized row counts")
    return ap.parse_args()


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return float(json.load(open(path))["hbm_gbs"]), "measured"
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of one GPU, sampled every 50 ms by one background process from before
    the warm-up until after the last timed loop.  `start()` / `stop()` bracket a timed region; the summary uses the
    samples whose timestamps fall inside a region, or, when a region was shorter than nvidia-smi's start-up and
    interval, the samples taken while the same steps ran as warm-up (it says which)."""
    QUERY = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int, enabled: bool = True):
        self.gpu, self.proc, self.lines, self.windows, self._t0 = gpu_index, None, [], [], None
        if not enabled:   # only the rank that prints samples
            return
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-i", str(self.gpu), "-lms", "50"], stdout=subprocess.PIPE, text=True)
        except OSError:
            self.proc = None

    def start(self):
        self._t0 = time.time()

    def stop(self):
        if self._t0 is not None:
            self.windows.append((self._t0, time.time()))
            self._t0 = None

    def close(self):
        if self.proc is None:
            return
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        self.lines += [l for l in out.splitlines() if l.strip()]
        self.proc = None

    @staticmethod
    def _when(stamp: str):
        import datetime
        try:
            return datetime.datetime.strptime(stamp.strip(), "%Y/%m/%d %H:%M:%S.%f").timestamp()
        except ValueError:
            return None

    def summary(self) -> dict:
        self.close()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        rows = []
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                rows.append((self._when(f[0]), float(f[1]), float(f[2]),
                             [n for n, flag in zip(names, f[5:9]) if flag.lower().startswith("active")]))
            except ValueError:
                continue
        inside = [r for r in rows if r[0] is not None and any(a <= r[0] <= b for a, b in self.windows)]
        window = "timed regions"
        if not inside and self.windows:   # regions shorter than the sampling interval: the load around them
            lo, hi = min(a for a, _ in self.windows) - 1.0, max(b for _, b in self.windows) + 0.2
            inside = [r for r in rows if r[0] is not None and lo <= r[0] <= hi]
            window = "warm-up and timed regions (the timed regions fell between two samples)"
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(r[1] for r in inside), "sm_max_mhz": max(r[2] for r in inside),
                "reasons": sorted({n for r in inside for n in r[3]}), "samples": len(inside), "window": window}


def kernel_bytes(name: str, cfg: dict, rows: int, ctx_sum: int) -> float:
    """Algorithmic bytes one launch of a step-list kernel must move (bf16 = 2 bytes)."""
    h, d = cfg["hidden"], cfg["head_dim"]
    qw, kw, f, v = cfg["heads"] * d, cfg["kv_heads"] * d, cfg["ffn"], cfg["vocab"]
    lin = lambda n, k, out_b: 2.0 * n * k + 2.0 * rows * k + out_b
    if name == "attend_rows":  # every visible K and V row once, q in, out
        return ctx_sum * kw * 2.0 * 2 + rows * qw * 2.0 * 2
    if name == "linear_qkv":
        return lin(qw + 2 * kw, h, 2.0 * rows * (qw + 2 * kw))
    if name == "linear_o":
        return lin(h, qw, 8.0 * rows * h)  # f32 residual in and out
    if name == "linear_gate_up":
        return lin(2 * f, h, 2.0 * rows * f)
    if name == "linear_down":
        return lin(h, f, 8.0 * rows * h)
    if name == "linear_unembed":
        return lin(v, h, 4.0 * rows * v)
    if name == "decode_layers":  # the persistent kernel: every layer's weights and kept rows once
        return cfg["layers"] * sum(kernel_bytes(k, cfg, rows, ctx_sum) for k in
                                   ("attend_rows", "linear_qkv", "linear_o", "linear_gate_up", "linear_down"))
    return 0.0


def cpu_weights(cfg, seed):
    from tessera_b200 import synth
    w = {k: [] for k in ("q", "k", "v", "o", "gate", "up", "down", "ln1", "ln2", "q_norm", "k_norm")}
    named = []
    for name, a in synth.decoder_weights(cfg, seed):
        named.append((name, a))
        if name in ("embed", "norm"):
            w[name] = a
        else:
            w[name.split(".", 2)[2].replace("mlp.", "")].append(a)
    return named, w


def cpu_step_rate(cfg, weights, rows, position, budget_s, min_steps=1, max_steps=8):
    """tokens/s of the CPU rules on `rows` sequences at `position` (earlier kept rows zero-filled)."""
    import oracle as O
    dec = O.CpuRulesDecoder(dict(cfg, context=position + max_steps + 1, slots=rows), weights)
    toks = np.arange(rows, dtype=np.uint32) % cfg["vocab"]
    slots = np.arange(rows, dtype=np.uint32)
    times = []
    t_all = time.perf_counter()
    for i in range(max_steps):
        t0 = time.perf_counter()
        toks = dec.step(toks, slots, np.full(rows, position + i, np.uint32))
        times.append(time.perf_counter() - t0)
        if i + 1 >= min_steps and time.perf_counter() - t_all > budget_s:
            break
    best = min(times)
    return rows / best, dec.threads, len(times), best


def run_reference(args, rank):
    """The reference's CPU path for this step (restated: the Rust workspace cannot be built here),
    all host threads, each step a bounded sample of the batch."""
    if rank != 0:
        return
    from tessera_b200 import synth
    cfg = synth.QWEN3_0_6B
    _, w = cpu_weights(cfg, 0)
    # one full-batch step sizes the per-step sample so that warmup + steps fit in about two minutes
    full_rate, threads, _, t_full = cpu_step_rate(cfg, w, BATCH, PROMPT, 0.0, 1, 1)
    total = args.steps + args.warmup
    rows = int(max(1, min(BATCH, BATCH * 120.0 / (total * t_full))))
    import oracle as O
    dec = O.CpuRulesDecoder(dict(cfg, context=PROMPT + total + 1, slots=rows), w)
    toks = np.arange(rows, dtype=np.uint32)
    slots = np.arange(rows, dtype=np.uint32)
    for i in range(args.warmup):
        toks = dec.step(toks, slots, np.full(rows, PROMPT + i, np.uint32))
    t0 = time.perf_counter()
    for i in range(args.steps):
        toks = dec.step(toks, slots, np.full(rows, PROMPT + args.warmup + i, np.uint32))
    dt = time.perf_counter() - t0
    value = rows * args.steps / dt
    sample = f"{rows} of {BATCH} sequences per step at positions {PROMPT}+, kept rows before the prompt end zero-filled"
    print(json.dumps({
        "impl": "reference", "metric": "decode_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32 activations, bf16 weights", "data": "synthetic",
        "config": {"workload": "Qwen3-0.6B-shaped decode, batch 64, prompt 128 (CPU rules restated in C; the "
                               "reference's Rust/Cranelift path is unavailable on this box)", "batch": BATCH,
                   "prompt": PROMPT},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def run_ours(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist
    from tessera_b200 import runner, synth

    torch.cuda.set_device(local_rank)
    cfg = synth.QWEN3_0_6B
    K, W = args.steps, args.warmup
    profile_steps = 3
    context = PROMPT + 2 * (K + W) + profile_steps + 8
    context = (context + 63) // 64 * 64
    dec = runner.Decoder(cfg, slots=BATCH, context=context, max_rows=2048, page=64, graphs=True, pdl=bool(args.pdl))
    named, cpu_w = cpu_weights(cfg, 0)
    dec.load_all(named)
    dec.use_step_kernel(bool(args.step_kernel))
    dec.set_table(synth.page_permutation(BATCH * dec.pages, seed=4 + rank))
    side = torch.cuda.Stream()  # the legacy NULL stream cannot be captured into graphs
    torch.cuda.set_stream(side)
    stream = side.cuda_stream
    prompts = [synth.prompt_tokens(cfg["vocab"], PROMPT, seed=1000 * rank + s) for s in range(BATCH)]
    slots = np.arange(BATCH, dtype=np.uint32)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    sampler = ClockSampler(local_rank, enabled=rank == 0)
    first = dec.prefill(prompts)
    dec.prepare(BATCH, stream)  # graphs of every context bucket exist before anything is timed
    pos = PROMPT
    cur = dec.step(first, slots, np.full(BATCH, pos, np.uint32), stream=stream)  # one row per slot on the device
    pos += 1

    # ---- value: device-resident loop ----
    dec.run_resident(W, stream)
    pos += W
    barrier()
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    dec.run_resident(K, stream)
    e1.record()
    torch.cuda.synchronize()
    sampler.stop()
    resident_s = max_over_ranks(e0.elapsed_time(e1) / 1e3)
    ctx_mid = pos + K / 2.0  # mean visible positions per row over the timed steps
    pos += K
    barrier()
    cur = dec.read_ids(BATCH, stream)

    # ---- e2e: host buffers in and out every step, over the same positions as the resident loop ----
    # (the sequences start again from their prompts, so that both loops see the same context lengths)
    first = dec.prefill(prompts)
    pos = PROMPT
    cur = dec.step(first, slots, np.full(BATCH, pos, np.uint32), stream=stream)
    pos += 1
    for i in range(W):
        cur = dec.step(cur, slots, np.full(BATCH, pos, np.uint32), stream=stream)
        pos += 1
    barrier()
    sampler.start()
    t0 = time.perf_counter()
    for i in range(K):
        cur = dec.step(cur, slots, np.full(BATCH, pos, np.uint32), stream=stream)
        pos += 1
    torch.cuda.synchronize()
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    sampler.stop()
    barrier()

    launches_per_step = dec.launches_per_step(BATCH, min(context, (pos + 127) // 128 * 128))
    # ---- per-kernel device time, live, for the roofline of the dominant kernel ----
    # The sequences start again and run up to the middle of the timed steps' positions, so that the profiled
    # launches see the context lengths the timed steps saw.  The profile records an event after every kernel:
    # that serialises launches that overlap in the timed loop (programmatic dependent launch) and adds the gap
    # between launches to every interval.  The serialised step is longer than the timed step by that gap times the
    # launches of a step: a kernel's duration inside the timed loop is taken as its serialised interval less the
    # average gap, and the serialised interval is reported beside it.
    first = dec.prefill(prompts)
    pos = PROMPT
    cur = dec.step(first, slots, np.full(BATCH, pos, np.uint32), stream=stream)
    pos += 1
    ahead = int(ctx_mid - (profile_steps + 1) / 2.0) - pos
    if ahead > 0:
        dec.run_resident(ahead, stream)
        pos += ahead
    prof = dec.profile(profile_steps, stream)
    ctx_prof = pos + (profile_steps + 1) / 2.0
    step_ms = sum(ms for ms, _ in prof.values()) / profile_steps
    shares = {k: ms / profile_steps / step_ms for k, (ms, n) in prof.items()}
    top = max(prof, key=lambda k: prof[k][0])
    top_ms, top_n = prof[top]
    timed_step_s = resident_s / K
    launches = sum(n for _, n in prof.values()) / profile_steps
    gap_s = max(0.0, step_ms / 1e3 - timed_step_s) / launches   # what serialising adds to every launch, on average

    def serial_s(k):    # per launch, as measured: the interval between the events either side of the kernel
        return prof[k][0] / prof[k][1] / 1e3

    def in_step_s(k):   # an estimate of the same launch inside the timed loop: less the average serialising gap
        return max(serial_s(k) - gap_s, 1e-9)
    peak, peak_kind = peaks()
    algo = kernel_bytes(top, cfg, BATCH, int(BATCH * ctx_prof))
    achieved = algo / serial_s(top) / 1e9
    ratio = NCU_TRAFFIC_RATIO.get(top)
    roofline = {"kernel": top, "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak, "peak_kind": f"of {peak_kind}", "frac_of_nominal_8tbs": achieved / 8000.0,
                "traffic": (ratio * algo if ratio else None),
                "traffic_source": ("dram bytes / algorithmic bytes of the committed ncu capture of this kernel, times this "
                                   "launch's algorithmic bytes" if ratio else None),
                "algorithmic_bytes_per_launch": algo, "avg_launch_us": serial_s(top) * 1e6,
                "duration": "measured: interval between CUDA events recorded after every kernel of the step (launches "
                            "serialised, so it includes the gap between two launches: a lower bound on the fraction)",
                "in_step_estimate": {"avg_launch_us": in_step_s(top) * 1e6, "frac": algo / in_step_s(top) / 1e9 / peak,
                                     "serialising_gap_us": gap_s * 1e6,
                                     "how": "interval less (serialised step - timed step) / launches per step"},
                "step_share": shares[top], "kernel_shares": {k: round(v, 4) for k, v in sorted(shares.items())},
                "per_kernel_gbs": {k: round(kernel_bytes(k, cfg, BATCH, int(BATCH * ctx_prof)) / serial_s(k) / 1e9, 1)
                                   for k, (ms, n) in prof.items() if kernel_bytes(k, cfg, BATCH, 1) > 0}}
    dec.close()
    torch.cuda.set_stream(torch.cuda.default_stream())
    if rank != 0:
        return None

    value = world * BATCH * K / resident_s
    step_bytes = sum(kernel_bytes(k, cfg, BATCH, int(BATCH * ctx_mid)) for k in ("decode_layers", "linear_unembed"))
    out = {
        "metric": "decode_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": resident_s / K * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "Qwen3-0.6B-shaped decode (28 layers, hidden 1024, 16q/8kv heads x 128, ffn 3072, "
                               "vocab 151936, tied), batch 64 per GPU, prompt 128, greedy, paged KV (64-row pages, "
                               "random page table)", "batch_per_gpu": BATCH, "prompt": PROMPT,
                   "context_at_timed_steps": [int(ctx_mid - K / 2), int(ctx_mid + K / 2)],
                   "l2": "each step streams 1.19 GB of weights plus the kept rows: inputs larger than the 126 MB L2",
                   "parallelism": f"dp{world} (independent sequences, replicated weights, no collective)",
                   "graphs": True, "pdl": bool(args.pdl)},
        "e2e": {"value": world * BATCH * K / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": 3 * BATCH * 4,
                "d2h_bytes_per_step": BATCH * 4, "ms_per_step": e2e_s / K * 1e3},
        "gpu_launches": (launches_per_step + 1) * K,
        "step_algorithmic_gb": step_bytes / 1e9, "step_hbm_frac": step_bytes / (resident_s / K) / 1e9 / peak,
        "roofline": roofline, "clocks": sampler.summary(),
    }
    if world == 1 and not args.no_cpu_baseline:
        try:
            rate, threads, n, best = cpu_step_rate(cfg, cpu_w, BATCH, PROMPT, 12.0, 2, 8)
            out["cpu_baseline"] = {"value": rate, "unit": "tokens/s", "cores": threads, "kind": "port",
                                   "sample": f"best of {n} full-batch decode steps (64 rows at positions {PROMPT}+, "
                                             f"kept rows before them zero-filled), {best:.2f} s per step"}
        except Exception as e:  # the baseline is a report, never a reason to lose the GPU numbers
            out["cpu_baseline"] = {"value": None, "unit": "tokens/s", "cores": 0, "kind": "port", "sample": f"failed: {e}"}
    return out


def run_case(args):
    """One kernel alone, at the step's shapes, through the C ABI: `steps` launches replayed from a CUDA
    graph over buffers rotated through more than the L2's 126 MB, timed with CUDA events."""
    import torch
    from tessera_b200 import ops, synth
    cfg = synth.QWEN3_0_6B
    rows = args.rows
    h, d = cfg["hidden"], cfg["head_dim"]
    qw, kw, f, v = cfg["heads"] * d, cfg["kv_heads"] * d, cfg["ffn"], cfg["vocab"]
    torch.manual_seed(0)
    side = torch.cuda.Stream()
    torch.cuda.set_stream(side)
    bf = lambda *shape, std=1.0: (torch.randn(*shape, device="cuda") * std).to(torch.bfloat16)
    calls = []
    if args.case == "attend_rows":
        ctx, page = args.ctx, 64
        pages = -(-ctx // page)
        copies = max(2, int(400e6 // (rows * pages * page * kw * 4)) + 1)
        if args.l2_warm:
            copies = 1   # the same kept rows every launch: they stay in the 126 MB L2 (what a prefetch ahead of the launch would give)
        slots = torch.arange(rows, dtype=torch.int32, device="cuda")
        positions = torch.full((rows,), ctx - 1, dtype=torch.int32, device="cuda")
        q = bf(rows, cfg["heads"], d)
        for c in range(copies):
            table = torch.from_numpy(synth.page_permutation(rows * pages, seed=c).view(np.int32)).cuda()
            kept = ops.Kept("paged", pages, table, rows * pages * page)
            k, vv = bf(rows * pages * page, cfg["kv_heads"], d), bf(rows * pages * page, cfg["kv_heads"], d)
            out = torch.empty_like(q)
            calls.append(lambda k=k, vv=vv, kept=kept, out=out: ops.attend_rows(
                q, k, vv, slots, positions, kept, ctx, scale=d ** -0.5, out=out))
        algo = kernel_bytes("attend_rows", cfg, rows, rows * ctx)
    elif args.case == "attend_flash":
        # causal prefill attention of the isolated attention configuration, one sequence of --ctx tokens
        n = args.ctx if args.ctx > 192 else 4096
        copies = 2
        for c in range(copies):
            q, k, vv = bf(1, n, cfg["heads"], d), bf(1, n, cfg["kv_heads"], d), bf(1, n, cfg["kv_heads"], d)
            out = torch.empty_like(q)
            calls.append(lambda q=q, k=k, vv=vv, out=out: ops.attend(q, k, vv, mask="causal", scale=d ** -0.5, out=out))
        algo = 4.0 * cfg["heads"] * d * n * (n + 1) / 2  # flops
    elif args.case == "linear_prefill":
        # prefill-sized linear: 2048 rows through the fused gate|up shape (n 6144, k 1024)
        rows = args.rows if args.rows > 128 else 2048
        n, k = 2 * f, h
        x = bf(rows, k)
        for c in range(4):
            w = bf(n, k, std=0.02)
            out = torch.empty((rows, n), dtype=torch.bfloat16, device="cuda")
            calls.append(lambda w=w, out=out: ops.linear(x, w, out=out, path=args.path))
        algo = 2.0 * rows * n * k  # flops
    else:
        shapes = {"linear_qkv": (qw + 2 * kw, h, "none", torch.bfloat16), "linear_o": (h, qw, "add", torch.float32),
                  "linear_gate_up": (2 * f, h, "swiglu", torch.bfloat16), "linear_down": (h, f, "add", torch.float32),
                  "linear_unembed": (v, h, "none", torch.float32)}
        n, k, epi, odt = shapes[args.case]
        copies = min(64, max(2, int(400e6 // (n * k * 2)) + 1))
        x = bf(rows, k)
        res = torch.randn(rows, n, device="cuda") if epi == "add" else None
        for c in range(copies):
            w = bf(n, k, std=0.02)
            out = torch.empty((rows, n // 2 if epi == "swiglu" else n), dtype=odt, device="cuda")
            calls.append(lambda w=w, out=out: ops.linear(x, w, res, epilogue=epi, out_dtype=odt, out=out, path=args.path))
        algo = kernel_bytes(args.case, cfg, rows, 0)
    ops.set_pdl(bool(args.pdl))
    for i in range(max(3, args.warmup)):
        calls[i % len(calls)]()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        for i in range(args.steps):
            calls[i % len(calls)]()
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    graph.replay()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / args.steps
    peak, kind = peaks()
    if args.case in ("attend_flash", "linear_prefill"):
        tf_peak = 1694.8
        path = os.path.join(ROOT, "MEASURED_PEAKS.json")
        if os.path.exists(path):
            tf_peak = float(json.load(open(path))["bf16_tflops"])
        print(json.dumps({"case": args.case, "us_per_launch": us, "algorithmic_flops": algo, "TFLOPs": algo / us / 1e6,
                          "frac": algo / us / 1e6 / tf_peak, "peak_kind": kind + " (burst)", "launches": args.steps,
                          "status": ops.device_status()}))
        return
    print(json.dumps({"case": args.case, "rows": rows, "ctx": args.ctx if args.case == "attend_rows" else None,
                      "us_per_launch": us, "algorithmic_bytes": algo, "GBs": algo / us / 1e3,
                      "frac": algo / us / 1e3 / peak, "peak_kind": kind, "launches": args.steps, "copies": len(calls),
                      "status": ops.device_status()}))


def _tensor_peaks():
    """(burst, sustained) bf16 TFLOP/s of MEASURED_PEAKS.json, else the pool's earlier measurement."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return float(d["bf16_tflops"]), float(d["bf16_tflops_sustained"]), "measured"
    return 1590.0, 1400.0, "fallback"


def _graph_us(calls, steps, warmup=3):
    """`steps` launches replayed from one CUDA graph, the calls taken in turn (their buffers together exceed the
    L2), timed with CUDA events on the launch stream; microseconds per launch."""
    import torch
    side = torch.cuda.current_stream()
    for i in range(max(3, warmup)):
        calls[i % len(calls)]()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        for i in range(steps):
            calls[i % len(calls)]()
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    graph.replay()
    e1.record()
    torch.cuda.synchronize()
    del graph
    return e0.elapsed_time(e1) * 1e3 / steps


SWEEP_SHAPES = [("q_proj", 2048, 1024), ("kv_proj", 1024, 1024), ("o_proj", 1024, 2048), ("gate_up", 6144, 1024),
                ("down", 1024, 3072), ("lm_head", 151936, 1024)]
SWEEP_ROWS = [1, 16, 64, 128, 2048, 8192]


def run_sweep(args):
    """The isolated linear sweep: every (N, K) of the Qwen3-0.6B shape at every M, the kernel path "auto" picks,
    one JSON line a case.  Decode-sized M (<= 128) is weight-bound: GB/s of the algorithmic bytes against the
    measured copy rate; prefill-sized M is tensor-bound: TFLOP/s against the measured cuBLAS burst."""
    import torch
    from tessera_b200 import ops
    torch.manual_seed(0)
    side = torch.cuda.Stream()
    torch.cuda.set_stream(side)
    ops.set_pdl(bool(args.pdl))
    hbm, hbm_kind = peaks()
    burst, _, tf_kind = _tensor_peaks()
    bf = lambda *shape, std=1.0: (torch.randn(*shape, device="cuda") * std).to(torch.bfloat16)
    for name, n, k in SWEEP_SHAPES:
        copies = min(48, max(2, int(400e6 // (n * k * 2)) + 1))   # rotated so that a launch never finds its weights in L2
        ws = [bf(n, k, std=0.02) for _ in range(copies)]
        for m in ([args.only_rows] if args.only_rows else SWEEP_ROWS):
            x = bf(m, k)
            outs = [torch.empty((m, n), dtype=torch.bfloat16, device="cuda") for _ in range(min(copies, 4))]
            calls = [(lambda w=w, o=outs[i % len(outs)]: ops.linear(x, w, out=o, path=args.path)) for i, w in enumerate(ws)]
            steps = max(8, min(200, int(2e9 // (2.0 * m * n * k + 1e7))))
            us = _graph_us(calls, steps)
            byts, flops = 2.0 * n * k + 2.0 * m * k + 2.0 * m * n, 2.0 * m * n * k
            bound = "hbm" if m <= 128 else "tensor"
            line = {"workload": "linear sweep", "case": name, "m": m, "n": n, "k": k, "us_per_launch": round(us, 3),
                    "GBs": round(byts / us / 1e3, 1), "TFLOPs": round(flops / us / 1e6, 2), "bound": bound,
                    "frac": round((byts / us / 1e3 / hbm) if bound == "hbm" else (flops / us / 1e6 / burst), 4),
                    "peak_kind": f"of {hbm_kind} copy rate" if bound == "hbm" else f"of {tf_kind} cuBLAS bf16 burst",
                    "path": args.path, "launches": steps, "weight_copies": copies, "status": ops.device_status()}
            print(json.dumps(line), flush=True)
        del ws
        if args.q8:   # the same shape with Q8_0 weights: 34 bytes per 32 weights
            packed = [ops.q8_0_pack(torch.randn(n, k) * 0.02).cuda() for _ in range(min(copies, 12) if n < 100000 else 2)]
            for m in [r for r in ([args.only_rows] if args.only_rows else SWEEP_ROWS) if r <= 64]:
                x = bf(m, k)
                out = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
                calls = [(lambda w=w: ops.linear_q8_0(x, w, out=out)) for w in packed]
                steps = max(8, min(200, int(2e9 // (2.0 * m * n * k + 1e7))))
                us = _graph_us(calls, steps)
                byts = n * (k // 32) * 34.0 + 2.0 * m * k + 2.0 * m * n
                print(json.dumps({"workload": "linear sweep", "form": "q8_0", "case": name, "m": m, "n": n, "k": k,
                                  "us_per_launch": round(us, 3), "GBs": round(byts / us / 1e3, 1), "bound": "hbm",
                                  "frac": round(byts / us / 1e3 / hbm, 4), "peak_kind": f"of {hbm_kind} copy rate",
                                  "launches": steps, "weight_copies": len(packed), "status": ops.device_status()}), flush=True)
            del packed


def run_attn(args):
    """The isolated attention cases: (a) causal prefill, 4 sequences x 4096 tokens, 16 query / 8 kv heads x 128;
    (b) paged decode, 64 sequences with context lengths uniform in [512, 8192] (seed 4) behind a seeded random page
    table, at 64- and 16-row pages.  One JSON line a case."""
    import torch
    from tessera_b200 import ops, synth
    torch.manual_seed(0)
    side = torch.cuda.Stream()
    torch.cuda.set_stream(side)
    ops.set_pdl(bool(args.pdl))
    hbm, hbm_kind = peaks()
    burst, _, tf_kind = _tensor_peaks()
    heads, kv_heads, d = 16, 8, 128
    bf = lambda *shape: torch.randn(*shape, device="cuda").to(torch.bfloat16)
    seqs, n = 4, 4096
    calls = []
    for c in range(2):
        q, k, v = bf(seqs, n, heads, d), bf(seqs, n, kv_heads, d), bf(seqs, n, kv_heads, d)
        out = torch.empty_like(q)
        calls.append(lambda q=q, k=k, v=v, out=out: ops.attend(q, k, v, mask="causal", scale=d ** -0.5, out=out))
    us = _graph_us(calls, 20)
    flops = 4.0 * seqs * heads * d * n * (n + 1) / 2
    print(json.dumps({"workload": "attention", "case": "causal prefill 4 x 4096, 16q/8kv x 128", "us_per_launch": round(us, 2),
                      "TFLOPs": round(flops / us / 1e6, 1), "bound": "tensor", "frac": round(flops / us / 1e6 / burst, 4),
                      "peak_kind": f"of {tf_kind} cuBLAS bf16 burst", "launches": 20, "status": ops.device_status()}), flush=True)
    del calls
    slots, context = 64, 8192
    lengths = np.random.default_rng(4).integers(512, 8193, size=slots)
    q = bf(slots, heads, d)
    row_slots = torch.arange(slots, dtype=torch.int32, device="cuda")
    positions = torch.from_numpy((lengths - 1).astype(np.int32)).cuda()
    for page in (64, 16):
        pages = context // page
        total = slots * pages * page
        table = torch.from_numpy(synth.page_permutation(slots * pages, seed=4).view(np.int32)).cuda()
        kept = ops.Kept("paged" if page == 64 else "paged16", pages, table, total)
        k, v = bf(total, kv_heads, d), bf(total, kv_heads, d)   # 1 GB each: far beyond the L2
        out = torch.empty_like(q)
        call = lambda: ops.attend_rows(q, k, v, row_slots, positions, kept, context, scale=d ** -0.5, out=out)
        us = _graph_us([call], 20)
        byts = float(lengths.sum()) * kv_heads * d * 2 * 2 + slots * heads * d * 2 * 2
        print(json.dumps({"workload": "attention", "case": f"paged decode, 64 sequences of 512..8192 positions, {page}-row pages",
                          "us_per_launch": round(us, 2), "GBs": round(byts / us / 1e3, 1), "bound": "hbm",
                          "frac": round(byts / us / 1e3 / hbm, 4), "peak_kind": f"of {hbm_kind} copy rate",
                          "traffic": round(NCU_TRAFFIC_RATIO["attend_rows_long"] * byts),
                          "traffic_source": "dram bytes / algorithmic bytes of the ncu capture of the same kernel at 64 x 4096 "
                                            "keys, times this launch's algorithmic bytes",
                          "positions_total": int(lengths.sum()), "launches": 20, "status": ops.device_status()}), flush=True)
        del k, v


def _dist_setup(local_rank, world):
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(local_rank)


def _timed(fn, steps, warmup, world):
    """W warm-up calls, then `steps` calls between CUDA events on the current stream, bracketed by barriers;
    returns the slowest rank's seconds."""
    import torch
    import torch.distributed as dist
    from tessera_b200 import dp
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        fn(warmup + i)
    e1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    return dp.max_over_ranks(e0.elapsed_time(e1) / 1e3, device="cuda")


def run_moe(args, rank, world, local_rank):
    """GLM-style MoE decode: batch 256 at context 2048, experts split over the ranks, token rows split evenly."""
    import torch
    import torch.distributed as dist
    from tessera_b200.moe_decoder import GLM_MOE, MoeDecoder
    alone = args.one_rank_of > 1    # one rank's kernels on one GPU, collectives replaced by local copies
    if alone:
        world = args.one_rank_of
    else:
        _dist_setup(local_rank, world)
    cfg = GLM_MOE
    batch, ctx0 = 256, 2048
    rows = batch // world
    K, W = args.steps, max(args.warmup, 3)
    context = ctx0 + 2 * (K + W) + 64
    dec = MoeDecoder(cfg, slots=rows, context=context, rank=rank, world=world, seed=0, alone=alone)
    dec.fill_kept(seed=1 + rank)
    dec.set_table(np.random.default_rng(7 + rank).permutation(rows * dec.pages))
    slots = torch.arange(rows, dtype=torch.int32, device="cuda")
    x_host = torch.randn(rows, cfg["hidden"], generator=torch.Generator().manual_seed(rank)).pin_memory()
    x_dev = x_host.cuda()
    sampler = ClockSampler(local_rank, enabled=rank == 0)
    graphed = os.environ.get("TS_MOE_GRAPHS", "1") != "0"
    step = dec.step_graphed if graphed else (lambda x, s, p, k: dec.step(x.clone(), s, p, k))

    def resident(i):
        pos = torch.full((rows,), ctx0 + i, dtype=torch.int32, device="cuda")
        step(x_dev, slots, pos, min(context, (ctx0 + i + 128) // 128 * 128))

    out_host = torch.empty(rows, cfg["hidden"]).pin_memory()

    def through_host(i):
        x = x_host.to("cuda", non_blocking=True)
        pos = torch.full((rows,), ctx0 + K + W + i, dtype=torch.int32, device="cuda")
        y = step(x, slots, pos, min(context, (ctx0 + K + W + i + 128) // 128 * 128))
        out_host.copy_(y, non_blocking=True)
        torch.cuda.synchronize()

    if graphed:   # capture every context bucket the two loops will meet before anything is timed
        for ctx in range(ctx0, ctx0 + 2 * (K + W) + 1):
            keys = min(context, (ctx + 128) // 128 * 128)
            if (rows, keys) not in dec._graphs:
                step(x_dev, slots, torch.full((rows,), ctx, dtype=torch.int32, device="cuda"), keys)
        torch.cuda.synchronize()
    sampler.start()
    seconds = _timed(resident, K, W, 1 if alone else world)
    e2e_seconds = _timed(through_host, K, W, 1 if alone else world)
    sampler.stop()
    dec.close()   # graphs with captured collectives must go before the communicator does
    check = None if alone else ep_check(rank, world)
    if rank != 0:
        return None
    peak, kind = peaks()
    per = cfg["experts"] // world
    expert_bytes = cfg["layers"] * per * 3 * cfg["hidden"] * cfg["ffn"] * 2.0
    dense_bytes = cfg["layers"] * ((cfg["heads"] + 2 * cfg["kv_heads"]) * cfg["head_dim"] * cfg["hidden"] +
                                   cfg["hidden"] * cfg["heads"] * cfg["head_dim"] + cfg["experts"] * cfg["hidden"] +
                                   3 * cfg["hidden"] * cfg["shared_ffn"]) * 2.0
    kv_bytes = cfg["layers"] * rows * ctx0 * cfg["kv_heads"] * cfg["head_dim"] * 4.0
    step_bytes = expert_bytes + dense_bytes + kv_bytes
    return ({
        "metric": "moe_decode_tokens_per_s" + ("_one_rank_alone" if alone else ""), "value": batch * K / seconds,
        "unit": "tokens/s", "n_gpus": 1 if alone else world, "steps": K,
        "warmup": W, "ms_per_step": seconds / K * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (seeded weights, kept rows filled with N(0,1), residual rows N(0,1))",
        "config": {"workload": "GLM-style MoE decoder: 8 layers, hidden 4096, 32q/8kv heads x 128, 128 experts top-8 "
                               "softmax + 1 shared expert, ffn 1536; decode batch 256 at context 2048, paged kept rows",
                   "parallelism": f"ep{world}: {per} experts and {rows} token rows per GPU; rows all-gathered, every rank runs its "
                                  "experts on all rows, outputs reduce-scattered (the reference's zero-fill scheme, no host "
                                  "reads)" + ("; step replayed from a CUDA graph" if graphed else "")
                                  + ("; ONE rank's kernels alone on one GPU, collectives replaced by local copies: a "
                                     "profiling aid, not a throughput" if alone else ""),
                   "l2": "expert weights per step exceed the 126 MB L2"},
        "e2e": {"value": batch * K / e2e_seconds, "unit": "tokens/s", "h2d_bytes_per_step": rows * cfg["hidden"] * 4,
                "d2h_bytes_per_step": rows * cfg["hidden"] * 4, "ms_per_step": e2e_seconds / K * 1e3},
        "roofline": {"kernel": "whole step (expert, dense and kept-row bytes of one rank)", "bound": "hbm",
                     "achieved": step_bytes / (seconds / K) / 1e9, "peak": peak, "unit": "GB/s",
                     "frac": step_bytes / (seconds / K) / 1e9 / peak, "peak_kind": f"of {kind}", "traffic": None,
                     "expert_kernel_traffic": NCU_TRAFFIC_RATIO["moe_grouped"] * expert_bytes,
                     "expert_kernel_traffic_source": "dram bytes / expert weight bytes of the ncu capture of moe_grouped_kernel "
                                                     "(one rank of eight), times this rank's expert weight bytes per step"},
        "ep_check": check, "clocks": sampler.summary()})


def ep_check(rank, world):
    """The expert-parallel exchange with this library's kernels on every rank, against the same block with every
    expert local: a small routed block (32 experts top-4, hidden 512, ffn 256, 16 rows a rank) with the same seeded
    weights on every rank; each rank takes its experts' slice, runs both schemes of tessera_b200.moe, and compares
    its own rows with the all-local result.  Ids must be equal bit for bit; outputs are sums in another order."""
    import torch
    import torch.distributed as dist
    from tessera_b200 import moe
    E, H, F, top, rows = 32, 512, 256, 4, 16
    g = torch.Generator().manual_seed(77)
    bf = lambda *shape, std: (torch.randn(*shape, generator=g) * std).to(torch.bfloat16).cuda()
    router, w_in, w_out = bf(E, H, std=0.05), bf(E, 2 * F, H, std=0.05), bf(E, H, F, std=0.05)
    h_all = bf(world * rows, H, std=1.0)
    h = h_all[rank * rows:(rank + 1) * rows].contiguous()
    full = moe.MoeWeights(router, w_in, w_out, first=0, experts_total=E)
    want, want_ids, _ = moe.moe_forward(h, full, top)
    if world == 1:
        return {"ranks": 1, "ids_equal": True, "max_rel_err": 0.0, "schemes": [], "note": "one rank: every expert is local"}
    per = E // world
    mine = moe.MoeWeights(router, w_in[rank * per:(rank + 1) * per].contiguous(), w_out[rank * per:(rank + 1) * per].contiguous(),
                          first=rank * per, experts_total=E)
    ep = moe.ExpertParallel()
    worst, same = 0.0, True
    for scheme in ("replicate", "dispatch"):
        y, ids, _ = ep.forward(h, mine, top, scheme=scheme)
        torch.cuda.synchronize()
        same = same and bool(torch.equal(ids, want_ids))
        worst = max(worst, float((y - want).abs().max() / want.abs().max()))
    t = torch.tensor([worst, 0.0 if same else 1.0], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return {"ranks": world, "ids_equal": bool(t[1].item() == 0.0), "max_rel_err": float(t[0].item()),
            "schemes": ["replicate", "dispatch"], "case": f"{E} experts top-{top}, hidden {H}, ffn {F}, {rows} rows a rank"}


def run_embed(args, rank, world, local_rank):
    """1024 ragged texts through the EmbeddingGemma-300M-shaped encoder, texts dealt to the ranks."""
    import torch
    import torch.distributed as dist
    from tessera_b200 import dp, synth
    from tessera_b200.encoder import EMBEDDING_300M, Encoder
    _dist_setup(local_rank, world)
    cfg = EMBEDDING_300M
    texts = 1024
    rng = np.random.default_rng(5)
    lens = rng.integers(32, 513, size=texts)
    tokens = [rng.integers(0, cfg["vocab"], size=int(n)).astype(np.int32) for n in lens]
    mine = dp.shard_by_length(lens, rank, world)
    my_lens = [int(lens[i]) for i in mine]
    packed = torch.from_numpy(np.concatenate([tokens[i] for i in mine])).pin_memory()
    cu = torch.from_numpy(np.concatenate([[0], np.cumsum(my_lens)]).astype(np.int32)).pin_memory()
    enc = Encoder(cfg, synth.decoder_weights(cfg, seed=0))
    tok_dev, cu_dev = packed.cuda(), cu.cuda()
    max_len = max(my_lens)
    K, W = args.steps, max(args.warmup, 3)
    sampler = ClockSampler(local_rank, enabled=rank == 0)
    # End to end, rank 0 ends up with all 1024 rows at their text indices: one gather of the 768-d rows over NCCL
    # (the only exchange the workload has), then one copy to the host.
    out_host = torch.empty(texts if rank == 0 else 0, cfg["hidden"]).pin_memory()
    widest = max(len(dp.shard_by_length(lens, r, world)) for r in range(world))

    def resident(i):
        enc.forward(tok_dev, cu_dev, max_len)

    def through_host(i):
        t, c = packed.to("cuda", non_blocking=True), cu.to("cuda", non_blocking=True)
        rows = dp.gather_rows(enc.forward(t, c, max_len), mine, texts, width=widest)
        if rows is not None:
            out_host.copy_(rows, non_blocking=True)
        torch.cuda.synchronize()

    sampler.start()
    seconds = _timed(resident, K, W, world)
    e2e_seconds = _timed(through_host, K, W, world)
    sampler.stop()
    del enc
    if rank != 0:
        return None
    total_tokens = int(lens.sum())
    params = cfg["layers"] * ((cfg["heads"] + 2 * cfg["kv_heads"]) * cfg["head_dim"] * cfg["hidden"] +
                              cfg["hidden"] * cfg["heads"] * cfg["head_dim"] + 3 * cfg["hidden"] * cfg["ffn"])
    flops = 2.0 * params * total_tokens + 4.0 * cfg["layers"] * cfg["heads"] * cfg["head_dim"] * float((lens.astype(np.float64) ** 2).sum())
    return ({
        "metric": "embedding_seqs_per_s", "value": texts * K / seconds, "unit": "sequences/s", "n_gpus": world, "steps": K,
        "warmup": W, "ms_per_step": seconds / K * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (seeded weights, uniform token ids, lengths uniform in [32, 512])",
        "config": {"workload": "EmbeddingGemma-300M-shaped bidirectional encoder: 24 layers, hidden 768, 3q/1kv heads x 256, "
                               "GeGLU 1152, vocab 262144, mean pooling to 768-d; batch 1024 texts", "tokens": total_tokens,
                   "parallelism": f"dp{world}: texts dealt by length, replicated weights, no collective in the pass; one gather of the "
                                  "result rows at the end (inside the end-to-end figure only)"},
        "e2e": {"value": texts * K / e2e_seconds, "unit": "sequences/s", "h2d_bytes_per_step": int(packed.numel() * 4 + cu.numel() * 4),
                "d2h_bytes_per_step": texts * cfg["hidden"] * 4, "ms_per_step": e2e_seconds / K * 1e3,
                "gathered": "rank 0 receives every rank's rows (dp.gather_rows) and copies all of them to the host"},
        "roofline": {"kernel": "whole pass (linear and attention flops)", "bound": "tensor",
                     "achieved": flops / (seconds / K) / 1e12 / world, "peak": 1418.9, "unit": "TFLOP/s",
                     "frac": flops / (seconds / K) / 1e12 / world / 1418.9, "peak_kind": "of measured (sustained)", "traffic": None},
        "clocks": sampler.summary()})


def main():
    args = parse_args()
    if args.case:
        run_case(args)
        return
    if args.workload == "sweep":
        run_sweep(args)
        return
    if args.workload == "attn":
        run_attn(args)
        return
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        if args.workload == "decode":
            out = run_ours(args, rank, world, local_rank)
            if not args.no_extras:
                # The other two sharded workloads, a few steps each, nested under the headline line.
                extra = argparse.Namespace(**vars(args))
                extra.one_rank_of = 0
                extra.steps, extra.warmup = min(args.steps, 8), 3
                moe_line = run_moe(extra, rank, world, local_rank)
                extra.steps = min(args.steps, 3)
                embed_line = run_embed(extra, rank, world, local_rank)
                if out is not None:
                    out["workloads"] = {"moe": moe_line, "embed": embed_line}
        else:
            out = (run_moe if args.workload == "moe" else run_embed)(args, rank, world, local_rank)
        if out is not None:
            print(json.dumps(out))
    finally:
        if world > 1 and dist.is_initialized():
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
