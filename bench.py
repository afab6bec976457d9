#!/usr/bin/env python
"""Benchmark of the padding-free BERT encoder path.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (N = 1..8): the whole-box configuration — BERT-base, 12 layers, 1024
sequences of max_seq 1024 with seeded lengths uniform in [16,1024] (about 556k
valid tokens), split over the N GPUs by packed-token cost (LPT), every GPU
holding a full weight replica; no collective on the data path.  One "step" is
one pass over all 1024 sequences.  Total work is fixed as N grows ("strong").

Printed JSON line (rank 0): `value` = valid tokens/s with inputs resident in
HBM; `e2e` = the same through the public packed-forward call with pinned HOST
buffers (H2D + compute + D2H inside the timed region); `roofline` = the GEMM
kernel's achieved algorithmic TFLOP/s from CUDA events around every GEMM launch
of the timed region against the measured dense bf16/fp16 peak; `cpu_baseline`
= the CPU oracle (the reference's fp32 PyTorch encoder restated) on a bounded
sample.  `--impl reference` times that CPU encoder alone.
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

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "bert_base_12L_packed_tokens_per_sec"
UNIT = "tokens/s"
WORKLOAD = "whole_box_1024x1024"
# dram__bytes_read.sum + dram__bytes_write.sum per GEMM launch and packed token, mean of the four GEMMs of a layer,
# from the two ncu captures summarised in profiles/gemm_kernels_microbatch18k.txt (18,645 tokens per launch: 95.2 MB)
# and profiles/gemm_kernels_microbatch76k.txt (70,734 tokens: 456.4 MB).  The algorithmic bytes of the same launches
# are 7,100 per token; DRAM sees less because a kernel's output is partly still in the 126 MB L2 when the next
# kernel reads it, the more so the smaller the launch.  Between the two launch sizes the figure is interpolated.
GEMM_DRAM_BYTES_PER_TOKEN = ((18645, 95.2e6 / 18645), (70734, 456.4e6 / 70734))


def gemm_dram_bytes_per_launch(tokens_per_launch: float) -> float:
    (t0, b0), (t1, b1) = GEMM_DRAM_BYTES_PER_TOKEN
    w = min(1.0, max(0.0, (tokens_per_launch - t0) / (t1 - t0)))
    return (b0 + w * (b1 - b0)) * tokens_per_launch


WORKLOAD_DESC = "bert-base 12L, 1024 seqs, max_seq 1024, lens U[16,1024] seed 1234, split by LPT over the GPUs"


# ----------------------------------------------------------------------------- peaks
def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"tflops": float(d.get("bf16_tflops_sustained", d.get("bf16_tflops"))),
                "tflops_burst": float(d.get("bf16_tflops")), "hbm_gbs": float(d["hbm_gbs"]), "source": "measured"}
    return {"tflops": 1400.0, "tflops_burst": 1590.0, "hbm_gbs": 6650.0, "source": "fallback"}


# ----------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while a region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.rows = []
        self.proc = None
        try:
            uuid = str(torch.cuda.get_device_properties(device_index).uuid)
            sel = uuid if uuid.startswith("GPU-") else "GPU-" + uuid
        except Exception:
            sel = str(device_index)
        self.cmd = ["nvidia-smi", "-i", sel, "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits", "-lms", "50"]
        self.skip = 0

    def start(self):
        try:
            self.proc = subprocess.Popen(self.cmd, stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
            # nvidia-smi needs a moment (longer on a box with eight GPUs) before its first line: wait for it, so that
            # a timed region of a few hundred milliseconds is sampled too; what came before the region is left out
            t0 = time.time()
            while not self.rows and time.time() - t0 < 10.0 and self.proc.poll() is None:
                time.sleep(0.01)
            self.skip = len(self.rows)
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.05)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows[self.skip:]:
            f = [x.strip() for x in r.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ----------------------------------------------------------------------------- CPU oracle timing
CPU_SAMPLE_SEQS = 32   # the CPU arm times the first 32 sequences of the workload (18,645 tokens), always the same ones


def host_threads() -> int:
    """The host threads this process may use (its CPU affinity), whatever OMP_NUM_THREADS says: torchrun
    exports OMP_NUM_THREADS=1 to its children, which would otherwise shrink the CPU arm to one thread."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def cpu_oracle_sample(lengths, reps=1):
    """Times the CPU oracle (the reference's fp32 PyTorch encoder restated, 12 layers) on the first
    CPU_SAMPLE_SEQS sequences of the workload with every host thread the process may use.
    Returns (tokens/s, sample text, threads, tokens, seconds)."""
    from oracle.bert_oracle import encoder_stack_packed
    from bytetransformer_b200.workloads import BERT_BASE, make_weights
    cores = host_threads()
    torch.set_num_threads(cores)
    layers = [[t.float() for t in w] for w in make_weights(BERT_BASE, seed=7)]
    g = torch.Generator().manual_seed(3)
    ids = list(range(min(CPU_SAMPLE_SEQS, len(lengths))))
    tok = int(sum(int(lengths[i]) for i in ids))
    cu = np.concatenate([[0], np.cumsum([int(lengths[i]) for i in ids])]).tolist()
    x = torch.randn(tok, BERT_BASE.hidden, generator=g)
    best = None
    with torch.no_grad():
        for _ in range(reps):
            t0 = time.perf_counter()
            encoder_stack_packed(x, cu, layers, BERT_BASE.head_num, 64, ln_eps=1e-6)
            dt = time.perf_counter() - t0
            best = dt if best is None else min(best, dt)
    sample = f"first {len(ids)} sequences ({tok} tokens) of the workload, 12 layers, fp32, {cores} threads"
    return tok / best, sample, cores, tok, best


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    from bytetransformer_b200.workloads import lengths_for
    lengths = lengths_for(WORKLOAD)
    # every step is the same bounded sample (a few seconds of CPU work)
    per_step = []
    sample, cores = "", host_threads()
    for i in range(args.warmup + args.steps):
        _, sample, cores, tok, dt = cpu_oracle_sample(lengths)
        if i >= args.warmup:
            per_step.append((tok, dt))
    tot_tok = sum(t for t, _ in per_step)
    tot_dt = sum(d for _, d in per_step)
    value = tot_tok / tot_dt
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1000.0 * tot_dt / max(1, len(per_step)),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "desc": WORKLOAD_DESC, "sample_per_step": sample},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


# ----------------------------------------------------------------------------- our arm
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-kernel-events", action="store_true", help="do not bracket kernels with events in the timed region")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-configs", action="store_true", help="skip the other BASELINE configurations (N = 1 extra key)")
    ap.add_argument("--token-budget", type=int, default=0)
    ap.add_argument("--e2e-token-budget", type=int, default=0, help="A/B aid: micro-batch budget of the host path")
    ap.add_argument("--fused-ln", type=int, default=-1,
                    help="A/B aid: LayerNorm inside the GEMM kernels: 0 never, 1 default policy, 2 always, 3 FFN2 only")
    ap.add_argument("--max-seqs", type=int, default=0,
                    help="profiling aid: keep only the first N sequences of the workload (small ncu captures)")
    ap.add_argument("--layers", type=int, default=0, help="profiling aid: run only the first L layers")
    ap.add_argument("--mixed-batches", action="store_true",
                    help="A/B aid: equal micro-batches with the same mix of lengths in each, instead of filling "
                         "one micro-batch after the other to the token budget in length order")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference_arm(args)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the encoder path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    from bytetransformer_b200.ranks import Ranks
    # barrier / max / sum around the work only; the data path has no collective, so the host-side gloo
    # backend is enough (and keeps NCCL's banner off stdout, which must carry one JSON line)
    ranks = Ranks(backend="gloo", device=dev)
    n_gpus = world

    from bytetransformer_b200.encoder import Encoder
    from bytetransformer_b200.runner import PackedRunner
    from bytetransformer_b200.sharding import lpt_shards
    from bytetransformer_b200.workloads import (BERT_BASE, attention_flops_per_layer, gemm_flops_per_layer,
                                                lengths_for, make_weights)

    lengths = lengths_for(WORKLOAD)
    if args.max_seqs > 0:
        lengths = lengths[:args.max_seqs]
    if args.layers > 0:
        BERT_BASE.layers = args.layers
    total_tokens = int(lengths.sum())
    shards = lpt_shards(lengths, n_gpus, BERT_BASE.hidden)
    mine = shards[rank]
    enc = Encoder(BERT_BASE.head_num, 64, make_weights(BERT_BASE, seed=7, device=dev), ln_eps=1e-6, gelu="erf")
    if args.fused_ln >= 0:
        from bytetransformer_b200 import _abi
        _abi.load().bt_debug_set_fused_layernorm(enc._h, args.fused_ln)
    # Inputs resident in device memory: nothing to overlap, so the largest launches (up to 75,776 tokens).  From
    # host memory (further down): at least four micro-batches per rank, so that the copies of one hide behind
    # the compute of its neighbours.  On one and two GPUs both give the same cut and one runner serves both.
    runner = PackedRunner(enc, lengths, mine, token_budget=args.token_budget, mix=args.mixed_batches, min_batches=1)
    budget = runner.token_budget
    xs, outs = runner.make_device_inputs(seed=rank)

    barrier = ranks.barrier
    max_over_ranks = ranks.max

    # ---- device-resident throughput -------------------------------------------------
    for _ in range(max(args.warmup, 3)):
        runner.run_device(xs, outs)
    barrier()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    barrier()
    runner.run_device(xs, outs)  # the GPUs idled while the sampler came up: one more untimed step
    enc.profile_enable(True)     # resets the launch counters ...
    enc.profile_enable(False)    # ... without bracketing kernels: the headline region runs undisturbed
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        runner.run_device(xs, outs)
    e1.record()
    barrier()
    ms_total = max_over_ranks(e0.elapsed_time(e1))
    launch_counts = enc.profile_read()
    # The same K steps once more with CUDA events around every kernel launch (on the
    # launching stream): per-kernel durations for the roofline.  The brackets cost a
    # few percent of step time, which is why the headline value is not taken here.
    ms_events_region = None
    prof = launch_counts
    if not args.no_kernel_events:
        enc.profile_enable(True)
        barrier()
        e0.record()
        for _ in range(args.steps):
            runner.run_device(xs, outs)
        e1.record()
        barrier()
        ms_events_region = e0.elapsed_time(e1) / args.steps
        prof = enc.profile_read()
        enc.profile_enable(False)
    clocks = sampler.stop() if sampler else None
    st = enc.device_status()
    if st != 0:
        raise SystemExit("a kernel reported a device-side error status (0x%x)" % st)
    ms_per_step = ms_total / args.steps
    value = total_tokens / (ms_per_step / 1000.0)

    # ---- end to end from pinned host memory ------------------------------------------
    e2e = None
    if not args.no_e2e:
        runner_e2e = PackedRunner(enc, lengths, mine, token_budget=args.e2e_token_budget or args.token_budget,
                                  mix=args.mixed_batches, min_batches=4)
        if runner_e2e.token_budget == runner.token_budget:
            runner_e2e = runner
        xh, oh = runner_e2e.make_host_inputs(seed=100 + rank)
        h2d = d2h = 0
        for _ in range(max(args.warmup, 3)):
            h2d, d2h = runner_e2e.run_host(xh, oh)
        barrier()
        e0.record()
        for _ in range(args.steps):
            h2d, d2h = runner_e2e.run_host(xh, oh)
        e1.record()
        barrier()
        ms_e2e = max_over_ranks(e0.elapsed_time(e1)) / args.steps
        h2d, d2h = (int(v) for v in ranks.sum(h2d, d2h))
        e2e = {"value": total_tokens / (ms_e2e / 1000.0), "unit": UNIT, "ms_per_step": ms_e2e,
               "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
               "micro_batch_token_budget": runner_e2e.token_budget, "micro_batches_rank0": len(runner_e2e.batches),
               "micro_batch_tokens_rank0": [mb.tokens for mb in runner_e2e.batches]}
        if runner_e2e is not runner:
            runner_e2e.workspace = None
        del xh, oh

    # ---- roofline of the dominant kernel (the GEMM), rank 0's launches -----------------
    peaks = measured_peaks()
    my_lengths = lengths[mine]
    my_tokens = int(my_lengths.sum())
    gemm_kinds = ("gemm_qkv", "gemm_attn_out", "gemm_ffn1", "gemm_ffn2")
    gemm_ms = sum(prof[k][0] for k in gemm_kinds)
    gemm_launches = sum(prof[k][1] for k in gemm_kinds)
    gemm_flops = args.steps * BERT_BASE.layers * gemm_flops_per_layer(my_tokens, BERT_BASE.hidden)
    roofline = None
    kernels = {}
    if not args.no_kernel_events and gemm_ms > 0:
        achieved = gemm_flops / (gemm_ms / 1000.0) / 1e12
        # per launch, like `achieved`: this rank's tokens per micro-batch times the captured per-token figure
        traffic = gemm_dram_bytes_per_launch(my_tokens / max(1, len(runner.batches))) if not args.layers else None
        roofline = {"bound": "tensor", "kernel": "the four GEMMs of a layer: gemm_f16_pair_kernel (QKV, FFN1 + GELU), gemm_f16_ln_kernel (attention output and FFN2, with LayerNorm)", "achieved": achieved,
                    "peak": peaks["tflops"], "unit": "TFLOP/s", "frac": achieved / peaks["tflops"],
                    "peak_source": peaks["source"] + " sustained bf16 dense", "traffic": traffic,
                    "launches": int(gemm_launches), "avg_launch_ms": gemm_ms / max(1, gemm_launches)}
        shape_flops = {"gemm_qkv": 6.0, "gemm_attn_out": 2.0, "gemm_ffn1": 8.0, "gemm_ffn2": 8.0}
        for k in gemm_kinds:
            fl = args.steps * BERT_BASE.layers * shape_flops[k] * my_tokens * BERT_BASE.hidden ** 2
            kernels[k] = {"ms": prof[k][0], "launches": int(prof[k][1]),
                          "tflops": fl / (prof[k][0] / 1000.0) / 1e12 if prof[k][0] > 0 else None}
        afl = args.steps * BERT_BASE.layers * attention_flops_per_layer(my_lengths, BERT_BASE.hidden)
        kernels["mha"] = {"ms": prof["mha"][0], "launches": int(prof["mha"][1]),
                          "tflops": afl / (prof["mha"][0] / 1000.0) / 1e12 if prof["mha"][0] > 0 else None}
        ln_bytes = args.steps * BERT_BASE.layers * 2 * my_tokens * BERT_BASE.hidden * 6.0  # fp32 in, fp16 out
        kernels["layernorm"] = {"ms": prof["layernorm"][0], "launches": int(prof["layernorm"][1]),
                                "gbs": ln_bytes / (prof["layernorm"][0] / 1000.0) / 1e9 if prof["layernorm"][0] > 0 else None,
                                "hbm_peak_gbs": peaks["hbm_gbs"]}
        if prof["layernorm"][1] == 0:
            kernels["layernorm"]["note"] = "LayerNorm ran inside the gemm_attn_out / gemm_ffn2 kernels (no separate launch)"
    launches = int(sum(v[1] for v in launch_counts.values()))
    launches = int(ranks.sum(launches)[0])

    # ---- CPU baseline (rank 0, N = 1 only) ---------------------------------------------
    cpu = None
    if rank == 0 and n_gpus == 1 and not args.no_cpu_baseline:
        tps, sample, cores, _, _ = cpu_oracle_sample(lengths_for(WORKLOAD), reps=2)
        cpu = {"value": tps, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample}

    # ---- the other BASELINE configurations (rank 0, N = 1 only): extra key, the headline is untouched ----
    configs = None
    if rank == 0 and n_gpus == 1 and not args.no_configs and not (args.max_seqs or args.layers):
        from bytetransformer_b200.latency_bench import baseline_configs
        enc.close()
        del xs, outs
        runner.workspace = None
        torch.cuda.empty_cache()
        configs = baseline_configs({"tflops": peaks["tflops"], "hbm_gbs": peaks["hbm_gbs"]}, device=dev, iters=20, warmup=5)

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": n_gpus, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": WORKLOAD if not (args.max_seqs or args.layers) else
                       f"{WORKLOAD} reduced: max_seqs={args.max_seqs} layers={args.layers} (profiling aid, not a bench line)",
                       "desc": WORKLOAD_DESC, "total_tokens": total_tokens,
                       "micro_batch_token_budget": budget, "micro_batches_rank0": len(runner.batches),
                       "l2": "inputs larger than L2 (>= 100 MB of activations per GPU per step)",
                       "roofline_measurement": "the K timed steps repeated right after, with CUDA events around every "
                                               "kernel launch on the launching stream",
                       "ms_per_step_with_kernel_events": ms_events_region},
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "roofline": roofline, "cpu_baseline": cpu,
            "kernels": kernels,
            "configs": configs,
        }
        print(json.dumps(line), flush=True)
    ranks.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
