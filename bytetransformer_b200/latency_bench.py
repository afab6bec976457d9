"""Latency sweep over the reference's published configurations.

Mirrors the reference's own benchmark loop (benchmark/bert_bench.sh:21-56): BERT-base,
12 layers, 12 heads x 64, fp16, average valid length 0.6 x max_seq, one padded
`[B,S,H]` batch with a `[B,S,S]` mask through the drop-in API — here the one-call stack
`bt_stack_forward_padded` (and, with --per-layer-op, the reference's per-layer operator
loop).  Prints one JSON line per (batch, max_seq) with milliseconds per 12-layer forward,
valid tokens/s, algorithmic TFLOP/s and the number the reference publishes for the same
point on an A100 (README.md:30-71) where there is one.

  python -m bytetransformer_b200.latency_bench --batch 1 --seqs 64,128,...,1024
  python -m bytetransformer_b200.latency_bench --batch 16 --seqs 512

Timing: CUDA events around each forward, L2 flushed (256 MB memset) before every timed
iteration, median of --iters after --warmup.
"""
from __future__ import annotations

import argparse
import json
import statistics
import sys

import torch

# ms per 12-layer forward published by the reference (A100, README.md:30-71)
README_MS = {
    1: {64: 0.90, 128: 0.97, 192: 1.36, 256: 1.43, 320: 1.69, 384: 1.72, 448: 1.86, 512: 2.00, 576: 2.19,
        640: 2.23, 704: 2.47, 768: 2.51, 832: 2.80, 896: 2.86, 960: 3.12, 1024: 3.16},
    16: {64: 2.09, 128: 3.18, 192: 5.08, 256: 6.85, 320: 7.49, 384: 8.44, 448: 8.89, 512: 9.22, 576: 10.15,
         640: 12.04, 704: 13.55, 768: 16.3, 832: 16.92, 896: 20.67, 960: 23.27, 1024: 24.70},
}


def lengths(batch: int, seq: int, seed: int):
    """batch 1: exactly round(0.6*S); otherwise uniform in [2*avg-S, S] with avg = 0.6*S,
    the reference's recipe (unit_test/python_scripts/bert_transformer_test.py:93-94)."""
    avg = int(round(0.6 * seq))
    if batch == 1:
        return torch.tensor([avg])
    g = torch.Generator().manual_seed(seed)
    return torch.randint(max(1, 2 * avg - seq), seq + 1, (batch,), generator=g)


def measure_config(name, shape, lens, max_seq, layers=None, iters=20, warmup=5, device=None, peaks=None, enc=None):
    """One BASELINE configuration through the one-call padded stack (`bt_stack_forward_padded`): median
    milliseconds per forward (CUDA events, L2 flushed before every timed iteration), valid tokens/s,
    algorithmic TFLOP/s and two roofline fractions - of the dense tensor peak, and of HBM bandwidth for the
    bytes every forward has to stream at least once (the layers' weights), which is what bounds the
    few-token configurations.  `shape` is a workloads.ModelShape, `lens` the valid lengths."""
    import numpy as np
    from .encoder import Encoder
    from .workloads import attention_flops_per_layer, gemm_flops_per_layer, make_weights
    dev = device or torch.device("cuda:0")
    layers = layers or shape.layers
    own = enc is None
    if own:
        import copy
        sh = copy.copy(shape)
        sh.layers = layers
        enc = Encoder(shape.head_num, 64, make_weights(sh, seed=7, device=dev))
    lens_t = torch.as_tensor(np.asarray(lens), dtype=torch.long)
    B, S, H = int(lens_t.numel()), int(max_seq), shape.hidden
    T = int(lens_t.sum())
    g = torch.Generator().manual_seed(S + B)
    x = torch.randn(B, S, H, generator=g).half().to(dev)
    mask = (torch.arange(S)[None, :] < lens_t[:, None]).unsqueeze(1).expand(B, S, S).contiguous().half().to(dev)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.int8, device=dev)
    times = []
    for i in range(warmup + iters):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        enc.forward(x, mask, n_layers=layers)
        e1.record()
        torch.cuda.synchronize()
        if i >= warmup:
            times.append(e0.elapsed_time(e1))
    status = enc.device_status()
    if own:
        enc.close()
    ms = statistics.median(times)
    fl = layers * (gemm_flops_per_layer(T, H) + attention_flops_per_layer(lens_t.numpy(), H))
    weight_bytes = layers * 24.0 * H * H
    out = {"config": name, "model": shape.name, "layers": layers, "batch": B, "max_seq": S, "valid_tokens": T,
           "ms": ms, "min_ms": min(times), "tokens_per_s": T / ms * 1e3, "algorithmic_tflops": fl / ms / 1e9,
           "weight_gbs": weight_bytes / ms / 1e6, "device_status": status}
    if peaks:
        out["frac_of_tensor_peak"] = out["algorithmic_tflops"] / peaks["tflops"]
        out["frac_of_hbm_peak_weights_only"] = out["weight_gbs"] / peaks["hbm_gbs"]
    return out


def baseline_configs(peaks=None, device=None, iters=20, warmup=5):
    """The BASELINE configurations that fit one GPU besides the whole-box one, each through the padded
    drop-in entry point: c1 (one layer, batch 16, max_seq 64), c2 (12 layers, batch 1, max_seq 64 / 512 /
    1024 at 0.6 x valid), c3 (12 layers, batch 16, max_seq 512) and c4 (BERT-large, 24 layers, batch 64,
    max_seq 384)."""
    from .workloads import BERT_BASE, BERT_LARGE, lengths_for
    out = {}
    out["c1_1L_b16_s64"] = measure_config("c1", BERT_BASE, lengths_for("single_layer_b16_s64"), 64, layers=1,
                                          iters=iters, warmup=warmup, device=device, peaks=peaks)
    for S in (64, 512, 1024):
        out[f"c2_12L_b1_s{S}"] = measure_config("c2", BERT_BASE, lengths_for(f"b1_sweep_s{S}"), S, iters=iters,
                                                 warmup=warmup, device=device, peaks=peaks)
    out["c3_12L_b16_s512"] = measure_config("c3", BERT_BASE, lengths_for("b16_s512"), 512, iters=iters, warmup=warmup,
                                            device=device, peaks=peaks)
    out["c4_large_24L_b64_s384"] = measure_config("c4", BERT_LARGE, lengths_for("large_b64_s384"), 384,
                                                  iters=max(5, iters // 2), warmup=3, device=device, peaks=peaks)
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--seqs", default="512")
    ap.add_argument("--iters", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--per-layer-op", action="store_true", help="call the one-layer operator 12 times, as the reference's loop")
    ap.add_argument("--graph", action="store_true", help="replay the forward from a CUDA graph")
    ap.add_argument("--no-pdl", action="store_true", help="launch without programmatic dependent launch (A/B)")
    ap.add_argument("--fused-ln", type=int, default=-1,
                    help="A/B aid: LayerNorm inside the GEMM kernels: 0 never, 1 default policy, 2 always, 3 FFN2 only")
    ap.add_argument("--mha-variant", type=int, default=-1,
                    help="A/B aid: 0 default policy, 1 one CTA per (query tile, head, sequence), 3 persistent CTAs")
    ap.add_argument("--split-k", type=int, default=0,
                    help="A/B aid: K ranges of the GEMMs that feed a LayerNorm: 0 policy, -1 never, n > 0 forced")
    ap.add_argument("--late-weights", action="store_true",
                    help="A/B aid: request the first weight blocks of a GEMM only after the wait for the kernel before")
    ap.add_argument("--general", choices=["padded", "causal"], default=None,
                    help="time the general-mask entry point instead (nothing packed, the whole [B,S,S] mask applied): "
                         "with the same right-padded mask, or with a causal mask over the valid keys")
    ap.add_argument("--front-back", action="store_true",
                    help="also time the embedding + LayerNorm front end (30522-word table) and the pooler for each shape")
    ap.add_argument("--baseline-configs", action="store_true",
                    help="instead of a sweep: the BASELINE configurations c1-c4 (BERT-base and BERT-large), one JSON line each")
    ap.add_argument("--breakdown", action="store_true",
                    help="add per-kernel-kind microseconds per forward (CUDA events around every launch, L2 warm)")
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("needs a CUDA device")
    if args.baseline_configs:
        import os
        peaks = None
        p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
        if os.path.exists(p):
            d = json.load(open(p))
            peaks = {"tflops": float(d["bf16_tflops_sustained"]), "hbm_gbs": float(d["hbm_gbs"])}
        for k, v in baseline_configs(peaks, iters=args.iters, warmup=args.warmup).items():
            print(json.dumps({"name": k, **v}), flush=True)
        return 0
    from .encoder import Encoder
    from .workloads import BERT_BASE, attention_flops_per_layer, gemm_flops_per_layer, make_weights
    dev = torch.device("cuda:0")
    enc = Encoder(BERT_BASE.head_num, 64, make_weights(BERT_BASE, seed=7, device=dev))
    if args.fused_ln >= 0:
        from . import _abi
        _abi.load().bt_debug_set_fused_layernorm(enc._h, args.fused_ln)
    if args.mha_variant >= 0:
        from . import _abi
        _abi.load().bt_debug_set_mha_tiles(args.mha_variant)
    if args.no_pdl:
        from . import _abi
        _abi.load().bt_debug_set(6, 0)
    if args.late_weights:
        from . import _abi
        _abi.load().bt_debug_set(8, 0)
    if args.split_k != 0:
        from . import _abi
        _abi.load().bt_debug_set(7, args.split_k)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.int8, device=dev)
    H = BERT_BASE.hidden
    for S in [int(s) for s in args.seqs.split(",")]:
        B = args.batch
        lens = lengths(B, S, seed=S)
        T = int(lens.sum())
        g = torch.Generator().manual_seed(S + 1)
        x = torch.randn(B, S, H, generator=g).half().to(dev)
        mask = (torch.arange(S)[None, :] < lens[:, None]).unsqueeze(1).expand(B, S, S).contiguous().half().to(dev)

        if args.general == "causal":
            mask = (mask.bool() & torch.tril(torch.ones(S, S, dtype=torch.bool, device=dev))[None]).half().contiguous()

        def fwd():
            if args.general is not None:
                return enc.forward_general(x, mask)
            if args.per_layer_op:
                h = x
                for l in range(BERT_BASE.layers):
                    h = enc.forward_layer(l, h, mask)
                return h
            return enc.forward(x, mask)

        graph = None
        if args.graph:
            fwd()
            torch.cuda.synchronize()
            s = torch.cuda.Stream()
            with torch.cuda.stream(s):
                fwd()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=s):
                    out_static = fwd()
            torch.cuda.synchronize()
        times = []
        for i in range(args.warmup + args.iters):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            if graph is not None:
                graph.replay()
            else:
                fwd()
            e1.record()
            torch.cuda.synchronize()
            if i >= args.warmup:
                times.append(e0.elapsed_time(e1))
        ms = statistics.median(times)
        fl = BERT_BASE.layers * (gemm_flops_per_layer(T, H) + attention_flops_per_layer(lens.numpy(), H))
        ref = README_MS.get(B, {}).get(S)
        breakdown = None
        if args.breakdown and graph is None:
            reps = 10
            enc.profile_enable(True)
            for _ in range(reps):
                fwd()
            torch.cuda.synchronize()
            breakdown = {k: {"us_per_forward": round(v[0] * 1e3 / reps, 2), "launches_per_forward": v[1] // reps}
                         for k, v in enc.profile_read().items() if v[1]}
            enc.profile_enable(False)
        extra = {}
        if args.front_back:
            from .encoder import embedding_layernorm, pooler
            gg = torch.Generator().manual_seed(3)
            vocab = 30522
            word = (torch.randn(vocab, H, generator=gg) * 0.02).half().to(dev)
            pos = (torch.randn(1024, H, generator=gg) * 0.02).half().to(dev)
            typ = (torch.randn(2, H, generator=gg) * 0.02).half().to(dev)
            gam, bet = torch.ones(H).half().to(dev), torch.zeros(H).half().to(dev)
            ids = torch.randint(0, vocab, (B, S), generator=gg, dtype=torch.int32).to(dev)
            pw, pb = (torch.randn(H, H, generator=gg) * 0.02).half().to(dev), torch.zeros(H).half().to(dev)

            def timed(fn):
                ts = []
                for i in range(args.warmup + args.iters):
                    flush.zero_()
                    a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a0.record()
                    fn()
                    a1.record()
                    torch.cuda.synchronize()
                    if i >= args.warmup:
                        ts.append(a0.elapsed_time(a1))
                return statistics.median(ts)

            t_emb = timed(lambda: embedding_layernorm(word, pos, typ, gam, bet, ids))
            t_pool = timed(lambda: pooler(x, pw, pb))
            emb_bytes = B * S * H * 2 * 4  # word row + position row + type row in, one row out
            extra = {"embedding_layernorm_us": round(t_emb * 1e3, 2),
                     "embedding_layernorm_gbs": round(emb_bytes / t_emb / 1e6, 1),
                     "pooler_us": round(t_pool * 1e3, 2)}
        api = ("general-mask stack (" + args.general + " mask)") if args.general else None
        print(json.dumps({
            "metric": "ms_per_12_layer_forward", "batch": B, "max_seq": S, "valid_tokens": T, "value": ms,
            "unit": "ms", "min_ms": min(times), "tokens_per_s": T / ms * 1e3, "algorithmic_tflops": fl / ms / 1e9,
            "higher_is_better": False, "reference_a100_ms": ref, "speedup_vs_reference_a100": (ref / ms) if ref else None,
            "api": (api or ("per-layer operator x12" if args.per_layer_op else "one-call padded stack")) + (", CUDA graph" if graph else "") + (", no PDL" if args.no_pdl else ""),
            "l2": "flushed before every timed iteration", "data": "synthetic", "dtype": "f16",
            **extra, **({"breakdown": breakdown} if breakdown else {})}), flush=True)
    if enc.device_status() != 0:
        print("device status non-zero", file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
