"""Stand-alone timing of the memory-bound kernels and of the attention kernels at small sequence lengths.

Each case runs one kernel through the C ABI on inputs of a few hundred MB (larger than the 126 MB L2, so
DRAM figures mean something), times it with CUDA events after warm-up and prints one JSON line with the
algorithmic bytes (or flops) per launch, achieved GB/s (TFLOP/s) and the fraction of the measured peak
(MEASURED_PEAKS.json beside the package's parent directory, else the pool's fallback figures).

  python -m bytetransformer_b200.kernel_bench                      # every case
  python -m bytetransformer_b200.kernel_bench --cases pack,gelu --iters 1 --warmup 1   # e.g. under a profiler

Cases and their reference counterparts: offsets (remove_padding.h:36-101), pack / restore
(remove_padding.h:104-121, layernorm.h:430-446), layernorm / layernorm_restore (layernorm.h:410-446),
gelu (gemm_bias_act.cu:32-66), softmax (softmax.h:191-297), embedding (layernorm.h:219-240), pooler,
mha_s64 / mha_s256 (attention_fused.cu:295-414, attention_fused_long.cu:171-312).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np
import torch

ALL_CASES = ["offsets", "pack", "restore", "layernorm", "layernorm_restore", "gelu", "softmax", "embedding", "pooler",
             "mha_s64", "mha_s256"]


def _peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": float(d["hbm_gbs"]), "tflops": float(d["bf16_tflops_sustained"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1400.0, "source": "fallback"}


def _time(fn, iters, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1e3  # microseconds


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--cases", default=",".join(ALL_CASES))
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("needs a CUDA device")
    from . import _abi
    from . import encoder as E
    from .workloads import BERT_BASE, make_weights
    dev = torch.device("cuda:0")
    lib = _abi.load()
    peaks = _peaks()
    H, F, nh = 768, 3072, 12
    g = torch.Generator().manual_seed(11)
    st = torch.cuda.current_stream().cuda_stream
    cases = [c for c in args.cases.split(",") if c]

    def report(case, kernel, us, nbytes=None, flops=None, note=""):
        line = {"case": case, "kernel": kernel, "us": round(us, 2), "note": note}
        if nbytes is not None:
            line.update({"algorithmic_bytes": int(nbytes), "gbs": round(nbytes / us / 1e3, 1),
                         "frac_of_hbm_peak": round(nbytes / us / 1e3 / peaks["hbm_gbs"], 3), "peak_gbs": peaks["hbm_gbs"]})
        if flops is not None:
            line.update({"algorithmic_flops": float(flops), "tflops": round(flops / us / 1e6, 1),
                         "frac_of_tensor_peak": round(flops / us / 1e6 / peaks["tflops"], 3), "peak_tflops": peaks["tflops"]})
        line["peak_source"] = peaks["source"]
        print(json.dumps(line), flush=True)

    # a padded batch of 512 sequences x 512 positions, valid lengths uniform in [1, 512]
    B, S = 512, 512
    lens = torch.randint(1, S + 1, (B,), generator=g)
    T = int(lens.sum())

    if "offsets" in cases:
        # only row 0 of each [S,S] mask is read; a [B,1,S] view with the same row stride would do, the full mask is 256 MB
        mask = (torch.arange(S)[None, :] < lens[:, None]).unsqueeze(1).expand(B, S, S).contiguous().half().to(dev)
        bi = torch.empty(B + 1, dtype=torch.int32, device=dev)
        wi = torch.empty(B * S, dtype=torch.int32, device=dev)
        us = _time(lambda: lib.bt_build_offsets(mask.data_ptr(), B, S, bi.data_ptr(), wi.data_ptr(), st), args.iters, args.warmup)
        report("offsets", "build_offsets_kernel", us, 2 * B * S + 4 * (B + 1) + 4 * T,
               note=f"B={B} S={S}: one CTA, latency-bound by design (runs once per forward)")
        del mask
    if any(c in cases for c in ("pack", "restore", "layernorm_restore")):
        bi = torch.tensor(np.concatenate([[0], np.cumsum(lens.numpy())]).astype(np.int32), device=dev)
    if "pack" in cases:
        x = torch.randn(B, S, H, generator=g).half().to(dev)
        xp = torch.empty(B * S, H, dtype=torch.float16, device=dev)
        us = _time(lambda: lib.bt_pack_rows(x.data_ptr(), xp.data_ptr(), bi.data_ptr(), None, B, S, H, st), args.iters, args.warmup)
        report("pack", "pack_rows_kernel", us, 4 * T * H, note=f"B={B} S={S} H={H} T={T}")
        del x, xp
    if "restore" in cases:
        xp = torch.randn(T, H, generator=g).half().to(dev)
        x = torch.empty(B, S, H, dtype=torch.float16, device=dev)
        us = _time(lambda: lib.bt_restore_rows(xp.data_ptr(), x.data_ptr(), bi.data_ptr(), B, S, H, st), args.iters, args.warmup)
        report("restore", "restore_rows_kernel", us, 2 * T * H + 2 * B * S * H, note=f"B={B} S={S} H={H} T={T} (zero fill included)")
        del x, xp
    M = 131072  # rows for the row kernels: 131072 x 768 fp32 = 403 MB in
    if "layernorm" in cases:
        x = torch.randn(M, H, generator=g).to(dev)
        gamma, beta = torch.ones(H).half().to(dev), torch.zeros(H).half().to(dev)
        out = torch.empty(M, H, dtype=torch.float16, device=dev)
        us = _time(lambda: lib.bt_add_bias_residual_layernorm(x.data_ptr(), 1, None, None, gamma.data_ptr(), beta.data_ptr(), 0,
                                                              out.data_ptr(), None, M, H, 1e-6, st), args.iters, args.warmup)
        report("layernorm", "layernorm_rows_kernel", us, 6 * M * H, note=f"rows={M} H={H}, fp32 sum in, fp16 out")
        del x, out
    if "layernorm_restore" in cases:
        x = torch.randn(T, H, generator=g).to(dev)
        gamma, beta = torch.ones(H).half().to(dev), torch.zeros(H).half().to(dev)
        out = torch.empty(B, S, H, dtype=torch.float16, device=dev)
        us = _time(lambda: lib.bt_add_bias_residual_layernorm_restore(x.data_ptr(), 1, None, None, gamma.data_ptr(), beta.data_ptr(), 0,
                                                                      out.data_ptr(), bi.data_ptr(), B, S, H, 1e-6, st),
                   args.iters, args.warmup)
        report("layernorm_restore", "layernorm_rows_kernel (scatter + zero fill)", us, 4 * T * H + 2 * B * S * H,
               note=f"B={B} S={S} H={H} T={T}")
        del x, out
    if "gelu" in cases:
        Mg = 65536
        x = torch.randn(Mg, F, generator=g).half().to(dev)
        bias = torch.randn(F, generator=g).half().to(dev)
        us = _time(lambda: lib.bt_add_bias_gelu(x.data_ptr(), bias.data_ptr(), None, Mg, F, _abi.BT_GELU_ERF, st), args.iters, args.warmup)
        report("gelu", "add_bias_gelu_kernel", us, 4 * Mg * F, note=f"rows={Mg} F={F}, in place")
        del x
    if "softmax" in cases:
        Bs, Ss = 32, 512
        logits = torch.randn(Bs, nh, Ss, Ss, generator=g).half().to(dev)
        lens_s = torch.randint(1, Ss + 1, (Bs,), generator=g)
        mask = (torch.arange(Ss)[None, :] < lens_s[:, None]).unsqueeze(1).expand(Bs, Ss, Ss).contiguous().half().to(dev)
        us = _time(lambda: lib.bt_masked_softmax(logits.data_ptr(), mask.data_ptr(), Bs, nh, Ss, 0.125, st), args.iters, args.warmup)
        report("softmax", "masked_softmax_kernel", us, 4 * nh * Bs * Ss * Ss + 2 * Bs * Ss * Ss,
               note=f"B={Bs} heads={nh} S={Ss}: logits read + written, mask read once per head group")
        del logits, mask
    if "embedding" in cases:
        vocab = 30522
        word = (torch.randn(vocab, H, generator=g) * 0.02).half().to(dev)
        pos = (torch.randn(1024, H, generator=g) * 0.02).half().to(dev)
        typ = (torch.randn(2, H, generator=g) * 0.02).half().to(dev)
        gam, bet = torch.ones(H).half().to(dev), torch.zeros(H).half().to(dev)
        Be, Se = 256, 512
        ids = torch.randint(0, vocab, (Be, Se), generator=g, dtype=torch.int32).to(dev)
        us = _time(lambda: E.embedding_layernorm(word, pos, typ, gam, bet, ids), args.iters, args.warmup)
        report("embedding", "embedding_layernorm_kernel", us, Be * Se * H * 2 * 4,
               note=f"B={Be} S={Se} H={H}: word + position + type rows in, one row out (the wrapper allocates the output)")
    if "pooler" in cases:
        Bp = 4096
        y = torch.randn(Bp, 8, H, generator=g).half().to(dev)
        W = (torch.randn(H, H, generator=g) * 0.02).half().to(dev)
        b = torch.zeros(H).half().to(dev)
        us = _time(lambda: E.pooler(y, W, b), args.iters, args.warmup)
        report("pooler", "pooler_kernel", us, flops=2.0 * Bp * H * H, note=f"B={Bp} H={H} (CUDA cores; weights 1.2 MB, L2 resident)")
    enc = None
    for case, L in (("mha_s64", 64), ("mha_s256", 256)):
        if case not in cases:
            continue
        if enc is None:
            import copy
            sh = copy.copy(BERT_BASE)
            sh.layers = 1
            enc = E.Encoder(nh, 64, make_weights(sh, seed=7, device=dev))
        nseq = 16
        lens_m = torch.randint(max(1, L // 5), L + 1, (nseq,), generator=g).tolist() if L == 64 else \
            torch.randint(1, L + 1, (nseq,), generator=g).tolist()
        cu = torch.tensor(np.concatenate([[0], np.cumsum(lens_m)]).astype(np.int32), device=dev)
        Tm = int(cu[-1])
        qkv = torch.randn(Tm, 3 * H, generator=g).half().to(dev)
        ctx = torch.empty(Tm, H, dtype=torch.float16, device=dev)
        us = _time(lambda: lib.bt_attention(enc._h, qkv.data_ptr(), ctx.data_ptr(), cu.data_ptr(), nseq, L, Tm, st),
                   args.iters, args.warmup)
        report(case, "attention (kernel chosen by shape)", us, nbytes=8 * Tm * H, flops=4.0 * H * sum(l * l for l in lens_m),
               note=f"16 sequences up to {L} tokens, T={Tm}: latency-bound (a few hundred items)")
    if enc is not None:
        st_word = enc.device_status()
        enc.close()
        if st_word != 0:
            print("device status non-zero", file=sys.stderr)
            return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
