"""Generate golden vectors by executing the reference's own test script on CPU.

The reference's `unit_test/python_scripts/bert_transformer_test.py` draws seeded
inputs and weights, runs its PyTorch encoder and (with --export_data) dumps the
tensors.  It hard-codes `.cuda()`; this script reads its source, drops those
calls, executes it unchanged otherwise (fp32, in a scratch directory) and keeps
the tensors it produced: the drawn lengths, the 12 weights per layer, the input,
the [B,S,S] mask and every layer's output.  The reference tree is only needed
to (re)generate the fixtures, which are committed next to this script.

Usage:  python tests/golden/make_golden.py <reference_root>
"""
import os
import runpy
import sys
import tempfile

import numpy as np

CASES = {
    # name: (batch, seqlen, head_num, head_size, n_layers, avg_seqlen)
    "ref_b3_s12_h1_l1": (3, 12, 1, 64, 1, 0),
    "ref_b4_s24_h2_l2_avg14": (4, 24, 2, 64, 2, 14),
    "ref_b5_s16_h1_l1_avg5": (5, 16, 1, 64, 1, 5),   # low=0: zero-length sequences possible
}

NAMES = ["qkv_kernel", "qkv_bias", "attr_output_kernel", "attr_output_bias",
         "attr_output_layernorm_gamma", "attr_output_layernorm_beta", "inter_kernel",
         "inter_bias", "output_kernel", "output_bias", "output_layernorm_gamma",
         "output_layernorm_beta"]


def run_case(script, args):
    b, s, hn, hs, nl, avg = args
    src = open(script).read().replace(".cuda()", "")
    with tempfile.TemporaryDirectory() as tmp:
        patched = os.path.join(tmp, "ref_script_cpu.py")
        with open(patched, "w") as f:
            f.write(src)
        argv = [patched, str(b), str(s), str(hn), str(hs), "--n_layers", str(nl),
                "--avg_seqlen", str(avg), "--dtype", "fp32", "--export_data",
                "--export_data_path", tmp]
        old_argv, old_cwd = sys.argv, os.getcwd()
        sys.argv = argv
        os.chdir(tmp)
        try:
            g = runpy.run_path(patched, run_name="__main__")
        finally:
            sys.argv = old_argv
            os.chdir(old_cwd)
    out = {"input_lens": g["input_lens"].numpy().astype(np.int64),
           "from_tensor": g["from_tensor"].numpy(),
           "attr_mask": g["attr_mask"].numpy(),
           "meta": np.array([b, s, hn, hs, nl, avg], dtype=np.int64)}
    for l in range(nl):
        for n in NAMES:
            out[f"l{l}_{n}"] = g[n][l].numpy()
        out[f"l{l}_out"] = g["transformer_output"][l].numpy()
    return out


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py <path to a checkout of the reference project>")
    ref = sys.argv[1]
    script = os.path.join(ref, "unit_test/python_scripts/bert_transformer_test.py")
    here = os.path.dirname(os.path.abspath(__file__))
    for name, args in CASES.items():
        data = run_case(script, args)
        path = os.path.join(here, name + ".npz")
        np.savez_compressed(path, **data)
        print(name, "lens", data["input_lens"].tolist(), os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
