"""Text test-vector files in the reference's own format.

The reference's benchmark script can export one single-layer case as fifteen text files, one
float per line in `%f` notation (unit_test/python_scripts/bert_transformer_test.py:160-180), and
its C++ test loads the same files and compares against `transformer_out.out`
(unit_test/bert_transformer_test.cc:88-188, unit_test/helper.h:39-85).  This module writes and
reads that directory layout, so that vectors made for the reference's C++ flow can be replayed
against this library (tests/cpp/text_case_driver.cc) and the other way round.

Shapes (H = head_num * size_per_head), all flattened row-major:
  qkv_kernel [H,3H]  qkv_bias [3H]  attr_output_kernel [H,H]  attr_output_bias [H]
  attr_output_layernorm_gamma/beta [H]  inter_kernel [H,4H]  inter_bias [4H]
  output_kernel [4H,H]  output_bias [H]  output_layernorm_gamma/beta [H]
  from_tensor [B,S,H]  atten_mask [B,S,S]  transformer_out [B,S,H] (padding rows zero)
"""
from __future__ import annotations

import os
from typing import Dict, Sequence

import numpy as np

WEIGHT_FILES = (
    "qkv_kernel.in", "qkv_bias.in",
    "attr_output_kernel.in", "attr_output_bias.in", "attr_output_layernorm_gamma.in", "attr_output_layernorm_beta.in",
    "inter_kernel.in", "inter_bias.in",
    "output_kernel.in", "output_bias.in", "output_layernorm_gamma.in", "output_layernorm_beta.in",
)
INPUT_FILE = "from_tensor.in"
MASK_FILE = "atten_mask.in"
OUTPUT_FILE = "transformer_out.out"


def weight_shapes(hidden: int):
    H, F = hidden, 4 * hidden
    return ((H, 3 * H), (3 * H,), (H, H), (H,), (H,), (H,), (H, F), (F,), (F, H), (H,), (H,), (H,))


def _save(path: str, a) -> None:
    a = np.asarray(a, dtype=np.float32).reshape(-1)
    # '%f' like the reference's np.savetxt call: six digits after the point
    with open(path, "w") as f:
        f.write("\n".join("%f" % v for v in a))
        f.write("\n")


def _load(path: str, shape) -> np.ndarray:
    a = np.loadtxt(path, dtype=np.float32).reshape(-1)
    n = int(np.prod(shape))
    if a.size != n:
        raise ValueError(f"{path}: {a.size} values, expected {n}")
    return a.reshape(shape)


def write_case(directory: str, weights: Sequence, from_tensor, atten_mask, transformer_out=None) -> None:
    """Write one single-layer case.  `weights` are the 12 tensors in the reference's order."""
    if len(weights) != len(WEIGHT_FILES):
        raise ValueError("expected 12 weight tensors")
    os.makedirs(directory, exist_ok=True)
    for name, w in zip(WEIGHT_FILES, weights):
        _save(os.path.join(directory, name), w)
    _save(os.path.join(directory, INPUT_FILE), from_tensor)
    _save(os.path.join(directory, MASK_FILE), atten_mask)
    if transformer_out is not None:
        _save(os.path.join(directory, OUTPUT_FILE), transformer_out)


def read_case(directory: str, batch_size: int, seq_len: int, head_num: int, size_per_head: int = 64) -> Dict[str, object]:
    """Read a case directory back: {'weights': [12 arrays], 'from_tensor', 'atten_mask', 'transformer_out' or None}."""
    H = head_num * size_per_head
    weights = [_load(os.path.join(directory, n), s) for n, s in zip(WEIGHT_FILES, weight_shapes(H))]
    out_path = os.path.join(directory, OUTPUT_FILE)
    return {
        "weights": weights,
        "from_tensor": _load(os.path.join(directory, INPUT_FILE), (batch_size, seq_len, H)),
        "atten_mask": _load(os.path.join(directory, MASK_FILE), (batch_size, seq_len, seq_len)),
        "transformer_out": _load(out_path, (batch_size, seq_len, H)) if os.path.exists(out_path) else None,
    }
