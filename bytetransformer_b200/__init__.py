"""bytetransformer_b200 — padding-free BERT encoder inference for NVIDIA B200 (sm_100a).

The hot path lives in `csrc/` (hand-written CUDA: TMA + tcgen05/TMEM GEMMs and
fused attention, vectorised row kernels) behind the C ABI of `include/bt_b200.h`;
this package is the Python host side over that ABI.  There is no CPU or
PyTorch fallback: importing the compute entry points without the built
`lib/libbt_b200.so` raises.
"""
from ._abi import BtError, LIB_PATH  # noqa: F401

__all__ = ["BtError", "LIB_PATH", "Encoder", "bert_transformer"]


def __getattr__(name):
    if name in ("Encoder", "bert_transformer", "build_offsets", "pack_rows", "restore_rows"):
        from . import encoder
        return getattr(encoder, name)
    raise AttributeError(name)
