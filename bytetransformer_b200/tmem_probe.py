"""Diagnostic: bytes per clock and SM that the warps of a CTA get out of tensor memory when they do
nothing but read it (`tcgen05.ld` of one shape, a wait after every load, a few XORs per word).

    python -m bytetransformer_b200.tmem_probe

The figure is a ceiling for judging kernels that consume tensor memory (GEMM epilogues, the attention
softmax): a kernel far below it is not bounded by tensor-memory bandwidth."""
import json
import sys

import torch


def read_rate(mode: int, warps: int, reps: int = 200, device=None) -> float:
    """mode 0/1/2 = .x32/.x64/.x128 loads; warps 4 or 8 per CTA; one CTA per SM.  Returns B/clk per SM."""
    from . import _abi
    lib = _abi.load()
    dev = torch.device("cuda:0") if device is None else torch.device(device)
    with torch.cuda.device(dev):
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        clocks = torch.zeros(sms, dtype=torch.int64, device=dev)
        sink = torch.zeros(sms * 256, dtype=torch.int32, device=dev)
        stream = torch.cuda.current_stream(dev).cuda_stream
        for _ in range(2):  # the first launch warms the instruction cache
            rc = lib.bt_debug_tmem_read_probe(mode, warps, sms, reps, clocks.data_ptr(), sink.data_ptr(), stream)
            if rc != 0:
                raise RuntimeError(f"bt_debug_tmem_read_probe returned {rc}")
        torch.cuda.synchronize(dev)
        clk = clocks.double().mean().item()
    return reps * warps * 32 * 256 * 4 / clk


def main() -> int:
    if not torch.cuda.is_available():
        raise SystemExit("needs a CUDA device")
    for warps in (4, 8):
        for mode, name in ((0, ".x32"), (1, ".x64"), (2, ".x128")):
            print(json.dumps({"metric": "tensor_memory_read_rate", "load": "tcgen05.ld.32x32b" + name,
                              "warps_per_cta": warps, "value": round(read_rate(mode, warps), 1),
                              "unit": "B/clk/SM"}), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
