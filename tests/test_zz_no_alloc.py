"""The allocation-free layer call, bt_layer_forward_padded_static().

Some users of this library run inside a host that forbids device allocation at
call time (an inference server after its memory plan is frozen, a plugin callback
of another runtime).  For them the library carries its scratch as a fixed array
in its device image.  This file checks, through the C ABI, that the call gives
the same output as bt_layer_forward_padded() with a caller workspace, twice in a
row (the array keeps the first call's bytes), and that a shape whose scratch
would not fit is refused.  It is collected last on purpose and also passes when
run alone in a fresh process.
"""
import ctypes as C

import pytest
import torch

from helpers import make_layer_weights, to_device_weights


def _make(dev, nh, B, S, seed, lens):
    from bytetransformer_b200.encoder import Encoder
    from oracle.bert_oracle import build_attr_mask
    g = torch.Generator().manual_seed(seed)
    H = nh * 64
    w = to_device_weights(make_layer_weights(H, g, recipe="uniform"), dev)
    enc = Encoder(nh, 64, [w])
    x = torch.empty(B, S, H).uniform_(-0.4, 0.4, generator=g).half().to(dev)
    mask = build_attr_mask(torch.as_tensor(lens), S, torch.float16).to(dev)
    return enc, x, mask


@pytest.mark.gpu
def test_static_scratch_matches_workspace_call_twice(cuda_device):
    from bytetransformer_b200 import _abi
    lib = _abi.load()
    B, S, nh = 6, 160, 12
    lens = [160, 1, 0, 77, 128, 129]
    enc, x, mask = _make(cuda_device, nh, B, S, 41, lens)
    stream = torch.cuda.current_stream(cuda_device).cuda_stream
    want = enc.forward_layer(0, x, mask)                      # existing entry point, caller workspace
    for attempt in range(2):
        out = torch.full_like(x, float("nan"))
        torch.cuda.synchronize(cuda_device)
        free_before = torch.cuda.mem_get_info(cuda_device)[0]  # cudaMemGetInfo: device-wide free bytes
        rc = lib.bt_layer_forward_padded_static(enc._h, 0, x.data_ptr(), mask.data_ptr(), out.data_ptr(), B, S, stream)
        assert rc == _abi.BT_OK, lib.bt_last_error(enc._h)
        torch.cuda.synchronize(cuda_device)
        if attempt == 1:
            # the property the entry point exists for: the call takes no device memory (the first call on a
            # device may still load the kernels' code, so the second one is the one that is held to it)
            assert torch.cuda.mem_get_info(cuda_device)[0] == free_before
        # same kernels, same inputs: the tolerance the encoder tests use is far from needed
        d = (out.float() - want.float()).abs()
        assert torch.isfinite(out).all()
        assert d.max().item() <= 2e-2 and d.mean().item() <= 1e-3, (attempt, d.max().item())
        assert torch.equal(out, want), f"call {attempt} differs from the workspace call"
    # a different shape right after: stale bytes of the previous call must not matter
    B2, S2 = 3, 96
    lens2 = [96, 5, 40]
    enc2, x2, mask2 = _make(cuda_device, nh, B2, S2, 42, lens2)
    want2 = enc2.forward_layer(0, x2, mask2)
    out2 = torch.full_like(x2, float("nan"))
    rc = lib.bt_layer_forward_padded_static(enc2._h, 0, x2.data_ptr(), mask2.data_ptr(), out2.data_ptr(), B2, S2,
                                            torch.cuda.current_stream(cuda_device).cuda_stream)
    assert rc == _abi.BT_OK
    torch.cuda.synchronize(cuda_device)
    assert torch.equal(out2, want2)
    assert enc.device_status() == 0 and enc2.device_status() == 0
    enc.close()
    enc2.close()


@pytest.mark.gpu
def test_static_scratch_rejects_shapes_beyond_its_size(cuda_device):
    from bytetransformer_b200 import _abi
    lib = _abi.load()
    B, S, nh = 8, 512, 12                                      # 4096 tokens: needs ~80 MB of scratch
    enc, x, mask = _make(cuda_device, nh, B, S, 43, [512] * B)
    n = C.c_size_t()
    assert lib.bt_workspace_bytes(enc._h, B, S, C.byref(n)) == _abi.BT_OK
    assert n.value > _abi.BT_STATIC_SCRATCH_BYTES
    out = torch.zeros_like(x)
    rc = lib.bt_layer_forward_padded_static(enc._h, 0, x.data_ptr(), mask.data_ptr(), out.data_ptr(), B, S,
                                            torch.cuda.current_stream(cuda_device).cuda_stream)
    assert rc == _abi.BT_ERR_WORKSPACE
    assert b"BT_STATIC_SCRATCH_BYTES" in lib.bt_last_error(enc._h)
    torch.cuda.synchronize(cuda_device)
    assert out.abs().max().item() == 0.0                       # nothing ran
    enc.close()


@pytest.mark.gpu
def test_handle_refuses_calls_while_another_device_is_current(cuda_device):
    """A handle belongs to the device it was created on; with another device current every entry point that takes
    the handle returns BT_ERR_INVALID_ARG before anything is launched (needs a second GPU to make one current)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from bytetransformer_b200 import _abi
    lib = _abi.load()
    B, S, nh = 2, 32, 2
    enc, x, mask = _make(cuda_device, nh, B, S, 44, [32, 7])
    out = torch.zeros_like(x)
    other = 1 if cuda_device.index in (None, 0) else 0
    with torch.cuda.device(other):
        rc = lib.bt_layer_forward_padded_static(enc._h, 0, x.data_ptr(), mask.data_ptr(), out.data_ptr(), B, S, 0)
        assert rc == _abi.BT_ERR_INVALID_ARG
        assert b"current device" in lib.bt_last_error(enc._h)
    torch.cuda.synchronize(cuda_device)
    assert out.abs().max().item() == 0.0
    enc.close()
