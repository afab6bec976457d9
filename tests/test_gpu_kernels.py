"""GPU parity tests of the individual steps of the path, through the C ABI,
against the CPU oracle (oracle/bert_oracle.py)."""
import math

import numpy as np
import pytest
import torch

from helpers import assert_close_fp16

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def enc(cuda_device):
    from bytetransformer_b200.encoder import Encoder
    from helpers import make_layer_weights, to_device_weights
    g = torch.Generator().manual_seed(0)
    w = to_device_weights(make_layer_weights(768, g), cuda_device)
    e = Encoder(12, 64, [w])
    yield e
    assert e.device_status() == 0
    e.close()


def _mask_from_lens(lens, S):
    from oracle.bert_oracle import build_attr_mask
    return build_attr_mask(torch.tensor(lens), S, torch.float16)


# ---------------------------------------------------------------- offsets / pack / restore
@pytest.mark.parametrize("B,S,lens", [
    (1, 8, [5]),
    (4, 24, [13, 7, 15, 13]),
    (5, 16, [3, 8, 5, 10, 0]),            # zero-length sequence
    (3, 13, [13, 0, 1]),                   # S not a multiple of 8, full + empty
    (40, 64, None),                        # more than 32 sequences: crosses the warp-scan boundary
    (1500, 32, None),                      # more than 1024 sequences: crosses the block-scan chunk
    (16, 512, None),
])
def test_offsets_bit_exact(cuda_device, B, S, lens):
    from bytetransformer_b200.encoder import build_offsets
    from oracle.bert_oracle import build_offsets as ref_offsets
    if lens is None:
        g = torch.Generator().manual_seed(B * 1000 + S)
        lens = torch.randint(0, S + 1, (B,), generator=g).tolist()
    mask = _mask_from_lens(lens, S)
    bi, wi = build_offsets(mask.to(cuda_device))
    rbi, rwi = ref_offsets(mask.numpy())
    assert np.array_equal(bi.cpu().numpy(), rbi)
    T = int(rbi[-1])
    assert np.array_equal(wi.cpu().numpy()[:T], rwi)


def test_offsets_counts_mask_values_ge_half(cuda_device):
    """Length is the COUNT of entries >= 0.5 in mask row 0 (remove_padding.h:51-54),
    whatever the other rows hold."""
    from bytetransformer_b200.encoder import build_offsets
    from oracle.bert_oracle import build_offsets as ref_offsets
    B, S = 3, 16
    m = torch.zeros(B, S, S, dtype=torch.float16)
    m[0, 0, :5] = 1.0
    m[1, 0, :7] = 0.5
    m[1, 0, 7:9] = 0.49
    m[2, 0, :3] = 2.0
    m[:, 1:, :] = 1.0  # other rows must not matter
    bi, wi = build_offsets(m.to(cuda_device))
    rbi, rwi = ref_offsets(m.numpy())
    assert rbi.tolist() == [0, 5, 12, 15]
    assert np.array_equal(bi.cpu().numpy(), rbi)
    assert np.array_equal(wi.cpu().numpy()[:15], rwi)


@pytest.mark.parametrize("B,S,H", [(5, 16, 64), (16, 64, 768), (3, 13, 128)])
def test_pack_restore_round_trip(cuda_device, B, S, H):
    from bytetransformer_b200.encoder import build_offsets, pack_rows, restore_rows
    from oracle.bert_oracle import build_offsets as ref_offsets, pack_rows as ref_pack, restore_rows as ref_restore
    g = torch.Generator().manual_seed(7)
    lens = torch.randint(0, S + 1, (B,), generator=g).tolist()
    mask = _mask_from_lens(lens, S)
    x = torch.randn(B, S, H, generator=g).half()
    bi, _ = build_offsets(mask.to(cuda_device))
    packed = pack_rows(x.to(cuda_device), bi)
    rbi, rwi = ref_offsets(mask.numpy())
    T = int(rbi[-1])
    want = ref_pack(x.numpy(), rwi)
    assert np.array_equal(packed.cpu().numpy()[:T], want)          # bit-exact copy
    back = restore_rows(packed, bi, B, S)
    assert np.array_equal(back.cpu().numpy(), ref_restore(want, rbi, B, S))  # zeros in padding rows


# ---------------------------------------------------------------- row kernels
@pytest.mark.parametrize("M,H,gb32", [(7, 64, False), (129, 768, False), (300, 1024, True), (33, 128, True)])
def test_add_bias_residual_layernorm(cuda_device, M, H, gb32):
    from bytetransformer_b200.encoder import add_bias_residual_layernorm
    from oracle.bert_oracle import add_bias_residual_layernorm as ref
    g = torch.Generator().manual_seed(M + H)
    x = torch.randn(M, H, generator=g).half()
    r = torch.randn(M, H, generator=g).half()
    b = torch.empty(H).uniform_(-0.4, 0.4, generator=g).half()
    gamma = torch.empty(H).uniform_(-0.4, 0.4, generator=g)
    beta = torch.empty(H).uniform_(-0.4, 0.4, generator=g)
    gd = gamma if gb32 else gamma.half()
    bd = beta if gb32 else beta.half()
    got = add_bias_residual_layernorm(x.to(cuda_device), b.to(cuda_device), r.to(cuda_device),
                                      gd.to(cuda_device), bd.to(cuda_device), eps=1e-6)
    want = ref(x.float(), b.float(), r.float(), gd.float(), bd.float(), eps=1e-6)
    assert_close_fp16(got, want, "layernorm", max_abs=4e-3, mean_abs=5e-4)


def test_layernorm_row_count_from_device(cuda_device):
    from bytetransformer_b200.encoder import add_bias_residual_layernorm
    g = torch.Generator().manual_seed(3)
    x = torch.randn(64, 256, generator=g).half().to(cuda_device)
    gamma = torch.ones(256).half().to(cuda_device)
    beta = torch.zeros(256).half().to(cuda_device)
    m_dev = torch.tensor([10], dtype=torch.int32, device=cuda_device)
    out = add_bias_residual_layernorm(x, None, None, gamma, beta, m_dev=m_dev)
    assert out[10:].abs().max().item() == 0.0      # rows beyond the device-side count untouched
    assert out[:10].abs().max().item() > 0.1


def test_layernorm_restore(cuda_device):
    from bytetransformer_b200.encoder import add_bias_residual_layernorm_restore, build_offsets
    from oracle.bert_oracle import add_bias_residual_layernorm as ref, build_offsets as ref_offsets, restore_rows
    B, S, H = 5, 16, 768
    lens = [3, 16, 0, 10, 1]
    mask = _mask_from_lens(lens, S)
    rbi, _ = ref_offsets(mask.numpy())
    T = int(rbi[-1])
    g = torch.Generator().manual_seed(11)
    x = torch.randn(T, H, generator=g).half()
    r = torch.randn(T, H, generator=g).half()
    b = torch.empty(H).uniform_(-0.4, 0.4, generator=g).half()
    gamma = torch.empty(H).uniform_(-0.4, 0.4, generator=g).half()
    beta = torch.empty(H).uniform_(-0.4, 0.4, generator=g).half()
    bi, _ = build_offsets(mask.to(cuda_device))
    got = add_bias_residual_layernorm_restore(x.to(cuda_device), b.to(cuda_device), r.to(cuda_device),
                                              gamma.to(cuda_device), beta.to(cuda_device), bi, B, S)
    want_packed = ref(x.float(), b.float(), r.float(), gamma.float(), beta.float(), eps=1e-6)
    want = torch.from_numpy(restore_rows(want_packed.numpy(), rbi, B, S))
    assert_close_fp16(got, want, "layernorm_restore", max_abs=4e-3, mean_abs=5e-4)
    pad = ~(torch.arange(S)[None, :] < torch.tensor(lens)[:, None])
    assert (got.cpu()[pad] == 0).all()            # exact zeros in padding rows


@pytest.mark.parametrize("kind", ["erf", "tanh"])
def test_add_bias_gelu(cuda_device, kind):
    from bytetransformer_b200.encoder import add_bias_gelu_
    from oracle.bert_oracle import add_bias_gelu as ref
    g = torch.Generator().manual_seed(5)
    x = (torch.randn(37, 3072, generator=g) * 2).half()
    b = torch.empty(3072).uniform_(-0.4, 0.4, generator=g).half()
    got = add_bias_gelu_(x.clone().to(cuda_device), b.to(cuda_device), kind)
    want = ref(x.float(), b.float(), kind)
    assert_close_fp16(got, want, "add_bias_gelu", max_abs=4e-3, mean_abs=3e-4)


@pytest.mark.parametrize("B,nh,S", [(2, 3, 64), (2, 2, 13), (1, 2, 512), (1, 1, 1024), (2, 1, 8), (1, 5, 264), (3, 2, 776)])
def test_masked_softmax(cuda_device, B, nh, S):
    from bytetransformer_b200.encoder import masked_softmax_
    from oracle.bert_oracle import masked_softmax as ref
    g = torch.Generator().manual_seed(S)
    lens = torch.randint(1, S + 1, (B,), generator=g).tolist()
    mask = _mask_from_lens(lens, S)
    x = (torch.randn(nh, B, S, S, generator=g) * 3).half()
    got = masked_softmax_(x.clone().to(cuda_device), mask.to(cuda_device), 0.125)
    want = ref(x.float(), mask.float(), 0.125)
    assert_close_fp16(got, want, "masked_softmax", max_abs=2e-3, mean_abs=1e-4)


# ---------------------------------------------------------------- GEMM
def _gemm_case(enc, dev, M, N, K, epi, gelu="erf", m_valid=None, seed=0):
    from bytetransformer_b200 import _abi
    g = torch.Generator().manual_seed(seed + M + N + K)
    a = torch.randn(M, K, generator=g).half()
    w = (torch.randn(K, N, generator=g) * 0.05).half()
    bias = torch.empty(N).uniform_(-0.4, 0.4, generator=g).half()
    res = torch.randn(M, N, generator=g).half()
    m_dev = None if m_valid is None else torch.tensor([m_valid], dtype=torch.int32, device=dev)
    got = enc.gemm(a.to(dev), w.to(dev), bias.to(dev), res.to(dev), epilogue=epi,
                   gelu=_abi.BT_GELU_ERF if gelu == "erf" else _abi.BT_GELU_TANH, m_dev=m_dev)
    want = a.float() @ w.float()
    if epi != _abi.BT_EPI_NONE:
        want = want + bias.float()
    if epi == _abi.BT_EPI_BIAS_GELU:
        want = torch.nn.functional.gelu(want, approximate="none" if gelu == "erf" else "tanh")
    if epi == _abi.BT_EPI_BIAS_RESIDUAL:
        want = want + res.float()
    mv = M if m_valid is None else m_valid
    scale = max(1.0, want.abs().max().item())
    assert_close_fp16(got[:mv], want[:mv], f"gemm {M}x{N}x{K} epi{epi}", max_abs=4e-3 * scale, mean_abs=4e-4 * scale)
    if mv < M:
        assert got[mv:].abs().max().item() == 0.0, "rows beyond the device-side row count were written"


@pytest.mark.parametrize("M,N,K", [
    (1, 64, 64), (7, 128, 64), (128, 256, 128), (129, 192, 192), (300, 768, 768),
    (640, 2304, 768), (1000, 768, 3072), (4500, 3072, 768), (257, 1024, 1024),
])
def test_gemm_plain(enc, cuda_device, M, N, K):
    from bytetransformer_b200 import _abi
    _gemm_case(enc, cuda_device, M, N, K, _abi.BT_EPI_NONE)


@pytest.mark.parametrize("epi,gelu", [(1, "erf"), (2, "erf"), (2, "tanh"), (3, "erf")])
@pytest.mark.parametrize("M,N,K", [(200, 768, 768), (515, 3072, 768)])
def test_gemm_epilogues(enc, cuda_device, M, N, K, epi, gelu):
    _gemm_case(enc, cuda_device, M, N, K, epi, gelu)


def test_gemm_row_count_from_device(enc, cuda_device):
    from bytetransformer_b200 import _abi
    _gemm_case(enc, cuda_device, 700, 768, 768, _abi.BT_EPI_BIAS, m_valid=333)
    _gemm_case(enc, cuda_device, 256, 256, 64, _abi.BT_EPI_NONE, m_valid=0)


@pytest.mark.parametrize("bn", [64, 128, 256])
def test_gemm_every_tile_width(enc, cuda_device, bn):
    from bytetransformer_b200 import _abi
    lib = _abi.load()
    lib.bt_debug_set(4, bn)
    try:
        _gemm_case(enc, cuda_device, 390, 768, 768, _abi.BT_EPI_BIAS_RESIDUAL)
        _gemm_case(enc, cuda_device, 4000, 768, 3072, _abi.BT_EPI_BIAS)
    finally:
        lib.bt_debug_set(4, 0)


def test_gemm_twice_bit_identical(enc, cuda_device):
    """Same launch twice must give bit-identical output (catches smem / TMEM races)."""
    g = torch.Generator().manual_seed(9)
    a = torch.randn(2000, 768, generator=g).half().to(cuda_device)
    w = (torch.randn(768, 2304, generator=g) * 0.05).half().to(cuda_device)
    o1 = enc.gemm(a, w)
    o2 = enc.gemm(a, w)
    assert torch.equal(o1, o2)


# ---------------------------------------------------------------- attention
@pytest.mark.parametrize("lens", [
    [1], [15], [16], [17], [64], [127], [128], [129], [255, 3], [300, 1, 128, 77],
    [512, 17, 0, 200], [1024], [5, 0, 0, 9],
])
def test_attention(enc, cuda_device, lens):
    from oracle.bert_oracle import attention_packed
    H = enc.hidden
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    T = int(cu[-1])
    g = torch.Generator().manual_seed(sum(lens))
    rows = T + 5                                   # a few allocated rows beyond T, filled with NaN
    qkv = torch.randn(rows, 3 * H, generator=g).half()
    qkv[T:] = float("nan")
    got = enc.attention(qkv.to(cuda_device), torch.from_numpy(cu).to(cuda_device), max(lens))
    want = attention_packed(qkv[:T].float(), cu.tolist(), enc.head_num, enc.head_size)
    assert_close_fp16(got[:T], want, f"attention {lens}", max_abs=5e-3, mean_abs=3e-4)
    assert got[T:].abs().max().item() == 0.0 if rows > T else True


def test_attention_twice_bit_identical(enc, cuda_device):
    lens = [300, 77, 129]
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]).astype(np.int32), device=cuda_device)
    g = torch.Generator().manual_seed(1)
    qkv = torch.randn(sum(lens), 3 * enc.hidden, generator=g).half().to(cuda_device)
    a = enc.attention(qkv, cu, 300)
    b = enc.attention(qkv, cu, 300)
    assert torch.equal(a, b)


def test_gemm_fp32_out_feeds_layernorm(enc, cuda_device):
    """The attention-output / FFN2 GEMMs keep the pre-LayerNorm sum in fp32
    (BT_EPI_BIAS_RESIDUAL_F32OUT) and the LayerNorm kernel reads it as float."""
    from bytetransformer_b200 import _abi
    from bytetransformer_b200.encoder import add_bias_residual_layernorm
    g = torch.Generator().manual_seed(21)
    M, N, K = 333, 768, 768
    a = torch.randn(M, K, generator=g).half()
    w = (torch.randn(K, N, generator=g) * 0.05).half()
    bias = torch.empty(N).uniform_(-0.4, 0.4, generator=g).half()
    res = torch.randn(M, N, generator=g).half()
    gamma = torch.empty(N).uniform_(0.5, 1.5, generator=g).half()
    beta = torch.empty(N).uniform_(-0.4, 0.4, generator=g).half()
    pre = enc.gemm(a.to(cuda_device), w.to(cuda_device), bias.to(cuda_device), res.to(cuda_device),
                   epilogue=_abi.BT_EPI_BIAS_RESIDUAL_F32OUT)
    assert pre.dtype == torch.float32
    want_pre = a.float() @ w.float() + bias.float() + res.float()
    assert (pre.cpu() - want_pre).abs().max().item() < 2e-4
    out = add_bias_residual_layernorm(pre, None, None, gamma.to(cuda_device), beta.to(cuda_device), eps=1e-6)
    want = torch.nn.functional.layer_norm(want_pre, (N,), gamma.float(), beta.float(), eps=1e-6)
    assert_close_fp16(out, want, "gemm->ln", max_abs=3e-3, mean_abs=3e-4)


@pytest.mark.parametrize("M,N,K,epi", [
    (256, 256, 64, 0), (300, 768, 768, 1), (1000, 2304, 768, 1), (777, 3072, 768, 2),
    (2049, 768, 3072, 3), (4500, 768, 768, 4), (18944, 768, 3072, 4), (129, 256, 128, 0),
])
def test_gemm_pair_kernel(enc, cuda_device, M, N, K, epi):
    """The two-CTA (cta_group::2, 256x256 tile) kernel, forced on for every shape."""
    from bytetransformer_b200 import _abi
    lib = _abi.load()
    lib.bt_debug_set(5, 1)
    try:
        if epi == 4:
            g = torch.Generator().manual_seed(M + N)
            a = torch.randn(M, K, generator=g).half()
            w = (torch.randn(K, N, generator=g) * 0.05).half()
            bias = torch.empty(N).uniform_(-0.4, 0.4, generator=g).half()
            res = torch.randn(M, N, generator=g).half()
            got = enc.gemm(a.to(cuda_device), w.to(cuda_device), bias.to(cuda_device), res.to(cuda_device),
                           epilogue=_abi.BT_EPI_BIAS_RESIDUAL_F32OUT)
            want = a.float() @ w.float() + bias.float() + res.float()
            assert (got.cpu() - want).abs().max().item() < 1e-3
        else:
            _gemm_case(enc, cuda_device, M, N, K, epi)
        _gemm_case(enc, cuda_device, M, N, K, _abi.BT_EPI_BIAS, m_valid=max(0, M - 131))
    finally:
        lib.bt_debug_set(5, 0)
    assert enc.device_status() == 0


def test_gemm_pair_twice_bit_identical_and_equal_to_single(enc, cuda_device):
    from bytetransformer_b200 import _abi
    lib = _abi.load()
    g = torch.Generator().manual_seed(19)
    a = torch.randn(5000, 768, generator=g).half().to(cuda_device)
    w = (torch.randn(768, 2304, generator=g) * 0.05).half().to(cuda_device)
    lib.bt_debug_set(5, 1)
    try:
        o1 = enc.gemm(a, w)
        o2 = enc.gemm(a, w)
    finally:
        lib.bt_debug_set(5, 2)
    try:
        o3 = enc.gemm(a, w)
    finally:
        lib.bt_debug_set(5, 0)
    assert torch.equal(o1, o2)
    assert torch.equal(o1, o3)          # same accumulation order: K is walked identically


@pytest.mark.parametrize("kernel", [0, 1, 3], ids=["by_shape", "cta_per_item", "persistent"])
def test_attention_variants(enc, cuda_device, kernel):
    """Both attention kernels (one CTA per item, persistent) forced for the same ragged batch, and the
    choice by shape, against the oracle; twice, bit-identical (race check)."""
    from bytetransformer_b200 import _abi
    from oracle.bert_oracle import attention_packed
    lib = _abi.load()
    lens = [300, 1, 128, 77, 513, 129, 1024, 64]
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    T = int(cu[-1])
    g = torch.Generator().manual_seed(4242)
    qkv = (torch.randn(T, 3 * enc.hidden, generator=g) * 1.5).half()   # logits with std ~ 2.8: sharp softmax
    want = attention_packed(qkv.float(), cu.tolist(), enc.head_num, enc.head_size)
    lib.bt_debug_set_mha_tiles(kernel)
    try:
        got = enc.attention(qkv.to(cuda_device), torch.from_numpy(cu).to(cuda_device), max(lens))
        got2 = enc.attention(qkv.to(cuda_device), torch.from_numpy(cu).to(cuda_device), max(lens))
    finally:
        lib.bt_debug_set_mha_tiles(0)
    assert torch.equal(got, got2)
    assert enc.device_status() == 0
    mx, mn = assert_close_fp16(got, want, f"attention kernel {kernel}", max_abs=8e-3, mean_abs=4e-4)
    print(f"attention kernel {kernel}: max-abs {mx:.3e} mean-abs {mn:.3e}")


@pytest.mark.parametrize("kernel", [1, 3], ids=["cta_per_item", "persistent"])
def test_attention_rejects_offsets_outside_the_allocation(enc, cuda_device, kernel):
    """cu_seqlens that do not describe rows of the buffers (a sequence running past the last row, one longer
    than max_len, a decreasing offset) must not be followed: the kernel leaves those sequences out, reports
    the bad-offsets status, and the rows of the well-formed sequences still come out right."""
    from bytetransformer_b200 import _abi
    from oracle.bert_oracle import attention_packed
    lib = _abi.load()
    good = [200, 130, 300]
    T = sum(good)
    g = torch.Generator().manual_seed(99)
    qkv = torch.randn(T, 3 * enc.hidden, generator=g).half()
    want = attention_packed(qkv.float(), np.concatenate([[0], np.cumsum(good)]).tolist(), enc.head_num, enc.head_size)
    qkv_dev = qkv.to(cuda_device)
    lib.bt_debug_set_mha_tiles(kernel)
    try:
        for bad_cu, ok_rows in (([0, 200, 330, 900], slice(0, 330)),        # last sequence runs past the 630 rows
                                ([0, 200, 100, 630], slice(0, 200)),        # decreasing offset
                                ([0, 200, 330, 630, 630 + 5000], slice(0, 630))):  # longer than max_len and the buffer
            cu = torch.tensor(bad_cu, dtype=torch.int32, device=cuda_device)
            out = torch.zeros(T, enc.hidden, dtype=torch.float16, device=cuda_device)
            rc = lib.bt_attention(enc._h, qkv_dev.data_ptr(), out.data_ptr(), cu.data_ptr(), len(bad_cu) - 1,
                                  300, T, torch.cuda.current_stream().cuda_stream)
            assert rc == 0
            torch.cuda.synchronize()
            assert enc.device_status() == 0x301
            assert torch.isfinite(out).all()
            if bad_cu[:3] == [0, 200, 330]:
                assert_close_fp16(out[ok_rows].cpu(), want[ok_rows], "rows of the well-formed sequences",
                                  max_abs=8e-3, mean_abs=4e-4)
    finally:
        lib.bt_debug_set_mha_tiles(0)
    assert enc.device_status() == 0


@pytest.mark.parametrize("M,N,K,gb32,m_valid", [
    (128, 256, 64, False, None), (333, 768, 768, False, None), (1000, 768, 3072, True, None),
    (18944, 768, 768, False, None), (700, 1024, 1024, True, 555), (40000, 768, 768, False, 39999), (130, 512, 128, False, 0),
])
@pytest.mark.parametrize("pair", [2, 1], ids=["one_cta", "sm_pairs"])
def test_gemm_with_fused_layernorm(enc, cuda_device, M, N, K, gb32, m_valid, pair):
    """bt_gemm_layernorm: GEMM + bias + residual + LayerNorm in one kernel, in its one-CTA form and in the
    form that runs the main loop on SM pairs (256-row tiles), each forced for every shape."""
    from bytetransformer_b200 import _abi
    _abi.load().bt_debug_set(9, pair)
    try:
        _fused_layernorm_case(enc, cuda_device, M, N, K, gb32, m_valid)
    finally:
        _abi.load().bt_debug_set(9, 0)


def _fused_layernorm_case(enc, cuda_device, M, N, K, gb32, m_valid):
    g = torch.Generator().manual_seed(M + N + K)
    a = torch.randn(M, K, generator=g).half()
    w = (torch.randn(K, N, generator=g) * 0.05).half()
    bias = torch.empty(N).uniform_(-0.4, 0.4, generator=g).half()
    res = (torch.randn(M, N, generator=g) + 0.5).half()          # non-zero mean exercises the one-pass variance
    gamma = torch.empty(N).uniform_(0.5, 1.5, generator=g)
    beta = torch.empty(N).uniform_(-0.4, 0.4, generator=g)
    gd, bd = (gamma, beta) if gb32 else (gamma.half(), beta.half())
    m_dev = None if m_valid is None else torch.tensor([m_valid], dtype=torch.int32, device=cuda_device)
    args = [t.to(cuda_device) for t in (a, w, bias, res, gd, bd)]
    got = enc.gemm_layernorm(*args, eps=1e-6, m_dev=m_dev)
    got2 = enc.gemm_layernorm(*args, eps=1e-6, m_dev=m_dev)
    assert torch.equal(got, got2)
    mv = M if m_valid is None else m_valid
    rows = slice(0, mv) if mv <= 4096 else torch.cat([torch.arange(0, 2048), torch.arange(mv - 2048, mv)])
    pre = a[rows].float() @ w.float() + bias.float() + res[rows].float()
    want = torch.nn.functional.layer_norm(pre, (N,), gd.float(), bd.float(), eps=1e-6)
    assert_close_fp16(got.cpu()[rows], want, f"gemm+ln {M}x{N}x{K}", max_abs=6e-3, mean_abs=4e-4)
    if mv < M:
        assert got[mv:].abs().max().item() == 0.0
    assert enc.device_status() == 0


# ---------------------------------------------------------------- failure path
def test_expired_wait_is_reported_and_the_context_stays_usable(enc, cuda_device):
    """A device-side wait that nothing satisfies (the library's own self-test kernel: an mbarrier
    nobody arrives on) gives up after its bound, the kernel returns normally, the status word
    carries the code, reading it clears it, and the next GEMM on the same handle is correct."""
    import time
    from bytetransformer_b200 import _abi
    gave_up = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    t0 = time.time()
    enc.selftest_bounded_wait(4_000_000, gave_up)      # ~2 ms of SM cycles
    torch.cuda.synchronize()
    assert time.time() - t0 < 5.0
    assert gave_up.item() == 1
    assert enc.device_status() == 0x7F1
    assert enc.device_status() == 0                     # read-and-clear
    _gemm_case(enc, cuda_device, 300, 768, 768, _abi.BT_EPI_BIAS)
    assert enc.device_status() == 0
