"""GPU parity of the encoder layer / stack through the C ABI against the oracle
(the reference's own fp32 PyTorch encoder, oracle/bert_oracle.py), on the
committed golden vectors and on seeded inputs with the benchmark shapes.

Tolerance (fp16 path vs fp32 oracle): max-abs <= 2e-2, mean-abs <= 1e-3."""
import glob
import os

import numpy as np
import pytest
import torch

from helpers import (MAX_ABS_TOL, MEAN_ABS_TOL, assert_close_fp16, fp16_round, make_layer_weights,
                     to_device_weights)

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _oracle(x, mask, layers, nh, hs, **kw):
    from oracle.bert_oracle import encoder_stack
    return encoder_stack(x, mask, layers, nh, hs, **kw)


def _valid(lens, S):
    return torch.arange(S)[None, :] < torch.as_tensor(lens)[:, None]


def _run_case(dev, B, S, nh, n_layers, lens, recipe, seed, gb32=False, gelu="erf", eps=1e-6, per_layer_op=False,
              fused_ln=None, split_k=None):
    from bytetransformer_b200.encoder import Encoder, bert_transformer
    from oracle.bert_oracle import build_attr_mask
    H = nh * 64
    g = torch.Generator().manual_seed(seed)
    layers = [make_layer_weights(H, g, recipe=recipe) for _ in range(n_layers)]
    x = torch.randn(B, S, H, generator=g) if recipe == "normal" else torch.empty(B, S, H).uniform_(-0.4, 0.4, generator=g)
    lens_t = torch.as_tensor(lens)
    mask = build_attr_mask(lens_t, S)
    want = _oracle(x.half().float(), mask, [fp16_round(w) for w in layers], nh, 64, ln_eps=eps, gelu_kind=gelu)[-1]
    dl = [to_device_weights(w, dev, gb32) for w in layers]
    xd, md = x.half().to(dev), mask.half().to(dev)
    if per_layer_op:
        h = xd
        for w in dl:
            h = bert_transformer(nh, 64, *w, h, md, True, True, ln_eps=eps, gelu=gelu)
        got = h
    else:
        enc = Encoder(nh, 64, dl, ln_eps=eps, gelu=gelu)
        if fused_ln is not None:  # 0 = LayerNorm as its own kernel, 2 = always inside the GEMM kernel
            from bytetransformer_b200 import _abi
            assert _abi.load().bt_debug_set_fused_layernorm(enc._h, fused_ln) == 0
        if split_k is not None:  # K ranges of the two GEMMs that feed a LayerNorm: -1 never, n > 0 forced
            from bytetransformer_b200 import _abi
            assert _abi.load().bt_debug_set(7, split_k) == 0
        try:
            got = enc.forward(xd, md)
        finally:
            if split_k is not None:
                _abi.load().bt_debug_set(7, 0)
        assert enc.device_status() == 0
        enc.close()
    v = _valid(lens, S)
    mx, mn = assert_close_fp16(got.cpu()[v], want[v], f"encoder B{B} S{S} L{n_layers} {recipe}")
    assert (got.cpu()[~v] == 0).all(), "padding rows must be exact zeros"
    return mx, mn


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLDEN, "*.npz"))), ids=os.path.basename)
def test_golden_vectors_from_reference_script(cuda_device, path):
    """Inputs, weights and outputs produced by the reference's own test script
    (tests/golden/make_golden.py); its PyTorch encoder uses exact GELU and the
    LayerNorm default eps 1e-5, so the library is configured the same way."""
    from bytetransformer_b200.encoder import Encoder
    from oracle.bert_oracle import WEIGHT_NAMES
    d = np.load(path)
    B, S, nh, hs, nl, _ = d["meta"].tolist()
    layers = [[torch.from_numpy(d[f"l{l}_{n}"]) for n in WEIGHT_NAMES] for l in range(nl)]
    x = torch.from_numpy(d["from_tensor"])
    mask = torch.from_numpy(d["attr_mask"])
    lens = d["input_lens"].tolist()
    dl = [to_device_weights(w, cuda_device) for w in layers]
    enc = Encoder(nh, hs, dl, ln_eps=1e-5, gelu="erf")
    h = x.half().to(cuda_device)
    md = mask.half().to(cuda_device)
    v = _valid(lens, S)
    # the reference's weights are U(-0.4,0.4): activations are O(10), so the bound scales with them
    for l in range(nl):
        h = enc.forward_layer(l, h, md)
        want = torch.from_numpy(d[f"l{l}_out"])
        # golden weights/inputs are fp32; the GPU sees them rounded to fp16 -> looser bound than the oracle test
        assert_close_fp16(h.cpu()[v], want[v], f"golden layer {l}", max_abs=6e-2, mean_abs=6e-3)
        assert (h.cpu()[~v] == 0).all()
    assert enc.device_status() == 0
    enc.close()


def test_config1_single_layer_b16_s64(cuda_device):
    """BERT-base layer, batch 16, max_seq 64, lengths uniform in [1,64] (seeded)."""
    g = torch.Generator().manual_seed(101)
    lens = torch.randint(1, 65, (16,), generator=g).tolist()
    _run_case(cuda_device, 16, 64, 12, 1, lens, "normal", seed=1)


def test_config1_reference_recipe_uniform_weights(cuda_device):
    """Same shape with the reference's own recipe (everything U(-0.4,0.4), lengths U[13,64]):
    exercises bias / gamma / beta.  Activations reach O(10), hence a scaled bound."""
    from bytetransformer_b200.encoder import Encoder
    from oracle.bert_oracle import build_attr_mask, encoder_stack
    g = torch.Generator().manual_seed(202)
    B, S, nh, H = 16, 64, 12, 768
    lens = torch.randint(13, 65, (B,), generator=g).tolist()
    layers = [make_layer_weights(H, g, recipe="uniform")]
    x = torch.empty(B, S, H).uniform_(-0.4, 0.4, generator=g)
    mask = build_attr_mask(torch.as_tensor(lens), S)
    want = encoder_stack(x.half().float(), mask, [fp16_round(w) for w in layers], nh, 64, ln_eps=1e-6)[-1]
    enc = Encoder(nh, 64, [to_device_weights(w, cuda_device) for w in layers])
    got = enc.forward(x.half().to(cuda_device), mask.half().to(cuda_device))
    v = _valid(lens, S)
    assert_close_fp16(got.cpu()[v], want[v], "uniform recipe")
    assert (got.cpu()[~v] == 0).all()
    enc.close()


def test_fp32_gamma_beta_and_tanh_gelu(cuda_device):
    g = torch.Generator().manual_seed(5)
    lens = torch.randint(0, 49, (6,), generator=g).tolist()
    _run_case(cuda_device, 6, 48, 2, 2, lens, "uniform", seed=3, gb32=True, gelu="tanh", eps=1e-5)


def test_per_layer_op_equals_stack(cuda_device):
    """Calling the one-layer operator N times (the reference's loop) and the one-call
    stack give the same result within tolerance (re-packing between layers is exact)."""
    g = torch.Generator().manual_seed(6)
    lens = torch.randint(1, 97, (4,), generator=g).tolist()
    _run_case(cuda_device, 4, 96, 12, 3, lens, "normal", seed=8, per_layer_op=True)
    _run_case(cuda_device, 4, 96, 12, 3, lens, "normal", seed=8, per_layer_op=False)


def test_config3_b16_s512_12_layers(cuda_device):
    """BERT-base 12 layers, batch 16, max_seq 512, lengths uniform in [1,512] (seeded)."""
    g = torch.Generator().manual_seed(303)
    lens = torch.randint(1, 513, (16,), generator=g).tolist()
    _run_case(cuda_device, 16, 512, 12, 12, lens, "normal", seed=4)


@pytest.mark.parametrize("fused_ln", [0, 2])
@pytest.mark.parametrize("nh,gb32", [(12, False), (16, True), (4, False)])
def test_layernorm_inside_gemm_or_separate(cuda_device, nh, gb32, fused_ln):
    """Both placements of LayerNorm (row kernel / inside the GEMM kernel by clusters of hidden/256
    CTAs) against the oracle, hidden 768 / 1024 / 256, ragged last row tile, 3 layers."""
    g = torch.Generator().manual_seed(77 + nh)
    lens = torch.randint(1, 301, (6,), generator=g).tolist()
    _run_case(cuda_device, 6, 300, nh, 3, lens, "normal", seed=21, gb32=gb32, fused_ln=fused_ln)


@pytest.mark.parametrize("split_k", [-1, 2, 4, 6])
@pytest.mark.parametrize("B,S,nh", [(1, 64, 12), (5, 130, 16)])
def test_split_k_sums(cuda_device, B, S, nh, split_k):
    """The attention-output and FFN2 GEMMs with K cut into ranges (one CTA and one fp32 partial sum per
    range, added up by the LayerNorm kernel) against the oracle; -1 = one range.  Hidden 768 has 12 and
    48 K blocks, hidden 1024 has 16 and 64, so 6 ranges only divide the former and the latter falls back
    to one range."""
    g = torch.Generator().manual_seed(5 + S)
    lens = [round(0.6 * S)] if B == 1 else torch.randint(1, S + 1, (B,), generator=g).tolist()
    _run_case(cuda_device, B, S, nh, 3, lens, "normal", seed=33, split_k=split_k, fused_ln=0)


@pytest.mark.parametrize("S", [64, 320, 1024])
def test_config2_batch1(cuda_device, S):
    """Batch 1, valid length round(0.6*S), 12 layers."""
    _run_case(cuda_device, 1, S, 12, 12, [round(0.6 * S)], "normal", seed=S)


def test_config4_bert_large_shapes_sampled(cuda_device):
    """BERT-large (hidden 1024, 16 heads), max_seq 384, truncated-normal lengths; 8 of the 64
    sequences and 3 of the 24 layers so that the CPU oracle finishes in seconds."""
    g = torch.Generator().manual_seed(404)
    lens = torch.clamp(torch.round(torch.randn(8, generator=g) * 80 + 230), 8, 384).long().tolist()
    _run_case(cuda_device, 8, 384, 16, 3, lens, "normal", seed=9)


def test_config4_bert_large_full_size(cuda_device):
    """BASELINE configuration 4 at full size through the padded drop-in entry point: BERT-large (24 layers,
    hidden 1024, 16 heads), batch 64, max_seq 384, lengths from the seeded truncated normal (13.7k valid
    tokens: the GEMM + LayerNorm kernels with four column tiles per row tile, 24 layers of error
    accumulation).  The CPU oracle cannot run the whole batch in test time, so:
      (a) the batch is run again with its sequences in reverse order: every sequence's rows must come out
          bit-identical, padding rows exact zeros;
      (b) all outputs are finite and every valid row is normalised (gamma 1, beta 0);
      (c) the longest, a middle and the shortest sequence are checked against the oracle run on that
          sequence alone (max-abs 2e-2, mean-abs 1e-3, the tolerance of the fp16 path)."""
    from bytetransformer_b200.encoder import Encoder
    from bytetransformer_b200.workloads import BERT_LARGE, lengths_for, make_weights
    from oracle.bert_oracle import build_attr_mask
    dev = cuda_device
    H, nh, S = BERT_LARGE.hidden, BERT_LARGE.head_num, 384
    lens = torch.as_tensor(lengths_for("large_b64_s384"))
    B = int(lens.numel())
    assert B == 64 and int(lens.max()) <= S
    weights = make_weights(BERT_LARGE, seed=7, device="cpu")
    assert len(weights) == 24
    enc = Encoder(nh, 64, [[t.to(dev) for t in layer] for layer in weights])
    g = torch.Generator().manual_seed(4004)
    x = torch.randn(B, S, H, generator=g).half()
    mask = build_attr_mask(lens, S, torch.float16)
    out = enc.forward(x.to(dev), mask.to(dev)).cpu()
    rev = torch.arange(B - 1, -1, -1)
    out_rev = enc.forward(x[rev].contiguous().to(dev), mask[rev].contiguous().to(dev)).cpu()
    assert enc.device_status() == 0
    enc.close()
    assert torch.equal(out, out_rev[rev]), "rows depend on the position of their sequence in the batch"
    v = _valid(lens.tolist(), S)
    assert (out[~v] == 0).all(), "padding rows must be exact zeros"
    of = out[v].float()
    assert torch.isfinite(of).all()
    assert of.mean(dim=1).abs().max().item() < 5e-3
    assert (of.var(dim=1, unbiased=False) - 1.0).abs().max().item() < 2e-2
    order = torch.argsort(lens, stable=True)
    layers32 = [[t.float() for t in layer] for layer in weights]
    for b in (int(order[-1]), int(order[B // 2]), int(order[0])):
        L = int(lens[b])
        want = _oracle(x[b, :L].float()[None], torch.ones(1, L, L), layers32, nh, 64, ln_eps=1e-6)[-1][0]
        assert_close_fp16(out[b, :L], want, f"config 4, sequence {b} of {L} tokens, 24 layers")


def test_packed_entry_matches_padded(cuda_device):
    """bt_stack_forward_packed on x[T,H] + cu_seqlens gives the rows of the padded call."""
    from bytetransformer_b200.encoder import Encoder, build_offsets, pack_rows
    from oracle.bert_oracle import build_attr_mask
    g = torch.Generator().manual_seed(12)
    B, S, nh, H, nl = 7, 200, 12, 768, 2
    lens = torch.randint(0, S + 1, (B,), generator=g).tolist()
    layers = [to_device_weights(make_layer_weights(H, g), cuda_device) for _ in range(nl)]
    x = torch.randn(B, S, H, generator=g).half().to(cuda_device)
    mask = build_attr_mask(torch.as_tensor(lens), S, torch.float16).to(cuda_device)
    enc = Encoder(nh, 64, layers)
    padded = enc.forward(x, mask)
    bi, _ = build_offsets(mask)
    T = int(bi[-1].item())
    xp = pack_rows(x, bi)[:T].contiguous()
    outp = enc.forward_packed(xp, bi, max(lens))
    v = _valid(lens, S)
    # same kernels except where the row count decides: the last LayerNorm (padded: separate kernel with
    # scatter, two-pass variance; packed: may be fused into the GEMM, one-pass variance) and the number of
    # K ranges the fp32 sums before a LayerNorm are accumulated in (B*S rows against T): equal up to an
    # fp16 ulp or two on a few elements
    d = (outp.cpu().float() - padded.cpu()[v].float()).abs()
    assert d.max().item() <= 4e-3 and d.mean().item() <= 1e-4, (d.max().item(), d.mean().item())
    assert enc.device_status() == 0
    enc.close()


def test_error_behaviour(cuda_device):
    """Bad input raises RuntimeError, as TORCH_CHECK does in the reference's plugin."""
    from bytetransformer_b200.encoder import Encoder
    g = torch.Generator().manual_seed(1)
    w = to_device_weights(make_layer_weights(128, g), cuda_device)
    enc = Encoder(2, 64, [w])
    x = torch.zeros(2, 8, 128, dtype=torch.float16, device=cuda_device)
    m = torch.ones(2, 8, 8, dtype=torch.float16, device=cuda_device)
    with pytest.raises(RuntimeError):
        enc.forward(x.float(), m)                       # wrong dtype
    with pytest.raises(RuntimeError):
        enc.forward(x.cpu(), m)                         # not CUDA
    with pytest.raises(RuntimeError):
        enc.forward(x.transpose(0, 1), m)               # not contiguous
    with pytest.raises(RuntimeError):
        enc.forward(torch.zeros(1, 1025, 128, dtype=torch.float16, device=cuda_device),
                    torch.ones(1, 1, 1, dtype=torch.float16, device=cuda_device))   # seq_len too long
    with pytest.raises(RuntimeError):
        Encoder(2, 32, [w])                             # head size must be 64
    enc.close()


def test_whole_box_workload_full_size_properties(cuda_device):
    """The benchmark workload at full size (1024 sequences of U[16,1024] tokens, BERT-base, 12 layers,
    cut into micro-batches of at most 148 x 128 packed tokens exactly as the benchmark does), through
    the packed entry point.  The CPU oracle cannot run 556k tokens in test time, so at this size:
      (a) every micro-batch is run a second time with its sequences in reverse order: a sequence's rows
          must come out bit-identical wherever the sequence sits in the batch;
      (b) all outputs are finite and every row is normalised (the last op is a LayerNorm with gamma 1,
          beta 0: row mean ~ 0, row variance ~ 1);
      (c) the longest, a middle and the shortest sequence are checked against the oracle run on that
          sequence alone (tolerance of the fp16 path: max-abs 2e-2, mean-abs 1e-3)."""
    from bytetransformer_b200.encoder import Encoder
    from bytetransformer_b200.runner import pick_token_budget
    from bytetransformer_b200.sharding import micro_batches
    from bytetransformer_b200.workloads import BERT_BASE, lengths_for, make_weights
    dev = cuda_device
    H, nh = BERT_BASE.hidden, BERT_BASE.head_num
    lens = lengths_for("whole_box_1024x1024")
    assert len(lens) == 1024 and lens.min() >= 16 and lens.max() <= 1024
    weights = make_weights(BERT_BASE, seed=7, device="cpu")
    enc = Encoder(nh, 64, [[t.to(dev) for t in layer] for layer in weights])
    mbs = micro_batches(lens, np.arange(len(lens)), pick_token_budget(int(lens.sum())), mix=False)   # as bench.py cuts them at N = 1
    assert sum(mb.tokens for mb in mbs) == int(lens.sum())
    order = np.argsort(lens, kind="stable")
    sampled = {int(order[-1]), int(order[len(order) // 2]), int(order[0])}
    kept = {}
    for k, mb in enumerate(mbs):
        g = torch.Generator(device=dev).manual_seed(1000 + k)
        x = torch.randn(mb.tokens, H, generator=g, device=dev, dtype=torch.float32).half()
        cu = torch.from_numpy(mb.cu_seqlens).to(dev)
        out = enc.forward_packed(x, cu, mb.max_len)
        # (a) reversed order of the sequences
        n = len(mb.seq_ids)
        ls = np.diff(mb.cu_seqlens)
        rev = np.arange(n)[::-1]
        cu_rev = np.zeros(n + 1, dtype=np.int32)
        np.cumsum(ls[rev], out=cu_rev[1:])
        x_rev = torch.cat([x[mb.cu_seqlens[i]:mb.cu_seqlens[i + 1]] for i in rev])
        out_rev = enc.forward_packed(x_rev, torch.from_numpy(cu_rev).to(dev), mb.max_len)
        back = torch.cat([out_rev[cu_rev[n - 1 - i]:cu_rev[n - i]] for i in range(n)])
        assert torch.equal(out, back), f"micro-batch {k}: rows depend on the position of their sequence"
        # (b)
        of = out.float()
        assert torch.isfinite(of).all()
        assert of.mean(dim=1).abs().max().item() < 5e-3
        assert (of.var(dim=1, unbiased=False) - 1.0).abs().max().item() < 2e-2
        for i, sid in enumerate(mb.seq_ids):
            if int(sid) in sampled:
                a, b = mb.cu_seqlens[i], mb.cu_seqlens[i + 1]
                kept[int(sid)] = (x[a:b].cpu(), out[a:b].cpu())
    assert enc.device_status() == 0
    enc.close()
    # (c)
    assert set(kept) == sampled
    layers32 = [[t.float() for t in layer] for layer in weights]
    for sid, (xs, got) in kept.items():
        L = xs.shape[0]
        want = _oracle(xs.float()[None], torch.ones(1, L, L), layers32, nh, 64, ln_eps=1e-6)[-1][0]
        assert_close_fp16(got, want, f"sequence {sid} of {L} tokens")


@pytest.mark.gpu
def test_end_to_end_runner_matches_the_device_resident_path(cuda_device):
    """PackedRunner.run_host (pinned host buffers, copies on their own streams, two device buffers each way) must give
    exactly what run_device gives on the same micro-batches, also when it is called again at once: the first copies
    of the second call are enqueued while the last micro-batches of the first may still be computing, and must
    wait for them."""
    from bytetransformer_b200.encoder import Encoder
    from bytetransformer_b200.runner import PackedRunner
    from bytetransformer_b200.workloads import BERT_BASE, make_weights
    import copy
    sh = copy.copy(BERT_BASE)
    sh.layers = 2
    enc = Encoder(sh.head_num, 64, make_weights(sh, seed=3, device=cuda_device))
    rng = np.random.default_rng(5)
    lens = rng.integers(1, 400, size=90)
    runner = PackedRunner(enc, lens, np.arange(len(lens)), token_budget=4096)
    assert len(runner.batches) >= 4
    xs_h, outs_h = runner.make_host_inputs(seed=1)
    xs_d = [x.to(cuda_device) for x in xs_h]
    outs_d = [torch.empty_like(x) for x in xs_d]
    runner.run_device(xs_d, outs_d)
    torch.cuda.synchronize(cuda_device)
    for attempt in range(3):
        for o in outs_h:
            o.zero_()
        runner.run_host(xs_h, outs_h)
        runner.run_host(xs_h, outs_h)      # back to back: no synchronisation in between
        torch.cuda.synchronize(cuda_device)
        for k, (oh, od) in enumerate(zip(outs_h, outs_d)):
            assert torch.equal(oh, od.cpu()), f"attempt {attempt}: micro-batch {k} differs"
    assert enc.device_status() == 0
    enc.close()
