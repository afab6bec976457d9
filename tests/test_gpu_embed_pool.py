"""Embedding front end and pooler back end (the steps either side of the encoder stack) through
the C ABI against their fp32 definitions in the oracle module."""
import pytest
import torch

from helpers import assert_close_fp16

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("B,S,H,gb32,ids", [(3, 17, 768, False, "default"), (2, 64, 1024, True, "given"),
                                            (5, 9, 64, False, "given"), (1, 512, 256, True, "default")])
def test_embedding_layernorm(cuda_device, B, S, H, gb32, ids):
    from bytetransformer_b200.encoder import embedding_layernorm
    from oracle.bert_oracle import embedding_layernorm as ref
    g = torch.Generator().manual_seed(B * 100 + S)
    V, P, Tn = 1000, 600, 2
    word = torch.randn(V, H, generator=g).half()
    pos = (torch.randn(P, H, generator=g) * 0.5).half()
    typ = (torch.randn(Tn, H, generator=g) * 0.5).half()
    gamma = torch.empty(H).uniform_(0.5, 1.5, generator=g)
    beta = torch.empty(H).uniform_(-0.4, 0.4, generator=g)
    gd, bd = (gamma, beta) if gb32 else (gamma.half(), beta.half())
    tok = torch.randint(0, V, (B, S), generator=g, dtype=torch.int32)
    tids = torch.randint(0, Tn, (B, S), generator=g, dtype=torch.int32) if ids == "given" else None
    pids = torch.randint(0, P, (B, S), generator=g, dtype=torch.int32) if ids == "given" else None
    dev = cuda_device
    got = embedding_layernorm(word.to(dev), pos.to(dev), typ.to(dev), gd.to(dev), bd.to(dev), tok.to(dev),
                              None if tids is None else tids.to(dev), None if pids is None else pids.to(dev), eps=1e-6)
    want = ref(word, pos, typ, gd, bd, tok, tids, pids, eps=1e-6)
    assert_close_fp16(got, want, "embedding_layernorm", max_abs=4e-3, mean_abs=4e-4)


def test_embedding_ids_outside_the_tables_are_clamped(cuda_device):
    from bytetransformer_b200.encoder import embedding_layernorm
    g = torch.Generator().manual_seed(1)
    H = 128
    word = torch.randn(10, H, generator=g).half().to(cuda_device)
    pos = torch.randn(4, H, generator=g).half().to(cuda_device)
    typ = torch.randn(2, H, generator=g).half().to(cuda_device)
    gamma = torch.ones(H).half().to(cuda_device)
    beta = torch.zeros(H).half().to(cuda_device)
    bad = torch.tensor([[-5, 3, 99, 9, 0, 1, 2, 3]], dtype=torch.int32, device=cuda_device)      # 8 positions, table of 4
    good = torch.tensor([[0, 3, 9, 9, 0, 1, 2, 3]], dtype=torch.int32, device=cuda_device)
    pids = torch.tensor([[0, 1, 2, 3, 3, 3, 3, 3]], dtype=torch.int32, device=cuda_device)
    a = embedding_layernorm(word, pos, typ, gamma, beta, bad)
    b = embedding_layernorm(word, pos, typ, gamma, beta, good, None, pids)
    assert torch.equal(a, b)


@pytest.mark.parametrize("B,S,H", [(1, 5, 64), (7, 33, 768), (16, 128, 1024)])
def test_pooler(cuda_device, B, S, H):
    from bytetransformer_b200.encoder import pooler
    from oracle.bert_oracle import pooler as ref
    g = torch.Generator().manual_seed(H + B)
    y = torch.randn(B, S, H, generator=g).half()
    W = (torch.randn(H, H, generator=g) * 0.05).half()
    b = torch.empty(H).uniform_(-0.4, 0.4, generator=g).half()
    got = pooler(y.to(cuda_device), W.to(cuda_device), b.to(cuda_device))
    assert_close_fp16(got, ref(y, W, b), "pooler", max_abs=3e-3, mean_abs=3e-4)


@pytest.mark.parametrize("B,S,H,gb32", [(6, 40, 768, False), (3, 129, 1024, True), (40, 17, 256, False)])
def test_embedding_written_packed_matches_embedding_then_pack(cuda_device, B, S, H, gb32):
    """The embedding front end fused with packing: rows of the valid tokens only, in packed order, bit for
    bit the rows that the unfused embedding followed by pack_rows gives (same arithmetic, other placement),
    and close to the fp32 definition; rows beyond the token count are not written."""
    from bytetransformer_b200.encoder import (EmbeddingWeights, build_offsets, embedding_layernorm,
                                              embedding_layernorm_packed, pack_rows)
    from oracle.bert_oracle import build_attr_mask, build_offsets as ref_offsets, embedding_layernorm as ref
    dev = cuda_device
    g = torch.Generator().manual_seed(7 * B + S)
    V, P, Tn = 500, 200, 2
    word = torch.randn(V, H, generator=g).half()
    pos = (torch.randn(P, H, generator=g) * 0.5).half()
    typ = (torch.randn(Tn, H, generator=g) * 0.5).half()
    gamma = torch.empty(H).uniform_(0.5, 1.5, generator=g)
    beta = torch.empty(H).uniform_(-0.4, 0.4, generator=g)
    gd, bd = (gamma, beta) if gb32 else (gamma.half(), beta.half())
    tok = torch.randint(0, V, (B, S), generator=g, dtype=torch.int32)
    tids = torch.randint(0, Tn, (B, S), generator=g, dtype=torch.int32)
    lens = torch.randint(0, S + 1, (B,), generator=g)
    lens[0] = S
    mask = build_attr_mask(lens, S, torch.float16).to(dev)
    bi, wi = build_offsets(mask)
    T = int(bi[-1].item())
    emb = EmbeddingWeights(word.to(dev), pos.to(dev), typ.to(dev), gd.to(dev), bd.to(dev), eps=1e-6)
    got = embedding_layernorm_packed(emb, tok.to(dev), bi, wi, type_ids=tids.to(dev))
    padded = embedding_layernorm(word.to(dev), pos.to(dev), typ.to(dev), gd.to(dev), bd.to(dev), tok.to(dev), tids.to(dev), None, eps=1e-6)
    want_packed = pack_rows(padded, bi)[:T]
    assert torch.equal(got[:T], want_packed)                     # bit-exact placement and values
    assert (got[T:] == 0).all()                                  # nothing written past the token count
    ref_bi, ref_wi = ref_offsets(mask.cpu().float())
    full = ref(word, pos, typ, gd, bd, tok, tids, None, eps=1e-6).reshape(B * S, H)
    assert_close_fp16(got[:T], full[torch.as_tensor(ref_wi[:T]).long()], "packed embedding vs fp32 definition",
                      max_abs=4e-3, mean_abs=4e-4)


def test_stack_from_token_ids_matches_embedding_then_stack(cuda_device):
    """bt_stack_forward_ids = embedding + LayerNorm (packed) -> layers -> scatter, in one call: the same
    numbers as the padded embedding followed by the padded stack (bit for bit: the packed rows are the
    same values and the layers run on them identically)."""
    from bytetransformer_b200.encoder import Encoder, EmbeddingWeights, embedding_layernorm
    from helpers import make_layer_weights, to_device_weights
    from oracle.bert_oracle import build_attr_mask
    dev = cuda_device
    g = torch.Generator().manual_seed(2024)
    nh, H, B, S, V = 12, 768, 5, 96, 300
    layers = [to_device_weights(make_layer_weights(H, g), dev) for _ in range(2)]
    word = (torch.randn(V, H, generator=g)).half().to(dev)
    pos = (torch.randn(S, H, generator=g) * 0.5).half().to(dev)
    typ = (torch.randn(2, H, generator=g) * 0.5).half().to(dev)
    gamma, beta = torch.ones(H).half().to(dev), torch.zeros(H).half().to(dev)
    tok = torch.randint(0, V, (B, S), generator=g, dtype=torch.int32).to(dev)
    lens = torch.tensor([96, 1, 0, 50, 77])
    mask = build_attr_mask(lens, S, torch.float16).to(dev)
    enc = Encoder(nh, 64, layers)
    emb = EmbeddingWeights(word, pos, typ, gamma, beta, eps=1e-6)
    got = enc.forward_ids(emb, tok, mask)
    x = embedding_layernorm(word, pos, typ, gamma, beta, tok, eps=1e-6)
    want = enc.forward(x, mask)
    assert enc.device_status() == 0
    enc.close()
    assert torch.equal(got, want)
