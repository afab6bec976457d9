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
