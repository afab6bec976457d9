"""CPU: pin the oracle (oracle/bert_oracle.py) to the golden vectors that the
reference's own test script produced (tests/golden/make_golden.py), and check
its offsets / pack / restore restatements on the reference's edge cases."""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import bert_oracle as O

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
FILES = sorted(glob.glob(os.path.join(GOLDEN, "*.npz")))


def test_golden_files_present():
    assert len(FILES) >= 3


@pytest.mark.parametrize("path", FILES, ids=os.path.basename)
def test_oracle_reproduces_reference_script_outputs(path):
    d = np.load(path)
    B, S, nh, hs, nl, _ = d["meta"].tolist()
    layers = [[torch.from_numpy(d[f"l{l}_{n}"]) for n in O.WEIGHT_NAMES] for l in range(nl)]
    x = torch.from_numpy(d["from_tensor"])
    mask = torch.from_numpy(d["attr_mask"])
    # the reference's encoder: exact GELU, F.layer_norm default eps (1e-5)
    outs = O.encoder_stack(x, mask, layers, nh, hs, ln_eps=1e-5, gelu_kind="erf")
    for l in range(nl):
        want = torch.from_numpy(d[f"l{l}_out"])
        assert torch.allclose(outs[l], want, rtol=0, atol=1e-5), (l, (outs[l] - want).abs().max())


@pytest.mark.parametrize("path", FILES, ids=os.path.basename)
def test_mask_recipe_matches_reference_script(path):
    d = np.load(path)
    B, S = d["meta"].tolist()[:2]
    lens = torch.from_numpy(d["input_lens"])
    assert np.array_equal(O.build_attr_mask(lens, S).numpy(), d["attr_mask"])
    bi, wi = O.build_offsets(d["attr_mask"])
    assert bi.dtype == np.int32 and wi.dtype == np.int32
    assert np.array_equal(np.diff(bi), d["input_lens"].astype(np.int32))


def _naive_offsets(mask):
    """Element-by-element definition, independent of the vectorised restatement."""
    B, S, _ = mask.shape
    bi, wi = [0], []
    for b in range(B):
        n = 0
        for j in range(S):
            if float(mask[b, 0, j]) >= 0.5:
                n += 1
        for i in range(n):
            wi.append(b * S + i)
        bi.append(bi[-1] + n)
    return np.array(bi, np.int32), np.array(wi, np.int32)


@pytest.mark.parametrize("B,S,seed", [(1, 1, 0), (5, 16, 1), (33, 40, 2), (70, 7, 3)])
def test_offsets_restatement(B, S, seed):
    g = torch.Generator().manual_seed(seed)
    lens = torch.randint(0, S + 1, (B,), generator=g)
    m = O.build_attr_mask(lens, S).numpy()
    bi, wi = O.build_offsets(m)
    nbi, nwi = _naive_offsets(m)
    assert np.array_equal(bi, nbi) and np.array_equal(wi, nwi)


def test_offsets_known_answer():
    m = O.build_attr_mask(torch.tensor([3, 0, 2]), 4).numpy()
    bi, wi = O.build_offsets(m)
    assert bi.tolist() == [0, 3, 3, 5]
    assert wi.tolist() == [0, 1, 2, 8, 9]


def test_pack_restore_round_trip():
    g = torch.Generator().manual_seed(4)
    lens = torch.tensor([3, 0, 5, 1])
    m = O.build_attr_mask(lens, 5).numpy()
    bi, wi = O.build_offsets(m)
    x = torch.randn(4, 5, 8, generator=g).numpy()
    p = O.pack_rows(x, wi)
    assert p.shape == (9, 8)
    r = O.restore_rows(p, bi, 4, 5)
    valid = (np.arange(5)[None, :] < lens.numpy()[:, None])
    assert np.array_equal(r[valid], x[valid]) and (r[~valid] == 0).all()


def test_packed_stack_equals_padded_stack_on_valid_rows():
    g = torch.Generator().manual_seed(5)
    H, nh = 128, 2
    lens = torch.tensor([5, 9, 0, 2])
    S = 9
    from helpers import make_layer_weights
    layers = [make_layer_weights(H, g, recipe="uniform") for _ in range(2)]
    x = torch.randn(4, S, H, generator=g)
    mask = O.build_attr_mask(lens, S)
    padded = O.encoder_stack(x, mask, layers, nh, 64)[-1]
    bi, wi = O.build_offsets(mask.numpy())
    xp = torch.from_numpy(O.pack_rows(x.numpy(), wi))
    packed = O.encoder_stack_packed(xp, bi.tolist(), layers, nh, 64)
    valid = torch.arange(S)[None, :] < lens[:, None]
    assert torch.allclose(packed, padded[valid], atol=2e-5)


def test_attention_packed_matches_layer_attention():
    g = torch.Generator().manual_seed(6)
    H, nh = 128, 2
    lens = [4, 7]
    cu = [0, 4, 11]
    qkv = torch.randn(11, 3 * H, generator=g)
    out = O.attention_packed(qkv, cu, nh, 64)
    # direct per-sequence computation
    for b in range(2):
        q, k, v = qkv[cu[b]:cu[b + 1]].chunk(3, -1)
        for h in range(nh):
            sl = slice(h * 64, (h + 1) * 64)
            p = torch.softmax(q[:, sl] @ k[:, sl].T / 8.0, -1)
            assert torch.allclose(out[cu[b]:cu[b + 1], sl], p @ v[:, sl], atol=1e-5)
