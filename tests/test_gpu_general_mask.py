"""The general-mask entry points (any [B,S,S] mask applied element by element, optional
attention_bias [heads,S,S]) against the oracle, and the device-side check that tells a
right-padding mask from any other.  Semantics: the reference's padded / unfused attention
(bytetransformer/include/softmax.h:41-45): score*scale + bias + (1 - mask) * -10000."""
import pytest
import torch

from helpers import assert_close_fp16, fp16_round, make_layer_weights, to_device_weights

pytestmark = pytest.mark.gpu


def _masks(kind, B, S, g):
    if kind == "causal":
        m = torch.tril(torch.ones(S, S)).expand(B, S, S).clone()
    elif kind == "prefix_lm":
        m = torch.tril(torch.ones(S, S)).expand(B, S, S).clone()
        for b in range(B):
            p = int(torch.randint(1, S, (1,), generator=g))
            m[b, :, :p] = 1.0
    elif kind == "block_diagonal":      # several documents packed into one row
        m = torch.zeros(B, S, S)
        for b in range(B):
            cuts = sorted(set([0, S] + torch.randint(1, S, (3,), generator=g).tolist()))
            for lo, hi in zip(cuts[:-1], cuts[1:]):
                m[b, lo:hi, lo:hi] = 1.0
    elif kind == "causal_blank_rows":   # a few query rows may see nothing at all
        m = torch.tril(torch.ones(S, S)).expand(B, S, S).clone()
        m[:, 5, :] = 0.0
        if S > 140:
            m[0, 130:140, :] = 0.0
    elif kind == "soft":                # entries other than 0 and 1: the bits cannot stand for the mask
        m = torch.tril(torch.ones(S, S)).expand(B, S, S).clone()
        m[:, :, ::7] *= 0.75
        m[:, 3, 1] = 0.25
    elif kind == "right_padded":
        lens = torch.randint(1, S + 1, (B,), generator=g)
        m = ((torch.arange(S)[None, :] < lens[:, None]).float().unsqueeze(1)).expand(B, S, S).clone()
    else:
        raise ValueError(kind)
    return m


def _run(dev, nh, B, S, kind, with_bias, n_layers, seed):
    from bytetransformer_b200.encoder import Encoder
    from oracle.bert_oracle import encoder_layer
    H = nh * 64
    g = torch.Generator().manual_seed(seed)
    layers = [make_layer_weights(H, g) for _ in range(n_layers)]
    x = torch.randn(B, S, H, generator=g).half()
    mask = _masks(kind, B, S, g)
    bias = (torch.randn(nh, S, S, generator=g) * 0.5).half() if with_bias else None
    h = x.float()
    for w in layers:
        h = encoder_layer(h, mask, fp16_round(w), nh, 64, ln_eps=1e-6,
                          attention_bias=None if bias is None else bias.float())
    enc = Encoder(nh, 64, [to_device_weights(w, dev) for w in layers])
    got = enc.forward_general(x.to(dev), mask.half().to(dev), None if bias is None else bias.to(dev))
    assert enc.device_status() == 0
    enc.close()
    if kind == "right_padded":      # rows that attend to nothing but themselves are meaningless: compare valid rows
        rows = mask[:, 0, :] > 0.5
        assert_close_fp16(got.cpu()[rows], h[rows], f"general {kind}")
    else:
        assert_close_fp16(got.cpu(), h, f"general {kind} bias={with_bias}")


@pytest.mark.parametrize("kind", ["causal", "prefix_lm", "block_diagonal", "right_padded"])
@pytest.mark.parametrize("with_bias", [False, True])
def test_general_mask_one_layer(cuda_device, kind, with_bias):
    _run(cuda_device, 4, 3, 200, kind, with_bias, 1, seed=11)


@pytest.mark.parametrize("S", [300, 77])
def test_rows_that_see_no_key_attend_to_all_keys(cuda_device, S):
    """A row whose mask is all zero has every score shifted by the same -10000, so its softmax runs over ALL
    keys (the reference's arithmetic mask): the key tiles of its query tile must not be cut short, while the
    other query tiles of a causal mask stop at the diagonal.  Every row is compared."""
    _run(cuda_device, 4, 2, S, "causal_blank_rows", False, 2, seed=19)


def test_general_mask_seq_len_not_multiple_of_8(cuda_device):
    """Rows of the mask / bias are then not 16-byte aligned: the scalar load path."""
    _run(cuda_device, 2, 2, 77, "causal", True, 1, seed=3)


def test_general_mask_long_sequence_three_layers(cuda_device):
    _run(cuda_device, 12, 2, 640, "prefix_lm", True, 3, seed=5)


@pytest.mark.parametrize("S,kind", [(77, "causal"), (640, "prefix_lm"), (96, "block_diagonal"), (1024, "causal")])
def test_binary_mask_without_bias_is_applied_from_bits(cuda_device, S, kind):
    """No bias and a mask of zeros and ones: a pre-pass turns the mask into one bit per (query, key) and the
    attention kernel applies it inside its softmax passes; sequence lengths that are not multiples of 8 / 32 /
    128 exercise the scalar pre-pass and the tail key tile."""
    _run(cuda_device, 2, 2, S, kind, False, 2, seed=S)


def test_mask_with_other_values_falls_back_to_the_additive_form(cuda_device):
    """(1 - mask) * -10000 for entries like 0.25 or 0.75 cannot be expressed in bits: the pre-pass raises its
    flag and the kernel adds the fp16 mask itself."""
    _run(cuda_device, 4, 2, 200, "soft", False, 1, seed=23)


def test_general_path_equals_packed_path_on_right_padded_masks(cuda_device):
    """On a right-padding mask both paths compute the same valid rows."""
    from bytetransformer_b200.encoder import Encoder
    g = torch.Generator().manual_seed(2)
    nh, B, S = 12, 5, 150
    w = [to_device_weights(make_layer_weights(nh * 64, g), cuda_device) for _ in range(2)]
    x = torch.randn(B, S, nh * 64, generator=g).half().to(cuda_device)
    mask = _masks("right_padded", B, S, g).half().to(cuda_device)
    enc = Encoder(nh, 64, w)
    a = enc.forward(x, mask)
    b = enc.forward_general(x, mask)
    rows = (mask[:, 0, :] > 0.5)
    d = (a[rows].float() - b[rows].float()).abs()
    assert d.max().item() <= 4e-3 and d.mean().item() <= 1e-4, (d.max().item(), d.mean().item())
    assert enc.device_status() == 0
    enc.close()


def test_mask_check_tells_right_padded_from_other_masks(cuda_device):
    from bytetransformer_b200.encoder import mask_is_right_padded
    g = torch.Generator().manual_seed(9)
    B, S = 6, 96
    rp = _masks("right_padded", B, S, g).half()
    assert mask_is_right_padded(rp.to(cuda_device)) is True
    outer = rp.clone()                            # padding rows all zero: the outer-product form of the reference's script
    lens = (rp[:, 0, :] > 0.5).sum(1)
    for b in range(B):
        outer[b, int(lens[b]):, :] = 0.0
    assert mask_is_right_padded(outer.to(cuda_device)) is True
    ones_below = rp.clone()                       # padding rows that allow keys beyond the length: refused
    for b in range(B):
        ones_below[b, int(lens[b]):, :] = 1.0
    assert mask_is_right_padded(ones_below.to(cuda_device)) is bool((lens == S).all())
    for kind in ("causal", "prefix_lm", "block_diagonal"):
        assert mask_is_right_padded(_masks(kind, B, S, g).half().to(cuda_device)) is False
    hole = rp.clone()
    b = int(torch.argmax(lens))
    hole[b, 0, 0] = 0.0                           # a hole in row 0: count and prefix disagree
    assert mask_is_right_padded(hole.to(cuda_device)) is False
    one_wrong = rp.clone()
    if int(lens[b]) >= 2:
        one_wrong[b, int(lens[b]) - 1, 0] = 0.0   # one element of one valid row
        assert mask_is_right_padded(one_wrong.to(cuda_device)) is False
