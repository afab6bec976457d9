"""Shared helpers of the test-suite: seeded inputs and tolerance checks."""
import numpy as np
import torch

# Tolerances of the fp16 path against the fp32 oracle (stated by the north star):
MAX_ABS_TOL = 2e-2
MEAN_ABS_TOL = 1e-3


def make_layer_weights(H, gen, std=0.02, recipe="normal", gb_fp32=False):
    """The 12 tensors of one layer (fp32, CPU) in the reference's order.

    recipe "normal":   weights ~ N(0, std), biases and beta 0, gamma 1.
    recipe "uniform":  everything ~ U(-0.4, 0.4), the recipe of the reference's
                       test (unit_test/python_scripts/bert_transformer_test.py:100-112);
                       exercises the bias / gamma / beta paths.
    """
    F = 4 * H
    shapes = [(H, 3 * H), (3 * H,), (H, H), (H,), (H,), (H,), (H, F), (F,), (F, H), (H,), (H,), (H,)]
    out = []
    for i, s in enumerate(shapes):
        if recipe == "uniform":
            t = torch.empty(*s).uniform_(-0.4, 0.4, generator=gen)
        else:
            if len(s) == 2:
                t = torch.randn(*s, generator=gen) * std
            elif i in (4, 10):
                t = torch.ones(*s)
            else:
                t = torch.zeros(*s)
        out.append(t)
    return out


def to_device_weights(w, device, gb_fp32=False):
    res = []
    for i, t in enumerate(w):
        if i in (4, 5, 10, 11) and gb_fp32:
            res.append(t.float().to(device).contiguous())
        else:
            res.append(t.half().to(device).contiguous())
    return res


def fp16_round(w):
    """What the GPU actually sees: weights rounded to fp16, as fp32 CPU tensors."""
    return [t.half().float() for t in w]


def assert_close_fp16(got, want, what="", max_abs=MAX_ABS_TOL, mean_abs=MEAN_ABS_TOL):
    got = got.float().cpu()
    want = want.float().cpu()
    assert got.shape == want.shape, (what, got.shape, want.shape)
    assert torch.isfinite(got).all(), f"{what}: non-finite values in the output"
    d = (got - want).abs()
    mx = d.max().item() if d.numel() else 0.0
    mn = d.mean().item() if d.numel() else 0.0
    assert mx <= max_abs and mn <= mean_abs, f"{what}: max-abs {mx:.4g} (tol {max_abs}), mean-abs {mn:.4g} (tol {mean_abs})"
    return mx, mn
