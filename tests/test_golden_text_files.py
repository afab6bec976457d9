"""Test vectors in the reference's text format (one float per line, the fifteen files its script
exports and its C++ test loads): writer / reader round trip on CPU, and on a GPU a case written
from the oracle replayed by the C++ driver tests/cpp/text_case_driver.cc through the class API."""
import os
import re
import shutil
import subprocess

import numpy as np
import pytest
import torch

from helpers import MAX_ABS_TOL, fp16_round, make_layer_weights

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _case(nh, B, S, seed):
    from oracle.bert_oracle import build_attr_mask, encoder_layer
    g = torch.Generator().manual_seed(seed)
    H = nh * 64
    w = [t.float() for t in fp16_round(make_layer_weights(H, g, recipe="normal"))]
    lens = torch.randint(0, S + 1, (B,), generator=g)
    lens[0] = S
    x = torch.randn(B, S, H, generator=g).half().float()
    mask = build_attr_mask(lens, S, torch.float32)
    out = encoder_layer(x, mask, w, nh, 64, ln_eps=1e-6, gelu_kind="erf")
    valid = (torch.arange(S)[None, :] < lens[:, None]).unsqueeze(-1).float()
    return w, x, mask, out * valid, lens


def test_write_read_round_trip(tmp_path):
    from bytetransformer_b200 import golden_files as gf
    w, x, mask, out, _ = _case(1, 2, 9, seed=1)
    gf.write_case(str(tmp_path), [t.numpy() for t in w], x.numpy(), mask.numpy(), out.numpy())
    assert sorted(os.listdir(tmp_path)) == sorted(list(gf.WEIGHT_FILES) + [gf.INPUT_FILE, gf.MASK_FILE, gf.OUTPUT_FILE])
    first = open(tmp_path / "qkv_bias.in").readline().strip()
    assert re.fullmatch(r"-?\d+\.\d{6}", first), first          # '%f' notation, one value per line
    back = gf.read_case(str(tmp_path), 2, 9, 1)
    for a, b in zip(back["weights"], w):
        assert a.shape == tuple(b.shape)
        assert np.abs(a - b.numpy()).max() <= 1e-6                # six decimals
    assert np.abs(back["from_tensor"] - x.numpy()).max() <= 1e-6
    assert np.array_equal(back["atten_mask"], mask.numpy())
    assert np.abs(back["transformer_out"] - out.numpy()).max() <= 1e-6
    with pytest.raises(ValueError):
        gf.read_case(str(tmp_path), 2, 10, 1)                     # wrong shape is refused


@pytest.fixture(scope="module")
def text_driver(tmp_path_factory):
    from bytetransformer_b200 import build
    build.build_core()
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cuda = os.path.dirname(os.path.dirname(nvcc))
    exe = str(tmp_path_factory.mktemp("textcase") / "text_case_driver")
    cmd = ["g++", "-std=c++17", "-O1", os.path.join(ROOT, "tests", "cpp", "text_case_driver.cc"), "-o", exe,
           "-I", os.path.join(ROOT, "include"), "-I", os.path.join(cuda, "include"),
           "-L", build.LIB_DIR, "-lbt_b200", "-Wl,-rpath," + build.LIB_DIR,
           "-L", os.path.join(cuda, "lib64"), "-lcudart", "-Wl,-rpath," + os.path.join(cuda, "lib64")]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return exe


def test_driver_builds_and_reports_missing_files(text_driver, tmp_path):
    r = subprocess.run([text_driver, "2", "8", "1", "64", str(tmp_path)], capture_output=True, text=True, timeout=120)
    assert r.returncode == 1 and "cannot open" in r.stderr


@pytest.mark.gpu
@pytest.mark.parametrize("gb32", [0, 1])
def test_text_case_replayed_through_the_class_api(text_driver, cuda_device, tmp_path, gb32):
    from bytetransformer_b200 import golden_files as gf
    nh, B, S = 2, 3, 40
    w, x, mask, out, lens = _case(nh, B, S, seed=5 + gb32)
    gf.write_case(str(tmp_path), [t.numpy() for t in w], x.numpy(), mask.numpy(), out.numpy())
    r = subprocess.run([text_driver, str(B), str(S), str(nh), "64", str(tmp_path), str(gb32), str(MAX_ABS_TOL)],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    m = re.search(r"max_diff ([0-9.]+) .* mean_diff ([0-9.]+)", r.stdout)
    assert m, r.stdout
    assert float(m.group(1)) <= MAX_ABS_TOL and float(m.group(2)) <= 1e-3
    got = np.loadtxt(tmp_path / "transformer_out.cuda.out", dtype=np.float32).reshape(B, S, nh * 64)
    pad = ~(np.arange(S)[None, :] < lens.numpy()[:, None])
    assert (got[pad] == 0).all()
