"""The header-only C++ shim (include/bert_transformer.h): compiles and links with a
plain C++ compiler, reports errors as exceptions (CPU), and — on a GPU — gives the
oracle's result through the reference's class API (the flow of the reference's
unit_test/bert_transformer_test.cc)."""
import os
import shutil
import struct
import subprocess

import numpy as np
import pytest
import torch

from helpers import assert_close_fp16, fp16_round, make_layer_weights

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def driver(tmp_path_factory):
    from bytetransformer_b200 import build
    build.build_core()
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cuda = os.path.dirname(os.path.dirname(nvcc))
    exe = str(tmp_path_factory.mktemp("shim") / "shim_driver")
    cmd = ["g++", "-std=c++17", "-O1", os.path.join(ROOT, "tests", "cpp", "shim_driver.cc"), "-o", exe,
           "-I", os.path.join(ROOT, "include"), "-I", os.path.join(cuda, "include"),
           "-L", build.LIB_DIR, "-lbt_b200", "-Wl,-rpath," + build.LIB_DIR,
           "-L", os.path.join(cuda, "lib64"), "-lcudart", "-Wl,-rpath," + os.path.join(cuda, "lib64")]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return exe


def test_shim_compiles_links_and_throws(driver):
    r = subprocess.run([driver, "--link-check"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "FP32 rejected" in r.stdout


@pytest.mark.gpu
@pytest.mark.parametrize("gb32", [0, 1])
def test_shim_infer_matches_oracle(driver, cuda_device, tmp_path, gb32):
    from oracle.bert_oracle import build_attr_mask, encoder_layer
    g = torch.Generator().manual_seed(77 + gb32)
    B, S, nh = 5, 72, 12
    H = nh * 64
    w = make_layer_weights(H, g, recipe="uniform")
    lens = torch.tensor([72, 0, 31, 64, 7])
    x = torch.empty(B, S, H).uniform_(-0.4, 0.4, generator=g).half()
    mask = build_attr_mask(lens, S, torch.float16)
    inp, outp = str(tmp_path / "in.bin"), str(tmp_path / "out.bin")
    with open(inp, "wb") as f:
        f.write(struct.pack("<4i", B, S, nh, gb32))
        for i, t in enumerate(w):
            a = t.float().numpy() if (gb32 and i in (4, 5, 10, 11)) else t.half().numpy()
            f.write(a.tobytes())
        f.write(x.numpy().tobytes())
        f.write(mask.numpy().tobytes())
    r = subprocess.run([driver, inp, outp], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    got = torch.from_numpy(np.fromfile(outp, dtype=np.float16).reshape(B, S, H))
    wr = [t if (gb32 and i in (4, 5, 10, 11)) else t.half().float() for i, t in enumerate(w)]
    want = encoder_layer(x.float(), mask.float(), wr, nh, 64, ln_eps=1e-6, gelu_kind="erf")
    valid = torch.arange(S)[None, :] < lens[:, None]
    assert_close_fp16(got[valid], want[valid], "C++ shim")
    assert (got[~valid] == 0).all()
