"""The PyTorch plugin (libths_bytetransformer.so): schema on CPU, behaviour on GPU."""
import io
import os

import pytest
import torch

from helpers import assert_close_fp16, fp16_round, make_layer_weights, to_device_weights

EXPECTED_SCHEMA = (
    "ByteTransformer::BertTransformer(int head_num, int head_size, Tensor qkv_kernel, Tensor qkv_bias, "
    "Tensor attr_output_kernel, Tensor attr_output_bias, Tensor attr_output_layernorm_gamma, "
    "Tensor attr_output_layernorm_beta, Tensor inter_kernel, Tensor inter_bias, Tensor output_kernel, "
    "Tensor output_bias, Tensor output_layernorm_gamma, Tensor output_layernorm_beta, Tensor input, "
    "Tensor attr_mask, bool is_remove_padding=True, bool use_fused_attention=True) -> Tensor")


@pytest.fixture(scope="module")
def plugin():
    from bytetransformer_b200 import build
    path = build.build_th_op()
    torch.ops.load_library(path)
    return path


def test_operator_schema_matches_reference(plugin):
    """Same schema string as the reference registers (th_op/ths_op_f.cc:85-95)."""
    schemas = torch._C._jit_get_schemas_for_operator("ByteTransformer::BertTransformer")
    assert len(schemas) == 1 and str(schemas[0]) == EXPECTED_SCHEMA


def test_custom_class_registered(plugin):
    cls = torch.classes.ByteTransformer.BertTransformer
    assert cls is not None


def test_cpu_tensors_are_rejected(plugin):
    g = torch.Generator().manual_seed(0)
    w = [t.half() for t in make_layer_weights(64, g)]
    x = torch.zeros(1, 4, 64, dtype=torch.float16)
    m = torch.ones(1, 4, 4, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        torch.ops.ByteTransformer.BertTransformer(1, 64, *w, x, m, True, True)


@pytest.mark.gpu
def test_functional_op_and_class_on_gpu(plugin, cuda_device):
    from oracle.bert_oracle import build_attr_mask, encoder_layer
    g = torch.Generator().manual_seed(31)
    nh, H, B, S = 12, 768, 5, 80
    w = make_layer_weights(H, g, recipe="normal")
    lens = torch.tensor([80, 3, 0, 64, 17])
    x = torch.randn(B, S, H, generator=g).half()
    mask = build_attr_mask(lens, S, torch.float16)
    want = encoder_layer(x.float(), mask.float(), fp16_round(w), nh, 64, ln_eps=1e-6, gelu_kind="erf")
    wd = to_device_weights(w, cuda_device)
    got = torch.ops.ByteTransformer.BertTransformer(nh, 64, *wd, x.to(cuda_device), mask.to(cuda_device), True, True)
    valid = torch.arange(S)[None, :] < lens[:, None]
    assert_close_fp16(got.cpu()[valid], want[valid], "th_op functional")
    assert (got.cpu()[~valid] == 0).all()

    obj = torch.classes.ByteTransformer.BertTransformer(nh, 64, *wd)
    got2 = obj.forward(x.to(cuda_device), mask.to(cuda_device))
    assert torch.equal(got2, got)
    # is_remove_padding = False: the padded path computes every row; on a right-padded mask its valid rows agree
    got3 = obj.forwardv2(x.to(cuda_device), mask.to(cuda_device), False, False)
    assert_close_fp16(got3.cpu()[valid], want[valid], "th_op class, is_remove_padding=False")
    assert_close_fp16(got3.cpu()[valid], got.cpu()[valid].float(), "padded path vs packed path", max_abs=8e-3, mean_abs=4e-4)

    # fp32 LayerNorm gamma/beta (use_fp32 of the reference) are accepted
    wd32 = to_device_weights(w, cuda_device, gb_fp32=True)
    got4 = torch.ops.ByteTransformer.BertTransformer(nh, 64, *wd32, x.to(cuda_device), mask.to(cuda_device), True, True)
    assert_close_fp16(got4.cpu()[valid], want[valid], "th_op fp32 gamma/beta")

    with pytest.raises(RuntimeError):
        torch.ops.ByteTransformer.BertTransformer(nh, 64, *wd, x.float().to(cuda_device), mask.to(cuda_device), True, True)


@pytest.mark.gpu
def test_causal_mask_needs_and_gets_the_padded_path(plugin, cuda_device):
    """A causal mask through the operator with is_remove_padding=False (the reference's padded semantics:
    whole [B,S,S] mask applied element by element, bytetransformer/src/attention_fused.cu:234-237,
    bytetransformer/include/softmax.h:41-45) against the oracle, through the functional op, the class's
    forwardv2 and, with an additive bias, forward_with_bias."""
    from oracle.bert_oracle import encoder_layer
    g = torch.Generator().manual_seed(77)
    nh, H, B, S = 12, 768, 3, 200
    w = make_layer_weights(H, g)
    x = torch.randn(B, S, H, generator=g).half()
    mask = torch.tril(torch.ones(S, S)).expand(B, S, S).contiguous()
    want = encoder_layer(x.float(), mask, fp16_round(w), nh, 64, ln_eps=1e-6)
    wd = to_device_weights(w, cuda_device)
    xd, md = x.to(cuda_device), mask.half().to(cuda_device)
    got = torch.ops.ByteTransformer.BertTransformer(nh, 64, *wd, xd, md, False, True)
    assert_close_fp16(got.cpu(), want, "functional op, causal mask, is_remove_padding=False")
    obj = torch.classes.ByteTransformer.BertTransformer(nh, 64, *wd)
    assert torch.equal(obj.forwardv2(xd, md, False, True), got)
    bias = (torch.randn(nh, S, S, generator=g) * 0.5).half()
    want_b = encoder_layer(x.float(), mask, fp16_round(w), nh, 64, ln_eps=1e-6, attention_bias=bias.float())
    got_b = obj.forward_with_bias(xd, md, bias.to(cuda_device))
    assert_close_fp16(got_b.cpu(), want_b, "class forward_with_bias, causal mask")
    # with packing on, the same mask means "length 1" (row 0 allows one key): not what a causal mask wants
    packed = torch.ops.ByteTransformer.BertTransformer(nh, 64, *wd, xd, md, True, True)
    assert (packed.cpu()[:, 1:] == 0).all()


@pytest.mark.gpu
def test_torchscript_pickle_round_trip(plugin, cuda_device):
    """Scripted module holding the custom class saves and loads (12 tensors + head info)."""
    g = torch.Generator().manual_seed(32)
    nh, H = 2, 128
    wd = to_device_weights(make_layer_weights(H, g), cuda_device)

    class M(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.enc = torch.classes.ByteTransformer.BertTransformer(nh, 64, *wd)

        def forward(self, x, m):
            return self.enc.forward(x, m)

    sm = torch.jit.script(M())
    buf = io.BytesIO()
    torch.jit.save(sm, buf)
    buf.seek(0)
    sm2 = torch.jit.load(buf)
    x = torch.randn(2, 16, H, generator=g).half().to(cuda_device)
    m = torch.ones(2, 16, 16, dtype=torch.float16, device=cuda_device)
    assert torch.equal(sm(x, m), sm2(x, m))


def test_stack_class_registered(plugin):
    assert torch.classes.ByteTransformer.BertEncoder is not None


@pytest.mark.gpu
def test_stack_class_equals_the_loop_over_one_layer_objects(plugin, cuda_device):
    """ByteTransformer.BertEncoder (all layers in one object, tokens packed once per forward) against the reference's
    way of running a model, a loop over one-layer objects, and against the oracle; with padding removal off it takes
    the padded path for a causal mask.  Also the pickle state (12 tensors per layer + head info)."""
    from oracle.bert_oracle import build_attr_mask, encoder_layer
    g = torch.Generator().manual_seed(77)
    nh, H, B, S, n_layers = 4, 256, 4, 96, 3
    layers = [make_layer_weights(H, g, recipe="normal") for _ in range(n_layers)]
    lens = torch.tensor([96, 1, 50, 77])
    x = torch.randn(B, S, H, generator=g).half()
    mask = build_attr_mask(lens, S, torch.float16)
    flat = [t for w in layers for t in to_device_weights(w, cuda_device)]
    enc = torch.classes.ByteTransformer.BertEncoder(nh, 64, flat)
    assert enc.num_layers() == n_layers
    xd, md = x.to(cuda_device), mask.to(cuda_device)
    got = enc.forward(xd, md)
    h = xd
    for l in range(n_layers):
        one = torch.classes.ByteTransformer.BertTransformer(nh, 64, *flat[12 * l:12 * (l + 1)])
        h = one.forward(h, md)
    valid = torch.arange(S)[None, :] < lens[:, None]
    d = (got.float() - h.float()).abs().cpu()[valid]
    assert d.max().item() <= 4e-3 and d.mean().item() <= 1e-4      # the last LayerNorm runs in different kernels
    assert (got.cpu()[~valid] == 0).all()
    want = x.float()
    for w in layers:
        want = encoder_layer(want, mask.float(), fp16_round(w), nh, 64, ln_eps=1e-6, gelu_kind="erf")
    assert_close_fp16(got.cpu()[valid], want[valid], "stack class vs oracle")
    # padded path: causal mask, every row computed
    causal = torch.tril(torch.ones(S, S)).expand(B, S, S).contiguous().half()
    want_c = x.float()
    for w in layers:
        want_c = encoder_layer(want_c, causal.float(), fp16_round(w), nh, 64, ln_eps=1e-6, gelu_kind="erf")
    got_c = enc.forwardv2(xd, causal.to(cuda_device), False)
    assert_close_fp16(got_c.cpu(), want_c, "stack class, causal mask, padded path")

    class M(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.enc = enc

        def forward(self, a, m):
            return self.enc.forward(a, m)

    sm = torch.jit.script(M())
    buf = io.BytesIO()
    torch.jit.save(sm, buf)
    buf.seek(0)
    sm2 = torch.jit.load(buf)
    assert torch.equal(sm(xd, md), sm2(xd, md))
