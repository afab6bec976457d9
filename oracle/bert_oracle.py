"""CPU oracle: the reference's own fp32 PyTorch encoder, restated as functions.

TEST INFRASTRUCTURE ONLY (checker for tests / smoke / the benchmark's CPU
baseline).  The product path never imports this module.

Parity status: PINNED.  `tests/golden/*.npz` hold inputs and outputs produced
by executing the reference's script
`unit_test/python_scripts/bert_transformer_test.py` itself on CPU (see
`tests/golden/make_golden.py`); `tests/test_oracle_golden.py` checks this
restatement against them in fp32 (max-abs <= 1e-5: the same torch calls in
the same order, so in practice identical) and checks the offsets restatement
against an element-by-element definition.  The optional `attention_bias` term
is NOT pinned that way: the reference's PyTorch encoder has no such term, it
is restated from the reference's unfused softmax kernel only.

What follows what (paths are relative to the reference project root):

* `encoder_layer` / `encoder_stack`  — layer math of
  `unit_test/python_scripts/bert_transformer_test.py:120-158`.
* `lengths_to_mask` / `build_attr_mask` — `bert_transformer_test.py:41-47,114`.
* `mask_output`                       — `bert_transformer_test.py:205-206`.
* `build_offsets`                     — `bytetransformer/include/remove_padding.h:36-86`
  (sequence length = number of entries >= 0.5 in mask row 0, exclusive scan,
  token -> padded-row map).
* `pack_rows` / `restore_rows`        — `remove_padding.h:104-121` and the
  zero-filling scatter of `bytetransformer/include/layernorm.h:334-373`.
* `gelu`  — erf form is what the reference's PyTorch encoder uses
  (`bert_transformer_test.py:151`); tanh form is what its CUDA kernels use
  (`bytetransformer/include/gemm_bias_act.h:78-96`).
* LayerNorm eps: the reference's PyTorch encoder uses the `F.layer_norm`
  default 1e-5; its CUDA kernels use 1e-6 (`layernorm.h:133`).  Both are
  parameters here.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, List, Sequence

import numpy as np
import torch
import torch.nn.functional as F

WEIGHT_NAMES = (
    "qkv_kernel", "qkv_bias",
    "attr_output_kernel", "attr_output_bias",
    "attr_output_layernorm_gamma", "attr_output_layernorm_beta",
    "inter_kernel", "inter_bias",
    "output_kernel", "output_bias",
    "output_layernorm_gamma", "output_layernorm_beta",
)


# --------------------------------------------------------------------------- offsets
def build_offsets(attr_mask: np.ndarray):
    """mask [B,S,S] -> (batch_idx int32[B+1], word_idx int32[T]).

    remove_padding.h:49-56: the length of sequence b is the COUNT of entries of
    mask row 0 (mask[b,0,:]) that are >= 0.5 — not the position of the first
    zero.  remove_padding.h:58-75: exclusive prefix sum.  remove_padding.h:81-85:
    word_idx[offset_b + i] = b*S + i for i < len_b (right padding is assumed).
    """
    m = np.asarray(attr_mask)
    B, S = m.shape[0], m.shape[1]
    lens = (m[:, 0, :].astype(np.float32) >= 0.5).sum(axis=1).astype(np.int32)
    batch_idx = np.zeros(B + 1, dtype=np.int32)
    np.cumsum(lens, out=batch_idx[1:])
    word_idx = np.concatenate(
        [np.arange(l, dtype=np.int32) + np.int32(b * S) for b, l in enumerate(lens)]
        + [np.zeros(0, dtype=np.int32)]
    ).astype(np.int32)
    return batch_idx, word_idx


def pack_rows(x_padded: np.ndarray, word_idx: np.ndarray) -> np.ndarray:
    """[B,S,H] -> [T,H]; remove_padding.h:104-121."""
    B, S, H = x_padded.shape
    return x_padded.reshape(B * S, H)[word_idx]


def restore_rows(x_packed: np.ndarray, batch_idx: np.ndarray, B: int, S: int) -> np.ndarray:
    """[T,H] -> [B,S,H] with exact zeros in padding rows; layernorm.h:345-358."""
    H = x_packed.shape[1]
    out = np.zeros((B, S, H), dtype=x_packed.dtype)
    for b in range(B):
        lo, hi = int(batch_idx[b]), int(batch_idx[b + 1])
        out[b, : hi - lo] = x_packed[lo:hi]
    return out


# --------------------------------------------------------------------------- masks
def lengths_to_mask(lengths: torch.Tensor, max_len: int) -> torch.Tensor:
    """bert_transformer_test.py:41-47 (bool [B,S])."""
    return torch.arange(max_len).unsqueeze(0).lt(lengths.to(torch.int64).unsqueeze(1))


def build_attr_mask(lengths: torch.Tensor, max_len: int, dtype=torch.float32) -> torch.Tensor:
    """bert_transformer_test.py:114: every query row of sequence b carries the
    same key mask (arange(S) < len_b).  Returns [B,S,S]."""
    m = lengths_to_mask(lengths, max_len)
    return m.unsqueeze(1).expand(-1, max_len, -1).contiguous().to(dtype)


def mask_output(out: torch.Tensor, lengths: torch.Tensor) -> torch.Tensor:
    """bert_transformer_test.py:205-206: zero the padding rows before comparing."""
    S = out.shape[1]
    return out * lengths_to_mask(lengths, S).unsqueeze(-1).to(out.dtype)


# --------------------------------------------------------------------------- layer math
def gelu(x: torch.Tensor, kind: str = "erf") -> torch.Tensor:
    if kind == "erf":
        return F.gelu(x)
    if kind == "tanh":
        return F.gelu(x, approximate="tanh")
    raise ValueError(kind)


def encoder_layer(x: torch.Tensor, attr_mask: torch.Tensor, w: Sequence[torch.Tensor],
                  head_num: int, head_size: int, *, ln_eps: float = 1e-5,
                  gelu_kind: str = "erf", tao: float = 1.0,
                  attention_bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One post-LN BERT encoder layer, bert_transformer_test.py:120-158.

    x [B,S,H], attr_mask [B,S,S] (1 attend / 0 masked), w = the 12 tensors in
    WEIGHT_NAMES order with GEMM weights stored [in,out].  `tao` is the softmax
    temperature of bytetransformer/include/attention.h:33-39 (scores / tao).
    `attention_bias` [head_num,S,S] is added to the scaled scores where the reference's
    unfused softmax adds it (bytetransformer/include/softmax.h:41-45); its PyTorch
    encoder has no such term.
    """
    (qkv_k, qkv_b, ao_k, ao_b, ln1_g, ln1_b, in_k, in_b, out_k, out_b, ln2_g, ln2_b) = w
    B, S, H = x.shape
    inp = x
    qkv = torch.matmul(x, qkv_k) + qkv_b
    q, k, v = qkv.chunk(3, dim=-1)

    def split(t):
        return t.view(B, S, head_num, head_size).permute(0, 2, 1, 3)

    q, k, v = split(q), split(k), split(v)
    scores = torch.matmul(q, k.transpose(-2, -1)) / (head_size ** 0.5) / tao
    if attention_bias is not None:
        scores = scores + attention_bias.unsqueeze(0)
    scores = scores - 10000.0 * (1.0 - attr_mask.unsqueeze(1))
    probs = F.softmax(scores, dim=-1)
    h = torch.matmul(probs, v).permute(0, 2, 1, 3).contiguous().view(B, S, H)
    h = torch.matmul(h, ao_k) + ao_b
    h = h + inp
    h = F.layer_norm(h, (H,), weight=ln1_g.to(h.dtype), bias=ln1_b.to(h.dtype), eps=ln_eps)
    res = h
    h = torch.matmul(h, in_k) + in_b
    h = gelu(h, gelu_kind)
    h = torch.matmul(h, out_k) + out_b
    h = h + res
    h = F.layer_norm(h, (H,), weight=ln2_g.to(h.dtype), bias=ln2_b.to(h.dtype), eps=ln_eps)
    return h


def encoder_stack(x, attr_mask, layers: Sequence[Sequence[torch.Tensor]], head_num, head_size,
                  **kw) -> List[torch.Tensor]:
    """The reference's `for layer in range(n_layers)` loop; returns every layer's output."""
    outs = []
    h = x
    for w in layers:
        h = encoder_layer(h, attr_mask, w, head_num, head_size, **kw)
        outs.append(h)
    return outs


def encoder_stack_packed(x_packed: torch.Tensor, cu_seqlens: Sequence[int],
                         layers, head_num, head_size, **kw) -> torch.Tensor:
    """Same math on a packed [T,H] batch: each sequence is run on its own
    (no padding, no mask needed).  Equivalent to the padded stack on valid rows
    because attention never crosses sequences."""
    outs = []
    for b in range(len(cu_seqlens) - 1):
        lo, hi = int(cu_seqlens[b]), int(cu_seqlens[b + 1])
        if hi == lo:
            continue
        xb = x_packed[lo:hi].unsqueeze(0)
        mb = torch.ones(1, hi - lo, hi - lo, dtype=xb.dtype)
        outs.append(encoder_stack(xb, mb, layers, head_num, head_size, **kw)[-1][0])
    if not outs:
        return x_packed.new_zeros((0, x_packed.shape[1]))
    return torch.cat(outs, dim=0)


# --------------------------------------------------------------------------- per-kernel restatements
def add_bias_gelu(x: torch.Tensor, bias: torch.Tensor, kind: str = "erf") -> torch.Tensor:
    """bytetransformer/src/gemm_bias_act.cu:32-66 (add_bias_gelu)."""
    return gelu(x + bias, kind)


def add_bias_residual_layernorm(x, bias, residual, gamma, beta, eps=1e-6):
    """bytetransformer/include/layernorm.h:273-296: LN(x + residual + bias)*gamma + beta."""
    H = x.shape[-1]
    return F.layer_norm(x + bias + residual, (H,), weight=gamma.to(x.dtype), bias=beta.to(x.dtype), eps=eps)


def masked_softmax(scores: torch.Tensor, attr_mask: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """bytetransformer/include/softmax.h:25-62: softmax(scale*scores + (1-mask)*-10000)
    with `1/(sum + 1e-6)` normalisation.  scores [nh,B,S,S] (softmax.h:33), attr_mask [B,S,S]."""
    s = scores * scale + (1.0 - attr_mask.unsqueeze(0)) * (-10000.0)
    m = s.max(dim=-1, keepdim=True).values
    e = torch.exp(s - m)
    return e / (e.sum(dim=-1, keepdim=True) + 1e-6)


def attention_packed(qkv: torch.Tensor, cu_seqlens, head_num, head_size, tao: float = 1.0):
    """Fused MHA on a packed [T,3H] QKV buffer (bias already added): for each
    sequence and head softmax(QK^T/sqrt(d)/tao) V over its own valid tokens.
    Semantics of bytetransformer/src/attention_fused.cu:295-414."""
    T, H3 = qkv.shape
    H = H3 // 3
    out = torch.zeros(T, H, dtype=qkv.dtype)
    for b in range(len(cu_seqlens) - 1):
        lo, hi = int(cu_seqlens[b]), int(cu_seqlens[b + 1])
        if hi == lo:
            continue
        L = hi - lo
        q, k, v = qkv[lo:hi].chunk(3, dim=-1)
        q = q.view(L, head_num, head_size).permute(1, 0, 2)
        k = k.view(L, head_num, head_size).permute(1, 0, 2)
        v = v.view(L, head_num, head_size).permute(1, 0, 2)
        p = F.softmax(torch.matmul(q, k.transpose(-2, -1)) / math.sqrt(head_size) / tao, dim=-1)
        out[lo:hi] = torch.matmul(p, v).permute(1, 0, 2).reshape(L, H)
    return out


def embedding_layernorm(word_emb, pos_emb, type_emb, gamma, beta, token_ids, type_ids=None, position_ids=None,
                        eps: float = 1e-6) -> torch.Tensor:
    """LayerNorm(word[token] + pos[position] + type[type]) in fp32: the standard BERT embedding block.
    The reference has no such step (only unused id fields, bytetransformer/include/bert_transformer.h:93-95),
    so this function is a definition, not a restatement: parity unpinned."""
    B, S = token_ids.shape
    if position_ids is None:
        position_ids = torch.arange(S).unsqueeze(0).expand(B, S)
    if type_ids is None:
        type_ids = torch.zeros(B, S, dtype=torch.long)
    x = word_emb.float()[token_ids.long()] + pos_emb.float()[position_ids.long()] + type_emb.float()[type_ids.long()]
    return F.layer_norm(x, (x.shape[-1],), gamma.float(), beta.float(), eps)


def pooler(encoder_out, W, bias) -> torch.Tensor:
    """tanh(first token @ W + bias), the standard BERT pooler (a definition, as above)."""
    return torch.tanh(encoder_out[:, 0, :].float() @ W.float() + bias.float())
