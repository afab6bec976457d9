"""Python host side over the C ABI: torch tensors supply device memory and
streams, every computation goes through libbt_b200.so.

`bert_transformer(...)` mirrors the reference's functional operator
`torch.ops.ByteTransformer.BertTransformer` (bytetransformer/th_op/ths_op_f.cc:28-95):
same argument order, names, defaults and error behaviour (RuntimeError on bad
input).  `Encoder` is the reusable object form (the reference's C++
`BertTransformer<HALF>` used through bytetransformer/th_op/bert_transformer_ext.h:40-118)
extended to a stack of layers.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence

import torch

from . import _abi

WEIGHT_NAMES = (
    "qkv_kernel", "qkv_bias", "attr_output_kernel", "attr_output_bias",
    "attr_output_layernorm_gamma", "attr_output_layernorm_beta", "inter_kernel", "inter_bias",
    "output_kernel", "output_bias", "output_layernorm_gamma", "output_layernorm_beta")
_LOOSE = {4, 5, 10, 11}  # LayerNorm gamma/beta: dtype not checked by the reference (CHECK_INPUT_LOOSE)


def _stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _check(t: torch.Tensor, name: str, dtype=None):
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise RuntimeError(f"Inconsistency of Tensor type: {name}")


class Encoder:
    """A stack of BERT encoder layers bound to one CUDA device."""

    def __init__(self, head_num: int, head_size: int, layers: Sequence[Sequence[torch.Tensor]], *,
                 max_batch_size: int = 65535, max_seq_len: int = 1024, ln_eps: float = 1e-6,
                 gelu: str = "erf", tao: float = 1.0):
        if not layers:
            raise RuntimeError("at least one layer of weights is required")
        self._lib = _abi.load()
        self.head_num, self.head_size = int(head_num), int(head_size)
        self.hidden = self.head_num * self.head_size
        first = layers[0]
        if len(first) != 12:
            raise RuntimeError("each layer needs 12 weight tensors")
        self.device = first[0].device
        if first[0].dtype != torch.float16:
            raise RuntimeError("only fp16 weights are supported (the fp32 template of the reference "
                               "is not built for sm_100a)")
        gb_fp32 = first[10].dtype == torch.float32  # bert_transformer_ext.h:60-63
        self._layers = []  # keeps the tensors alive: the library stores raw pointers only
        cfg = _abi.bt_config(self.head_num, self.head_size, int(max_batch_size), int(max_seq_len), 4,
                             float(ln_eps), _abi.BT_GELU_ERF if gelu == "erf" else _abi.BT_GELU_TANH,
                             float(tao), int(gb_fp32), self.device.index if self.device.index is not None else -1)
        if gelu not in ("erf", "tanh"):
            raise RuntimeError("gelu must be 'erf' or 'tanh'")
        h = C.c_void_p()
        rc = self._lib.bt_create(C.byref(cfg), C.byref(h))
        if rc != _abi.BT_OK:
            raise _abi.BtError(rc, "bt_create",
                               "head_size must be 64 and the device must be compute capability 10.x")
        self._h = h
        H = self.hidden
        shapes = [(H, 3 * H), (3 * H,), (H, H), (H,), (H,), (H,), (H, 4 * H), (4 * H,), (4 * H, H), (H,), (H,), (H,)]
        for li, w in enumerate(layers):
            if len(w) != 12:
                raise RuntimeError("each layer needs 12 weight tensors")
            for i, t in enumerate(w):
                _check(t, WEIGHT_NAMES[i], None if i in _LOOSE else torch.float16)
                if tuple(t.shape) != shapes[i]:
                    raise RuntimeError(f"{WEIGHT_NAMES[i]} has shape {tuple(t.shape)}, expected {shapes[i]}")
                if i in _LOOSE and t.dtype != (torch.float32 if gb_fp32 else torch.float16):
                    raise RuntimeError("LayerNorm gamma/beta must all be fp16 or all be fp32")
            lw = _abi.bt_layer_weights(*[t.data_ptr() for t in w])
            self._call("bt_set_layer_weights", self._h, li, C.byref(lw))
            self._layers.append(list(w))
        self.n_layers = len(self._layers)
        self._ws: Optional[torch.Tensor] = None

    # ------------------------------------------------------------------ helpers
    def _call(self, name, *args):
        rc = getattr(self._lib, name)(*args)
        if rc != _abi.BT_OK:
            raise _abi.BtError(rc, name, self._lib.bt_last_error(self._h).decode())
        return rc

    def close(self):
        if getattr(self, "_h", None):
            self._lib.bt_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _workspace(self, nbytes: int) -> torch.Tensor:
        if self._ws is None or self._ws.numel() < nbytes:
            self._ws = torch.empty(nbytes, dtype=torch.int8, device=self.device)
        return self._ws

    def device_status(self) -> int:
        st = C.c_int(0)
        self._call("bt_device_status", self._h, _stream_ptr(self.device), C.byref(st))
        return st.value

    def selftest_bounded_wait(self, max_cycles: int, gave_up: torch.Tensor | None = None):
        """Enqueue the library's failure-path self-test: a wait that nothing satisfies gives up after
        about `max_cycles` SM cycles and leaves BT_STATUS_SELFTEST_TIMEOUT in the status word."""
        if gave_up is not None:
            _check(gave_up, "gave_up", torch.int32)
        self._call("bt_selftest_bounded_wait", self._h, int(max_cycles),
                   gave_up.data_ptr() if gave_up is not None else None, _stream_ptr(self.device))

    def profile_enable(self, on: bool = True):
        self._call("bt_profile_enable", self._h, int(bool(on)))

    def profile_read(self):
        """{kind: (milliseconds, launches)} since the last profile_enable(True)."""
        n = len(_abi.PROF_KINDS)
        ms = (C.c_double * n)()
        cnt = (C.c_longlong * n)()
        self._call("bt_profile_read", self._h, ms, cnt)
        return {k: (ms[i], cnt[i]) for i, k in enumerate(_abi.PROF_KINDS)}

    # ----------------------------------------------------------------- forwards
    def _check_io(self, x, attr_mask):
        _check(x, "input", torch.float16)
        _check(attr_mask, "attr_mask", torch.float16)
        if x.dim() != 3 or x.shape[2] != self.hidden:
            raise RuntimeError("input must be [batch, seq_len, head_num*head_size]")
        B, S = int(x.shape[0]), int(x.shape[1])
        if S > 1024:
            raise RuntimeError("Input seq_len too long")  # th_op/util.h:40
        if tuple(attr_mask.shape) != (B, S, S):
            raise RuntimeError("attr_mask must be [batch, seq_len, seq_len]")
        return B, S

    def forward_layer(self, layer: int, x: torch.Tensor, attr_mask: torch.Tensor) -> torch.Tensor:
        """One layer, padded in / padded out, padding rows zero (the reference op)."""
        B, S = self._check_io(x, attr_mask)
        with torch.cuda.device(self.device):
            out = torch.empty_like(x)
            n = C.c_size_t()
            self._call("bt_workspace_bytes", self._h, B, S, C.byref(n))
            ws = self._workspace(n.value)
            self._call("bt_layer_forward_padded", self._h, int(layer), x.data_ptr(), attr_mask.data_ptr(),
                       out.data_ptr(), ws.data_ptr(), ws.numel(), B, S, _stream_ptr(self.device))
        return out

    def forward(self, x: torch.Tensor, attr_mask: torch.Tensor, n_layers: Optional[int] = None) -> torch.Tensor:
        """All layers in one call: pack once, run the stack packed, scatter once."""
        B, S = self._check_io(x, attr_mask)
        nl = self.n_layers if n_layers is None else int(n_layers)
        with torch.cuda.device(self.device):
            out = torch.empty_like(x)
            n = C.c_size_t()
            self._call("bt_workspace_bytes", self._h, B, S, C.byref(n))
            ws = self._workspace(n.value)
            self._call("bt_stack_forward_padded", self._h, nl, x.data_ptr(), attr_mask.data_ptr(), out.data_ptr(),
                       ws.data_ptr(), ws.numel(), B, S, _stream_ptr(self.device))
        return out

    def forward_ids(self, emb: "EmbeddingWeights", token_ids: torch.Tensor, attr_mask: torch.Tensor,
                    type_ids: Optional[torch.Tensor] = None, position_ids: Optional[torch.Tensor] = None,
                    n_layers: Optional[int] = None) -> torch.Tensor:
        """The whole model front to back: embeddings of the valid tokens straight into the packed
        activation, all layers, scatter once (the padded input tensor never exists)."""
        _check(token_ids, "token_ids", torch.int32)
        _check(attr_mask, "attr_mask", torch.float16)
        if token_ids.dim() != 2 or attr_mask.dim() != 3:
            raise RuntimeError("token_ids must be [batch, seq_len], attr_mask [batch, seq_len, seq_len]")
        B, S = int(token_ids.shape[0]), int(token_ids.shape[1])
        if tuple(attr_mask.shape) != (B, S, S):
            raise RuntimeError("attr_mask must be [batch, seq_len, seq_len]")
        for t, n in ((type_ids, "type_ids"), (position_ids, "position_ids")):
            if t is not None:
                _check(t, n, torch.int32)
                if tuple(t.shape) != (B, S):
                    raise RuntimeError(f"{n} must be [batch, seq_len]")
        nl = self.n_layers if n_layers is None else int(n_layers)
        with torch.cuda.device(self.device):
            out = torch.empty(B, S, self.hidden, dtype=torch.float16, device=self.device)
            n = C.c_size_t()
            self._call("bt_workspace_bytes", self._h, B, S, C.byref(n))
            ws = self._workspace(n.value)
            w = emb.as_struct()
            self._call("bt_stack_forward_ids", self._h, nl, C.byref(w), token_ids.data_ptr(),
                       type_ids.data_ptr() if type_ids is not None else None,
                       position_ids.data_ptr() if position_ids is not None else None, attr_mask.data_ptr(),
                       out.data_ptr(), ws.data_ptr(), ws.numel(), B, S, _stream_ptr(self.device))
        return out

    def forward_general(self, x: torch.Tensor, attr_mask: torch.Tensor, attention_bias: Optional[torch.Tensor] = None,
                        n_layers: Optional[int] = None) -> torch.Tensor:
        """All layers with the reference's padded-path attention semantics: nothing is packed, the whole
        [B,S,S] mask is applied element by element as (1 - mask) * -10000 and `attention_bias`
        ([head_num,S,S] fp16, optional) is added to the scaled scores; every output row is computed."""
        B, S = self._check_io(x, attr_mask)
        if attention_bias is not None:
            _check(attention_bias, "attention_bias", torch.float16)
            if tuple(attention_bias.shape) != (self.head_num, S, S):
                raise RuntimeError("attention_bias must be [head_num, seq_len, seq_len]")
        nl = self.n_layers if n_layers is None else int(n_layers)
        with torch.cuda.device(self.device):
            out = torch.empty_like(x)
            n = C.c_size_t()
            self._call("bt_workspace_bytes", self._h, B, S, C.byref(n))
            ws = self._workspace(n.value)
            self._call("bt_stack_forward_padded_general", self._h, nl, x.data_ptr(), attr_mask.data_ptr(),
                       attention_bias.data_ptr() if attention_bias is not None else None, out.data_ptr(),
                       ws.data_ptr(), ws.numel(), B, S, _stream_ptr(self.device))
        return out

    def packed_workspace_bytes(self, batch: int, total_tokens: int) -> int:
        n = C.c_size_t()
        self._call("bt_workspace_bytes_packed", self._h, int(batch), int(total_tokens), C.byref(n))
        return n.value

    def forward_packed(self, x_packed: torch.Tensor, cu_seqlens: torch.Tensor, max_len: int,
                       out: Optional[torch.Tensor] = None, workspace: Optional[torch.Tensor] = None,
                       n_layers: Optional[int] = None) -> torch.Tensor:
        """Packed in / packed out: x_packed [T,H] fp16, cu_seqlens int32 [B+1] on the device."""
        _check(x_packed, "x_packed", torch.float16)
        _check(cu_seqlens, "cu_seqlens", torch.int32)
        if x_packed.dim() != 2 or x_packed.shape[1] != self.hidden:
            raise RuntimeError("x_packed must be [total_tokens, head_num*head_size]")
        T = int(x_packed.shape[0])
        B = int(cu_seqlens.numel()) - 1
        nl = self.n_layers if n_layers is None else int(n_layers)
        with torch.cuda.device(self.device):
            if out is None:
                out = torch.empty_like(x_packed)
            ws = workspace if workspace is not None else self._workspace(self.packed_workspace_bytes(B, T))
            self._call("bt_stack_forward_packed", self._h, nl, x_packed.data_ptr(), cu_seqlens.data_ptr(), B,
                       int(max_len), T, out.data_ptr(), ws.data_ptr(), ws.numel(), _stream_ptr(self.device))
        return out

    # -------------------------------------------------------- single steps (tests, tools)
    def gemm(self, a: torch.Tensor, w: torch.Tensor, bias=None, residual=None, *, epilogue=_abi.BT_EPI_NONE,
             gelu=_abi.BT_GELU_ERF, m_dev: Optional[torch.Tensor] = None) -> torch.Tensor:
        _check(a, "a", torch.float16)
        _check(w, "w", torch.float16)
        M, K = a.shape
        N = w.shape[1]
        odt = torch.float32 if epilogue == _abi.BT_EPI_BIAS_RESIDUAL_F32OUT else torch.float16
        out = torch.zeros(M, N, dtype=odt, device=a.device)
        self._call("bt_gemm", self._h, a.data_ptr(), w.data_ptr(), out.data_ptr(),
                   bias.data_ptr() if bias is not None else None,
                   residual.data_ptr() if residual is not None else None,
                   m_dev.data_ptr() if m_dev is not None else None, int(M), int(N), int(K), int(epilogue), int(gelu),
                   _stream_ptr(a.device))
        return out

    def gemm_layernorm(self, a, w, bias, residual, gamma, beta, eps=1e-6, m_dev=None) -> torch.Tensor:
        """LayerNorm(a @ w + bias + residual) * gamma + beta in one kernel (bt_gemm_layernorm)."""
        M, K = a.shape
        N = w.shape[1]
        scratch = torch.empty(M, N, dtype=torch.float32, device=a.device)
        out = torch.zeros(M, N, dtype=torch.float16, device=a.device)
        self._call("bt_gemm_layernorm", self._h, a.data_ptr(), w.data_ptr(), bias.data_ptr(), residual.data_ptr(),
                   gamma.data_ptr(), beta.data_ptr(), int(gamma.dtype == torch.float32), float(eps),
                   scratch.data_ptr(), out.data_ptr(), m_dev.data_ptr() if m_dev is not None else None,
                   int(M), int(N), int(K), _stream_ptr(a.device))
        return out

    def attention(self, qkv: torch.Tensor, cu_seqlens: torch.Tensor, max_len: int) -> torch.Tensor:
        _check(qkv, "qkv", torch.float16)
        _check(cu_seqlens, "cu_seqlens", torch.int32)
        rows = int(qkv.shape[0])
        ctx = torch.zeros(rows, self.hidden, dtype=torch.float16, device=qkv.device)
        self._call("bt_attention", self._h, qkv.data_ptr(), ctx.data_ptr(), cu_seqlens.data_ptr(),
                   int(cu_seqlens.numel()) - 1, int(max_len), rows, _stream_ptr(qkv.device))
        return ctx


# ---------------------------------------------------------------------------------------------
# free functions over the stateless entry points
def embedding_layernorm(word_emb: torch.Tensor, pos_emb: torch.Tensor, type_emb: torch.Tensor, gamma: torch.Tensor,
                        beta: torch.Tensor, token_ids: torch.Tensor, type_ids: Optional[torch.Tensor] = None,
                        position_ids: Optional[torch.Tensor] = None, eps: float = 1e-6) -> torch.Tensor:
    """Encoder input [B,S,H] = LayerNorm(word[token] + position + type) (the step before the stack)."""
    for t, n in ((word_emb, "word_emb"), (pos_emb, "pos_emb"), (type_emb, "type_emb")):
        _check(t, n, torch.float16)
    _check(token_ids, "token_ids", torch.int32)
    if token_ids.dim() != 2:
        raise RuntimeError("token_ids must be [batch, seq_len]")
    gb32 = gamma.dtype == torch.float32
    _check(gamma, "gamma", torch.float32 if gb32 else torch.float16)
    _check(beta, "beta", gamma.dtype)
    B, S = int(token_ids.shape[0]), int(token_ids.shape[1])
    H = int(word_emb.shape[1])
    for t, n in ((type_ids, "type_ids"), (position_ids, "position_ids")):
        if t is not None:
            _check(t, n, torch.int32)
            if tuple(t.shape) != (B, S):
                raise RuntimeError(f"{n} must be [batch, seq_len]")
    lib = _abi.load()
    with torch.cuda.device(word_emb.device):
        out = torch.empty(B, S, H, dtype=torch.float16, device=word_emb.device)
        rc = lib.bt_embedding_layernorm(word_emb.data_ptr(), pos_emb.data_ptr(), type_emb.data_ptr(), gamma.data_ptr(),
                                        beta.data_ptr(), int(gb32), token_ids.data_ptr(),
                                        type_ids.data_ptr() if type_ids is not None else None,
                                        position_ids.data_ptr() if position_ids is not None else None, out.data_ptr(),
                                        B, S, H, int(word_emb.shape[0]), int(pos_emb.shape[0]), int(type_emb.shape[0]),
                                        float(eps), _stream_ptr(word_emb.device))
    if rc != 0:
        raise _abi.BtError(rc, "bt_embedding_layernorm")
    return out


class EmbeddingWeights:
    """Tables and LayerNorm parameters of the embedding front end (fp16 tables, gamma/beta fp16 or fp32)."""

    def __init__(self, word_emb, pos_emb, type_emb, gamma, beta, eps: float = 1e-6):
        for t, n in ((word_emb, "word_emb"), (pos_emb, "pos_emb"), (type_emb, "type_emb")):
            _check(t, n, torch.float16)
        self.gb32 = gamma.dtype == torch.float32
        _check(gamma, "gamma", torch.float32 if self.gb32 else torch.float16)
        _check(beta, "beta", torch.float32 if self.gb32 else torch.float16)
        self.tensors = (word_emb, pos_emb, type_emb, gamma, beta)   # keeps the device memory alive
        self.eps = float(eps)

    def as_struct(self) -> "_abi.bt_embedding_weights":
        w, p, t, g, b = self.tensors
        return _abi.bt_embedding_weights(w.data_ptr(), p.data_ptr(), t.data_ptr(), g.data_ptr(), b.data_ptr(),
                                         1 if self.gb32 else 0, int(w.shape[0]), int(p.shape[0]), int(t.shape[0]), self.eps)


def embedding_layernorm_packed(emb: EmbeddingWeights, token_ids: torch.Tensor, batch_idx: torch.Tensor,
                               word_idx: torch.Tensor, type_ids: Optional[torch.Tensor] = None,
                               position_ids: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Embedding + LayerNorm of the valid tokens only, packed: row r of the result is the token at padded
    position word_idx[r] (offsets from build_offsets); rows from the token count on stay zero."""
    _check(token_ids, "token_ids", torch.int32)
    _check(batch_idx, "batch_idx", torch.int32)
    _check(word_idx, "word_idx", torch.int32)
    B, S = int(token_ids.shape[0]), int(token_ids.shape[1])
    H = int(emb.tensors[0].shape[1])
    out = torch.zeros(B * S, H, dtype=torch.float16, device=token_ids.device)
    w = emb.as_struct()
    rc = _abi.load().bt_embedding_layernorm_packed(
        C.byref(w), token_ids.data_ptr(), type_ids.data_ptr() if type_ids is not None else None,
        position_ids.data_ptr() if position_ids is not None else None, batch_idx.data_ptr(), word_idx.data_ptr(),
        out.data_ptr(), B, S, H, _stream_ptr(token_ids.device))
    if rc != _abi.BT_OK:
        raise RuntimeError(f"bt_embedding_layernorm_packed failed ({_abi.ERROR_NAMES.get(rc, rc)})")
    return out


def pooler(encoder_out: torch.Tensor, W: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """pooled [B,H] = tanh(encoder_out[:,0,:] @ W + bias) (the step after the stack)."""
    _check(encoder_out, "encoder_out", torch.float16)
    _check(W, "W", torch.float16)
    _check(bias, "bias", torch.float16)
    B, S, H = (int(v) for v in encoder_out.shape)
    if tuple(W.shape) != (H, H) or tuple(bias.shape) != (H,):
        raise RuntimeError("W must be [hidden, hidden] and bias [hidden]")
    lib = _abi.load()
    with torch.cuda.device(encoder_out.device):
        out = torch.empty(B, H, dtype=torch.float16, device=encoder_out.device)
        rc = lib.bt_pooler(encoder_out.data_ptr(), W.data_ptr(), bias.data_ptr(), out.data_ptr(), B, S, H,
                           _stream_ptr(encoder_out.device))
    if rc != 0:
        raise _abi.BtError(rc, "bt_pooler")
    return out


def mask_is_right_padded(attr_mask: torch.Tensor) -> bool:
    """True when the packed entry points would honour `attr_mask` [B,S,S] (they look at row 0 only, as the
    reference's prefix-sum kernel does); otherwise use Encoder.forward_general.  Synchronises the stream."""
    _check(attr_mask, "attr_mask", torch.float16)
    if attr_mask.dim() != 3 or attr_mask.shape[1] != attr_mask.shape[2]:
        raise RuntimeError("attr_mask must be [batch, seq_len, seq_len]")
    lib = _abi.load()
    with torch.cuda.device(attr_mask.device):
        scratch = torch.empty(1, dtype=torch.int32, device=attr_mask.device)
        res = C.c_int(0)
        rc = lib.bt_mask_is_right_padded(attr_mask.data_ptr(), int(attr_mask.shape[0]), int(attr_mask.shape[1]),
                                         scratch.data_ptr(), C.byref(res), _stream_ptr(attr_mask.device))
    if rc != 0:
        raise _abi.BtError(rc, "bt_mask_is_right_padded")
    return bool(res.value)


def build_offsets(attr_mask: torch.Tensor):
    """(batch_idx int32[B+1], word_idx int32[B*S]) on the device; only the first
    batch_idx[B] entries of word_idx are defined."""
    lib = _abi.load()
    _check(attr_mask, "attr_mask", torch.float16)
    B, S = int(attr_mask.shape[0]), int(attr_mask.shape[1])
    batch_idx = torch.empty(B + 1, dtype=torch.int32, device=attr_mask.device)
    word_idx = torch.full((B * S,), -1, dtype=torch.int32, device=attr_mask.device)
    rc = lib.bt_build_offsets(attr_mask.data_ptr(), B, S, batch_idx.data_ptr(), word_idx.data_ptr(),
                              _stream_ptr(attr_mask.device))
    if rc != _abi.BT_OK:
        raise _abi.BtError(rc, "bt_build_offsets")
    return batch_idx, word_idx


def pack_rows(x_padded: torch.Tensor, batch_idx: torch.Tensor, out: Optional[torch.Tensor] = None):
    lib = _abi.load()
    B, S, H = x_padded.shape
    if out is None:
        out = torch.zeros(B * S, H, dtype=torch.float16, device=x_padded.device)
    rc = lib.bt_pack_rows(x_padded.data_ptr(), out.data_ptr(), batch_idx.data_ptr(), None, B, S, H,
                          _stream_ptr(x_padded.device))
    if rc != _abi.BT_OK:
        raise _abi.BtError(rc, "bt_pack_rows")
    return out


def restore_rows(x_packed: torch.Tensor, batch_idx: torch.Tensor, B: int, S: int):
    lib = _abi.load()
    H = x_packed.shape[1]
    out = torch.full((B, S, H), float("nan"), dtype=torch.float16, device=x_packed.device)
    rc = lib.bt_restore_rows(x_packed.data_ptr(), out.data_ptr(), batch_idx.data_ptr(), B, S, H,
                             _stream_ptr(x_packed.device))
    if rc != _abi.BT_OK:
        raise _abi.BtError(rc, "bt_restore_rows")
    return out


def add_bias_residual_layernorm(x, bias, residual, gamma, beta, eps=1e-6, m_dev=None):
    lib = _abi.load()
    M, H = x.shape
    out = torch.zeros(M, H, dtype=torch.float16, device=x.device)
    rc = lib.bt_add_bias_residual_layernorm(
        x.data_ptr(), int(x.dtype == torch.float32), bias.data_ptr() if bias is not None else None,
        residual.data_ptr() if residual is not None else None, gamma.data_ptr(), beta.data_ptr(),
        int(gamma.dtype == torch.float32), out.data_ptr(), m_dev.data_ptr() if m_dev is not None else None,
        M, H, float(eps), _stream_ptr(x.device))
    if rc != _abi.BT_OK:
        raise _abi.BtError(rc, "bt_add_bias_residual_layernorm")
    return out


def add_bias_residual_layernorm_restore(x, bias, residual, gamma, beta, batch_idx, B, S, eps=1e-6):
    lib = _abi.load()
    H = x.shape[1]
    out = torch.full((B, S, H), float("nan"), dtype=torch.float16, device=x.device)
    rc = lib.bt_add_bias_residual_layernorm_restore(
        x.data_ptr(), int(x.dtype == torch.float32), bias.data_ptr() if bias is not None else None,
        residual.data_ptr() if residual is not None else None, gamma.data_ptr(), beta.data_ptr(),
        int(gamma.dtype == torch.float32), out.data_ptr(), batch_idx.data_ptr(), B, S, H, float(eps),
        _stream_ptr(x.device))
    if rc != _abi.BT_OK:
        raise _abi.BtError(rc, "bt_add_bias_residual_layernorm_restore")
    return out


def add_bias_gelu_(x, bias, gelu="erf"):
    lib = _abi.load()
    M, N = x.shape
    rc = lib.bt_add_bias_gelu(x.data_ptr(), bias.data_ptr(), None, M, N,
                              _abi.BT_GELU_ERF if gelu == "erf" else _abi.BT_GELU_TANH, _stream_ptr(x.device))
    if rc != _abi.BT_OK:
        raise _abi.BtError(rc, "bt_add_bias_gelu")
    return x


def masked_softmax_(logits, attr_mask, scale=1.0):
    """logits [nh,B,S,S] (the reference's layout), in place."""
    lib = _abi.load()
    nh, B, S, _ = logits.shape
    rc = lib.bt_masked_softmax(logits.data_ptr(), attr_mask.data_ptr(), B, nh, S, float(scale),
                               _stream_ptr(logits.device))
    if rc != _abi.BT_OK:
        raise _abi.BtError(rc, "bt_masked_softmax")
    return logits


def bert_transformer(head_num: int, head_size: int,
                     qkv_kernel, qkv_bias, attr_output_kernel, attr_output_bias,
                     attr_output_layernorm_gamma, attr_output_layernorm_beta,
                     inter_kernel, inter_bias, output_kernel, output_bias,
                     output_layernorm_gamma, output_layernorm_beta,
                     input, attr_mask, is_remove_padding: bool = True,
                     use_fused_attention: bool = True, *, ln_eps: float = 1e-6, gelu: str = "erf"):
    """Drop-in for `torch.ops.ByteTransformer.BertTransformer` (ths_op_f.cc:85-95).

    is_remove_padding=True: the packed path (lengths = valid keys of mask row 0, right padding, padding rows
    of the output zero).  False: the reference's padded semantics (nothing packed, the whole [B,S,S] mask
    applied element by element, every output row computed), which is what a causal or block-diagonal mask
    needs.  `use_fused_attention` is accepted for signature compatibility: attention is fused on both paths.
    The encoder object is built per call, as the reference does (bert_transformer_ext.h:86-110)."""
    w = [qkv_kernel, qkv_bias, attr_output_kernel, attr_output_bias, attr_output_layernorm_gamma,
         attr_output_layernorm_beta, inter_kernel, inter_bias, output_kernel, output_bias,
         output_layernorm_gamma, output_layernorm_beta]
    enc = Encoder(head_num, head_size, [w], ln_eps=ln_eps, gelu=gelu)
    try:
        if not is_remove_padding:
            return enc.forward_general(input, attr_mask, n_layers=1)
        return enc.forward_layer(0, input, attr_mask)
    finally:
        enc.close()
