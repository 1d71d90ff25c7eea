"""The kernels of ``csrc/`` as Python functions on torch CUDA tensors.

Each function checks shapes, dtypes and devices, allocates its output with
torch and launches on torch's current stream.  There is no other
implementation behind these names: on a machine without the compiled
libraries (or without nvcc to make them) they raise.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from .csrc import build as _build

F32, BF16 = 0, 1
_P = ctypes.c_void_p
_I = ctypes.c_int
_L = ctypes.c_longlong
_F = ctypes.c_float

_SIGNATURES = {
    ("elementwise", "ri_embed_rows"): [_P, _P, _P, _I, _I, _I, _I, _P, _P],
    ("elementwise", "ri_embed_rows_scaled"): [_P, _P, _P, _I, _I, _I, _F, _I, _I, _P, _P],
    ("elementwise", "ri_activation"): [_P, _P, _L, _I, _I, _P],
    ("elementwise", "ri_embed_rows_same"): [_P, _P, _P, _L, _I, _I, _I, _I, _P, _P],
    ("norm_gains", "ri_norm_gains_post"): [_P] * 6 + [_P, _I, _F] + [_P] * 6 + [_I, _I, _F, _P, _F, _L, _I, _P, _I, _I, _P, _P],
    ("qkv_prep", "ri_qkv_prep_norm"): [_P, _L, _I, _I, _I] + [_P] * 9 + [_I, _I, _I, _I, _F, _P, _P, _I, _F] + [_I] * 10 + [_P, _P],
    ("moe", "ri_moe_route_rule"): [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _F, _I, _I, _P],
    ("gla", "ri_gla_recurrent_scalar"): [_P, _L, _I, _I, _I, _P, _I, _I, _F, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    ("mlstm", "ri_mlstm_gates"): [_P, _L, _I, _I, _P, _P, _F, _P, _P, _P, _P, _I, _I, _I, _I, _P],
    ("mlstm", "ri_mlstm_head_norm_gate"): [_P, _P, _P, _F, _P, _L, _P, _I, _I, _I, _I, _I, _P],
    ("elementwise", "ri_gate_heads"): [_P, _P, _L, _I, _I, _I, _I, _I, _I, _P],
    ("streams", "ri_stream_norm"): [_P] * 8 + [_I, _I, _I, _F, _I, _I, _P],
    ("streams", "ri_stream_norm2"): [_P] * 13 + [_I, _I, _I, _F, _I, _I, _P],
    ("pair_embedding", "ri_embed_pair_hash"): [_P] * 9 + [_I, _I, _I, _I, _I, _L, _L, _I, _I, _P, _P],
    ("delta_rule", "ri_short_conv"): [_P, _L, _I, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    ("delta_rule", "ri_delta_rule_recurrent"): [_P, _I, _I, _I, _I, _P, _L, _I, _P, _P, _P, _F] + [_P] * 6 + [_I] * 8 + [_P],
    ("elementwise", "ri_gated_act"): [_P, _P, _I, _I, _I, _I, _F, _F, _I, _P],
    ("elementwise", "ri_scale_f32"): [_P, _L, _F, _P],
    ("moe", "ri_moe_route"): [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P],
    ("moe", "ri_moe_plan"): [_P, _P, _P, _P, _I, _I, _I, _I, _P],
    ("moe", "ri_moe_grouped_linear"): [_P, _L, _P, _P, _L, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P],
    ("moe", "ri_moe_combine"): [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P],
    ("rope_kv", "ri_qk_norm_rope_append_pairs"): [_P] * 10 + [_F, _P, _I, _I] + [_I] * 10 + [_P, _P],
    ("latent_attention", "ri_latent_prep"): [_P, _L, _I, _I] + [_P] * 8 + [_F, _P] + [_I] * 11 + [_P, _P],
    ("gla", "ri_gla_recurrent"): [_P, _L, _I, _I, _I, _P, _P, _F, _F, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    ("gla", "ri_gla_head_norm_gate"): [_P, _P, _F, _P, _L, _P, _I, _I, _I, _I, _I, _P],
    ("linear_f32", "ri_linear_heads_f32"): [_P, _P, _P, _I, _I, _I, _I, _L, _L, _L, _L, _P],
    ("elementwise", "ri_rmsnorm"): [_P, _P, _P, _P, _P, _I, _I, _F, _I, _I, _P, _I, _I, _P],
    ("elementwise", "ri_add_rows"): [_P, _P, _L, _I, _P],
    ("elementwise", "ri_silu_mul"): [_P, _P, _I, _I, _I, _I, _P],
    ("rope_kv", "ri_qk_norm_rope_append"): [_P] * 10 + [_F, _P, _I, _I] + [_I] * 9 + [_P, _P],
    ("attention_rows", "ri_attention_rows"): [_P] * 8 + [_I] * 8 + [_F, _I, _P, _F, _I, _P, _P],
    ("elementwise", "ri_softcap_f32"): [_P, _L, _F, _P],
    ("norm_gains", "ri_norm_gains"): [_P] * 6 + [_P, _I, _F] + [_P] * 6 + [_I, _I, _F, _I, _P, _I, _I, _P, _P],
    ("qkv_prep", "ri_qkv_prep"): [_P, _L, _I, _I, _I] + [_P] * 9 + [_I, _I, _I, _I, _F] + [_I] * 10 + [_P, _P],
    ("linear_f32", "ri_linear_f32"): [_P, _P, _P, _I, _I, _I, _P],
    ("sampling", "ri_sample"): [_P, _L, _I, _I, _P, _P, _L, _P, _P, _P, _P, _P, _P, _P, _L, _I, _I, _P, _I, _P],
    ("sampling", "ri_sample_work_bytes"): [_I, _I],
    ("sampling", "ri_argmax"): [_P, _L, _I, _I, _P, _P, _P, _P],
    ("sampling", "ri_mark_seen"): [_P, _L, _P, _P, _I, _I, _P],
    ("attention_decode", "ri_attention_decode_sink"): [_P] * 9 + [_I] * 8 + [_F, _I, _P, _P, _P],
    ("attention_decode", "ri_attention_decode_cap"): [_P] * 9 + [_I] * 8 + [_F, _I, _P, _F, _P, _P],
    ("linear_skinny", "ri_linear_skinny"): [_P, _P, _P, _I, _I, _I, _I, _I, _P, _P],
    ("linear_skinny", "ri_linear_skinny_act"): [_P, _P, _P, _I, _I, _I, _I, _I, _I, _P, _P],
    ("linear_skinny", "ri_linear_skinny_gated"): [_P, _P, _P, _I, _I, _I, _I, _P, _P],
    ("linear_skinny", "ri_linear_skinny_gated_with"): [_P, _P, _P, _I, _I, _I, _I, _F, _F, _P, _P],
    ("linear_stream_tc", "ri_linear_stream_tc"): [_P, _P, _P, _I, _I, _I, _I, _I, _P, _P],
    ("linear_stream_tc", "ri_linear_stream_tc_gate"): [_P, _P, _P, _I, _I, _I, _I, _I, _F, _F, _P, _P],
    ("attention_prefill_tc", "ri_attention_prefill_tc"): [_P] * 8 + [_I] * 9 + [_F, _I, _P, _F, _P, _P],
    ("attention_prefill", "ri_attention_prefill"): [_P] * 8 + [_I] * 8 + [_F, _I, _P, _I, _F, _P, _P],
}
DECODE_CHUNK = 128          # keys per partial result of the decode attention kernel
MAX_FAST_HEAD_DIM = 256
TCGEN05_HEAD_DIMS = (64, 128)   # head sizes the tcgen05 prefill attention kernel is built for
_NO_TCGEN05 = os.environ.get("RUST_INFERENCE_B200_NO_TCGEN05") == "1"   # for comparisons
# the skinny linear applies the SiLU gate in its epilogue (one kernel less per layer: 2 % faster at batch 1 of
# Qwen3-8B shapes, 0.3 % at batch 8); RUST_INFERENCE_B200_FUSED_SWIGLU=0 takes the separate kernel, for comparisons
_FUSED_SWIGLU = os.environ.get("RUST_INFERENCE_B200_FUSED_SWIGLU", "1") != "0"
_WEIGHT_HINTS = os.environ.get("RUST_INFERENCE_B200_WEIGHT_HINTS", "1") != "0"
# likewise an activation after a product of a handful of tokens (RUST_INFERENCE_B200_FUSED_ACT=0: a kernel of its own)
_FUSED_ACT = os.environ.get("RUST_INFERENCE_B200_FUSED_ACT", "1") != "0"
# Up to here the bfloat16 linear is this package's mma.sync weight-streaming kernel whatever the matrix; the kernel takes
# up to 16 tokens, and from 13 to 16 it is taken for the matrices whose grid of 16-row blocks sits well on the SMs: all
# blocks there at once, and either at most two per SM (they then have the ring of three stages) or nearly three
# (with two or three blocks of the two-stage ring an SM has enough bytes on their way; a grid that leaves most SMs
# two of them does not).  The others go to the tcgen05 kernel below.  Measured inside the decode step (ms a step;
# everything on the mma.sync kernel / everything on the tcgen05 one / by this rule, with the gate/up product on the
# tcgen05 kernel): Qwen3-8B shapes (grids of 384, 256 and 256 blocks for 148 SMs) 13 tokens 4.73 / 4.59 / 4.34,
# 16 tokens 5.48 / 4.91 / 4.71; Qwen3-14B shapes (448, 320 and 320 blocks: none sits well) 16 tokens 7.87 / 7.20 / 7.20,
# and 7.51 with the matrices of 320 blocks on the mma.sync kernel.
# RUST_INFERENCE_B200_SKINNY_MAX=8..16 moves the first limit, for comparisons.
SKINNY_MAX_TOKENS = min(16, max(1, int(os.environ.get("RUST_INFERENCE_B200_SKINNY_MAX", "12"))))
SKINNY_KERNEL_TOKENS = 16          # what the kernel takes
SKINNY_BLOCKS_PER_SM = 3           # its blocks of 16 rows that share an SM (two with the ring of three stages)
_sm_count = {}


def _takes_skinny(M: int, N: int, K: int, device) -> bool:
    """Whether a bfloat16 linear of M tokens with a matrix [N, K] runs on the mma.sync weight-streaming kernel."""
    if K % 8 or M > SKINNY_KERNEL_TOKENS:
        return False
    if M <= SKINNY_MAX_TOKENS:
        return True
    key = str(device)
    if key not in _sm_count:
        _sm_count[key] = torch.cuda.get_device_properties(device).multi_processor_count
    fill = -(-N // 16) / _sm_count[key]                  # blocks per SM
    return fill <= 2.0 or 2.5 <= fill <= SKINNY_BLOCKS_PER_SM
# For 13 to 128 tokens there is a tcgen05 weight-streaming kernel of this package (linear_stream_tc).  Measured inside
# the decode step at Qwen3-8B shapes against the library product (cuBLAS): the step is 2.8 % faster with it at 24
# tokens and 1.9 % at 32, the same at 40, and 1.5 to 2 % slower from 48 on (at 64 tokens a layer's products are
# half tensor-core-bound, and the library's tiles do better there); the output head (65,536 outputs and more) is
# faster on it at every token count.  So it is taken up to STREAM_TC_SMALL tokens and for wide matrices;
# RUST_INFERENCE_B200_STREAM_TC=1 takes it for all linears of 13 to 128 tokens, =0 for none but the wide ones.
STREAM_TC_MAX_TOKENS = 128
STREAM_TC_SMALL = 32
STREAM_TC_WIDE = int(os.environ.get("RUST_INFERENCE_B200_STREAM_TC_WIDE", "65536"))   # from this many outputs on it is taken anyway
_STREAM_TC = os.environ.get("RUST_INFERENCE_B200_STREAM_TC", "")
# the selection of a token other than the greedy one: from this many logits a row on, several blocks per row
SAMPLE_WIDE_VOCAB = 16384
_SAMPLE_WIDE = os.environ.get("RUST_INFERENCE_B200_SAMPLE_WIDE", "1") != "0"
# ... and those passes as one kernel whose blocks meet at barriers per row (0: a kernel per pass, for comparisons)
SAMPLE_ONE_KERNEL = os.environ.get("RUST_INFERENCE_B200_SAMPLE_ONE_KERNEL", "1") != "0"
_fn_cache = {}


class KernelError(RuntimeError):
    pass


def _fn(lib_name: str, fn_name: str, defines=None):
    key = (lib_name, fn_name, tuple(sorted((defines or {}).items())))
    f = _fn_cache.get(key)
    if f is None:
        lib = _build.library(lib_name, defines)
        f = getattr(lib, fn_name)
        f.argtypes = _SIGNATURES[(lib_name, fn_name)]
        f.restype = _L if fn_name.endswith("_bytes") else _I
        _fn_cache[key] = f = (f, lib)
    return f


_launches = [0]


def launch_count() -> int:
    """Kernels of this package launched so far (graph replays count what they replay)."""
    return _launches[0]


def add_launches(n: int) -> None:
    _launches[0] += n


def _call(lib_name: str, fn_name: str, *args, defines=None):
    f, lib = _fn(lib_name, fn_name, defines)
    rc = f(*args)
    _launches[0] += 1
    if rc != 0:
        raise KernelError(f"{fn_name}: {lib.ri_last_error().decode(errors='replace')} (code {rc})")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"the kernels work in float32 or bfloat16, not {dtype}")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _need(t: torch.Tensor, name: str, dtype=None, shape=None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if shape is not None and tuple(t.shape) != tuple(shape):
        raise KernelError(f"{name} must have shape {tuple(shape)}, got {tuple(t.shape)}")


_err_flags = {}


def error_flag(device) -> torch.Tensor:
    """One int32 per device that kernels set when they meet an index they must
    not follow (an unmapped page, a token id or position out of range).  The
    engine reads it whenever it synchronises anyway."""
    dev = torch.device(device)
    key = (dev.type, dev.index if dev.index is not None else torch.cuda.current_device())
    f = _err_flags.get(key)
    if f is None:
        f = torch.zeros(1, dtype=torch.int32, device=dev)
        _err_flags[key] = f
    return f


ERROR_TEXT = {1: "token id outside the vocabulary", 2: "cache write to an unmapped page",
              3: "position beyond the rotary table", 4: "attention read from an unmapped page",
              5: "a bounded wait inside a kernel ran out (copy or tensor-core completion never arrived)",
              6: "the tcgen05 attention kernel's shared memory does not start on a multiple of 1024 bytes "
                 "(set RUST_INFERENCE_B200_NO_TCGEN05=1 to use the mma.sync kernel)",
              7: "a sequence is longer than the scratch memory given to the decode attention covers "
                 "(max_chunks x 128 keys): the keys beyond were left out"}


# ---------------------------------------------------------------------------------------
def embed(ids: torch.Tensor, table: torch.Tensor, scale: float = 1.0, copies: int = 1) -> torch.Tensor:
    """float32 rows ``table[ids] * scale``: [tokens, dim], or [tokens, copies, dim] with every row ``copies`` times
    (the streams of a residual that is kept several times over all start as the embedding)."""
    _need(ids, "ids", torch.int32)
    _need(table, "table")
    tokens, (vocab, dim) = ids.numel(), table.shape
    shape = (tokens, dim) if copies == 1 else (tokens, copies, dim)
    out = torch.empty(shape, dtype=torch.float32, device=table.device)
    _call("elementwise", "ri_embed_rows_scaled", ids.data_ptr(), table.data_ptr(), out.data_ptr(), tokens, dim, vocab,
          float(scale), int(copies), _code(table.dtype), error_flag(table.device).data_ptr(), _stream())
    return out


NORM_KINDS = {"layernorm": 0, "rmsnorm": 1}


def stream_norm(resid: torch.Tensor, gain: torch.Tensor, eps: float, out_dtype: torch.dtype, kind: str = "layernorm",
                delta: Optional[torch.Tensor] = None, mix: Optional[torch.Tensor] = None,
                out_w: Optional[torch.Tensor] = None, read: Optional[torch.Tensor] = None,
                rows: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None, more=()) -> torch.Tensor:
    """The norm in front of a sublayer over a residual of S streams ``resid`` [n, S, dim] (float32).

    ``bias`` [dim] (float32) is added to the normed row.  ``more``: up to two further pending outputs as pairs
    (tensor [n, dim], weights [S] or None for ones), added like ``delta`` with ``out_w``, in this order, in float32.

    First the pending update: with ``delta`` [n, dim] (the output of the sublayer before, compute dtype) every
    stream t becomes sum_s mix[s, t] x_s + out_w[t] delta (``mix`` absent: the identity; ``out_w`` absent: ones),
    written back into ``resid`` unless ``rows`` is given.  Then the input u = sum_t read[t] x_t (``read`` absent:
    the plain sum) is normed with ``gain`` (``kind``: "layernorm" without bias, or "rmsnorm").  With ``rows``
    (int32 indices) only those rows are read, in that order.  Returns [n or len(rows), dim] in ``out_dtype``."""
    _need(resid, "resid", torch.float32)
    if resid.dim() != 3:
        raise KernelError(f"stream_norm: resid must be [tokens, streams, dim], got {tuple(resid.shape)}")
    n, S, dim = resid.shape
    _need(gain, "gain", torch.float32, (dim,))
    if delta is not None:
        _need(delta, "delta", out_dtype, (n, dim))
    for t, name, shape in ((mix, "mix", (S, S)), (out_w, "out_w", (S,)), (read, "read", (S,))):
        if t is not None:
            _need(t, name, torch.float32, shape)
    if rows is not None:
        _need(rows, "rows", torch.int32)
    n_out = n if rows is None else rows.numel()
    out = torch.empty((n_out, dim), dtype=out_dtype, device=resid.device)
    more = list(more)
    if len(more) > 2 or (more and delta is None):
        raise KernelError("stream_norm: at most three pending outputs, the first of them in ``delta``")
    if bias is not None:
        _need(bias, "bias", torch.float32, (dim,))
    for y, w in more:
        _need(y, "pending output", out_dtype, (n, dim))
        if w is not None:
            _need(w, "weights of a pending output", torch.float32, (S,))
    more += [(None, None)] * (2 - len(more))
    _call("streams", "ri_stream_norm2", resid.data_ptr(), _ptr(delta), _ptr(mix), _ptr(out_w), _ptr(read), _ptr(rows),
          gain.data_ptr(), out.data_ptr(), _ptr(more[0][0]), _ptr(more[0][1]), _ptr(more[1][0]), _ptr(more[1][1]), _ptr(bias),
          n_out, S, dim, float(eps), NORM_KINDS[kind], _code(out_dtype), _stream())
    return out


ACTIVATIONS = {"relu2": 0, "gelu_tanh": 1, "gelu": 2}


def activation(x: torch.Tensor, kind: str) -> torch.Tensor:
    """Element by element: "relu2" relu(x)^2, "gelu_tanh" 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))), "gelu" the
    exact form 0.5 x (1 + erf(x / sqrt(2)))."""
    _need(x, "x")
    if kind not in ACTIVATIONS:
        raise KernelError(f"activation {kind!r} is not built (known: {', '.join(sorted(ACTIVATIONS))})")
    out = torch.empty_like(x)
    _call("elementwise", "ri_activation", x.data_ptr(), out.data_ptr(), x.numel(), ACTIVATIONS[kind], _code(x.dtype), _stream())
    return out


def _columns(t: torch.Tensor, name: str, dtype) -> int:
    """``t`` is a block of columns of a dense matrix (a slice ``m[:, a:b]``): returns its row pitch in elements."""
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if t.dtype != dtype or t.dim() != 2 or (t.shape[1] > 1 and t.stride(1) != 1):
        raise KernelError(f"{name} must be columns of a {dtype} matrix, got {t.dtype} with strides {t.stride()}")
    return t.stride(0) if t.shape[0] > 1 else max(t.stride(0), t.shape[1])


def gate_heads(x: torch.Tensor, g: torch.Tensor, fn: str = "sigmoid") -> torch.Tensor:
    """In place: x[t, h, j] *= f(g[t, h]) when ``g`` has one column per head, or f(g[t, h * width + j]) when it has
    one per element; f "sigmoid" or "silu".  ``g`` may be a block of columns of a wider matrix."""
    _need(x, "x")
    tokens, heads, width = x.shape
    ldg = _columns(g, "g", x.dtype)
    if g.shape[0] != tokens or g.shape[1] not in (heads, heads * width):
        raise KernelError(f"gate_heads: gates {tuple(g.shape)} do not fit {tuple(x.shape)}")
    per_head = 1 if g.shape[1] == heads else 0
    _call("elementwise", "ri_gate_heads", x.data_ptr(), g.data_ptr(), ldg, tokens, heads, width, per_head,
          {"sigmoid": 0, "silu": 1}[fn], _code(x.dtype), _stream())
    return x


def linear_heads(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """One product per head: y[t, h, :] = w[h] x[t, h, :] for x [tokens, H, K] (any strides with dense last
    dimension, e.g. a slice of a projection), w [H, N, K] dense; y [tokens, H, N] dense.
    float32: this package's FMA kernel (the arithmetic of ``linear``); bfloat16: the library's batched product."""
    if x.dim() != 3 or w.dim() != 3 or x.shape[1] != w.shape[0] or x.shape[2] != w.shape[2]:
        raise KernelError(f"linear_heads: x {tuple(x.shape)} and w {tuple(w.shape)} do not fit")
    _need(w, "w", x.dtype)
    M, H, K = x.shape
    N = w.shape[1]
    if not x.is_cuda or (K > 1 and x.stride(2) != 1):
        raise KernelError("linear_heads: x must be a CUDA tensor whose last dimension is dense")
    y = torch.empty((M, H, N), dtype=x.dtype, device=x.device)
    if M == 0:
        return y
    if x.dtype == torch.float32:
        _call("linear_f32", "ri_linear_heads_f32", x.data_ptr(), w.data_ptr(), y.data_ptr(), M, H, N, K,
              x.stride(0), x.stride(1), H * N, N, _stream())
        return y
    if x.dtype != torch.bfloat16:
        raise KernelError(f"linear_heads: dtype {x.dtype}")
    torch.bmm(x.transpose(0, 1), w.transpose(1, 2), out=y.transpose(0, 1))
    return y


def latent_prep(proj: torch.Tensor, q_col: int, dkv_col: int, qa: torch.Tensor, heads: int, dim: int, rot: int, rank: int,
                gain: torch.Tensor, eps: float, rope_table: Optional[torch.Tensor], pool: Optional[torch.Tensor],
                page_table: torch.Tensor, tok_seq: torch.Tensor, tok_pos: torch.Tensor, seq_slot: torch.Tensor,
                write: bool = True) -> torch.Tensor:
    """Latent attention between its projections and the attention over the cache.  ``proj`` [tokens, N] holds the
    heads' queries ([dim plain, rot to rotate] each) from column ``q_col`` and the down projection (rank + rot) from
    ``dkv_col``; ``qa`` [tokens, H, rank] the plain query parts already multiplied by the key up-projection.  Appends
    [RMS-normed latent, rotated shared key part] to ``pool`` [pages, 1, page_size, rank + rot] and returns the
    query rows [tokens, H, rank + rot].  Rotation turns neighbouring pairs by ``rope_table`` [positions, rot/2, 2]."""
    _need(proj, "proj")
    tokens, ld = proj.shape
    _need(qa, "qa", proj.dtype, (tokens, heads, rank))
    _need(gain, "gain", torch.float32, (rank,))
    Dk = rank + rot
    if q_col + heads * (dim + rot) > ld or dkv_col + Dk > ld:
        raise KernelError("latent_prep: the projection is narrower than its columns")
    rows = 0
    if rot:
        if rope_table is None:
            raise KernelError("latent_prep: a rotated part needs the table of angles")
        _need(rope_table, "rope_table", torch.float32)
        if rope_table.dim() != 3 or rope_table.shape[1] != rot // 2 or rope_table.shape[2] != 2:
            raise KernelError(f"rope table must be [positions, {rot // 2}, 2], got {tuple(rope_table.shape)}")
        rows = rope_table.shape[0]
    else:
        rows = 1 << 30
    if write:
        if pool is None:
            raise KernelError("latent_prep: appending needs the cache pool")
        _need(pool, "pool", proj.dtype)
        pages, kvh, page_size, dk = pool.shape
        if kvh != 1 or dk != Dk:
            raise KernelError(f"latent_prep: pool {tuple(pool.shape)} does not fit one row of {Dk} per token")
    else:
        pages, page_size = 1, 1
    _need(page_table, "page_table", torch.int32)
    for t, n in ((tok_seq, "tok_seq"), (tok_pos, "tok_pos"), (seq_slot, "seq_slot")):
        _need(t, n, torch.int32)
    qf = torch.empty((tokens, heads, Dk), dtype=proj.dtype, device=proj.device)
    _call("latent_attention", "ri_latent_prep", proj.data_ptr(), ld, int(q_col), int(dkv_col), qa.data_ptr(), qf.data_ptr(),
          _ptr(pool) if write else None, page_table.data_ptr(), tok_seq.data_ptr(), tok_pos.data_ptr(), seq_slot.data_ptr(),
          gain.data_ptr(), float(eps), _ptr(rope_table), rows, tokens, heads, dim, rot, rank, page_table.shape[1], page_size,
          pages, 1 if write else 0, _code(proj.dtype), error_flag(proj.device).data_ptr(), _stream())
    return qf


def gla_recurrent(proj: torch.Tensor, q_col: int, k_col: int, v_col: int, z: torch.Tensor, bias: torch.Tensor, tau: float,
                  qscale: float, state: torch.Tensor, seq_slot: torch.Tensor, seq_start: torch.Tensor, heads: int, dim: int,
                  vdim: int, single: bool = False) -> torch.Tensor:
    """Gated linear attention over the step's new tokens.  Per (sequence, head) the state S [dim, vdim] (float32, in
    ``state`` [slots, H, dim, vdim], updated in place) goes S <- diag(a_t) S + k_t v_t^T with the decay
    a_t = sigmoid(z_t + bias)^(1/tau) per key channel, and o_t = S^T (q_t qscale).  q, k, v are columns of ``proj``
    [tokens, N] from ``q_col``, ``k_col``, ``v_col`` (head after head); ``z`` [tokens, H*dim].  ``single``: every sequence
    brings one token (the kernel then stages one token at a time; the results are the same bits).  Returns
    o [tokens, H, vdim] in float32."""
    _need(proj, "proj")
    tokens, ld = proj.shape
    _need(z, "z", proj.dtype, (tokens, heads * dim))
    _need(bias, "bias", torch.float32, (heads * dim,))
    _need(state, "state", torch.float32)
    if tuple(state.shape[1:]) != (heads, dim, vdim):
        raise KernelError(f"gla_recurrent: state {tuple(state.shape)} does not fit {heads} heads of {dim} x {vdim}")
    seqs = seq_slot.numel()
    _need(seq_slot, "seq_slot", torch.int32, (seqs,))
    _need(seq_start, "seq_start", torch.int32, (seqs + 1,))
    if max(q_col, k_col) + heads * dim > ld or v_col + heads * vdim > ld:
        raise KernelError("gla_recurrent: the projection is narrower than its columns")
    o = torch.empty((tokens, heads, vdim), dtype=torch.float32, device=proj.device)
    _call("gla", "ri_gla_recurrent", proj.data_ptr(), ld, int(q_col), int(k_col), int(v_col), z.data_ptr(), bias.data_ptr(),
          float(tau), float(qscale), state.data_ptr(), o.data_ptr(), seq_slot.data_ptr(), seq_start.data_ptr(), seqs, heads,
          dim, vdim, 1 if single and tokens == seqs else 0, _code(proj.dtype), _stream())
    return o


def head_norm_gate(o: torch.Tensor, gain: torch.Tensor, eps: float, g: torch.Tensor, out_dtype: torch.dtype,
                   fn: str = "silu") -> torch.Tensor:
    """y[t, h, :] = rmsnorm(o[t, h, :]) * gain * f(g[t, h*width ..]) for float32 o [tokens, H, width]; ``g`` [tokens,
    H*width] may be a block of columns of a wider matrix of the compute dtype.  Returns [tokens, H*width]."""
    _need(o, "o", torch.float32)
    tokens, H, width = o.shape
    _need(gain, "gain", torch.float32, (width,))
    ldg = _columns(g, "g", out_dtype)
    if tuple(g.shape) != (tokens, H * width):
        raise KernelError(f"head_norm_gate: gates {tuple(g.shape)} do not fit {tuple(o.shape)}")
    y = torch.empty((tokens, H * width), dtype=out_dtype, device=o.device)
    _call("gla", "ri_gla_head_norm_gate", o.data_ptr(), gain.data_ptr(), float(eps), g.data_ptr(), ldg, y.data_ptr(), tokens,
          H, width, {"sigmoid": 0, "silu": 1}[fn], _code(out_dtype), _stream())
    return y


def mlstm_gates(proj: torch.Tensor, i_col: int, f_col: int, i_bias: torch.Tensor, f_bias: torch.Tensor, cap: float,
                m_state: torch.Tensor, seq_slot: torch.Tensor, seq_start: torch.Tensor, heads: int,
                single: bool = False) -> torch.Tensor:
    """The gates of the matrix memory for the step's new tokens.  ``proj`` [tokens, N] holds the input gate's
    pre-activation of head h at column ``i_col`` + h and the forget gate's at ``f_col`` + h.  With
    li = cap tanh((zi + i_bias) / cap), lf = log_sigmoid(cap tanh((zf + f_bias) / cap)) and the running maximum
    m_t = max(lf + m_(t-1), li) (``m_state`` [slots, H] float32, updated in place; 0 at a sequence's start), returns
    float32 [tokens, H, 3]: exp(lf + m_(t-1) - m_t), exp(li - m_t), exp(-m_t).  ``single``: every sequence brings one
    token (another shape of kernel; the same bits)."""
    _need(proj, "proj")
    tokens, ld = proj.shape
    _need(i_bias, "i_bias", torch.float32, (heads,))
    _need(f_bias, "f_bias", torch.float32, (heads,))
    _need(m_state, "m_state", torch.float32)
    if m_state.dim() != 2 or m_state.shape[1] != heads:
        raise KernelError(f"mlstm_gates: m_state {tuple(m_state.shape)} does not fit {heads} heads")
    if max(i_col, f_col) + heads > ld:
        raise KernelError("mlstm_gates: the projection is narrower than its columns")
    seqs = seq_slot.numel()
    _need(seq_slot, "seq_slot", torch.int32, (seqs,))
    _need(seq_start, "seq_start", torch.int32, (seqs + 1,))
    gates = torch.empty((tokens, heads, 3), dtype=torch.float32, device=proj.device)
    _call("mlstm", "ri_mlstm_gates", proj.data_ptr(), ld, int(i_col), int(f_col), i_bias.data_ptr(), f_bias.data_ptr(),
          float(cap), m_state.data_ptr(), gates.data_ptr(), seq_slot.data_ptr(), seq_start.data_ptr(), seqs, heads,
          1 if single and tokens == seqs else 0, _code(proj.dtype), _stream())
    return gates


def scalar_decay_recurrent(proj: torch.Tensor, q_col: int, k_col: int, v_col: int, gates: torch.Tensor, qscale: float,
                           state: torch.Tensor, seq_slot: torch.Tensor, seq_start: torch.Tensor, heads: int, dim: int,
                           vdim: int, ones: bool = True, single: bool = False) -> torch.Tensor:
    """The recurrence S <- a_t S + (b_t k_t) v_t^T, o_t = S^T (q_t qscale) per (sequence, head) with one decay a_t and
    one key factor b_t per token and head: ``gates`` [tokens, H, >= 2] float32 holds them at [.., 0] and [.., 1].  With
    ``ones`` the values get one more column that is 1 for every token: ``state`` is [slots, H, dim, vdim + 1] and the
    result [tokens, H, vdim + 1], whose last column is n_t . q_t with n_t = a_t n_(t-1) + b_t k_t.  q, k, v are columns
    of ``proj`` as for ``gla_recurrent``; the state is float32 and updated in place."""
    _need(proj, "proj")
    tokens, ld = proj.shape
    _need(gates, "gates", torch.float32)
    if gates.dim() != 3 or tuple(gates.shape[:2]) != (tokens, heads) or gates.shape[2] < 2:
        raise KernelError(f"scalar_decay_recurrent: gates {tuple(gates.shape)} do not fit {tokens} tokens of {heads} heads")
    wide = vdim + (1 if ones else 0)
    _need(state, "state", torch.float32)
    if tuple(state.shape[1:]) != (heads, dim, wide):
        raise KernelError(f"scalar_decay_recurrent: state {tuple(state.shape)} does not fit {heads} heads of {dim} x {wide}")
    seqs = seq_slot.numel()
    _need(seq_slot, "seq_slot", torch.int32, (seqs,))
    _need(seq_start, "seq_start", torch.int32, (seqs + 1,))
    if max(q_col, k_col) + heads * dim > ld or v_col + heads * vdim > ld:
        raise KernelError("scalar_decay_recurrent: the projection is narrower than its columns")
    o = torch.empty((tokens, heads, wide), dtype=torch.float32, device=proj.device)
    _call("gla", "ri_gla_recurrent_scalar", proj.data_ptr(), ld, int(q_col), int(k_col), int(v_col), gates.data_ptr(),
          int(gates.shape[2]), 1 if ones else 0, float(qscale), state.data_ptr(), o.data_ptr(), seq_slot.data_ptr(),
          seq_start.data_ptr(), seqs, heads, dim, vdim, 1 if single and tokens == seqs else 0, _code(proj.dtype), _stream())
    return o


def mlstm_head_norm_gate(o: torch.Tensor, gates: torch.Tensor, gain: torch.Tensor, eps: float, g: torch.Tensor,
                         out_dtype: torch.dtype) -> torch.Tensor:
    """Behind the matrix memory's recurrence: o [tokens, H, vdim + 1] float32 (last column n . q), ``gates``
    [tokens, H, 3] (exp(-m) at [.., 2]).  h = o[.., :vdim] / (max(|n . q|, exp(-m)) + 1e-6), then per head
    y = h / sqrt(mean(h^2) + eps) * gain[h, :] * sigmoid(g[t, h vdim ..]); ``gain`` [H vdim] float32; ``g`` [tokens,
    H vdim] may be a block of columns of a wider matrix (float32 or the compute dtype).  Returns [tokens, H vdim]."""
    _need(o, "o", torch.float32)
    tokens, H, wide = o.shape
    vdim = wide - 1
    _need(gates, "gates", torch.float32, (tokens, H, 3))
    _need(gain, "gain", torch.float32, (H * vdim,))
    ldg = _columns(g, "g", g.dtype)
    if tuple(g.shape) != (tokens, H * vdim):
        raise KernelError(f"mlstm_head_norm_gate: gates {tuple(g.shape)} do not fit {tuple(o.shape)}")
    y = torch.empty((tokens, H * vdim), dtype=out_dtype, device=o.device)
    _call("mlstm", "ri_mlstm_head_norm_gate", o.data_ptr(), gates.data_ptr(), gain.data_ptr(), float(eps), g.data_ptr(), ldg,
          y.data_ptr(), tokens, H, vdim, _code(g.dtype), _code(out_dtype), _stream())
    return y


def _weight_hint(then: Optional[torch.Tensor], tokens: int) -> Optional[torch.Tensor]:
    """``then`` if the linear over it will be the weight-streaming kernel for ``tokens`` rows."""
    if (_WEIGHT_HINTS and then is not None and tokens <= SKINNY_MAX_TOKENS and then.dtype == torch.bfloat16
            and then.dim() == 2 and then.is_contiguous()):
        return then
    return None


def rmsnorm(resid: torch.Tensor, gain: torch.Tensor, eps: float, out_dtype: torch.dtype,
            delta: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None,
            then: Optional[torch.Tensor] = None) -> torch.Tensor:
    """RMSNorm of the float32 residual stream ``resid`` [n, dim].

    With ``delta`` (compute dtype, same shape) the sum resid + delta is normed,
    and written back into ``resid`` unless ``rows`` is given.  With ``rows``
    (int32 indices) only those rows are normed, in that order.  ``then`` names the
    weight matrix [N, K] of the linear that reads the result next: for a handful of
    rows in bfloat16 the kernel asks for the start of it to be brought into L2 (a
    hint; it changes no result)."""
    _need(resid, "resid", torch.float32)
    n, dim = resid.shape
    _need(gain, "gain", torch.float32, (dim,))
    if delta is not None:
        _need(delta, "delta", out_dtype, (n, dim))
    if rows is not None:
        _need(rows, "rows", torch.int32)
    n_out = n if rows is None else rows.numel()
    out = torch.empty((n_out, dim), dtype=out_dtype, device=resid.device)
    hint = _weight_hint(then, n_out)
    _call("elementwise", "ri_rmsnorm", resid.data_ptr(), _ptr(delta), _ptr(rows), gain.data_ptr(), out.data_ptr(),
          n_out, dim, float(eps), 1, _code(out_dtype), _ptr(hint), hint.shape[0] if hint is not None else 0,
          hint.shape[1] if hint is not None else 0, _stream())
    return out


def add_rows(resid: torch.Tensor, delta: torch.Tensor) -> None:
    """resid += delta (float32 += compute dtype)."""
    _need(resid, "resid", torch.float32)
    _need(delta, "delta", None, resid.shape)
    _call("elementwise", "ri_add_rows", resid.data_ptr(), delta.data_ptr(), resid.numel(), _code(delta.dtype), _stream())


def silu_mul(gate_up: torch.Tensor, block: Optional[int] = None) -> torch.Tensor:
    """silu(gate) * up for ``gate_up`` [rows, 2*inter], in which gate and up columns alternate
    in blocks of ``block`` channels (default: all gates, then all ups)."""
    _need(gate_up, "gate_up")
    rows, two = gate_up.shape
    if two % 2:
        raise KernelError("silu_mul: the last dimension must be even")
    inter = two // 2
    block = inter if block is None else int(block)
    out = torch.empty((rows, inter), dtype=gate_up.dtype, device=gate_up.device)
    _call("elementwise", "ri_silu_mul", gate_up.data_ptr(), out.data_ptr(), rows, inter, block,
          _code(gate_up.dtype), _stream())
    return out


def linear_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor, block: int) -> torch.Tensor:
    """silu(x Wg^T) * (x Wu^T) for ``w_gate_up`` [2*inter, K] with gate and up rows alternating in
    blocks of ``block``.  A handful of bfloat16 tokens with block 8 run as one kernel (the product's
    epilogue applies the gate); otherwise the product and ``silu_mul`` run one after the other."""
    M, K = x.shape
    N = w_gate_up.shape[0]
    if (x.dtype == torch.bfloat16 and block == 8 and N % 16 == 0 and K % 8 == 0 and _FUSED_SWIGLU
            and _gated_on_stream_tc(M, N, K, x.device)):
        return linear_stream_tc(x, w_gate_up, gated=True)
    if (x.dtype == torch.bfloat16 and _takes_skinny(M, N, K, x.device) and block == 8 and N % 16 == 0
            and _FUSED_SWIGLU):
        _need(x, "x")
        _need(w_gate_up, "w_gate_up", x.dtype)
        y = torch.empty((M, N // 2), dtype=torch.bfloat16, device=x.device)
        _call("linear_skinny", "ri_linear_skinny", x.data_ptr(), w_gate_up.data_ptr(), y.data_ptr(), M, N, K, 0, 1,
              error_flag(x.device).data_ptr(), _stream())
        return y
    if (x.dtype == torch.bfloat16 and block == 8 and N % 16 == 0 and _FUSED_SWIGLU
            and _takes_stream_tc(M, N, K)):
        return linear_stream_tc(x, w_gate_up, gated=True)
    return silu_mul(linear(x, w_gate_up), block)


# The gate/up product of a handful of tokens is the one layer linear that the tcgen05 kernel does better than the
# mma.sync one, where its grid fills the device: a large matrix (many waves of 16-row blocks for the mma.sync kernel,
# whose successor can only come in with the last wave) that the tcgen05 kernel covers in one wave with at least two
# shares of K per tile.  Measured inside the decode step at Qwen3-8B shapes (24,576 x 4,096; ms a step, tcgen05 /
# mma.sync): 12 tokens 4.24 / 4.46, 8 tokens 3.75 / 3.90, 4 tokens 3.35 / 3.43, 3 tokens 3.30 / 3.33; 2 tokens
# 3.16 / 3.13 and 1 token 3.02 / 3.01 the other way round; at 14B and 32B shapes (one share of K: 272 and 400 blocks
# for 148 SMs) 6.01 / 5.93 and 12.52 / 12.44, so those stay where they are.  The other layer linears at 8B shapes lose
# 1 to 3 % on it each.  Against the library product above 32 tokens: 40 tokens 7.47 / 7.58, 64 tokens 10.03 / 10.11.
GATED_STREAM_TC_MIN_TOKENS = 3
GATED_STREAM_TC_MIN_ELEMENTS = 90_000_000
_GATED_STREAM_TC = os.environ.get("RUST_INFERENCE_B200_GATED_STREAM_TC", "1") != "0"
_splits_cache = {}


def _gated_on_stream_tc(M: int, N: int, K: int, device) -> bool:
    if not _GATED_STREAM_TC or M < GATED_STREAM_TC_MIN_TOKENS or M > STREAM_TC_MAX_TOKENS or N * K < GATED_STREAM_TC_MIN_ELEMENTS:
        return False
    key = (N, K, str(device))
    if key not in _splits_cache:
        _, lib = _fn("linear_stream_tc", "ri_linear_stream_tc")
        sms = torch.cuda.get_device_properties(device).multi_processor_count
        _splits_cache[key] = int(lib.ri_linear_stream_tc_splits(int(N), int(K), int(sms)))
    return _splits_cache[key] >= 2


def _takes_stream_tc(M: int, N: int, K: int) -> bool:
    """Whether a bfloat16 linear of M tokens (more than the mma.sync kernel takes) runs on the tcgen05 streaming kernel."""
    return M <= STREAM_TC_MAX_TOKENS and K % 8 == 0 and (
        _STREAM_TC == "1" or N >= STREAM_TC_WIDE or (M <= STREAM_TC_SMALL and _STREAM_TC != "0"))


def linear_act(x: torch.Tensor, w: torch.Tensor, act: str) -> torch.Tensor:
    """act(x w^T) with ``act`` one of ``ACTIVATIONS``.  A handful of bfloat16 tokens run as one kernel (the
    weight-streaming product applies the activation to its float32 sums before it stores them); otherwise the product
    and ``activation`` run one after the other."""
    if act not in ACTIVATIONS:
        raise KernelError(f"activation {act!r} is not built (known: {', '.join(sorted(ACTIVATIONS))})")
    M, K = x.shape
    N = w.shape[0]
    if x.dtype == torch.bfloat16 and w.shape[1] == K and _FUSED_ACT and _takes_skinny(M, N, K, x.device):
        _need(x, "x")
        _need(w, "w", x.dtype)
        y = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
        _call("linear_skinny", "ri_linear_skinny_act", x.data_ptr(), w.data_ptr(), y.data_ptr(), M, N, K, 0, 0,
              ACTIVATIONS[act] + 1, error_flag(x.device).data_ptr(), _stream())
        return y
    return activation(linear(x, w), act)


def linear(x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """y = x w^T for x [M, K], w [N, K].

    float32: this package's own FMA kernel (no tensor cores, no TF32).
    bfloat16, up to 12 tokens (up to 16 for matrices of one wave of blocks): this package's weight-streaming
    tensor-core kernel (mma.sync).
    bfloat16, from there to 32 tokens (and up to 128 for wide matrices such as the output head): this package's
    tcgen05 weight-streaming kernel.
    bfloat16, more tokens: the library GEMM (cuBLAS through torch), as the
    reference engine uses cuBLAS for its linears (src/cuda/mod.rs:186-232 there).
    ``out_dtype`` float32 keeps the float32 accumulator (used for the logits)."""
    _need(x, "x")
    _need(w, "w", x.dtype)
    M, K = x.shape
    N, K2 = w.shape
    if K != K2:
        raise KernelError(f"linear: x has {K} columns, w has {K2}")
    if x.data_ptr() % 16:
        x = x.clone()            # a one-row slice of a wider matrix: the kernels read 16-byte pieces
    if x.dtype == torch.float32:
        y = torch.empty((M, N), dtype=torch.float32, device=x.device)
        _call("linear_f32", "ri_linear_f32", x.data_ptr(), w.data_ptr(), y.data_ptr(), M, N, K, _stream())
        return y
    if x.dtype != torch.bfloat16:
        raise KernelError(f"linear: dtype {x.dtype}")
    if _takes_skinny(M, N, K, x.device):
        # a handful of tokens: the weight-streaming kernel of this package
        y = torch.empty((M, N), dtype=torch.float32 if out_dtype == torch.float32 else torch.bfloat16, device=x.device)
        _call("linear_skinny", "ri_linear_skinny", x.data_ptr(), w.data_ptr(), y.data_ptr(), M, N, K,
              1 if out_dtype == torch.float32 else 0, 0, error_flag(x.device).data_ptr(), _stream())
        return y
    if _takes_stream_tc(M, N, K):
        return linear_stream_tc(x, w, out_dtype)
    if out_dtype == torch.float32:
        return torch.mm(x, w.t(), out_dtype=torch.float32)
    return torch.mm(x, w.t())


_STREAM_TC_GATES = {"silu": 1, "gelu_tanh": 2, "clamped_swish": 3}


def linear_stream_tc(x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
                     gated: bool = False, gate: str = "silu", limit: float = 0.0, alpha: float = 1.0) -> torch.Tensor:
    """y = x w^T in bfloat16 for up to 128 tokens on tcgen05: weight rows as the M side of the product, tokens as N,
    K split over a thread-block cluster whose partial tiles are added through distributed shared memory.
    ``gated``: w holds gate and up rows alternating in blocks of 8, and y [M, N/2] = f(gate) * up' with the gate function
    ``gate`` ("silu", "gelu_tanh", or "clamped_swish" with ``limit`` and ``alpha``: see ``gated_act``)."""
    _need(x, "x", torch.bfloat16)
    _need(w, "w", torch.bfloat16)
    M, K = x.shape
    if M > STREAM_TC_MAX_TOKENS or K % 8 or w.shape[1] != K:
        raise KernelError(f"linear_stream_tc: x {tuple(x.shape)}, w {tuple(w.shape)}: at most {STREAM_TC_MAX_TOKENS} tokens, K a multiple of 8")
    N = w.shape[0]
    if gated and N % 16:
        raise KernelError(f"linear_stream_tc: {N} gate and up rows are not whole blocks of 8 and 8")
    y = torch.empty((M, N // 2 if gated else N), dtype=torch.float32 if out_dtype == torch.float32 else torch.bfloat16,
                    device=x.device)
    _call("linear_stream_tc", "ri_linear_stream_tc_gate", x.data_ptr(), w.data_ptr(), y.data_ptr(), M, N, K,
          1 if out_dtype == torch.float32 else 0, _STREAM_TC_GATES[gate] if gated else 0, float(limit), float(alpha),
          error_flag(x.device).data_ptr(), _stream())
    return y


def qk_norm_rope_append(qkv: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int,
                        q_gain: Optional[torch.Tensor], k_gain: Optional[torch.Tensor], eps: float,
                        rope_table: Optional[torch.Tensor], rotary_dim: int,
                        k_pool: torch.Tensor, v_pool: torch.Tensor, page_table: torch.Tensor,
                        tok_seq: torch.Tensor, tok_pos: torch.Tensor, seq_slot: torch.Tensor,
                        write_kv: bool = True, pairs: bool = False) -> torch.Tensor:
    """Norm and rotate the q and k heads of ``qkv`` [tokens, (H+2KV)*Dh], append k
    and v to the pools [pages, KV, page_size, Dh]; returns q [tokens, H, Dh].  ``pairs``: the
    rotation turns neighbouring elements (2i, 2i+1) instead of elements half a rotated part apart."""
    _need(qkv, "qkv")
    tokens = qkv.shape[0]
    if qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim:
        raise KernelError(f"qkv has {qkv.shape[1]} columns, expected {(num_heads + 2 * num_kv_heads) * head_dim}")
    if k_pool is None:                 # nothing is appended (write_kv False): any valid pointers will do
        if write_kv:
            raise KernelError("qk_norm_rope_append: appending needs the cache pools")
        pages, page_size = 1, 1
        k_pool = v_pool = qkv
        page_table = tok_seq.view(1, -1) if page_table is None else page_table
    else:
        pages, kvh, page_size, dh = k_pool.shape
        if (kvh, dh) != (num_kv_heads, head_dim) or v_pool.shape != k_pool.shape:
            raise KernelError(f"cache pools {tuple(k_pool.shape)} / {tuple(v_pool.shape)} do not fit {num_kv_heads} kv heads of {head_dim}")
        _need(k_pool, "k_pool", qkv.dtype)
        _need(v_pool, "v_pool", qkv.dtype)
    _need(page_table, "page_table", torch.int32)
    for t, n in ((tok_seq, "tok_seq"), (tok_pos, "tok_pos"), (seq_slot, "seq_slot")):
        _need(t, n, torch.int32)
    for g, n in ((q_gain, "q_gain"), (k_gain, "k_gain")):
        if g is not None:
            _need(g, n, torch.float32, (head_dim,))
    rope_rows = 0
    if rope_table is not None:
        _need(rope_table, "rope_table", torch.float32)
        if rope_table.dim() != 3 or rope_table.shape[1] != rotary_dim // 2 or rope_table.shape[2] != 2:
            raise KernelError(f"rope table must be [positions, {rotary_dim // 2}, 2], got {tuple(rope_table.shape)}")
        rope_rows = rope_table.shape[0]
    q = torch.empty((tokens, num_heads, head_dim), dtype=qkv.dtype, device=qkv.device)
    _call("rope_kv", "ri_qk_norm_rope_append_pairs", qkv.data_ptr(), q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(),
          page_table.data_ptr(), tok_seq.data_ptr(), tok_pos.data_ptr(), seq_slot.data_ptr(), _ptr(q_gain),
          _ptr(k_gain), float(eps), _ptr(rope_table), rope_rows, rotary_dim, tokens, num_heads, num_kv_heads,
          head_dim, page_table.shape[1], page_size, pages, 1 if write_kv else 0, 1 if pairs else 0, _code(qkv.dtype),
          error_flag(qkv.device).data_ptr(), _stream())
    return q


def rms_gains(resid: torch.Tensor, gains, eps: float, out_dtype: torch.dtype, terms=(), entry=None,
              rows: Optional[torch.Tensor] = None, then: Optional[torch.Tensor] = None, post=None, out=None):
    """RMS norm of the float32 residual ``resid`` [n, dim] with one or two gains: a tuple of x / sqrt(mean(x^2) + eps) * g
    for every g of ``gains``, from one pass.  First whatever joins the residual, in float32: ``terms``, up to two pending
    outputs as pairs (tensor [n, dim] of the compute dtype, a float32 factor [1] or None for 1), two of them summed
    before they are added (x + (a + b)); then ``entry`` (an object with ``ids``, ``table``, ``scale``, ``vec``):
    table[ids] * scale (``ids`` None: not) and the vector ``vec`` [dim].  The new residual is written back unless ``rows``
    (int32 indices: only those rows are read, in that order) is given.  ``then``: the weight matrix of the linear that
    reads the first result next; for a handful of bfloat16 rows the kernel asks for its start to be brought into L2 (a
    hint; it changes no result).

    ``post`` (a pair (gain float32 [dim], eps)): the pending outputs' weighted sum s is normed on its own before it joins,
    x + s / sqrt(mean(s^2) + eps) * gain (a norm behind the sublayer; the gain may hold a layer scale as well).
    Without ``gains`` nothing is normed in front: whatever joins joins, the residual is written back, and ``out`` (if
    given: the left ``dim`` columns of a wider matrix of the compute dtype) gets the new residual's rows; returns ()."""
    _need(resid, "resid", torch.float32)
    n, dim = resid.shape
    gains = tuple(gains)
    if len(gains) > 2 or (not gains and (rows is not None or then is not None)):
        raise KernelError(f"rms_gains: {len(gains)} gains (one or two; none only for whole steps)")
    for g in gains:
        _need(g, "gain", torch.float32, (dim,))
    terms = list(terms)
    if len(terms) > 2:
        raise KernelError("rms_gains: at most two pending outputs")
    for y, w in terms:
        _need(y, "pending output", out_dtype, (n, dim))
        if w is not None:
            _need(w, "factor of a pending output", torch.float32, (1,))
    terms += [(None, None)] * (2 - len(terms))
    ids = table = vec = None
    scale, vocab = 1.0, 0
    if entry is not None:
        ids, table, scale, vec = entry.ids, entry.table, float(entry.scale), entry.vec
        if ids is not None:
            _need(ids, "ids", torch.int32, (n,))
            _need(table, "table", out_dtype)
            if table.dim() != 2 or table.shape[1] != dim:
                raise KernelError(f"rms_gains: table {tuple(table.shape)} does not fit rows of {dim}")
            vocab = table.shape[0]
        if vec is not None:
            _need(vec, "vec", torch.float32, (dim,))
        if rows is not None and (ids is not None or vec is not None):
            raise KernelError("rms_gains: the terms of an entry join whole steps, not selected rows")
    if rows is not None:
        _need(rows, "rows", torch.int32)
    n_out = n if rows is None else rows.numel()
    outs = tuple(torch.empty((n_out, dim), dtype=out_dtype, device=resid.device) for _ in gains)
    hint = _weight_hint(then, n_out) if out_dtype == torch.bfloat16 else None
    post_gain, post_eps = (None, 0.0) if post is None else post
    if post_gain is not None:
        _need(post_gain, "gain of the norm behind the sublayer", torch.float32, (dim,))
        if terms[0][0] is None:
            raise KernelError("rms_gains: a norm behind the sublayer needs its output")
    pitch = 0
    if not gains and out is not None:
        pitch = _columns(out, "out", out_dtype)
        if tuple(out.shape) != (n, dim):
            raise KernelError(f"rms_gains: out {tuple(out.shape)} does not fit {n} rows of {dim}")
    first = gains[0].data_ptr() if gains else None
    first_out = outs[0].data_ptr() if gains else (_ptr(out) if out is not None else None)
    _call("norm_gains", "ri_norm_gains_post", resid.data_ptr(), _ptr(terms[0][0]), _ptr(terms[0][1]), _ptr(terms[1][0]),
          _ptr(terms[1][1]), _ptr(ids), _ptr(table), int(vocab), scale, _ptr(vec), _ptr(rows), first,
          gains[1].data_ptr() if len(gains) > 1 else None, first_out, outs[1].data_ptr() if len(gains) > 1 else None,
          n_out, dim, float(eps), _ptr(post_gain), float(post_eps), int(pitch), _code(out_dtype), _ptr(hint),
          hint.shape[0] if hint is not None else 0, hint.shape[1] if hint is not None else 0,
          error_flag(resid.device).data_ptr(), _stream())
    return outs


def embed_same(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor) -> None:
    """out[t] = table[ids[t]] in the table's own dtype; ``out`` [tokens, dim] may be a block of columns of a wider
    matrix (one half of the input of a product over two concatenated vectors)."""
    _need(ids, "ids", torch.int32)
    _need(table, "table")
    tokens, (vocab, dim) = ids.numel(), table.shape
    pitch = _columns(out, "out", table.dtype)
    if tuple(out.shape) != (tokens, dim):
        raise KernelError(f"embed_same: out {tuple(out.shape)} does not fit {tokens} rows of {dim}")
    _call("elementwise", "ri_embed_rows_same", ids.data_ptr(), table.data_ptr(), out.data_ptr(), int(pitch), tokens, dim, vocab,
          _code(table.dtype), error_flag(table.device).data_ptr(), _stream())


def qkv_prep(proj: torch.Tensor, q_col: int, k_col: int, v_col: int, heads: int, kv_heads: int, Dp: int, Dk: int,
             bias: Optional[torch.Tensor], rope_table: Optional[torch.Tensor], rot: int, pairs: bool, unit: bool,
             eps: float, k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor], page_table: torch.Tensor,
             tok_seq: torch.Tensor, tok_pos: torch.Tensor, seq_slot: torch.Tensor, write_kv: bool = True,
             norm: str = "", q_gain: Optional[torch.Tensor] = None, k_gain: Optional[torch.Tensor] = None,
             norm_eps: float = 0.0) -> torch.Tensor:
    """Between the q/k/v product and the attention kernels: ``proj`` [tokens, N] holds the q heads from column ``q_col``,
    the k heads from ``k_col`` and the v heads from ``v_col`` (< 0: none, the values are the keys as cached), every head
    ``Dp`` columns wide with ``Dk`` true elements.  ``bias`` (float32, by column of the product) is added first; the first
    ``rot`` elements of q and k heads are turned by ``rope_table`` [positions, rot/2, 2] (``pairs``: partners are
    neighbours, else half a rotated part apart); with ``unit`` q and k heads are then divided by their root mean square
    over ``Dk`` (eps inside the root, no gain).  k (and v) go to the token's place in the pools
    [pages, KV, page_size, Dp]; returns q [tokens, H, Dp].  All of it in float32.

    ``norm``: an RMS norm of q and k before the rotation, "head" over each head's ``Dk`` elements with the gains
    ``q_gain`` and ``k_gain`` [Dp] for all heads, or "all" over all q heads (all k heads) of the token at once with gains
    [H, Dp] and [KV, Dp]; eps ``norm_eps`` inside the root; the gains' padding columns are zero."""
    _need(proj, "proj")
    tokens, ld = proj.shape
    if norm not in ("", "head", "all"):
        raise KernelError(f"qkv_prep: norm {norm!r} (head, all or none)")
    if norm:
        for g, name, n in ((q_gain, "q_gain", heads), (k_gain, "k_gain", kv_heads)):
            _need(g, name, torch.float32, (Dp,) if norm == "head" else (n, Dp))
    nv = 0 if v_col < 0 else kv_heads
    if q_col + heads * Dp > ld or k_col + kv_heads * Dp > ld or (nv and v_col + nv * Dp > ld):
        raise KernelError("qkv_prep: the projection is narrower than its columns")
    if bias is not None:
        _need(bias, "bias", torch.float32)
        if bias.numel() < max(q_col + heads * Dp, k_col + kv_heads * Dp, v_col + nv * Dp):
            raise KernelError("qkv_prep: the bias vector is shorter than the columns it is indexed by")
    rope_rows = 0
    if rope_table is not None:
        _need(rope_table, "rope_table", torch.float32)
        if rope_table.dim() != 3 or rope_table.shape[1] != rot // 2 or rope_table.shape[2] != 2:
            raise KernelError(f"rope table must be [positions, {rot // 2}, 2], got {tuple(rope_table.shape)}")
        rope_rows = rope_table.shape[0]
    if write_kv:
        if k_pool is None:
            raise KernelError("qkv_prep: appending needs the cache pools")
        _need(k_pool, "k_pool", proj.dtype)
        pages, kvh, page_size, dp = k_pool.shape
        if (kvh, dp) != (kv_heads, Dp):
            raise KernelError(f"qkv_prep: pool {tuple(k_pool.shape)} does not fit {kv_heads} kv heads of {Dp}")
        if nv:
            _need(v_pool, "v_pool", proj.dtype, k_pool.shape)
    else:
        pages, page_size = 1, 1
    _need(page_table, "page_table", torch.int32)
    for t, n in ((tok_seq, "tok_seq"), (tok_pos, "tok_pos"), (seq_slot, "seq_slot")):
        _need(t, n, torch.int32)
    q = torch.empty((tokens, heads, Dp), dtype=proj.dtype, device=proj.device)
    _call("qkv_prep", "ri_qkv_prep_norm", proj.data_ptr(), ld, int(q_col), int(k_col), int(v_col), _ptr(bias), q.data_ptr(),
          _ptr(k_pool) if write_kv else None, _ptr(v_pool) if write_kv and nv else None, page_table.data_ptr(),
          tok_seq.data_ptr(), tok_pos.data_ptr(), seq_slot.data_ptr(), _ptr(rope_table), rope_rows, int(rot),
          1 if pairs else 0, 1 if unit else 0, float(eps), _ptr(q_gain) if norm else None, _ptr(k_gain) if norm else None,
          {"": 0, "head": 1, "all": 2}[norm], float(norm_eps), tokens, heads, kv_heads, Dp, Dk, page_table.shape[1], page_size,
          pages, 1 if write_kv else 0, _code(proj.dtype), error_flag(proj.device).data_ptr(), _stream())
    return q


def _mask(window: int, chunk: int) -> int:
    """The kernels' one mask integer: a window of the last ``window`` keys, or (negative) chunks of ``chunk``
    positions counted from the sequence's start, of which a query sees its own up to itself."""
    if window < 0 or chunk < 0 or (window and chunk):
        raise KernelError(f"attention: window {window} and chunk {chunk}: at most one of them, none negative")
    return int(window) if window else -int(chunk)


def _cap(softcap: float) -> float:
    softcap = float(softcap or 0.0)
    if softcap < 0.0:
        raise KernelError(f"a soft cap is positive (0: none), got {softcap}")
    return softcap


def _sink(sink: Optional[torch.Tensor], heads: int) -> Optional[int]:
    if sink is None:
        return None
    _need(sink, "sink", torch.float32, (heads,))
    return sink.data_ptr()


def attention(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, page_table: torch.Tensor,
              seq_slot: torch.Tensor, seq_start: torch.Tensor, seq_len: torch.Tensor, max_new: int, scale: float,
              window: int = 0, sink: Optional[torch.Tensor] = None, chunk: int = 0, softcap: float = 0.0) -> torch.Tensor:
    """Causal attention of the step's new tokens (q [tokens, H, Dh], sequences back to back as
    ``seq_start`` says) over the paged cache, which already holds their keys and values: float32 or
    bfloat16, any head size up to 512, any page size.  Every (token, head) is computed in one fixed
    order that depends on its own position only, so the result does not depend on the step's cutting.
    ``sink`` [H] (float32): exp(sink[h]) joins head h's softmax denominator, with no key and no value.
    ``softcap`` > 0: score <- softcap * tanh(score / softcap) after the scale.
    ``v_pool`` may be ``k_pool`` itself (values that are the keys: latent attention)."""
    _need(q, "q")
    tokens, H, Dh = q.shape
    pages, KV, page_size, dh = k_pool.shape
    if dh != Dh or v_pool.shape != k_pool.shape:
        raise KernelError(f"attention: pools {tuple(k_pool.shape)} do not fit head_dim {Dh}")
    _need(k_pool, "k_pool", q.dtype)
    _need(v_pool, "v_pool", q.dtype)
    _need(page_table, "page_table", torch.int32)
    seqs = seq_slot.numel()
    _need(seq_slot, "seq_slot", torch.int32, (seqs,))
    _need(seq_start, "seq_start", torch.int32, (seqs + 1,))
    _need(seq_len, "seq_len", torch.int32, (seqs,))
    out = torch.empty_like(q)
    _call("attention_rows", "ri_attention_rows", q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), out.data_ptr(),
          page_table.data_ptr(), seq_slot.data_ptr(), seq_start.data_ptr(), seq_len.data_ptr(), seqs, int(max_new),
          H, KV, Dh, page_table.shape[1], page_size, pages, float(scale), _mask(window, chunk), _sink(sink, H), _cap(softcap),
          _code(q.dtype), error_flag(q.device).data_ptr(), _stream())
    return out


def fast_attention_supported(dtype: torch.dtype, head_dim: int, page_size: int) -> bool:
    """Whether the tensor-core attention kernels take this case (else the float32-order kernel of ``attention`` does)."""
    return dtype == torch.bfloat16 and head_dim % 16 == 0 and 16 <= head_dim <= MAX_FAST_HEAD_DIM and page_size == 32


def _decode_parts(head_dim: int, chunks: int) -> int:
    """Partial results per (sequence, head) that the decode attention's scratch memory must have room for."""
    _, lib = _fn("attention_decode", "ri_attention_decode_sink", {"RI_HEAD_DIM": head_dim})
    return int(lib.ri_attention_decode_parts(int(chunks)))


def attention_decode(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, page_table: torch.Tensor,
                     seq_slot: torch.Tensor, seq_len: torch.Tensor, scale: float, window: int,
                     max_len: int, sink: Optional[torch.Tensor] = None, chunk: int = 0, softcap: float = 0.0) -> torch.Tensor:
    """Attention of one new token per sequence (q [seqs, H, Dh], bfloat16) over the
    paged cache, keys split into chunks of ``DECODE_CHUNK``; ``max_len`` bounds the
    sequences' lengths after this step and sizes the scratch memory."""
    _need(q, "q", torch.bfloat16)
    seqs, H, Dh = q.shape
    pages, KV, page_size, dh = k_pool.shape
    if dh != Dh or v_pool.shape != k_pool.shape:
        raise KernelError(f"attention_decode: pools {tuple(k_pool.shape)} do not fit head_dim {Dh}")
    if not fast_attention_supported(q.dtype, Dh, page_size):
        raise KernelError(f"attention_decode: head_dim {Dh} with pages of {page_size} is not supported")
    _need(k_pool, "k_pool", torch.bfloat16)
    _need(v_pool, "v_pool", torch.bfloat16)
    _need(page_table, "page_table", torch.int32)
    _need(seq_slot, "seq_slot", torch.int32, (seqs,))
    _need(seq_len, "seq_len", torch.int32, (seqs,))
    chunks = max(1, -(-int(max_len) // DECODE_CHUNK))
    parts = _decode_parts(Dh, chunks)
    o_part = torch.empty((seqs, H, parts, Dh), dtype=torch.float32, device=q.device)
    ml_part = torch.empty((seqs, H, parts, 2), dtype=torch.float32, device=q.device)
    out = torch.empty_like(q)
    _call("attention_decode", "ri_attention_decode_cap", q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(),
          out.data_ptr(), o_part.data_ptr(), ml_part.data_ptr(), page_table.data_ptr(), seq_slot.data_ptr(),
          seq_len.data_ptr(), seqs, H, KV, Dh, page_table.shape[1], page_size, pages, chunks, float(scale),
          _mask(window, chunk), _sink(sink, H), _cap(softcap), error_flag(q.device).data_ptr(), _stream(),
          defines={"RI_HEAD_DIM": Dh})
    return out


def attention_prefill(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, page_table: torch.Tensor,
                      seq_slot: torch.Tensor, seq_start: torch.Tensor, seq_len: torch.Tensor, max_new: int,
                      scale: float, window: int, sink: Optional[torch.Tensor] = None, v_dims: int = 0,
                      chunk: int = 0, softcap: float = 0.0) -> torch.Tensor:
    """Attention of the step's new tokens (q [tokens, H, Dh], bfloat16, sequences back
    to back as ``seq_start`` says) over the paged cache, which already holds their keys
    and values; ``max_new`` is the most tokens one sequence brings.  ``v_pool`` may be ``k_pool``
    itself (values that are the keys): the mma.sync kernel then reads each tile once; ``v_dims`` > 0
    says that only that many leading elements of the result are wanted (the rest may be zeros)."""
    _need(q, "q", torch.bfloat16)
    tokens, H, Dh = q.shape
    pages, KV, page_size, dh = k_pool.shape
    if dh != Dh or v_pool.shape != k_pool.shape:
        raise KernelError(f"attention_prefill: pools {tuple(k_pool.shape)} do not fit head_dim {Dh}")
    if not fast_attention_supported(q.dtype, Dh, page_size):
        raise KernelError(f"attention_prefill: head_dim {Dh} with pages of {page_size} is not supported")
    _need(k_pool, "k_pool", torch.bfloat16)
    _need(v_pool, "v_pool", torch.bfloat16)
    _need(page_table, "page_table", torch.int32)
    seqs = seq_slot.numel()
    _need(seq_slot, "seq_slot", torch.int32, (seqs,))
    _need(seq_start, "seq_start", torch.int32, (seqs + 1,))
    _need(seq_len, "seq_len", torch.int32, (seqs,))
    out = torch.empty_like(q)
    if Dh in TCGEN05_HEAD_DIMS and not _NO_TCGEN05:
        # head sizes of 64 and 128: the tcgen05 / tensor-memory kernel
        _call("attention_prefill_tc", "ri_attention_prefill_tc", q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(),
              out.data_ptr(), page_table.data_ptr(), seq_slot.data_ptr(), seq_start.data_ptr(), seq_len.data_ptr(),
              q.shape[0], seqs, int(max_new), H, KV, Dh, page_table.shape[1], page_size, pages, float(scale),
              _mask(window, chunk), _sink(sink, H), _cap(softcap), error_flag(q.device).data_ptr(), _stream(),
              defines={"RI_HEAD_DIM": Dh})
        return out
    _call("attention_prefill", "ri_attention_prefill", q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(),
          out.data_ptr(), page_table.data_ptr(), seq_slot.data_ptr(), seq_start.data_ptr(), seq_len.data_ptr(),
          seqs, int(max_new), H, KV, Dh, page_table.shape[1], page_size, pages, float(scale), _mask(window, chunk),
          _sink(sink, H), int(v_dims), _cap(softcap), error_flag(q.device).data_ptr(), _stream(), defines={"RI_HEAD_DIM": Dh})
    return out


def argmax(logits: torch.Tensor) -> torch.Tensor:
    """First index of each row's maximum: int32 [rows]."""
    _need(logits, "logits", torch.float32)
    rows, vocab = logits.shape
    out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    slices = min(128, max(1, -(-vocab // 2048)))           # ri_argmax_slices of the library
    part_val = part_idx = None
    if slices > 1:
        part_val = torch.empty((rows, slices), dtype=torch.float32, device=logits.device)
        part_idx = torch.empty((rows, slices), dtype=torch.int32, device=logits.device)
    _call("sampling", "ri_argmax", logits.data_ptr(), logits.stride(0), rows, vocab, out.data_ptr(), _ptr(part_val),
          _ptr(part_idx), _stream())
    return out


def sample(logits: torch.Tensor, temperature: torch.Tensor, uniform: torch.Tensor,
           top_k: Optional[torch.Tensor] = None, top_p: Optional[torch.Tensor] = None,
           penalty: Optional[torch.Tensor] = None, seen: Optional[torch.Tensor] = None,
           seen_rows: Optional[torch.Tensor] = None, uses_top_k: bool = True, uses_top_p: bool = True) -> torch.Tensor:
    """One token per row of float32 ``logits`` [rows, vocab]; the options are
    per-row device tensors (temperature float32, top_k int32, top_p float32,
    penalty float32), ``uniform`` the per-row number in [0, 1).

    From ``SAMPLE_WIDE_VOCAB`` logits a row on, several blocks work on each row (the same
    token, bit for bit); a caller that knows that no row has a top-k or a top-p says so
    with ``uses_top_k`` / ``uses_top_p`` and saves those searches."""
    _need(logits, "logits", torch.float32)
    rows, vocab = logits.shape
    _need(temperature, "temperature", torch.float32, (rows,))
    _need(uniform, "uniform", torch.float32, (rows,))
    if top_k is not None:
        _need(top_k, "top_k", torch.int32, (rows,))
    if top_p is not None:
        _need(top_p, "top_p", torch.float32, (rows,))
    if penalty is not None:
        _need(penalty, "penalty", torch.float32, (rows,))
    seen_stride = 0
    if seen is not None:
        _need(seen, "seen", torch.uint8)
        if seen.shape[1] != vocab:
            raise KernelError("seen must be [rows, vocab]")
        seen_stride = seen.stride(0)
        if seen_rows is not None:
            _need(seen_rows, "seen_rows", torch.int32, (rows,))
    out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    work, work_bytes = None, 0
    if _SAMPLE_WIDE and vocab >= SAMPLE_WIDE_VOCAB:
        f, _ = _fn("sampling", "ri_sample_work_bytes")
        work_bytes = int(f(rows, vocab))
        work = torch.empty(work_bytes, dtype=torch.uint8, device=logits.device)
    k_on, p_on = bool(uses_top_k and top_k is not None), bool(uses_top_p and top_p is not None)
    _call("sampling", "ri_sample", logits.data_ptr(), logits.stride(0), rows, vocab, _ptr(seen), _ptr(seen_rows),
          seen_stride, temperature.data_ptr(), _ptr(top_k), _ptr(top_p), _ptr(penalty), uniform.data_ptr(),
          out.data_ptr(), _ptr(work), work_bytes, int(k_on), int(p_on), error_flag(logits.device).data_ptr(),
          int(SAMPLE_ONE_KERNEL), _stream())
    if work is not None and not SAMPLE_ONE_KERNEL:
        add_launches(2 + 12 * (1 + k_on + p_on) + p_on)          # one was counted by the call
    return out


def mark_seen(seen: torch.Tensor, rows: torch.Tensor, tokens: torch.Tensor) -> None:
    """seen[rows[i], tokens[i]] = 1."""
    _need(seen, "seen", torch.uint8)
    _need(rows, "rows", torch.int32)
    _need(tokens, "tokens", torch.int32, rows.shape)
    _call("sampling", "ri_mark_seen", seen.data_ptr(), seen.stride(0), rows.data_ptr(), tokens.data_ptr(),
          rows.numel(), seen.shape[1], _stream())


# ---------------------------------------------------------------------------------------
def scale_(x: torch.Tensor, factor: float) -> torch.Tensor:
    """x *= factor in place (float32)."""
    _need(x, "x", torch.float32)
    if factor != 1.0:
        _call("elementwise", "ri_scale_f32", x.data_ptr(), x.numel(), float(factor), _stream())
    return x


def softcap_(x: torch.Tensor, cap: float) -> torch.Tensor:
    """x <- cap * tanh(x / cap) in place (float32); ``cap`` 0: nothing."""
    _need(x, "x", torch.float32)
    if cap:
        _call("elementwise", "ri_softcap_f32", x.data_ptr(), x.numel(), _cap(cap), _stream())
    return x


def embed_pair_hash(ids: torch.Tensor, table: torch.Tensor, pairs: torch.Tensor, last_token: torch.Tensor,
                    tok_seq: torch.Tensor, tok_pos: torch.Tensor, seq_slot: torch.Tensor, seq_start: torch.Tensor,
                    mul_prev: int, mul_cur: int, single: bool = False) -> torch.Tensor:
    """float32 rows ``table[id] + pairs[(previous id * mul_prev + id * mul_cur) mod buckets]`` with ``pairs``
    [buckets + 1, dim]; a sequence's first token (position 0) takes row ``buckets``.  The token before a step's first
    one comes from ``last_token`` [slots] (int32), which is brought up to date.  ``single``: every sequence brings
    one token (one launch instead of two)."""
    _need(ids, "ids", torch.int32)
    _need(table, "table")
    _need(pairs, "pairs", table.dtype)
    _need(last_token, "last_token", torch.int32)
    tokens, (vocab, dim) = ids.numel(), table.shape
    if pairs.dim() != 2 or pairs.shape[1] != dim or pairs.shape[0] < 2:
        raise KernelError(f"embed_pair_hash: pair table {tuple(pairs.shape)} does not fit rows of {dim}")
    seqs = seq_slot.numel()
    for t, n in ((tok_seq, "tok_seq"), (tok_pos, "tok_pos"), (seq_slot, "seq_slot"), (seq_start, "seq_start")):
        _need(t, n, torch.int32)
    out = torch.empty((tokens, dim), dtype=torch.float32, device=table.device)
    _call("pair_embedding", "ri_embed_pair_hash", ids.data_ptr(), table.data_ptr(), pairs.data_ptr(), out.data_ptr(),
          last_token.data_ptr(), tok_seq.data_ptr(), tok_pos.data_ptr(), seq_slot.data_ptr(), seq_start.data_ptr(), tokens,
          seqs, dim, vocab, pairs.shape[0] - 1, int(mul_prev), int(mul_cur), 1 if single else 0, _code(table.dtype),
          error_flag(table.device).data_ptr(), _stream())
    if not (single and tokens == seqs):
        add_launches(1)
    return out


def short_conv(x: torch.Tensor, col0: int, weight: torch.Tensor, state: torch.Tensor, tok_seq: torch.Tensor,
               seq_slot: torch.Tensor, seq_start: torch.Tensor, single: bool = False,
               weight_t: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal convolution over time per channel, then silu: channels are columns ``col0 .. col0 + C`` of ``x``
    [tokens, N]; ``weight`` [C, taps] float32 (the last column is the current token's); ``state`` [slots, taps-1, C]
    float32 holds every sequence's last inputs (zeros at its start) and is brought up to date.  ``weight_t``: the
    weights once more as [taps, C]; with it bfloat16 inputs take a kernel of eight channels per thread (the same
    results).  float32 [tokens, C]."""
    _need(x, "x")
    _need(weight, "weight", torch.float32)
    C, taps = weight.shape
    tokens, ld = x.shape
    if col0 < 0 or col0 + C > ld:
        raise KernelError("short_conv: the channels lie outside the matrix")
    _need(state, "state", torch.float32)
    if tuple(state.shape[1:]) != (taps - 1, C):
        raise KernelError(f"short_conv: state {tuple(state.shape)} does not fit {taps} taps on {C} channels")
    seqs = seq_slot.numel()
    for t, n in ((tok_seq, "tok_seq"), (seq_slot, "seq_slot"), (seq_start, "seq_start")):
        _need(t, n, torch.int32)
    y = torch.empty((tokens, C), dtype=torch.float32, device=x.device)
    if weight_t is not None:
        _need(weight_t, "weight_t", torch.float32, (taps, C))
    _call("delta_rule", "ri_short_conv", x.data_ptr(), ld, int(col0), weight.data_ptr(), _ptr(weight_t), y.data_ptr(), state.data_ptr(),
          tok_seq.data_ptr(), seq_slot.data_ptr(), seq_start.data_ptr(), tokens, seqs, C, taps, 1 if single else 0,
          _code(x.dtype), _stream())
    if not (single and tokens == seqs) and taps > 1:
        add_launches(1)
    return y


def delta_rule_recurrent(qkv: torch.Tensor, q_col: int, k_col: int, v_col: int, proj: torch.Tensor, beta_col: int,
                         z: torch.Tensor, dt_bias: torch.Tensor, a_log: torch.Tensor, qscale: float, state: torch.Tensor,
                         seq_slot: torch.Tensor, seq_start: torch.Tensor, heads: int, qk_heads: int, dim: int, vdim: int,
                         single: bool = False) -> torch.Tensor:
    """The gated delta rule over the step's new tokens.  Per head h (with q/k head h // (heads // qk_heads)) the state S
    [dim, vdim] (float32, in ``state`` [slots, H, dim, vdim], updated in place) goes
    S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q, with q and k made unit vectors (q also times
    ``qscale``), g = exp(-exp(a_log[h]) softplus(z + dt_bias)) per key channel and beta = sigmoid of column
    ``beta_col + h`` of ``proj``.  ``qkv`` [tokens, C] float32 holds q, k, v from ``q_col``, ``k_col``, ``v_col``;
    ``z`` [tokens, H*dim] in the compute dtype.  The q and k columns of ``qkv`` are made unit vectors in place.
    Returns o [tokens, H, vdim] float32."""
    _need(qkv, "qkv", torch.float32)
    tokens, C = qkv.shape
    _need(proj, "proj")
    _need(z, "z", proj.dtype, (tokens, heads * dim))
    _need(dt_bias, "dt_bias", torch.float32, (heads * dim,))
    _need(a_log, "a_log", torch.float32, (heads,))
    _need(state, "state", torch.float32)
    if tuple(state.shape[1:]) != (heads, dim, vdim):
        raise KernelError(f"delta_rule_recurrent: state {tuple(state.shape)} does not fit {heads} heads of {dim} x {vdim}")
    if heads % qk_heads or max(q_col, k_col) + qk_heads * dim > C or v_col + heads * vdim > C or beta_col + heads > proj.shape[1]:
        raise KernelError("delta_rule_recurrent: the columns do not fit the matrices")
    seqs = seq_slot.numel()
    _need(seq_slot, "seq_slot", torch.int32, (seqs,))
    _need(seq_start, "seq_start", torch.int32, (seqs + 1,))
    o = torch.empty((tokens, heads, vdim), dtype=torch.float32, device=qkv.device)
    decay = torch.empty((tokens, heads * dim), dtype=torch.float32, device=qkv.device)
    beta = torch.empty((tokens, heads + qk_heads), dtype=torch.float32, device=qkv.device)
    _call("delta_rule", "ri_delta_rule_recurrent", qkv.data_ptr(), C, int(q_col), int(k_col), int(v_col), proj.data_ptr(),
          proj.shape[1], int(beta_col), z.data_ptr(), dt_bias.data_ptr(), a_log.data_ptr(), float(qscale), decay.data_ptr(),
          beta.data_ptr(), state.data_ptr(), o.data_ptr(), seq_slot.data_ptr(), seq_start.data_ptr(), tokens, seqs, heads,
          qk_heads, dim, vdim, 1 if single and tokens == seqs else 0, _code(proj.dtype), _stream())
    add_launches(1)
    return o


GATES = {"silu": 0, "gelu_tanh": 1, "clamped_swish": 2}


def gated_act(gate_up: torch.Tensor, kind: str, block: Optional[int] = None, limit: float = 0.0,
              alpha: float = 1.0) -> torch.Tensor:
    """f(gate) * up' for ``gate_up`` [rows, 2*inter] whose gate and up columns alternate in blocks of ``block``
    channels (default: all gates, then all ups).  ``kind``: "silu", "gelu_tanh", or "clamped_swish":
    g sigmoid(alpha g) (u + 1) with g = min(gate, limit), u = clamp(up, -limit, limit)."""
    _need(gate_up, "gate_up")
    if kind not in GATES:
        raise KernelError(f"gate {kind!r} is not built (known: {', '.join(sorted(GATES))})")
    rows, two = gate_up.shape
    if two % 2:
        raise KernelError("gated_act: the last dimension must be even")
    inter = two // 2
    block = inter if block is None else int(block)
    out = torch.empty((rows, inter), dtype=gate_up.dtype, device=gate_up.device)
    _call("elementwise", "ri_gated_act", gate_up.data_ptr(), out.data_ptr(), rows, inter, block, GATES[kind], float(limit),
          float(alpha), _code(gate_up.dtype), _stream())
    return out


def linear_gated(x: torch.Tensor, w_gate_up: torch.Tensor, block: int, kind: str = "silu", limit: float = 0.0,
                 alpha: float = 1.0) -> torch.Tensor:
    """f(x Wg^T) * (x Wu^T)' for the stacked matrix of ``linear_swiglu``; "silu" takes that function's fused kernels; the
    other gates (see ``gated_act``) take the same weight-streaming kernels with the gate in their epilogues for up to 32
    bfloat16 tokens (in the same order of choice), and run the product and the gate one after the other beyond."""
    if kind == "silu":
        return linear_swiglu(x, w_gate_up, block)
    M, K = x.shape
    N = w_gate_up.shape[0]
    fusable = (kind in _STREAM_TC_GATES and x.dtype == torch.bfloat16 and block == 8 and N % 16 == 0 and K % 8 == 0
               and _FUSED_SWIGLU and w_gate_up.shape[1] == K)
    if fusable and _gated_on_stream_tc(M, N, K, x.device):
        # a large matrix and a few tokens: the tcgen05 weight-streaming product, the gate in its epilogue
        return linear_stream_tc(x, w_gate_up, gated=True, gate=kind, limit=limit, alpha=alpha)
    if fusable and not _takes_skinny(M, N, K, x.device) and _takes_stream_tc(M, N, K):
        return linear_stream_tc(x, w_gate_up, gated=True, gate=kind, limit=limit, alpha=alpha)
    if (kind in ("gelu_tanh", "clamped_swish") and x.dtype == torch.bfloat16 and block == 8 and N % 16 == 0 and _FUSED_SWIGLU
            and _takes_skinny(M, N, K, x.device) and w_gate_up.shape[1] == K):
        # a handful of tokens: the weight-streaming product applies the gate to its float32 sums
        _need(x, "x")
        _need(w_gate_up, "w_gate_up", x.dtype)
        if x.data_ptr() % 16:
            x = x.clone()
        y = torch.empty((M, N // 2), dtype=torch.bfloat16, device=x.device)
        _call("linear_skinny", "ri_linear_skinny_gated_with", x.data_ptr(), w_gate_up.data_ptr(), y.data_ptr(), M, N, K,
              {"gelu_tanh": 2, "clamped_swish": 3}[kind], float(limit), float(alpha), error_flag(x.device).data_ptr(), _stream())
        return y
    return gated_act(linear(x, w_gate_up), kind, block, limit, alpha)


MOE_SCORES = {"softmax": 0, "sigmoid": 1}


def moe_route(x: torch.Tensor, router: torch.Tensor, correction: torch.Tensor, top: int, score: str = "softmax",
              groups: int = 1, keep: int = 1, group_top: int = 2, scale: float = 1.0, renormalize: bool = True):
    """Per token the ``top`` router outputs with the largest softmax(router x) + correction (ties: the lower index),
    and as weights their softmax scores divided by their sum (+ 1e-20).  ``router`` [N, D] and ``correction`` [N]
    float32.  Returns (int32 [tokens, top], float32 [tokens, top]).

    ``score`` "sigmoid": the scores are the sigmoid of every output on its own.  ``groups`` > 1: the outputs form that
    many equal runs of neighbours, a run's score is the sum of its ``group_top`` largest choice scores, and only outputs
    of the ``keep`` best runs can be chosen.  The weights are multiplied by ``scale``; ``renormalize`` False leaves out
    the division by their sum."""
    _need(x, "x")
    tokens, D = x.shape
    _need(router, "router", torch.float32)
    N = router.shape[0]
    if router.shape[1] != D:
        raise KernelError(f"moe_route: router {tuple(router.shape)} does not fit rows of {D}")
    _need(correction, "correction", torch.float32, (N,))
    idx = torch.empty((tokens, top), dtype=torch.int32, device=x.device)
    weight = torch.empty((tokens, top), dtype=torch.float32, device=x.device)
    if score not in MOE_SCORES:
        raise KernelError(f"moe_route: score {score!r} (known: {', '.join(sorted(MOE_SCORES))})")
    _call("moe", "ri_moe_route_rule", x.data_ptr(), router.data_ptr(), correction.data_ptr(), idx.data_ptr(), weight.data_ptr(),
          tokens, D, N, int(top), MOE_SCORES[score], int(groups), int(keep), int(group_top), float(scale),
          1 if renormalize else 0, _code(x.dtype), _stream())
    return idx, weight


MOE_TILE_ROWS, MOE_TILE_ROWS_WIDE = 32, 64


def moe_plan(idx: torch.Tensor, experts: int, wide: bool = False):
    """The step's (token, choice) pairs grouped by expert for the grouped products: (perm int32 [pairs], tiles int32
    [max_tiles, 3] of (expert, first row, rows), meta int32 [2] = (tiles, rows), rows per tile); choices >= ``experts``
    are left out.  ``wide``: tiles of 64 rows instead of 32 (many pairs per expert; bfloat16 products whose rows are whole
    16-byte pieces).  Everything stays on the device."""
    _need(idx, "idx", torch.int32)
    pairs = idx.numel()
    bm = MOE_TILE_ROWS_WIDE if wide else MOE_TILE_ROWS
    _, lib = _fn("moe", "ri_moe_plan")
    max_tiles = int(lib.ri_moe_max_tiles(int(pairs), int(experts), bm))
    perm = torch.empty(max(pairs, 1), dtype=torch.int32, device=idx.device)
    tiles = torch.empty((max_tiles, 3), dtype=torch.int32, device=idx.device)
    meta = torch.empty(2, dtype=torch.int32, device=idx.device)
    _call("moe", "ri_moe_plan", idx.data_ptr(), perm.data_ptr(), tiles.data_ptr(), meta.data_ptr(), pairs, int(experts),
          max_tiles, bm, _stream())
    return perm, tiles, meta, bm


def moe_grouped_linear(a: torch.Tensor, w: torch.Tensor, plan, rows_out: int, gather_div: int = 0, scatter: bool = False,
                       out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """y[out(r)] = w[e] a[in(r)] for every row r of the plan's tiles; ``w`` [E, N, K]; in(r) = perm[r] // gather_div
    (``gather_div`` > 0) or r; out(r) = perm[r] (``scatter``) or r.  Rows that no tile covers are not written."""
    perm, tiles, meta, bm = plan
    _need(a, "a")
    _need(w, "w", a.dtype)
    E, N, K = w.shape
    if a.dim() != 2 or a.shape[1] != K:
        raise KernelError(f"moe_grouped_linear: a {tuple(a.shape)} and w {tuple(w.shape)} do not fit")
    out_dtype = out_dtype or a.dtype
    if out_dtype not in (a.dtype, torch.float32):
        raise KernelError("moe_grouped_linear: the result is float32 or the compute dtype")
    y = torch.empty((rows_out, N), dtype=out_dtype, device=a.device)
    _call("moe", "ri_moe_grouped_linear", a.data_ptr(), a.stride(0), w.data_ptr(), y.data_ptr(), N, perm.data_ptr(),
          tiles.data_ptr(), meta.data_ptr(), tiles.shape[0], int(bm), N, K, int(gather_div), 1 if scatter else 0,
          1 if out_dtype == torch.float32 else 0, _code(a.dtype), _stream())
    return y


def moe_combine(pair_out: torch.Tensor, idx: torch.Tensor, weight: torch.Tensor, x: torch.Tensor, experts: int,
                extra: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y[t] = sum_j weight[t, j] * (idx[t, j] >= experts ? x[t] : pair_out[t * top + j]) (+ extra[t]), in float32, j
    ascending, rounded once to x's dtype."""
    _need(x, "x")
    tokens, D = x.shape
    top = idx.shape[1]
    _need(pair_out, "pair_out", torch.float32, (tokens * top, D))
    _need(idx, "idx", torch.int32, (tokens, top))
    _need(weight, "weight", torch.float32, (tokens, top))
    if extra is not None:
        _need(extra, "extra", x.dtype, (tokens, D))
    y = torch.empty_like(x)
    _call("moe", "ri_moe_combine", pair_out.data_ptr(), idx.data_ptr(), weight.data_ptr(), x.data_ptr(), _ptr(extra),
          y.data_ptr(), tokens, D, top, int(experts), _code(x.dtype), _stream())
    return y
