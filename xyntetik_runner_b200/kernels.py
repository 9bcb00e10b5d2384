"""Python face of the CUDA library: one function per launcher, torch tensors in.

Every function checks what the kernel cannot (device, dtype, contiguity),
launches on torch's current stream and raises on a refusal.  Nothing here has
another way to compute its result: if the library cannot be built or loaded,
the first call raises.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .csrc import build as _build

F32, BF16 = 0, 1
_ERR = {-1: "the kernel refuses these sizes or dtypes", -2: "CUDA refused the launch", -3: "tensor map encoding failed",
        -4: "size beyond the entry point's fixed limit", -5: "set-up of the entry point failed"}

_lib = None


class KernelError(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        path = _build.library_path()
        try:
            _lib = ctypes.CDLL(path)
        except OSError as e:
            raise KernelError(f"cannot load {path}: {e}") from None
        _declare(_lib)
    return _lib


def library_file() -> str:
    lib()
    return _build.library_path(build=False)


_vp, _i, _ll, _f = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float


def _declare(L: ctypes.CDLL) -> None:
    sig = {
        "xr_embed": [_vp, _i, _vp, _vp, _i, _vp, _i, _i, _i, _f, _vp],
        "xr_rmsnorm": [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _f, _vp],
        "xr_rope_store": [_vp, _i, _vp, _vp, _vp, _vp, _vp, _ll, _ll, _i, _i, _i, _i, _i, _i, _i, _i, _f, _vp],
        "xr_act_mul": [_vp, _vp, _i, _i, _i, _i, _i, _f, _vp],
        "xr_residual_add": [_vp, _vp, _i, _i, _i, _vp],
        "xr_gemm_simt": [_vp, _i, _vp, _i, _vp, _vp, _i, _i, _i, _i, _i, _ll, _ll, _vp],
        "xr_attention_simt": [_vp, _vp, _i, _vp, _vp, _vp, _vp, _ll, _ll, _ll, _i, _i, _i, _i, _i, _i, _i, _f, _vp, _f, _vp],
        "xr_gemm_tc": [_vp, _vp, _vp, _vp, _i, _i, _i, _f, _i, _i, _i, _ll, _ll, _vp, _ll, _vp, _i, _i, ctypes.POINTER(ctypes.c_int), _i, _vp],
        "xr_finish_add_rmsnorm": [_vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _f, _vp],
        "xr_finish_plain": [_vp, _i, _vp, _vp, _i, _i, _i, _i, _ll, _vp],
        "xr_finish_rope_store": [_vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _ll, _ll, _i, _i, _i, _i, _i, _i, _i, _i, _f, _vp],
        "xr_attention_mma": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _ll, _ll, _ll, _i, _i, _i, _i, _i, _i, _i, _f,
                             _i, _i, _i, _i, _i, _vp, _ll, _i, _i, _vp, _vp, _i, _i, _ll, _vp, _f, _vp],
        "xr_attention_mma_splits": [_i, _i, _ll],
        "xr_attention_even_launches": [],
        "xr_attention_wait_probe": [_vp, _vp, ctypes.c_uint, _vp],
        "xr_attention_tc_supported": [_i, _i, _i, _i],
        "xr_attention_tc": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _ll, _i, _i, _i, _i, _i, _i, _i, _i, _f, _i, _ll, _ll, _i, _i, _vp, _f, _vp],
        "xr_sample": [_vp, _ll, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp],
        "xr_sample_one_block": [_vp, _ll, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp],
        "xr_logprob": [_vp, _ll, _i, _i, _vp, _vp, _vp],
        "xr_random_normal": [_vp, _i, _ll, ctypes.c_ulonglong, ctypes.c_ulonglong, _f, _f, _vp],
        "xr_scaled_add": [_vp, _vp, _f, _i, _i, _vp],
        "xr_stream_step": [_vp, _vp, _vp, _i, _i, _vp],
        "xr_sigmoid_gate": [_vp, _ll, _vp, _ll, _i, _i, _i, _i, _i, _i, _vp],
        "xr_concat_cast": [_vp, _vp, _vp, _i, _i, _i, _vp],
        "xr_softcap": [_vp, _f, _ll, _vp],
        "xr_latent_prep": [_vp, _i, _ll, _vp, _ll, _vp, _vp, _vp, _vp, _vp, _vp, _ll, _i, _i, _i, _i, _i, _i, _i, _i, _f, _i, _vp],
        "xr_head_matmul": [_vp, _i, _ll, _i, _vp, _i, _ll, _ll, _ll, _vp, _i, _ll, _vp, _i, _ll, _i, _i, _i, _i, _i, _vp],
        "xr_latent_attention": [_vp, _vp, _i, _ll, _i, _vp, _vp, _ll, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _i, _vp],
        "xr_latent_attention_mma_supported": [_i, _i],
        "xr_latent_attention_mma": [_vp, _ll, _ll, _vp, _ll, _i, _vp, _vp, _ll, _ll, _vp, _vp, _vp, _ll, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _i, _i, _i, _vp],
        "xr_heads_gather": [_vp, _ll, _i, _vp, _i, _i, _i, _i, _vp],
        "xr_heads_scatter_gate": [_vp, _vp, _vp, _ll, _i, _i, _i, _i, _i, _vp],
        "xr_qk_norm_rope_store": [_vp, _i, _ll, _vp, _ll, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _ll, _ll, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _i, _f, _i,
                                  _vp, _i, _vp, _i, _f, _i, _vp],
        "xr_rmsnorm_act": [_vp, _i, _ll, _vp, _vp, _ll, _i, _i, _f, _vp],
        "xr_delta": [_vp, _i, _ll, _vp, _vp, _vp, _vp, _vp, _ll, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp],
        "xr_head_norm_gate": [_vp, _vp, _i, _ll, _vp, _i, _i, _vp, _i, _i, _i, _i, _f, _vp],
        "xr_mlstm": [_vp, _i, _ll, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _f, _vp],
        "xr_route_topk": [_vp, _vp, _vp, _i, _i, _i, _vp, _i, _vp],
        "xr_moe_plan": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp],
        "xr_moe_gather": [_vp, _i, _ll, _vp, _vp, _vp, _i, _i, _i, _i, _vp],
        "xr_gemm_tc_grouped": [_vp, _vp, _vp, _i, _i, _i, _f, _i, _i, _i, _ll, _ll, _i, _vp, _i, _vp, _vp],
        "xr_moe_tile_rows": [],
        "xr_moe_gemm": [_vp, _i, _ll, _vp, _i, _vp, _i, _ll, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _vp],
        "xr_moe_combine": [_vp, _vp, _vp, _vp, _i, _i, _i, _vp],
        "xr_embed_pair": [_vp, _vp, _i, _vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _ll, _ll, _ll, _vp],
        "xr_last_token": [_vp, _vp, _i, _vp, _vp, _vp, _vp, _i, _i, _vp],
        "xr_norm_add": [_vp, _vp, _vp, _vp, _i, _i, _i, _f, _i, _vp, _vp, _i, _vp],
        "xr_cast_rows": [_vp, _vp, _i, _ll, _vp],
        "xr_depth_average": [_vp, _vp, _vp, _vp, _vp, _i, _i, _ll, _vp],
        "xr_rotate_heads": [_vp, _i, _ll, _i, _i, _i, _i, _i, _i, _vp, _vp, _f, _f, _i, _vp],
        "xr_rglru": [_vp, _ll, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _ll, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i,
                     _f, _vp],
        "xr_row_norm_gate": [_vp, _vp, _ll, _vp, _vp, _i, _i, _i, _f, _f, _vp],
        "xr_decay_attention": [_vp, _ll, _i, _i, _i, _vp, _vp, _ll, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp],
    }
    for name, args in sig.items():
        fn = getattr(L, name)
        fn.argtypes = args
        fn.restype = ctypes.c_int


def _check(code: int, what: str) -> None:
    if code != 0:
        raise KernelError(f"{what}: {_ERR.get(code, f'error {code}')}")


try:
    _raw_stream, _raw_device = torch._C._cuda_getCurrentRawStream, torch._C._cuda_getDevice
except AttributeError:                   # (another torch: the documented way, a few microseconds a call)
    _raw_stream = _raw_device = None


def _stream() -> int:
    """The current CUDA stream's handle.  Asked for at every launch: a step of a few hundred tokens is a few hundred
    launches whose host time nothing hides, so it is the two C calls, not the Stream object that torch builds."""
    if _raw_stream is not None:
        return _raw_stream(_raw_device())
    return torch.cuda.current_stream().cuda_stream


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"dtype {dt} is not float32 or bfloat16")


def _dev(*ts) -> None:
    for t in ts:
        if t is not None and (not t.is_cuda or not t.is_contiguous()):
            raise KernelError("kernel arguments must be contiguous CUDA tensors")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


launch_count = 0   # kernels launched through this module since import (bench reports it)


def _count(n: int = 1) -> None:
    global launch_count
    launch_count += n


# ---------------------------------------------------------------------------
def embed(table: torch.Tensor, ids: torch.Tensor, x: torch.Tensor, feed: Optional[torch.Tensor] = None, scale: float = 1.0) -> None:
    """x[t] = table[ids[t]] widened to float32, times `scale`; ids outside the table read row 0.  With `feed` (int32
    on the device), ids[t] = -(1 + j) reads token feed[j]."""
    _dev(table, ids, x, feed)
    n, d = x.shape
    assert ids.dtype == torch.int32 and ids.numel() >= n and x.dtype == torch.float32 and table.shape[1] == d
    assert feed is None or feed.dtype == torch.int32
    _check(lib().xr_embed(table.data_ptr(), dtype_code(table.dtype), ids.data_ptr(), _ptr(feed),
                          0 if feed is None else feed.numel(), x.data_ptr(), n, d, table.shape[0], float(scale), _stream()), "embed")
    _count()


def _second_norm(w2, out2, out, d):
    assert (w2 is None) == (out2 is None)
    if w2 is not None:
        assert w2.dtype == torch.float32 and w2.numel() == d and out2.shape == out.shape and out2.dtype == out.dtype and out2.is_contiguous()


def rmsnorm(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, eps: float, rows: Optional[torch.Tensor] = None,
            w2: Optional[torch.Tensor] = None, out2: Optional[torch.Tensor] = None) -> None:
    """out[i] = x[rows[i] or i] * rsqrt(mean(x^2) + eps) * w; x float32, w float32.  With `w2`, `out2`: the same rows times a second
    weight into `out2`, in the same pass (one root mean square for both)."""
    _dev(x, w, out, rows, w2, out2)
    n, d = out.shape
    assert x.dtype == torch.float32 and w.dtype == torch.float32 and x.shape[1] == d and w.numel() == d
    assert rows is None or (rows.dtype == torch.int32 and rows.numel() >= n)
    _second_norm(w2, out2, out, d)
    _check(lib().xr_rmsnorm(x.data_ptr(), _ptr(rows), w.data_ptr(), out.data_ptr(), _ptr(w2), _ptr(out2), dtype_code(out.dtype), n, d,
                            float(eps), _stream()), "rmsnorm")
    _count()


def rope_store(qkv: torch.Tensor, positions, tok_seg, block_tables, inv_freq: Optional[torch.Tensor],
               cache_k_ptr: Optional[int], page_stride: int, v_offset: int, H: int, K: int, hd: int,
               rotary_dim: int, max_pages: int, page_size: int, adjacent: bool = False, mscale: float = 1.0) -> None:
    """Rotate Q in place, rotate K and store K, V into their pages (cache_k_ptr None: store nothing).  Pair j of
    a head is elements (j, j + rotary_dim/2), or (2j, 2j + 1) with `adjacent`; cosines and sines are multiplied
    by `mscale` (src/model.c:3514-3532)."""
    _dev(qkv, positions, tok_seg, block_tables, inv_freq)
    n = qkv.shape[0]
    assert qkv.shape[1] == (H + 2 * K) * hd
    assert rotary_dim == 0 or (inv_freq is not None and inv_freq.dtype == torch.float32 and inv_freq.numel() >= rotary_dim // 2)
    _check(lib().xr_rope_store(qkv.data_ptr(), dtype_code(qkv.dtype), positions.data_ptr(), tok_seg.data_ptr(),
                               block_tables.data_ptr(), _ptr(inv_freq), cache_k_ptr, page_stride, v_offset,
                               n, H, K, hd, rotary_dim, max_pages, page_size, int(adjacent), float(mscale), _stream()),
           "rope_store")
    _count()


ACT_NONE, ACT_SILU, ACT_GELU_TANH, ACT_SWISH_CLAMP = 0, 1, 2, 3
# "swish_clamp" exists for gated products only and takes a `limit`: with g' = min(g, limit) and u' = u clamped to
# [-limit, limit] the product stores g' sigmoid(1.702 g') (u' + 1).
ACTIVATIONS = {"none": ACT_NONE, "silu": ACT_SILU, "gelu_tanh": ACT_GELU_TANH, "swish_clamp": ACT_SWISH_CLAMP}


def rmsnorm_act(inp: torch.Tensor, w: torch.Tensor, out: torch.Tensor, eps: float) -> None:
    """out[t] = inp[t] * rsqrt(mean(inp[t]^2) + eps) * w for rows in the activation dtype (rows may be strided); w float32."""
    _dev(w)
    n, d = inp.shape
    assert out.shape == (n, d) and inp.dtype == out.dtype and inp.stride(1) == 1 and out.stride(1) == 1 and inp.is_cuda and out.is_cuda
    assert w.dtype == torch.float32 and w.numel() == d
    _check(lib().xr_rmsnorm_act(inp.data_ptr(), dtype_code(inp.dtype), inp.stride(0), w.data_ptr(), out.data_ptr(), out.stride(0), n, d,
                                float(eps), _stream()), "rmsnorm_act")
    _count()


def qk_norm_rope_store(inp: torch.Tensor, q_out: torch.Tensor, positions, tok_seg, block_tables, freq: Optional[torch.Tensor],
                       q_w: Optional[torch.Tensor], k_w: Optional[torch.Tensor], cache_k_ptr: Optional[int], page_stride: int, v_offset: int,
                       H: int, K: int, D: int, Vd: int, hd: int, rotary_dim: int, max_pages: int, page_size: int, adjacent: bool,
                       eps: float, unit_norm: bool = False, q_coef: float = 0.0, q_every: int = 0, partial: Optional[torch.Tensor] = None,
                       splits: int = 0, bias: Optional[torch.Tensor] = None, mscale: float = 1.0, norm_after: bool = False) -> None:
    """inp [n, >= (H + K) D + K Vd] (rows may be strided): Q heads, K heads (D each), V heads (Vd each).  Every Q and K head is
    RMS-normed with the weight q_w / k_w (float32 [D], shared by the heads; None: no norm), its first `rotary_dim` elements rotated
    (freq: float64 [rotary_dim / 2]); Q goes to q_out [n, *] (head h at column h * hd), K and V into the token's cache rows, every
    head filled up to `hd` elements with zeros (cache_k_ptr None: nothing is stored).  `unit_norm` (with no weights): every Q
    and K head is divided by its root mean square all the same.  `q_every` > 0: the Q heads of the token at position p are
    multiplied by 1 + q_coef ln(floor((p + 1) / q_every) + 1).  `partial` (float32 [splits][n][inp.shape[1]], with `bias`): the rows are
    still the partial sums of a product cut along K; the kernel sums them (+ bias) into `inp`, every column, before it reads them.
    `mscale` multiplies every cosine and sine; `norm_after` (with `unit_norm`): the root mean square is that of the rotated head."""
    _dev(positions, tok_seg, block_tables, freq, q_w, k_w, partial, bias)
    n = inp.shape[0]
    assert partial is None or (partial.dtype == torch.float32 and splits >= 1 and partial.numel() >= splits * n * inp.shape[1])
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == inp.shape[1])
    assert inp.stride(1) == 1 and q_out.stride(1) == 1 and inp.dtype == q_out.dtype and q_out.shape[0] == n and q_out.shape[1] >= H * hd
    assert inp.shape[1] >= (H + K) * D + K * Vd and (freq is None or (freq.dtype == torch.float64 and freq.numel() >= rotary_dim // 2))
    assert q_w is None or (q_w.dtype == torch.float32 and k_w.dtype == torch.float32 and q_w.numel() == D and k_w.numel() == D)
    _check(lib().xr_qk_norm_rope_store(inp.data_ptr(), dtype_code(inp.dtype), inp.stride(0), q_out.data_ptr(), q_out.stride(0),
                                       positions.data_ptr(), tok_seg.data_ptr(), block_tables.data_ptr(), _ptr(freq), _ptr(q_w), _ptr(k_w),
                                       cache_k_ptr, page_stride, v_offset, n, H, K, D, Vd, hd, rotary_dim, max_pages, page_size,
                                       int(adjacent), float(eps), int(unit_norm), float(q_coef), int(q_every), _ptr(partial), int(splits),
                                       _ptr(bias) if partial is not None else None, inp.shape[1], float(mscale), int(norm_after),
                                       _stream()),
           "qk_norm_rope_store")
    _count()


def act_mul(gu: torch.Tensor, h: torch.Tensor, act: int = ACT_SILU, gated: bool = True, limit: float = 0.0) -> None:
    """Gated: h[t][f] = act(gu[t][f]) * gu[t][F + f] for gu [n, 2F] (ACT_SWISH_CLAMP: see ACTIVATIONS); ungated:
    h = act(gu) for gu [n, F] (h may be gu)."""
    _dev(gu, h)
    n, F = h.shape
    assert gu.shape == (n, 2 * F if gated else F) and gu.dtype == h.dtype
    _check(lib().xr_act_mul(gu.data_ptr(), h.data_ptr(), dtype_code(h.dtype), n, F, int(act), int(gated), float(limit), _stream()), "act_mul")
    _count()


def silu_mul(gu: torch.Tensor, h: torch.Tensor) -> None:
    act_mul(gu, h, ACT_SILU, True)


def residual_add(x: torch.Tensor, delta: torch.Tensor) -> None:
    _dev(x, delta)
    n, d = x.shape
    assert x.dtype == torch.float32 and delta.shape == x.shape
    _check(lib().xr_residual_add(x.data_ptr(), delta.data_ptr(), dtype_code(delta.dtype), n, d, _stream()), "residual_add")
    _count()


def gemm_simt(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
              accumulate: bool = False) -> None:
    """out[t][r] (+)= sum_k x[t][k] w[r][k] (+ bias[r]) in float32 FMA.  Rows of x and out may be strided."""
    for t in (x, w, out, bias):
        if t is not None and not t.is_cuda:
            raise KernelError("kernel arguments must be CUDA tensors")
    n, k = x.shape
    n_out = w.shape[0]
    assert w.shape[1] == k and out.shape == (n, n_out) and w.is_contiguous()
    assert x.stride(1) == 1 and out.stride(1) == 1
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == n_out)
    _check(lib().xr_gemm_simt(x.data_ptr(), dtype_code(x.dtype), w.data_ptr(), dtype_code(w.dtype), _ptr(bias),
                              out.data_ptr(), dtype_code(out.dtype), int(accumulate), n, n_out, k,
                              x.stride(0), out.stride(0), _stream()), "gemm_simt")
    _count()


def attention_simt(q: torch.Tensor, q_row_stride: int, out: torch.Tensor, cache_k_ptr: int, positions, tok_seg,
                   block_tables, page_stride: int, v_offset: int, H: int, K: int, hd: int, max_pages: int,
                   page_size: int, window: int, scale: float, sink: Optional[torch.Tensor] = None, softcap: float = 0.0) -> None:
    """Causal attention of every token of the step over its request's pages, float32 arithmetic.  `sink`: float32 [H];
    exp(sink[h]) joins the denominator of head h's softmax once (it has no key and no value).  `softcap` c > 0: every scaled
    score s becomes c tanh(s / c)."""
    _dev(out, positions, tok_seg, block_tables, sink)
    assert sink is None or (sink.dtype == torch.float32 and sink.numel() == H)
    n = out.shape[0]
    assert out.shape[1] == H * hd and q.dtype == out.dtype
    _check(lib().xr_attention_simt(q.data_ptr(), out.data_ptr(), dtype_code(out.dtype), cache_k_ptr,
                                   positions.data_ptr(), tok_seg.data_ptr(), block_tables.data_ptr(), page_stride,
                                   v_offset, q_row_stride, n, H, K, hd, max_pages, page_size, window, float(scale),
                                   _ptr(sink), float(softcap), _stream()), "attention_simt")
    _count()


EXEMPT_IDS = 8          # ids per row that a penalty window never holds, as the sampling kernel takes them


def sample(logits: torch.Tensor, temp, top_k, top_p, min_p, penalty, draw, recent: Optional[torch.Tensor],
           scratch: torch.Tensor, out: torch.Tensor, any_sampled: bool = True, one_block: bool = False,
           shortcuts: bool = True, pending: Optional[torch.Tensor] = None, feed: Optional[torch.Tensor] = None,
           exempt: Optional[torch.Tensor] = None) -> None:
    """One token per row of float32 logits by the reference's sampling chain (see csrc/sampling.cu).
    `scratch` must hold rows * vocab floats unless every row is greedy (`any_sampled` False).  `shortcuts` (the
    default): one block a row that selects the top-k, or gathers the head of the distribution, sorts that and walks
    it as the reference does; rows where that does not apply are left to a second launch that goes the long way for
    them alone.  Without: the long way for every row, by threshold descents that never sort, spread over a cluster of
    eight blocks a row when the rows are few and have more than 1,024 values (`one_block`: in one block whatever the width).
    `pending` (int32 [rows, 3]) with `feed` and `exempt` (int32 [rows, EXEMPT_IDS]): row r's window lacks the token that
    the step before sampled and the host has not read yet; it is feed[pending[r, 0]] (-1: the window is complete),
    takes window entry pending[r, 1], and is left out if it is among the first pending[r, 2] ids of exempt[r].
    `out` must not be `feed` then."""
    _dev(temp, top_k, top_p, min_p, penalty, draw, recent, scratch, out)
    rows, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    assert not any_sampled or scratch.numel() >= rows * V
    assert out.dtype == torch.int32 and top_k.dtype == torch.int32
    # (rows that are all greedy are one argmax each: nothing for a cluster to share)
    args = (logits.data_ptr(), logits.stride(0), rows, V, temp.data_ptr(), top_k.data_ptr(), top_p.data_ptr(), min_p.data_ptr(),
            penalty.data_ptr(), draw.data_ptr(), _ptr(recent), scratch.data_ptr(), out.data_ptr())
    if pending is not None:
        _dev(pending, feed, exempt)
        assert pending.dtype == torch.int32 and pending.numel() >= 3 * rows and exempt.dtype == torch.int32
        assert exempt.numel() >= EXEMPT_IDS * rows and feed.dtype == torch.int32 and recent is not None
        assert out.data_ptr() != feed.data_ptr() and any_sampled and not one_block
    if one_block or not any_sampled:
        _check(lib().xr_sample_one_block(*args, _stream()), "sample")
    else:
        _check(lib().xr_sample(*args, int(shortcuts), _ptr(pending), _ptr(feed), _ptr(exempt), _stream()), "sample")
    _count()


def logprob(logits: torch.Tensor, target: torch.Tensor, out: torch.Tensor) -> None:
    """out[i] = log softmax(logits[i])[target[i]] (float maximum, double sum of exponentials, float result)."""
    _dev(target, out)
    rows, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and logits.is_cuda
    assert target.dtype == torch.int32 and target.numel() >= rows and out.dtype == torch.float32 and out.numel() >= rows
    _check(lib().xr_logprob(logits.data_ptr(), logits.stride(0), rows, V, target.data_ptr(), out.data_ptr(), _stream()), "logprob")
    _count()


def random_normal(out: torch.Tensor, key: int, mean: float, std: float, first: int = 0) -> None:
    """out.flat[i] = mean + std * z(key, first + i): the counter-based generator of csrc/random_fill.cu, whose
    values equal ``weights.random_fill.normal_values`` bit for bit."""
    _dev(out)
    _check(lib().xr_random_normal(out.data_ptr(), dtype_code(out.dtype), out.numel(), key & 0xFFFFFFFFFFFFFFFF, first,
                                  float(mean), float(std), _stream()), "random_normal")
    _count()


# ---------------------------------------------------------------------------
EPI_STORE, EPI_ADD, EPI_GATED = 0, 1, 2
EPI_SWIGLU = EPI_GATED          # the gated epilogue with the SiLU activation
_TC_SCRATCH_FLOATS = 32 << 20
_HANDOVER_FLAGS = 2048          # one word per CTA of the decode attention in even shares
_tc_state = {}


class Workspace:
    """Split-K scratch and status word of the tensor-core product on one device.

    A product that is cut along K leaves float32 partial sums here.  When its caller defers the sum to its next
    kernel the slab stays taken until that kernel has been launched (``PartialSums.release``), and products
    launched meanwhile get room behind it: two deferred sums can never share memory, whatever order a block
    runs its parts in.  Slabs are handed out by a bump pointer that returns to the start whenever nothing is
    outstanding, so the usual order (product, then the kernel that sums it) always uses the same addresses,
    which CUDA graphs need.  ``reset`` (called at the start of every engine step) drops slabs that a failed
    step left behind."""

    def __init__(self, device: torch.device):
        self.scratch = torch.empty(_TC_SCRATCH_FLOATS, dtype=torch.float32, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self.status_ptr = self.status.data_ptr()
        self.flags = torch.zeros(_HANDOVER_FLAGS, dtype=torch.int32, device=device)   # raised and lowered inside one launch
        self.top = 0            # floats taken from the start of the scratch
        self.live = 0           # slabs outstanding

    def reset(self) -> None:
        self.top = self.live = 0

    def room(self):
        """(address, floats) of the free part."""
        if self.live == 0:
            self.top = 0
        return self.scratch.data_ptr() + 4 * self.top, self.scratch.numel() - self.top

    def take(self, floats: int) -> torch.Tensor:
        at = self.top
        self.top += (floats + 63) // 64 * 64
        self.live += 1
        return self.scratch[at:at + floats]

    def give_back(self) -> None:
        self.live = max(0, self.live - 1)
        if self.live == 0:
            self.top = 0


def workspace(device: torch.device) -> Workspace:
    key = device.index if device.index is not None else torch.cuda.current_device()
    ws = _tc_state.get(key)
    if ws is None:
        ws = _tc_state[key] = Workspace(device)
    return ws


def tc_workspace(device: torch.device):
    """(split-K scratch, status word) of the tensor-core product on `device`, made on first use."""
    ws = workspace(device)
    return ws.scratch, ws.status


def tc_workspace_reset(device: torch.device) -> None:
    """Forget deferred sums that were never finished (a step that failed half way)."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key in _tc_state:
        _tc_state[key].reset()


def tc_check_status(device: torch.device) -> None:
    """Raise if a tensor-core kernel gave up a wait since the last check (reads one word from the device)."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    ws = _tc_state.get(key)
    if ws is not None:
        code = int(ws.status.item())
        if code != 0:
            ws.status.zero_()
            ws.flags.zero_()                  # a launch that gave up may have left some raised
            what = {1: "a tcgen05 product", 2: "the bulk-copy decode attention", 3: "the tcgen05 attention", 4: "the tcgen05 attention (shared memory not 1 KB aligned)"}.get(code, "a kernel")
            raise KernelError(f"{what} gave up waiting on a barrier; its output is not valid")


def gemm_tc_supported(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> bool:
    k = x.shape[1]
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and k >= 8 and k % 8 == 0 and x.stride(1) == 1
            and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and w.is_contiguous()
            and out.stride(1) == 1)


TILE_ROWS, TILE_K = 128, 64
GATED_FEATURES = 64        # features per 128-row tile of a gated product


def pack_weight(w: torch.Tensor, halves: int = 1) -> torch.Tensor:
    """Re-lay a [rows, K] bfloat16 matrix tile by tile for the tensor-core product:
    [row tile][K block][128][64], rows and K padded with zeros to whole tiles, so that every tile the
    kernel fetches is one contiguous 16 KB read.

    `halves` = 2: the rows are F gate rows followed by F up rows of a gated product.  They are interleaved so that
    a 128-row tile holds 64 features: its rows 32 q .. 32 q + 15 are the gate rows of features 64 tile + 16 q + (0..15)
    and rows 32 q + 16 .. 32 q + 31 their up rows (q = 0..3: the four quarters of the accumulator's lanes), which
    lets the product's epilogue combine a feature's two sums inside one warp."""
    assert w.dtype == torch.bfloat16 and w.dim() == 2 and w.shape[0] % halves == 0 and halves in (1, 2)
    rows, k = w.shape[0] // halves, w.shape[1]
    kp = -(-k // TILE_K) * TILE_K
    if halves == 2:
        fp = -(-rows // GATED_FEATURES) * GATED_FEATURES
        both = torch.zeros((2, fp, kp), dtype=w.dtype, device=w.device)
        both[0, :rows, :k] = w[:rows]
        both[1, :rows, :k] = w[rows:]
        # [half][tile][quarter][16][K] -> [tile][quarter][half][16][K]
        src = both.view(2, fp // GATED_FEATURES, 4, 16, kp).permute(1, 2, 0, 3, 4).reshape(fp * 2, kp)
        del both
    else:
        rp = -(-rows // TILE_ROWS) * TILE_ROWS
        if rp != rows or kp != k:
            src = torch.zeros((rp, kp), dtype=w.dtype, device=w.device)
            src[:rows, :k] = w
        else:
            src = w
    rp = src.shape[0]
    return src.view(rp // TILE_ROWS, TILE_ROWS, kp // TILE_K, TILE_K).permute(0, 2, 1, 3).contiguous()


class PartialSums:
    """float32 partial sums [splits][n][rows] of a product that was cut along K and whose sum is left to the
    caller's next kernel.  The slab of the workspace they lie in is this object's until ``release``."""

    def __init__(self, ws: Workspace, partial: torch.Tensor, splits: int):
        self._ws, self.partial, self.splits = ws, partial, splits

    def release(self) -> None:
        if self._ws is not None:
            self._ws.give_back()
            self._ws = None


_SPLITS_USED = ctypes.c_int(1)           # where xr_gemm_tc says how it cut the product (read at once after the call)
_SPLITS_USED_REF = ctypes.byref(_SPLITS_USED)


def _gemm_tc(x, w, out, bias, epilogue, act, force_splits, defer, packed_rows, act_limit=0.0):
    n, k = x.shape
    gated = epilogue == EPI_GATED
    if packed_rows is not None:
        # w comes from pack_weight(); packed_rows is the logical number of output features
        n_out = packed_rows
        tiles = -(-n_out // GATED_FEATURES) if gated else -(-n_out // TILE_ROWS)
        assert w.dim() == 4 and w.shape[0] == tiles and w.shape[1] == -(-k // TILE_K) and out.shape == (n, n_out)
        assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and k % 8 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0
    else:
        if gated:
            raise KernelError("the gated product takes weights from pack_weight(w, halves=2)")
        n_out = w.shape[0]
        assert w.shape[1] == k and out.shape == (n, n_out) and gemm_tc_supported(x, w, out)
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == n_out and not gated)
    assert not defer or not gated
    ws = workspace(x.device)
    at, room = ws.room()
    _check(lib().xr_gemm_tc(x.data_ptr(), w.data_ptr(), _ptr(bias), out.data_ptr(), dtype_code(out.dtype), epilogue, int(act), float(act_limit),
                            n, n_out, k, x.stride(0), out.stride(0), at, room,
                            ws.status_ptr, force_splits, int(defer), _SPLITS_USED_REF,
                            int(packed_rows is not None), _stream()), "gemm_tc")
    splits = _SPLITS_USED.value
    _count(1 if (splits == 1 or defer) else 2)
    if defer and splits > 1:
        rows = tiles * TILE_ROWS if (gated and packed_rows is not None) else n_out
        return PartialSums(ws, ws.take(splits * n * rows), splits)
    return splits


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
            epilogue: int = EPI_STORE, force_splits: int = 0, packed_rows: Optional[int] = None, act: Optional[int] = None,
            act_limit: float = 0.0) -> int:
    """bfloat16 product on tcgen05.  EPI_STORE: out[t][r] = act(x.w + bias); EPI_ADD: float32 out += x.w + bias;
    EPI_GATED: w from ``pack_weight(w, halves=2)``, out[t][f] = act(x.w_gate[f]) * (x.w_up[f]) (act defaults to SiLU).
    Returns the number of K splits used."""
    if act is None:
        act = ACT_SILU if epilogue == EPI_GATED else ACT_NONE
    return _gemm_tc(x, w, out, bias, epilogue, act, force_splits, False, packed_rows, act_limit)


def gemm_tc_deferred(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
                     epilogue: int = EPI_STORE, force_splits: int = 0, packed_rows: Optional[int] = None) -> Optional[PartialSums]:
    """The same product, its sum left to the caller when it was cut along K: returns ``PartialSums`` ([splits][n][n_out]
    float32 in a slab of the workspace; `out` is NOT written, and the bias not added) for the caller's next kernel
    (``finish_*``) to sum, then ``release()``.  Returns None when the product was not cut: `out` is complete."""
    r = _gemm_tc(x, w, out, bias, epilogue, ACT_NONE, force_splits, True, packed_rows)
    return r if isinstance(r, PartialSums) else None


def finish_add_rmsnorm(partial: torch.Tensor, splits: int, bias: Optional[torch.Tensor], x: torch.Tensor,
                       w: torch.Tensor, out: torch.Tensor, eps: float, w2: Optional[torch.Tensor] = None,
                       out2: Optional[torch.Tensor] = None) -> None:
    """x += sum of the split-K partials (+ bias); out = RMSNorm(x) * w (and out2 = RMSNorm(x) * w2).  One pass over each row."""
    _dev(x, w, out, bias, w2, out2)
    n, d = x.shape
    assert x.dtype == torch.float32 and w.dtype == torch.float32 and out.shape == (n, d) and partial.numel() >= splits * n * d
    _second_norm(w2, out2, out, d)
    _check(lib().xr_finish_add_rmsnorm(partial.data_ptr(), splits, _ptr(bias), x.data_ptr(), w.data_ptr(), out.data_ptr(), _ptr(w2),
                                       _ptr(out2), dtype_code(out.dtype), n, d, float(eps), _stream()), "finish_add_rmsnorm")
    _count()


def finish_plain(partial: torch.Tensor, splits: int, bias: Optional[torch.Tensor], out: torch.Tensor,
                 accumulate: bool) -> None:
    """out (+)= sum of the split-K partials (+ bias)."""
    n, width = out.shape
    assert out.stride(1) == 1 and partial.numel() >= splits * n * width
    _check(lib().xr_finish_plain(partial.data_ptr(), splits, _ptr(bias), out.data_ptr(), dtype_code(out.dtype),
                                 int(accumulate), n, width, out.stride(0), _stream()), "finish_plain")
    _count()


def finish_rope_store(partial: torch.Tensor, splits: int, bias: Optional[torch.Tensor], qkv: torch.Tensor, positions,
                      tok_seg, block_tables, inv_freq: Optional[torch.Tensor], cache_k_ptr: Optional[int],
                      page_stride: int, v_offset: int, H: int, K: int, hd: int, rotary_dim: int, max_pages: int,
                      page_size: int, adjacent: bool = False, mscale: float = 1.0) -> None:
    """Sum the partials of the fused QKV product (+ bias), rotate Q and K, write Q into `qkv` and K, V into
    their pages (into `qkv` when cache_k_ptr is None)."""
    _dev(qkv, positions, tok_seg, block_tables, inv_freq, bias)
    n = qkv.shape[0]
    assert qkv.dtype == torch.bfloat16 and qkv.shape[1] == (H + 2 * K) * hd and partial.numel() >= splits * n * qkv.shape[1]
    _check(lib().xr_finish_rope_store(partial.data_ptr(), splits, _ptr(bias), qkv.data_ptr(), positions.data_ptr(),
                                      tok_seg.data_ptr(), block_tables.data_ptr(), _ptr(inv_freq), cache_k_ptr, page_stride,
                                      v_offset, n, H, K, hd, rotary_dim, max_pages, page_size, int(adjacent), float(mscale),
                                      _stream()), "finish_rope_store")
    _count()


# ---------------------------------------------------------------------------
def attention_mma_supported(dtype: torch.dtype, H: int, K: int, hd: int) -> bool:
    return dtype == torch.bfloat16 and hd % 16 == 0 and 16 <= hd <= 128 and H % K == 0 and H // K <= 16


def attention_mma_splits(max_kv_len: int, window: int, items: int) -> int:
    """Slots of scratch per (segment, kv head) pair that the key-split kernel needs for a step with `items` such
    pairs: its spans per request, or its CTAs over the pairs where it cuts the step's tiles into even shares."""
    return int(lib().xr_attention_mma_splits(max_kv_len, window, items))


def long_row_tiles(seg_len_host, heads_per_kv_head: int, rows_per_tile: int) -> int:
    """Row tiles of the portions that the prompt attention kernels take (more than 16 packed rows = tokens x query heads
    per kv head), summed: the x extent of their grids.  seg_len_host: the portions' lengths (numpy, on the host)."""
    rows = seg_len_host.astype("int64") * heads_per_kv_head
    return int(((rows + rows_per_tile - 1) // rows_per_tile)[rows > 16].sum())


def attention_even_launches() -> int:
    """How often the decode attention was launched in even shares (rather than in spans) so far."""
    return int(lib().xr_attention_even_launches())


def attention_wait_probe(device: torch.device, limit: int = 1 << 12) -> None:
    """Run the decode attention's bounded wait on a flag that nothing raises: it runs out after `limit` looks and the
    status word of `device` says so, as it would for a hand-over that never came (``tc_check_status`` then raises).
    Nothing faults and nothing hangs; this exists so that tests can drive the host's handling of that word."""
    ws = workspace(device)
    _check(lib().xr_attention_wait_probe(ws.flags.data_ptr() + 4 * (ws.flags.numel() - 1), ws.status.data_ptr(), int(limit),
                                         _stream()), "attention_wait_probe")


def attention_mma(q: torch.Tensor, q_row_stride: int, out: torch.Tensor, cache_k_ptr: int, seg_start, seg_len, seg_pos0,
                  block_tables, part_acc: Optional[torch.Tensor], part_ml: Optional[torch.Tensor], page_stride: int,
                  v_offset: int, H: int, K: int, hd: int, max_pages: int, page_size: int, window: int, scale: float,
                  n_seg: int, max_seg_len: int, max_kv_len: int, splits: int, any_short: bool, any_long: bool,
                  group: Optional[tuple] = None, uneven: bool = False, row_tiles: int = 0,
                  sink: Optional[torch.Tensor] = None, softcap: float = 0.0) -> None:
    """Causal attention over the pages on tensor cores (bfloat16); `softcap` c > 0: every scaled score s becomes c tanh(s / c).  Portions with at most 16 packed rows
    (tokens x heads per kv head) go through the key-split kernel and need `part_acc` [n_seg*K*splits*16*hd]
    and `part_ml` [n_seg*K*splits*32] float32 scratch; longer portions through the row-tiled kernel.
    `group` = (pointer to the cache group's array, its pages, its layers, this layer's index) lets the
    key-split kernel fetch whole page blocks with bulk copies (head sizes 64 and 128, power-of-two pages).
    `uneven`: the requests' lengths differ much; the kernel then cuts the tiles of all requests into even shares from
    fewer requests on than it does otherwise.  row_tiles: ``long_row_tiles(lengths, H // K, 64)``, which sizes the
    row-tiled kernel's grid exactly; 0: every portion gets the blocks of the longest.  `sink`: float32 [H]; exp(sink[h])
    joins the denominator of head h's softmax once."""
    _dev(out, seg_start, seg_len, seg_pos0, block_tables, part_acc, part_ml, sink)
    assert sink is None or (sink.dtype == torch.float32 and sink.numel() == H)
    assert q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and out.shape[1] == H * hd
    if any_short:
        assert part_acc is not None and part_acc.numel() >= n_seg * K * splits * 16 * hd
        assert part_ml is not None and part_ml.numel() >= n_seg * K * splits * 32
    ws = workspace(out.device)
    _check(lib().xr_attention_mma(q.data_ptr(), out.data_ptr(), cache_k_ptr, seg_start.data_ptr(), seg_len.data_ptr(),
                                  seg_pos0.data_ptr(), block_tables.data_ptr(), _ptr(part_acc), _ptr(part_ml),
                                  q_row_stride, page_stride, v_offset, n_seg, H, K, hd, max_pages, page_size, window,
                                  float(scale), max_seg_len, max_kv_len, splits, int(any_short), int(any_long),
                                  group[0] if group else None, group[1] if group else 0, group[2] if group else 1,
                                  group[3] if group else 0, ws.status.data_ptr() if group else None,
                                  ws.flags.data_ptr() if group else None, ws.flags.numel() if group else 0, int(uneven),
                                  row_tiles, _ptr(sink), float(softcap), _stream()), "attention_mma")
    _count((1 if any_long else 0) + (2 if any_short else 0))


def attention_tc_supported(dtype: torch.dtype, H: int, K: int, hd: int, page_size: int) -> bool:
    return dtype == torch.bfloat16 and bool(lib().xr_attention_tc_supported(H, K, hd, page_size))


def attention_tc(qkv: torch.Tensor, out: torch.Tensor, seg_start, seg_len, seg_pos0, block_tables, group: tuple,
                 H: int, K: int, hd: int, max_pages: int, page_size: int, window: int, scale: float, n_seg: int,
                 max_seg_len: int, row_tiles: int = 0, sink: Optional[torch.Tensor] = None, softcap: float = 0.0) -> None:
    """Causal attention of the portions with more than 16 packed rows on tcgen05 (S and O in tensor memory).
    qkv: the step's fused rows (Q heads first); group = (pointer to the cache group's array, pages, layers, layer).
    row_tiles: ``long_row_tiles(lengths, H // K, 128)``, which sizes the grid exactly; 0: every portion gets the blocks
    of the longest.  `sink`: float32 [H]; exp(sink[h]) joins the denominator of head h's softmax once."""
    _dev(qkv, out, seg_start, seg_len, seg_pos0, block_tables, sink)
    assert sink is None or (sink.dtype == torch.float32 and sink.numel() == H)
    n = qkv.shape[0]
    assert qkv.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and out.shape == (n, H * hd)
    status = tc_workspace(out.device)[1]
    _check(lib().xr_attention_tc(qkv.data_ptr(), out.data_ptr(), group[0], seg_start.data_ptr(), seg_len.data_ptr(),
                                 seg_pos0.data_ptr(), block_tables.data_ptr(), status.data_ptr(), qkv.stride(0), n, n_seg,
                                 H, K, hd, max_pages, page_size, window, float(scale), max_seg_len, row_tiles, group[1], group[2],
                                 group[3], _ptr(sink), float(softcap), _stream()), "attention_tc")
    _count()


# ---------------------------------------------------------------------------
# Kernels of blocks that run their sublayers side by side, of joined streams and of capped logits
def scaled_add(x: torch.Tensor, d: torch.Tensor, m: float) -> None:
    """x += m * d on float32 streams."""
    _dev(x, d)
    assert x.dtype == torch.float32 and d.dtype == torch.float32 and x.shape == d.shape
    _check(lib().xr_scaled_add(x.data_ptr(), d.data_ptr(), float(m), x.shape[0], x.shape[1], _stream()), "scaled_add")
    _count()


def stream_step(x: torch.Tensor, x0: Optional[torch.Tensor], v: Optional[torch.Tensor]) -> None:
    """x[t] += x0[t] + v on float32 streams [n, width]; v a float32 vector of width values; either may be None."""
    _dev(x, x0, v)
    assert x.dtype == torch.float32 and x.is_contiguous() and (x0 is None or (x0.dtype == torch.float32 and x0.shape == x.shape and x0.is_contiguous()))
    assert v is None or (v.dtype == torch.float32 and v.numel() == x.shape[1] and v.is_contiguous())
    _check(lib().xr_stream_step(x.data_ptr(), _ptr(x0), _ptr(v), x.shape[0], x.shape[1], _stream()), "stream_step")
    _count()


def sigmoid_gate(o: torch.Tensor, g: torch.Tensor, H: int, hd: int, Vd: int, each: bool) -> None:
    """o [n, H * hd] (hd columns a head, of which the first Vd are the head's) times sigmoid(g), in place: g [n, H * Vd], a gate
    per element (`each`), or g [n, H], a gate per head.  Rows of g may be strided (columns of a wider product)."""
    _dev(o)
    n = o.shape[0]
    assert g.is_cuda and o.dtype == g.dtype and o.stride(1) == 1 and g.stride(1) == 1 and o.shape[1] == H * hd and g.shape == (n, H * Vd if each else H)
    _check(lib().xr_sigmoid_gate(o.data_ptr(), o.stride(0), g.data_ptr(), g.stride(0), dtype_code(o.dtype), n, H, hd, Vd, int(each),
                                 _stream()), "sigmoid_gate")
    _count()


def concat_cast(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor) -> None:
    """out[t] = [a[t]; b[t]] of two float32 streams [n, width], in out's dtype."""
    _dev(a, b, out)
    n, width = a.shape
    assert a.dtype == torch.float32 and b.dtype == torch.float32 and b.shape == a.shape and out.shape == (n, 2 * width)
    _check(lib().xr_concat_cast(a.data_ptr(), b.data_ptr(), out.data_ptr(), dtype_code(out.dtype), n, width, _stream()), "concat_cast")
    _count()


def softcap(z: torch.Tensor, cap: float) -> None:
    """z <- cap * tanh(z / cap) in place on float32 logits."""
    _dev(z)
    assert z.dtype == torch.float32
    _check(lib().xr_softcap(z.data_ptr(), float(cap), z.numel(), _stream()), "softcap")
    _count()


# ---------------------------------------------------------------------------
# Latent attention (csrc/latent_attention.cu)
def latent_prep(q: torch.Tensor, down: Optional[torch.Tensor], positions, tok_seg, block_tables, freq: Optional[torch.Tensor],
                norm_w: Optional[torch.Tensor], cache_ptr: Optional[int], page_stride: int, H: int, D: int, R: int, C: int,
                rot_dims: int, max_pages: int, page_size: int, eps: float, adjacent: bool = False) -> None:
    """Rotate the rotated part of every head's query in `q` ([n, >= H (D + R)], rows may be strided) in place; from `down`
    ([n, >= C + R], rows may be strided) write the token's cache row [normed latent (C) | rotated key part (R)] (cache_ptr
    None: write nothing, `down` may be None).  freq: float64 [rot_dims / 2]; `adjacent`: pairs (2i, 2i + 1), else
    (i, i + rot_dims / 2)."""
    _dev(positions, tok_seg, block_tables, freq, norm_w)
    assert q.stride(1) == 1 and q.is_cuda and q.shape[1] >= H * (D + R)
    assert freq is None or freq.dtype == torch.float64
    if cache_ptr is not None:
        assert down is not None and down.stride(1) == 1 and down.dtype == q.dtype and down.shape[1] >= C + R
        assert norm_w.dtype == torch.float32 and norm_w.numel() == C
    _check(lib().xr_latent_prep(q.data_ptr(), dtype_code(q.dtype), q.stride(0), _ptr(down), 0 if down is None else down.stride(0),
                                positions.data_ptr(), tok_seg.data_ptr(), block_tables.data_ptr(), _ptr(freq), _ptr(norm_w), cache_ptr,
                                page_stride, q.shape[0], H, D, R, C, rot_dims, max_pages, page_size, float(eps), int(adjacent), _stream()),
           "latent_prep")
    _count()


def head_matmul(inp: torch.Tensor, in_col: int, head_in: int, w: torch.Tensor, transposed: bool, out: torch.Tensor,
                n: int, H: int, Kd: int, J: int, gate: Optional[torch.Tensor] = None, gate_col: int = 0, gate_each: bool = False) -> None:
    """out[t, h, j] = sum_k inp[t, in_col + h * head_in + k] * W_h(k, j) (* sigmoid(gate[t, gate_col + h]), or with `gate_each`
    * sigmoid(gate[t, gate_col + h * J + j])), float32 sums.
    w [H * Kd, J] with W_h(k, j) = w[h * Kd + k, j], or `transposed`: w [H * J, Kd] with W_h(k, j) = w[h * J + j, k].
    out is [n, H * J] (any of the two dtypes)."""
    assert w.is_contiguous() and inp.stride(1) == 1 and out.is_contiguous() and out.shape == (n, H * J)
    assert tuple(w.shape) == ((H * J, Kd) if transposed else (H * Kd, J))
    es = inp.element_size()
    w_head, w_k, w_j = (J * Kd, 1, Kd) if transposed else (Kd * J, J, 1)
    gptr = None if gate is None else gate.data_ptr() + gate_col * gate.element_size()
    _check(lib().xr_head_matmul(inp.data_ptr() + in_col * es, dtype_code(inp.dtype), inp.stride(0), head_in, w.data_ptr(),
                                dtype_code(w.dtype), w_head, w_k, w_j, out.data_ptr(), dtype_code(out.dtype), out.stride(0),
                                gptr, 0 if gate is None else dtype_code(gate.dtype), 0 if gate is None else gate.stride(0),
                                n, H, Kd, J, int(gate_each), _stream()), "head_matmul")
    _count()


def latent_attention(ql: torch.Tensor, proj: torch.Tensor, qr_col: int, head_qr: int, out: torch.Tensor, cache_ptr: int,
                     page_stride: int, positions, tok_seg, block_tables, H: int, C: int, R: int, max_pages: int,
                     page_size: int, scale: float, window: int = 0) -> None:
    """Causal softmax attention of every token over its request's cached rows [latent (C) | rotated key part (R)] (all of
    them, or the last `window` > 0 up to the token itself):
    ql [n, H * C] float32 (queries in the latent space), rotated query parts in `proj` (head h at column
    qr_col + h * head_qr), out [n, H * C] float32 = sum_j a_j latent_j."""
    _dev(ql, out, positions, tok_seg, block_tables)
    n = ql.shape[0]
    assert ql.dtype == torch.float32 and out.dtype == torch.float32 and ql.shape == (n, H * C) and out.shape == (n, H * C)
    _check(lib().xr_latent_attention(ql.data_ptr(), proj.data_ptr() + qr_col * proj.element_size(), dtype_code(proj.dtype),
                                     proj.stride(0), head_qr, out.data_ptr(), cache_ptr, page_stride, positions.data_ptr(),
                                     tok_seg.data_ptr(), block_tables.data_ptr(), n, H, C, R, max_pages, page_size, float(scale),
                                     int(window), _stream()), "latent_attention")
    _count()


def latent_attention_mma_supported(dtype: torch.dtype, D: int, R: int, C: int) -> bool:
    """Whether the tensor-core kernel takes these sizes: bfloat16, latent size a multiple of 64 up to 512, rotated part
    a multiple of 8, an even plain part (the query's pieces are read in pairs)."""
    return dtype == torch.bfloat16 and D % 2 == 0 and bool(lib().xr_latent_attention_mma_supported(C, R))


def latent_attention_splits(n: int, H: int, max_kv_len: int, sms: int = 148) -> tuple:
    """(keys per split, splits) for a step of n tokens whose longest context is max_kv_len: one split when the tokens
    alone fill the machine twice, else ranges of at least 128 keys, a multiple of 32."""
    base = n * (-(-H // 16))
    if base >= 2 * sms or max_kv_len <= 128:
        return max(32, -(-max_kv_len // 32) * 32), 1
    splits = max(1, min(-(-2 * sms // base), -(-max_kv_len // 128)))
    chunk = -(-(-(-max_kv_len // splits)) // 32) * 32
    return chunk, -(-max_kv_len // chunk)


def latent_attention_mma(ql: torch.Tensor, proj: torch.Tensor, qr_col: int, head_qr: int, out: torch.Tensor,
                         part_o: Optional[torch.Tensor], part_ml: Optional[torch.Tensor], cache_ptr: int, page_stride: int,
                         positions, tok_seg, block_tables, H: int, C: int, R: int, max_pages: int, page_size: int, scale: float,
                         chunk: int, splits: int, n_pad: Optional[int] = None, window: int = 0) -> None:
    """``latent_attention`` on tensor cores, bfloat16 queries and cache.  Token-major (n_pad None): ql [n, H * C], out
    [n, H * C] float32.  Head-major (n_pad given): ql and out are [H * n_pad, C] bfloat16, head h of token t in row
    h * n_pad + t (the layout of the grouped per-head products).  With `splits` > 1 every range of `chunk` keys is a
    CTA of its own and part_o [n * ceil(H/16) * splits * 16 * C] and part_ml [n * ceil(H/16) * splits * 32] (float32)
    carry their results to the kernel that merges them; the ranges start at the first key a token sees (`window` > 0: the
    last `window` keys up to the token itself)."""
    _dev(ql, out, positions, tok_seg, block_tables, part_o, part_ml)
    n = positions.numel()
    mt = -(-H // 16)
    assert ql.dtype == torch.bfloat16 and proj.dtype == torch.bfloat16
    if n_pad is None:
        assert out.dtype == torch.float32 and ql.shape == (n, H * C) and out.shape == (n, H * C)
        q_tok, q_head, o32, o16, o_tok, o_head = H * C, C, out.data_ptr(), None, 0, 0
    else:
        assert out.dtype == torch.bfloat16 and ql.shape == (H * n_pad, C) and out.shape == (H * n_pad, C) and n_pad >= n
        q_tok, q_head, o32, o16, o_tok, o_head = C, n_pad * C, None, out.data_ptr(), C, n_pad * C
    if splits > 1:
        assert part_o.numel() >= n * mt * splits * 16 * C and part_ml.numel() >= n * mt * splits * 32
    _check(lib().xr_latent_attention_mma(ql.data_ptr(), q_tok, q_head, proj.data_ptr() + qr_col * 2, proj.stride(0), head_qr, o32, o16,
                                         o_tok, o_head, _ptr(part_o), _ptr(part_ml), cache_ptr, page_stride, positions.data_ptr(),
                                         tok_seg.data_ptr(), block_tables.data_ptr(), n, H, C, R, max_pages, page_size, float(scale),
                                         chunk, splits, int(window), _stream()), "latent_attention_mma")
    _count(2 if splits > 1 else 1)


def heads_gather(inp: torch.Tensor, in_col: int, head_in: int, out: torch.Tensor, n: int, n_pad: int, H: int, Kd: int) -> None:
    """out[h * n_pad + t] = inp[t, in_col + h * head_in : ... + Kd] (bfloat16; rows t >= n are zeros)."""
    _dev(out)
    assert inp.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and out.shape == (H * n_pad, Kd) and inp.stride(1) == 1
    _check(lib().xr_heads_gather(inp.data_ptr() + 2 * in_col, inp.stride(0), head_in, out.data_ptr(), n, n_pad, H, Kd, _stream()), "heads_gather")
    _count()


def heads_scatter_gate(inp: torch.Tensor, y: torch.Tensor, gate: Optional[torch.Tensor], gate_col: int, n: int, n_pad: int, H: int, J: int,
                       gate_each: bool = False) -> None:
    """y[t, h * J + j] = inp[h * n_pad + t, j] * sigmoid(gate[t, gate_col + h]) (inp float32, y and gate bfloat16); with
    `gate_each` the gate is gate[t, gate_col + h * J + j]."""
    _dev(inp, y)
    assert inp.dtype == torch.float32 and y.dtype == torch.bfloat16 and inp.shape == (H * n_pad, J) and y.shape == (n, H * J)
    gptr = None if gate is None else gate.data_ptr() + 2 * gate_col
    _check(lib().xr_heads_scatter_gate(inp.data_ptr(), y.data_ptr(), gptr, 0 if gate is None else gate.stride(0), n, n_pad, H, J, int(gate_each), _stream()),
           "heads_scatter_gate")
    _count()


# ---------------------------------------------------------------------------
# Matrix-memory recurrence (csrc/mlstm.cu)
def mlstm_state_floats(H: int, D: int, V: int) -> int:
    return H * (D * V + D + 1)


def mlstm(proj: torch.Tensor, cols, gates: torch.Tensor, state: torch.Tensor, coef: torch.Tensor, o: torch.Tensor,
          norm_w: torch.Tensor, y: torch.Tensor, seg_start, seg_len, seg_slot, n_seg: int, H: int, D: int, V: int,
          cap: float, eps: float) -> None:
    """The recurrence over the step's tokens, request by request, from and into `state` [slots, H * (D V + D + 1)].
    proj [n, *]: q, k, v and the output gate at the columns `cols` = (q, k, v, g); gates [n, 2H] float32; coef
    [n, 3H] and o [n, H V] float32 scratch; y [n, H V] = o / rms(o per head) * norm_w * sigmoid(g)."""
    _dev(gates, state, coef, o, norm_w, y, seg_start, seg_len, seg_slot)
    n = proj.shape[0]
    assert proj.stride(1) == 1 and gates.dtype == torch.float32 and gates.shape == (n, 2 * H) and state.dtype == torch.float32
    assert state.shape[1] == mlstm_state_floats(H, D, V) and coef.numel() >= 3 * n * H and o.shape == (n, H * V)
    assert y.shape == (n, H * V) and y.dtype == proj.dtype and norm_w.dtype == torch.float32 and norm_w.numel() == H * V
    _check(lib().xr_mlstm(proj.data_ptr(), dtype_code(proj.dtype), proj.stride(0), cols[0], cols[1], cols[2], cols[3],
                          gates.data_ptr(), state.data_ptr(), coef.data_ptr(), o.data_ptr(), norm_w.data_ptr(), y.data_ptr(),
                          seg_start.data_ptr(), seg_len.data_ptr(), seg_slot.data_ptr(), n, n_seg, H, D, V, float(cap), float(eps),
                          _stream()), "mlstm")
    _count(3)


def head_norm_gate(o: torch.Tensor, gate: torch.Tensor, gate_col: int, w: torch.Tensor, y: torch.Tensor, H: int, V: int, eps: float,
                   per_head_weight: bool = False, silu: bool = False) -> None:
    """y [n, H V] = o / rms(o per head) * w * act(gate[:, gate_col + h V + i]): o float32 [n, H V]; y in the activation dtype, gate
    in y's dtype or float32; w float32, V values for all heads or (`per_head_weight`) H V; act the sigmoid, or SiLU with `silu`."""
    _dev(o, w, y)
    n = o.shape[0]
    assert o.dtype == torch.float32 and o.shape == (n, H * V) and y.shape == (n, H * V) and gate.stride(1) == 1
    assert gate.dtype in (y.dtype, torch.float32)
    assert w.dtype == torch.float32 and w.numel() == (H * V if per_head_weight else V) and gate.shape[1] >= gate_col + H * V
    _check(lib().xr_head_norm_gate(o.data_ptr(), gate.data_ptr() + gate_col * gate.element_size(), dtype_code(gate.dtype), gate.stride(0),
                                   w.data_ptr(), V if per_head_weight else 0, int(silu), y.data_ptr(), dtype_code(y.dtype), n, H, V,
                                   float(eps), _stream()), "head_norm_gate")
    _count()


# ---------------------------------------------------------------------------
# Gated delta rule (csrc/delta.cu)
def delta_state_floats(H: int, G: int, D: int, V: int, taps: int) -> int:
    """float32 values per request slot: S [H][V][D], then the last taps - 1 inputs of the convolutions' 2 G D + H V channels."""
    return H * V * D + (taps - 1) * (2 * G * D + H * V)


def delta(proj: torch.Tensor, conv_w: torch.Tensor, gates: torch.Tensor, neg_a: torch.Tensor, dt_bias: torch.Tensor,
          state: torch.Tensor, qkv: torch.Tensor, coef: torch.Tensor, o: torch.Tensor, tok_seg, seg_start, seg_len, seg_slot,
          n_seg: int, H: int, G: int, D: int, V: int, taps: int) -> None:
    """The gated delta rule over the step's tokens, request by request, from and into `state` [slots, delta_state_floats].
    proj [n, >= CH] (rows may be strided): the convolutions' channels q [G D], k [G D], v [H V] from column 0; conv_w [CH, taps]
    float32; gates [n, 2H] float32 (pre-activations of beta, then of the decay); neg_a = -exp(A_log) and dt_bias [H] float32;
    qkv [n, CH] and coef [n, 2H] float32 scratch; o [n, H V] float32 receives the read-outs."""
    _dev(conv_w, gates, neg_a, dt_bias, state, qkv, coef, o, tok_seg, seg_start, seg_len, seg_slot)
    n = proj.shape[0]
    CH = 2 * G * D + H * V
    assert proj.stride(1) == 1 and proj.shape[1] >= CH and conv_w.shape == (CH, taps) and conv_w.dtype == torch.float32
    assert gates.dtype == torch.float32 and gates.shape == (n, 2 * H) and state.dtype == torch.float32 and state.dim() == 2
    assert state.shape[1] >= delta_state_floats(H, G, D, V, taps) and neg_a.numel() == H and dt_bias.numel() == H
    assert neg_a.dtype == torch.float32 and dt_bias.dtype == torch.float32
    assert qkv.shape == (n, CH) and qkv.dtype == torch.float32 and coef.numel() >= 2 * n * H and coef.dtype == torch.float32
    assert o.shape == (n, H * V) and o.dtype == torch.float32
    _check(lib().xr_delta(proj.data_ptr(), dtype_code(proj.dtype), proj.stride(0), conv_w.data_ptr(), gates.data_ptr(), neg_a.data_ptr(),
                          dt_bias.data_ptr(), state.data_ptr(), state.stride(0), qkv.data_ptr(), coef.data_ptr(), o.data_ptr(),
                          tok_seg.data_ptr(), seg_start.data_ptr(), seg_len.data_ptr(), seg_slot.data_ptr(), n, n_seg, H, G, D, V, taps,
                          _stream()), "delta")
    _count(2)


# ---------------------------------------------------------------------------
# Routed experts (csrc/moe.cu)
def route_topk(z: torch.Tensor, ids: torch.Tensor, wts: torch.Tensor, top: int, sigmoid_scores: bool = False,
               correction: Optional[torch.Tensor] = None) -> None:
    """ids[t], wts[t]: the `top` largest of z[t] (ties: lower index) and the softmax over them alone.  With `sigmoid_scores` the
    scores are s = sigmoid(z): the `top` largest s + correction (float32 [E], optional) are chosen, and their weights are s as it is."""
    _dev(z, ids, wts, correction)
    assert correction is None or (sigmoid_scores and correction.dtype == torch.float32 and correction.numel() == z.shape[1])
    n, E = z.shape
    assert z.dtype == torch.float32 and ids.dtype == torch.int32 and wts.dtype == torch.float32
    assert ids.shape == (n, top) and wts.shape == (n, top)
    _check(lib().xr_route_topk(z.data_ptr(), ids.data_ptr(), wts.data_ptr(), n, E, top, _ptr(correction), int(sigmoid_scores),
                               _stream()), "route_topk")
    _count()


def moe_tile_rows() -> int:
    """Rows per tile of the FMA kernel of the experts' products (the alignment its plan needs)."""
    return int(lib().xr_moe_tile_rows())


def moe_max_tiles(pairs: int, E: int, align: int) -> int:
    """Tiles of `align` rows that a plan over `pairs` rows and E experts can need at most."""
    return pairs // align + E + 1


def moe_plan(ids: torch.Tensor, row_src, pair_row, tile_group, E: int, align: int) -> None:
    """Sort the (token, choice) pairs by expert on the device, every expert's rows starting at a multiple of `align`:
    row_src [max_tiles * align] (pair of a row, -1: padding), pair_row [pairs], tile_group [max_tiles] (expert of a
    tile, -1: no rows); see k_moe_plan in csrc/moe.cu."""
    _dev(ids, row_src, pair_row, tile_group)
    pairs = ids.numel()
    max_tiles = moe_max_tiles(pairs, E, align)
    assert row_src.numel() >= max_tiles * align and pair_row.numel() >= pairs and tile_group.numel() >= max_tiles
    _check(lib().xr_moe_plan(ids.data_ptr(), row_src.data_ptr(), pair_row.data_ptr(), tile_group.data_ptr(), pairs, E, align,
                             max_tiles, _stream()), "moe_plan")
    _count()


def moe_gather(h: torch.Tensor, out: torch.Tensor, row_src, tile_group, top: int, align: int) -> None:
    """out[r] = h[row_src[r] // top] for the rows of the plan's tiles (zeros for rows of padding)."""
    _dev(out, row_src, tile_group)
    assert h.stride(1) == 1 and out.shape[1] == h.shape[1] and out.dtype == h.dtype and out.shape[0] % align == 0
    _check(lib().xr_moe_gather(h.data_ptr(), dtype_code(h.dtype), h.stride(0), out.data_ptr(), row_src.data_ptr(),
                               tile_group.data_ptr(), top, h.shape[1], align, out.shape[0], _stream()), "moe_gather")
    _count()


def moe_gemm(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, row_src, tile_group, top: int,
             gated: bool, act: int = ACT_NONE, limit: float = 0.0) -> None:
    """The experts' products over the planned rows (a plan with align = moe_tile_rows()), float32 FMA.  gated:
    a = h [n, K], w [E, 2F, K], out [rows, F] = gate_act(h . w_gate, h . w_up); else a [rows, K], w [E, N, K], out [rows, N]."""
    _dev(a, w, out)
    E, rows, K = w.shape
    N = rows // 2 if gated else rows
    assert a.shape[1] == K and out.shape[1] == N and out.shape[0] % moe_tile_rows() == 0
    _check(lib().xr_moe_gemm(a.data_ptr(), dtype_code(a.dtype), a.stride(0), w.data_ptr(), dtype_code(w.dtype), out.data_ptr(),
                             dtype_code(out.dtype), out.stride(0), row_src.data_ptr(), tile_group.data_ptr(),
                             out.shape[0] // moe_tile_rows(), top, N, K, int(gated), int(act), float(limit), _stream()), "moe_gemm")
    _count()


def pack_weight_groups(w: torch.Tensor, halves: int = 1) -> torch.Tensor:
    """``pack_weight`` of every matrix of w [groups, rows, K], one after another: [groups, row tiles, K blocks, 128, 64]."""
    return torch.stack([pack_weight(w[g], halves) for g in range(w.shape[0])]).contiguous()


def gemm_tc_grouped(x: torch.Tensor, w_packed: torch.Tensor, out: torch.Tensor, tile_group: torch.Tensor, bn: int, n_out: int,
                    epilogue: int = EPI_STORE, act: int = ACT_NONE, act_limit: float = 0.0) -> None:
    """bfloat16 product on tcgen05 of rows sorted by group: tile t of `bn` rows of x multiplies by matrix
    tile_group[t] of w_packed (from ``pack_weight_groups``); tiles with tile_group below zero are skipped.
    EPI_STORE: out[r] = x[r] . w^T; EPI_GATED (halves = 2 packing): out[r][f] = gate_act(x . w_gate[f], x . w_up[f])."""
    _dev(x, w_packed, out, tile_group)
    n, k = x.shape
    assert x.dtype == torch.bfloat16 and w_packed.dtype == torch.bfloat16 and w_packed.dim() == 5 and n % bn == 0
    tiles = -(-n_out // GATED_FEATURES) if epilogue == EPI_GATED else -(-n_out // TILE_ROWS)
    assert w_packed.shape[1] == tiles and w_packed.shape[2] == -(-k // TILE_K) and out.shape == (n, n_out)
    assert tile_group.dtype == torch.int32 and tile_group.numel() >= n // bn
    ws = workspace(x.device)
    _check(lib().xr_gemm_tc_grouped(x.data_ptr(), w_packed.data_ptr(), out.data_ptr(), dtype_code(out.dtype), epilogue, int(act),
                                    float(act_limit), n, n_out, k, x.stride(0), out.stride(0), bn, tile_group.data_ptr(),
                                    w_packed.shape[0], ws.status_ptr, _stream()), "gemm_tc_grouped")
    _count()


def moe_combine(d: torch.Tensor, z: torch.Tensor, wts: torch.Tensor, pair_row: torch.Tensor, top: int) -> None:
    """d[t] += sum_j wts[t, j] * z[pair_row[t * top + j]] (float32)."""
    _dev(d, z, wts, pair_row)
    n, width = d.shape
    assert d.dtype == torch.float32 and z.dtype == torch.float32 and z.shape[1] == width
    _check(lib().xr_moe_combine(d.data_ptr(), z.data_ptr(), wts.data_ptr(), pair_row.data_ptr(), n, width, top, _stream()), "moe_combine")
    _count()


# ---------------------------------------------------------------------------
# Streams with other arrangements than the pre-norm block (csrc/stream.cu)
def embed_pair(table: torch.Tensor, pairs: torch.Tensor, ids, positions, tok_seg, seg_start, seg_slot, last: torch.Tensor, x: torch.Tensor,
               mul_prev: int, mul_cur: int, feed: Optional[torch.Tensor] = None) -> None:
    """x[t] = table[id_t] + pairs[(prev_t * mul_prev + id_t * mul_cur) mod buckets], buckets = pairs' rows - 1; a request's first
    token reads pairs' last row; prev_t of a portion's first token is last[slot] (int32 [slots], see ``last_token``)."""
    _dev(table, pairs, ids, positions, tok_seg, seg_start, seg_slot, last, x, feed)
    n, d = x.shape
    assert table.dtype == pairs.dtype and table.shape[1] == d and pairs.shape[1] == d and pairs.shape[0] >= 2
    assert x.dtype == torch.float32 and last.dtype == torch.int32 and ids.dtype == torch.int32
    _check(lib().xr_embed_pair(table.data_ptr(), pairs.data_ptr(), dtype_code(table.dtype), ids.data_ptr(), _ptr(feed),
                               0 if feed is None else feed.numel(), positions.data_ptr(), tok_seg.data_ptr(), seg_start.data_ptr(),
                               seg_slot.data_ptr(), last.data_ptr(), x.data_ptr(), n, d, table.shape[0], pairs.shape[0] - 1, int(mul_prev),
                               int(mul_cur), _stream()), "embed_pair")
    _count()


def last_token(ids, seg_start, seg_len, seg_slot, last: torch.Tensor, n_seg: int, vocab: int, feed: Optional[torch.Tensor] = None) -> None:
    """last[slot of portion s] = the portion's last token."""
    _dev(ids, seg_start, seg_len, seg_slot, last, feed)
    _check(lib().xr_last_token(ids.data_ptr(), _ptr(feed), 0 if feed is None else feed.numel(), seg_start.data_ptr(), seg_len.data_ptr(),
                               seg_slot.data_ptr(), last.data_ptr(), n_seg, vocab, _stream()), "last_token")
    _count()


def norm_add(d: torch.Tensor, x: torch.Tensor, gain: torch.Tensor, eps: float, cast: Optional[torch.Tensor] = None, clear: bool = False,
             partial: Optional[torch.Tensor] = None, splits: int = 0, bias: Optional[torch.Tensor] = None) -> None:
    """x[t] += d[t] / sqrt(mean(d[t]^2) + eps) * gain (one float32 number on the device); `cast` also receives the new x in its
    dtype; `clear` zeroes d behind the read.  `partial` (float32 [splits][n][width], with `bias`): partial sums of products cut
    along K that belong to d; the kernel adds them (split order, then the bias) to d's rows before it takes the norm."""
    _dev(d, x, gain, cast, partial, bias)
    assert partial is None or (partial.dtype == torch.float32 and splits >= 1 and partial.numel() >= splits * d.numel())
    assert bias is None or (partial is not None and bias.dtype == torch.float32 and bias.numel() == d.shape[1])
    n, w = x.shape
    assert d.shape == (n, w) and d.dtype == torch.float32 and x.dtype == torch.float32 and gain.dtype == torch.float32 and gain.numel() == 1
    assert cast is None or cast.shape == (n, w)
    _check(lib().xr_norm_add(d.data_ptr(), x.data_ptr(), gain.data_ptr(), _ptr(cast), 0 if cast is None else dtype_code(cast.dtype), n, w,
                             float(eps), int(clear), _ptr(partial), _ptr(bias), int(splits), _stream()), "norm_add")
    _count()


def row_norm_gate(o: torch.Tensor, gate: torch.Tensor, gate_col: int, w: torch.Tensor, y: torch.Tensor, eps: float, scale: float = 1.0) -> None:
    """y[t] = o[t] / sqrt(mean(o[t]^2) + eps) * w * sigmoid(gate[t, gate_col:gate_col + width]) * scale: one norm over the whole row;
    o, gate, w float32, y in the activation dtype."""
    _dev(o, w, y)
    n, width = o.shape
    assert o.dtype == torch.float32 and gate.dtype == torch.float32 and gate.stride(1) == 1 and gate.shape[1] >= gate_col + width
    assert w.dtype == torch.float32 and w.numel() == width and y.shape == (n, width)
    _check(lib().xr_row_norm_gate(o.data_ptr(), gate.data_ptr() + 4 * gate_col, gate.stride(0), w.data_ptr(), y.data_ptr(), dtype_code(y.dtype),
                                  n, width, float(eps), float(scale), _stream()), "row_norm_gate")
    _count()


def cast_rows(x: torch.Tensor, out: torch.Tensor) -> None:
    """out = x in out's dtype (x float32)."""
    _dev(x, out)
    assert x.dtype == torch.float32 and out.numel() == x.numel()
    _check(lib().xr_cast_rows(x.data_ptr(), out.data_ptr(), dtype_code(out.dtype), x.numel(), _stream()), "cast_rows")
    _count()


def depth_average(x: torch.Tensor, x0: torch.Tensor, hist: torch.Tensor, w: torch.Tensor, k: int, cast: Optional[torch.Tensor] = None) -> None:
    """hist[k-1] <- x;  x <- w[0] x0 + sum_(j=1..k-1) w[j] hist[j-1] + w[k] x (the old x); float32; `cast` also receives the new x."""
    _dev(x, x0, hist, w, cast)
    assert x.dtype == torch.float32 and x0.shape == x.shape and hist.dtype == torch.float32 and hist.shape[0] >= k and hist[0].numel() == x.numel()
    assert w.dtype == torch.float32 and w.numel() == k + 1
    _check(lib().xr_depth_average(x.data_ptr(), x0.data_ptr(), hist.data_ptr(), w.data_ptr(), _ptr(cast),
                                  0 if cast is None else dtype_code(cast.dtype), k, x.numel(), _stream()), "depth_average")
    _count()


def rotate_heads(rows: torch.Tensor, col0: int, heads: int, head_stride: int, dims: int, live: int, adjacent: bool, freq: torch.Tensor,
                 positions, sign: float = 1.0, scale: float = 1.0) -> None:
    """In place, for every row t and head h: the first `dims` elements at column col0 + h * head_stride are turned in pairs by
    sign * position_t * freq[m] (freq float64), then the head's first `live` elements are multiplied by `scale`."""
    _dev(freq, positions)
    assert rows.stride(1) == 1 and rows.is_cuda and rows.shape[1] >= col0 + (heads - 1) * head_stride + live
    assert freq.dtype == torch.float64 and freq.numel() >= dims // 2
    _check(lib().xr_rotate_heads(rows.data_ptr(), dtype_code(rows.dtype), rows.stride(0), col0, heads, head_stride, dims, live, int(adjacent),
                                 freq.data_ptr(), positions.data_ptr(), float(sign), float(scale), rows.shape[0], _stream()), "rotate_heads")
    _count()


# ---------------------------------------------------------------------------
# Linear recurrences (csrc/recurrent.cu)
def rglru_state_floats(R: int, taps: int) -> int:
    """float32 values per request slot: S [R], then the last taps - 1 inputs of the convolution [taps - 1][R]."""
    return R * taps


def rglru(proj: torch.Tensor, conv_w, conv_b, wa_t, wi_t, wa, wi, ba, bi, lam, state: torch.Tensor, tok_seg, seg_start, seg_len, seg_slot,
          a_s: torch.Tensor, b_s: torch.Tensor, u_s: torch.Tensor, out: torch.Tensor, n_seg: int, R: int, B: int, taps: int, c: float) -> None:
    """The real-gated linear recurrent unit over the step's tokens, request by request, from and into `state`.  proj [n, >= 2R]
    float32 (rows may be strided): the gated branch's pre-activations in columns [0, R), the convolution's inputs in [R, 2R).
    out [n, R] = S * gelu_tanh(gated branch).  wa, wi: the gates' matrices [B, out, in]; wa_t, wi_t: the same transposed to
    [B, in, out] (steps of many tokens read those).  See csrc/recurrent.cu for the other arguments."""
    _dev(conv_w, conv_b, wa_t, wi_t, wa, wi, ba, bi, lam, state, tok_seg, seg_start, seg_len, seg_slot, a_s, b_s, u_s, out)
    n = proj.shape[0]
    Bs = R // B
    assert u_s.dtype == torch.float32 and u_s.numel() >= n * R
    assert proj.dtype == torch.float32 and proj.stride(1) == 1 and proj.shape[1] >= 2 * R and out.shape == (n, R)
    assert all(t.dtype == torch.float32 for t in (conv_w, conv_b, wa_t, wi_t, wa, wi, ba, bi, lam, state, a_s, b_s))
    assert conv_w.shape == (R, taps) and all(t.shape == (B, Bs, Bs) for t in (wa_t, wi_t, wa, wi)) and a_s.numel() >= n * R and b_s.numel() >= n * R
    assert state.dim() == 2 and state.shape[1] >= rglru_state_floats(R, taps)
    _check(lib().xr_rglru(proj.data_ptr(), proj.stride(0), 0, R, conv_w.data_ptr(), conv_b.data_ptr(), wa_t.data_ptr(), wi_t.data_ptr(),
                          wa.data_ptr(), wi.data_ptr(), ba.data_ptr(), bi.data_ptr(), lam.data_ptr(), state.data_ptr(), state.stride(0), tok_seg.data_ptr(),
                          seg_start.data_ptr(), seg_len.data_ptr(), seg_slot.data_ptr(), a_s.data_ptr(), b_s.data_ptr(), u_s.data_ptr(), out.data_ptr(),
                          dtype_code(out.dtype), n, n_seg, R, B, taps, float(c), _stream()), "rglru")
    _count(3 if n <= 16 else 2)


def decay_attention(proj: torch.Tensor, cols, decay: torch.Tensor, state: torch.Tensor, seg_start, seg_len, seg_slot, o: torch.Tensor,
                    n_seg: int, H: int, D: int, V: int) -> None:
    """Linear attention with a constant decay per head: S <- decay_h S + k v^T, o = S^T q, with q, k, v = silu of proj's columns at
    cols = (q, k, v); proj float32 [n, *] (a step of many tokens activates those columns in place), state float32 [slots, >= H D V],
    o float32 [n, H V]."""
    _dev(decay, state, seg_start, seg_len, seg_slot, o)
    n = proj.shape[0]
    assert proj.dtype == torch.float32 and proj.stride(1) == 1 and o.shape == (n, H * V) and o.dtype == torch.float32
    assert decay.dtype == torch.float32 and decay.numel() == H and state.dtype == torch.float32 and state.shape[1] >= H * D * V
    _check(lib().xr_decay_attention(proj.data_ptr(), proj.stride(0), cols[0], cols[1], cols[2], decay.data_ptr(), state.data_ptr(),
                                    state.stride(0), seg_start.data_ptr(), seg_len.data_ptr(), seg_slot.data_ptr(), o.data_ptr(), n, n_seg, H, D, V,
                                    _stream()), "decay_attention")
    _count(2 if n > 16 else 1)
