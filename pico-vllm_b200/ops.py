"""Python face of the CUDA kernels: one function per kernel family.

Each function checks shapes, dtypes and devices on the host, refuses sizes the kernels do not
take with a :class:`KernelError`, and launches on torch's current CUDA stream.  The library is
loaded (and, if needed, compiled) at the first call.  There is no CPU path: tensors on another
device are refused.

Matrix products go to the library (``torch.mm``, cuBLAS), as in the reference, whose
projections are ``nn.Linear`` (pico_vllm/model.py:147-152, 309-312); everything else on the
forward path is a kernel of ``csrc/``.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .errors import KernelError

_F32, _BF16 = 0, 1
NORM_NONE, NORM_RMS, NORM_CENTRED = 0, 1, 2      # kinds of norm the row kernels have
NORM_COPY = 3      # as the output kind: no norm, the (added-to) stream row written out in the activation type
_lib = None
launches = 0  # kernels of this package launched so far (graph replays add their captured count)


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return _F32
    if t.dtype == torch.bfloat16:
        return _BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {t.dtype}")


def library():
    """The loaded kernel library (ctypes); loads and builds it at first use."""
    global _lib
    if _lib is not None:
        return _lib
    if not torch.cuda.is_available():
        raise KernelError("no CUDA device: this engine runs on a GPU only (there is no CPU path)")
    from .csrc import library_path
    path = library_path()
    try:
        lib = ctypes.CDLL(path)
    except OSError as e:
        raise KernelError(f"cannot load the kernel library {path}: {e}") from None
    vp, i32, f32, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong
    sigs = {
        "pico_embedding": [vp, vp, i32, vp, i32, i32, i32, vp, vp],
        "pico_add_rmsnorm": [vp, vp, vp, vp, vp, i32, i32, f32, i32, vp],
        "pico_swiglu": [vp, vp, i32, i32, i32, vp],
        "pico_rope_store": [vp, i32, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, vp],
        "pico_paged_attention_generic": [vp, i32, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32,
                                         i32, i32, f32, i32, f32, i32, vp, i32, vp, vp],
        "pico_paged_prefill_mma": [vp, i32, vp, vp, vp, vp, i32, vp, i32, vp, vp, i32, i32, i32, i32, i32, i32, f32, f32, vp, i32,
                                   vp, vp],
        "pico_paged_decode_mma": [vp, i32, vp, vp, vp, vp, vp, vp, i32, vp, vp, vp, i32, i32, i32, i32, i32, i32,
                                  f32, i32, f32, vp, i32, vp, vp],
        "pico_skinny_linear": [vp, i32, vp, vp, vp, i32, i32, i32, i32, i32, vp, f32, vp, vp],
        "pico_skinny_argmax": [vp, i32, vp, vp, i32, i32, i32, vp, f32, vp, vp],
        "pico_skinny_norm_fits": [i32, i32],
        "pico_skinny_linear_residual": [vp, i32, vp, vp, i32, i32, i32, vp],
        "pico_skinny_gate_up_swiglu": [vp, i32, vp, vp, i32, i32, i32, vp, f32, vp],
        "pico_skinny_qkv_rope_store": [vp, i32, vp, vp, vp, vp, vp, i32, vp, vp, vp, i32, i32, i32, i32, i32, i32, vp, f32,
                                       vp],
        "pico_make_kv_tensor_map": [vp, vp, i64, i32, i32],
        "pico_paged_decode_tma": [vp, vp, vp, i32, vp, vp, vp, vp, i32, vp, vp, vp, i32, i32, i32, i32, i32, i32,
                                  f32, i32, i32, f32, vp],
        "pico_tma_status": [vp],
        "pico_make_kv_tensor_map_2d": [vp, vp, i64, i32, i32, i32],
        "pico_paged_prefill_tcgen05": [vp, vp, vp, i32, vp, vp, i32, vp, i32, vp, vp, i32, i32, i32, i32, i32, i32, f32, i32,
                                       vp, i32, vp, i32, f32, vp, i32, vp, vp],
        "pico_tca_status": [vp],
        "pico_gemm_tcgen05_pair": [vp, i32, vp, vp, vp, i32, i32, i32, i32, i32, vp],
        "pico_tp_status": [vp],
        "pico_sample": [vp, i32, i32, i32, vp, vp, vp, vp, vp],
        "pico_post_add_norm": [vp, vp, vp, i32, f32, vp, i32, f32, vp, vp, i32, i32, i32, vp],
        "pico_scale_softcap": [vp, i32, i32, i32, f32, f32, vp],
        "pico_latent_norm_store": [vp, i32, i32, i32, vp, vp, i32, i32, vp, vp, vp, i32, i32, i32, vp, f32, i32, i32, vp],
        "pico_head_scale": [vp, vp, i32, i32, i32, i32, vp],
        "pico_moe_route": [vp, vp, vp, i32, i32, i32, i32, i32, vp, vp, i32, vp, f32, i32, i32, i32, vp],
        "pico_moe_group": [vp, i32, i32, i32, vp, vp, vp, vp, vp],
        "pico_moe_tile_rows": [i32, i32, i32, i32, i32],
        "pico_moe_gather": [vp, vp, i32, i32, i32, vp, vp],
        "pico_moe_combine_placed": [vp, vp, vp, i32, i32, i32, vp, vp, i32, vp, i32, vp, vp],
        "pico_moe_gemm": [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, vp, vp, vp, i32, f32, i32, vp],
        "pico_moe_combine": [vp, vp, i32, i32, i32, vp, vp, i32, vp, i32, vp, vp],
        "pico_moe_scaled_act": [vp, vp, vp, i32, i32, i32, vp, i32, vp],
        "pico_qk_norm_rope_store": [vp, i32, vp, vp, vp, f32, vp, vp, f32, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32,
                                    i32, i32, vp],
        "pico_sigmoid_gate": [vp, vp, i32, i32, i32, i32, vp],
        "pico_decay_linear_attention": [vp, i32, i32, i32, i32, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, vp,
                                        vp, i32, i32, vp],
        "pico_gated_rms_norm": [vp, vp, vp, i32, f32, vp, i32, i32, i32, vp],
        "pico_hyper_step": [vp, vp, vp, vp, vp, vp, f32, vp, vp, vp, i32, i32, i32, i32, vp],
        "pico_hyper_expand": [vp, vp, i32, i32, i32, vp],
        "pico_scale_add_rows": [vp, f32, vp, vp, i32, i32, i32, vp],
        "pico_gated_linear_attention": [vp, i32, vp, i32, vp, i32, vp, i32, i32, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32,
                                        i32, i32, i32, vp, vp, vp],
        "pico_scaled_sum": [vp, f32, vp, f32, vp, i64, i32, vp],
        "pico_mlstm_prepare": [vp, i32, i32, i32, i32, i32, i32, vp, vp, f32, f32, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32,
                               i32, i32, i32, i32, vp],
        "pico_hgrn2_prepare": [vp, i32, i32, i32, i32, vp, vp, vp, i32, i32, i32, i32, vp],
        "pico_causal_conv_silu": [vp, i32, i32, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, vp],
        "pico_mamba2_prepare": [vp, i32, i32, vp, vp, vp, i32, vp, vp, i32, i32, i32, i32, vp],
        "pico_group_rms_norm": [vp, i32, i32, i32, i32, vp, f32, vp, vp, i32, vp, i32, vp, i32, vp, i32, vp, i32, i32, vp],
        "pico_delta_prepare": [vp, i32, i32, i32, vp, i32, i32, vp, i32, vp, vp, vp, i32, i32, i32, i32, f32, f32, i32, vp],
        "pico_gated_delta_rule": [vp, vp, i32, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, vp],
        "pico_pair_rope_norm_store": [vp, i32, i32, i32, i32, vp, vp, i32, i32, vp, vp, f32, vp, vp, vp, vp, i32, i32, i32, i32,
                                      i32, i32, i32, i32, vp],
        "pico_sum_add_norm": [vp, vp, vp, i32, f32, f32, vp, vp, i32, f32, f32, vp, vp, i32, f32, f32, vp, i32, f32, vp, vp, i32,
                              i32, i32, vp],
        "pico_gelu_gate_rows": [vp, vp, i32, i32, vp, vp, i32, i32, i32, vp, i32, vp],
        "pico_capped_glu": [vp, i32, i32, i32, f32, f32, i32, vp, i32, vp],
        "pico_whole_norm_store": [vp, i32, i32, i32, i32, vp, vp, f32, i32, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32,
                                  i32, vp],
    }
    for name, args in sigs.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = ctypes.c_int
    _lib = lib
    return lib


def _check(code: int, what: str) -> None:
    if code == 0:
        return
    reasons = {-2: "an element type the kernel does not take", -3: "a size the kernel does not take",
               -4: "a misaligned row stride"}
    if code in reasons:
        raise KernelError(f"{what}: {reasons[code]}")
    raise KernelError(f"{what}: CUDA error {code} at launch")


def _stream() -> int:
    """The current CUDA stream's handle (the raw getter: torch.cuda.current_stream() costs ~14 us a call,
    which at ten launches a layer was a third of a step's host time)."""
    return torch._C._cuda_getCurrentRawStream(torch.cuda.current_device())


def _cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernel arguments must be CUDA tensors (there is no CPU path)")


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _count(n: int = 1) -> None:
    global launches
    launches += n


# ------------------------------------------------------------------------------------------
def embedding(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor,
              feedback: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t, :] = float32(table[ids[t], :]).  ids int32 [T]; table [V, H]; out float32 [T, H].
    With ``feedback`` (int32), an id -(j+1) means feedback[j]: the token the sampling kernel chose
    in the step before, which the host may not have read yet."""
    _cuda(ids, table, out, feedback)
    if feedback is not None and feedback.dtype != torch.int32:
        raise KernelError("embedding: feedback must be int32")
    T, (V, H) = ids.shape[0], table.shape
    if ids.dtype != torch.int32 or out.dtype != torch.float32 or out.shape != (T, H):
        raise KernelError("embedding: ids must be int32 [T] and out float32 [T, H]")
    if not (table.is_contiguous() and out.is_contiguous() and ids.is_contiguous()):
        raise KernelError("embedding: tensors must be contiguous")
    _check(library().pico_embedding(_ptr(ids), _ptr(table), _dtype_code(table), _ptr(out), T, H, V, _ptr(feedback),
                                    _stream()), "embedding")
    _count()
    return out


def add_rmsnorm(x: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Residual add and RMS norm in one pass.

    x float32 [T, H] is the residual stream.  Without ``rows``: x += delta (written back) and
    out = norm(x) * weight for every row.  With ``rows`` (int32 [R]): out[r] = norm(x[rows[r]] +
    delta[rows[r]]) * weight and x is not changed.  delta may be None.  weight float32 [H].
    """
    _cuda(x, delta, weight, out, rows)
    H = x.shape[1]
    R = rows.shape[0] if rows is not None else x.shape[0]
    if x.dtype != torch.float32 or weight.dtype != torch.float32 or weight.shape != (H,):
        raise KernelError("add_rmsnorm: x must be float32 [T, H] and weight float32 [H]")
    if out.shape != (R, H) or (delta is not None and (delta.shape != x.shape or delta.dtype != out.dtype)):
        raise KernelError("add_rmsnorm: out must be [rows, H] and delta like x in out's dtype")
    if rows is not None and rows.dtype != torch.int32:
        raise KernelError("add_rmsnorm: rows must be int32")
    if not (x.is_contiguous() and out.is_contiguous() and (delta is None or delta.is_contiguous())):
        raise KernelError("add_rmsnorm: tensors must be contiguous")
    _check(library().pico_add_rmsnorm(_ptr(x), _ptr(delta), _ptr(weight), _ptr(out), _ptr(rows), R, H,
                                      float(eps), _dtype_code(out), _stream()), f"add_rmsnorm (width {H})")
    _count()
    return out


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out = silu(gate_up[:, :I]) * gate_up[:, I:], float32 inside."""
    _cuda(gate_up, out)
    T, I = out.shape
    if gate_up.shape != (T, 2 * I) or gate_up.dtype != out.dtype:
        raise KernelError("swiglu: gate_up must be [T, 2*I] in out's dtype")
    if not (gate_up.is_contiguous() and out.is_contiguous()):
        raise KernelError("swiglu: tensors must be contiguous")
    _check(library().pico_swiglu(_ptr(gate_up), _ptr(out), T, I, _dtype_code(out), _stream()), "swiglu")
    _count()
    return out


def rope_store(qkv: torch.Tensor, bias: Optional[torch.Tensor], positions: torch.Tensor,
               inv_freq: torch.Tensor, slots: Optional[torch.Tensor], k_pages: Optional[torch.Tensor],
               v_pages: Optional[torch.Tensor], n_heads: int, n_kv_heads: int, head_dim: int,
               page_size: int, pairing: str = "half") -> None:
    """Adds the bias, rotates q (in place) and k, and stores k and v into their cache pages.
    ``pairing``: which dims rotate together; the kernels have "half" only (d with d + head_dim/2).

    qkv [T, (n_heads + 2 n_kv_heads) head_dim]; bias float32 or None; positions, slots int32 [T]
    (slot = page * page_size + offset, -1 = do not store); inv_freq float32 [rot_dim / 2];
    pages [num_pages, n_kv_heads, page_size, head_dim] in qkv's dtype.  With slots None only q
    is rotated.
    """
    _cuda(qkv, bias, positions, inv_freq, slots, k_pages, v_pages)
    _check_pairing(pairing, "rope_store")
    T = qkv.shape[0]
    width = (n_heads + 2 * n_kv_heads) * head_dim
    if qkv.shape[1] != width or qkv.stride(1) != 1:
        raise KernelError(f"rope_store: qkv must have {width} contiguous columns")
    if bias is not None and (bias.dtype != torch.float32 or bias.shape != (width,)):
        raise KernelError("rope_store: bias must be float32 of the qkv width")
    if positions.dtype != torch.int32 or inv_freq.dtype != torch.float32:
        raise KernelError("rope_store: positions int32, inv_freq float32")
    if slots is not None:
        if slots.dtype != torch.int32 or k_pages is None or v_pages is None:
            raise KernelError("rope_store: slots must be int32 and come with pages")
        for p in (k_pages, v_pages):
            if p.dtype != qkv.dtype or not p.is_contiguous() or tuple(p.shape[1:]) != (n_kv_heads, page_size, head_dim):
                raise KernelError("rope_store: pages must be contiguous [pages, kv_heads, page_size, head_dim] in qkv's dtype")
    _check(library().pico_rope_store(_ptr(qkv), qkv.stride(0), _ptr(bias), _ptr(positions), _ptr(inv_freq),
                                     _ptr(slots), _ptr(k_pages), _ptr(v_pages), T, n_heads, n_kv_heads,
                                     head_dim, 2 * inv_freq.shape[0], page_size, _dtype_code(qkv), _stream()),
           f"rope_store (head_dim {head_dim})")
    _count()


def _check_pairing(pairing: str, what: str) -> None:
    if pairing != "half":
        raise KernelError(f"{what}: rotary pairing {pairing!r} is not built (the kernels pair dim d with d + head_dim/2)")


def attention_scratch_floats(T: int, n_heads: int, head_dim: int, n_splits: int) -> int:
    """Float32 elements of scratch that paged_attention needs for n_splits > 1."""
    return 0 if n_splits <= 1 else T * n_heads * n_splits * (head_dim + 2)


def paged_attention(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, out: torch.Tensor,
                    tok_seg: torch.Tensor, positions: torch.Tensor, block_table: torch.Tensor,
                    n_heads: int, n_kv_heads: int, head_dim: int, page_size: int, window: Optional[int],
                    scale: float, n_splits: int = 1, scratch: Optional[torch.Tensor] = None,
                    softcap: Optional[float] = None, slopes: Optional[torch.Tensor] = None, chunk: Optional[int] = None,
                    sinks: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal attention of every token of the batch over its request's cache pages.
    ``softcap`` c: the scaled score s becomes c * tanh(s / c) before the softmax.
    ``slopes`` float32 [n_heads]: slopes[h] * (query position - key position) is taken off head h's scores.
    ``chunk`` C: the token at position p sees only keys from floor(p / C) * C on (positions count from the request's start).
    ``sinks`` float32 [n_heads]: head h's softmax has one more term exp(sinks[h]) in its denominator and no value for it.

    q: [T, >= n_heads*head_dim] rows (the qkv buffer, queries first); out [T, n_heads*head_dim];
    tok_seg int32 [T]: row of block_table for each token; positions int32 [T]; block_table int32
    [segments, width].  The token at position p sees keys max(0, p+1-window) .. p.  n_splits > 1
    cuts each token's key range into parts that run in parallel and needs ``scratch`` (float32,
    attention_scratch_floats elements).
    """
    _cuda(q, k_pages, v_pages, out, tok_seg, positions, block_table, scratch)
    T = q.shape[0]
    if head_dim % 16 != 0 or head_dim > 256:
        raise KernelError(f"paged_attention: head_dim must be a multiple of 16 up to 256, got {head_dim}")
    if n_heads % n_kv_heads != 0:
        raise KernelError("paged_attention: n_heads must be a multiple of n_kv_heads")
    if q.stride(1) != 1 or q.shape[1] < n_heads * head_dim or out.shape != (T, n_heads * head_dim):
        raise KernelError("paged_attention: bad q or out shape")
    if not (out.is_contiguous() and k_pages.is_contiguous() and v_pages.is_contiguous() and block_table.stride(1) == 1):
        raise KernelError("paged_attention: out, pages and block_table rows must be contiguous")
    if tuple(k_pages.shape[1:]) != (n_kv_heads, page_size, head_dim) or k_pages.shape != v_pages.shape:
        raise KernelError("paged_attention: pages must be [pages, kv_heads, page_size, head_dim]")
    if not (q.dtype == k_pages.dtype == v_pages.dtype == out.dtype):
        raise KernelError("paged_attention: q, pages and out must share one dtype")
    for t in (tok_seg, positions, block_table):
        if t.dtype != torch.int32:
            raise KernelError("paged_attention: index tensors must be int32")
    _cuda(slopes, sinks)
    for t in (slopes, sinks):
        if t is not None and (t.dtype != torch.float32 or t.shape != (n_heads,)):
            raise KernelError("paged_attention: slopes and sinks must be float32 [n_heads]")
    part_o = part_ml = None
    if n_splits > 1:
        need = attention_scratch_floats(T, n_heads, head_dim, n_splits)
        if scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need:
            raise KernelError(f"paged_attention: n_splits={n_splits} needs {need} float32 of scratch")
        part_o = scratch.data_ptr()
        part_ml = part_o + 4 * T * n_heads * n_splits * head_dim
    _check(library().pico_paged_attention_generic(
        _ptr(q), q.stride(0), _ptr(k_pages), _ptr(v_pages), _ptr(out), part_o, part_ml, _ptr(tok_seg),
        _ptr(positions), _ptr(block_table), block_table.stride(0), T, n_heads, n_kv_heads, head_dim, page_size,
        int(window) if window else 0, float(scale), n_splits, float(softcap) if softcap else 0.0, _dtype_code(q),
        _ptr(slopes), int(chunk) if chunk else 0, _ptr(sinks), _stream()),
        f"paged_attention (head_dim {head_dim})")
    _count(2 if n_splits > 1 else 1)
    return out


def mma_attention_takes(dtype: torch.dtype, n_heads: int, n_kv_heads: int, head_dim: int) -> bool:
    """True when the tensor-core attention kernels take these sizes (else use paged_attention)."""
    return (dtype == torch.bfloat16 and head_dim % 16 == 0 and 16 <= head_dim <= 256
            and n_heads % n_kv_heads == 0 and n_heads // n_kv_heads <= 16)


def make_kv_tensor_map(pages: torch.Tensor):
    """A TMA tensor map over the cache pages of one layer ([pages, kv_heads, page_size, head_dim]
    bfloat16, contiguous), for the TMA-fed decode kernel; None when the sizes are not taken (head_dim
    64 or 128, page size 8, 16, 32 or 64).  The returned object must be kept alive while it is used."""
    if not pages.is_cuda or pages.dtype != torch.bfloat16 or not pages.is_contiguous() or pages.dim() != 4:
        return None
    n_pages, nkv, ps, hd = pages.shape
    if hd not in (64, 128) or ps not in (8, 16, 32, 64):
        return None
    buf = (ctypes.c_ubyte * 192)()
    addr = ctypes.addressof(buf)
    aligned = (addr + 63) & ~63                      # a tensor map is 128 bytes on a 64-byte boundary
    rc = library().pico_make_kv_tensor_map(aligned, pages.data_ptr(), n_pages * nkv * ps, hd, ps)
    if rc != 0:
        return None
    return (buf, aligned)


def make_kv_tensor_map_2d(pages: torch.Tensor, values: bool = False):
    """Like :func:`make_kv_tensor_map`, with boxes of [page_size rows, 64 dims]: the operand layout of
    the tcgen05 prefill attention kernel; for the ``values`` a box holds all 64-dim blocks of the
    page rows, one after the other.  None when the sizes are not taken."""
    if not pages.is_cuda or pages.dtype != torch.bfloat16 or not pages.is_contiguous() or pages.dim() != 4:
        return None
    n_pages, nkv, ps, hd = pages.shape
    if hd not in (64, 128) or ps not in (8, 16, 32, 64):
        return None
    buf = (ctypes.c_ubyte * 192)()
    aligned = (ctypes.addressof(buf) + 63) & ~63
    if library().pico_make_kv_tensor_map_2d(aligned, pages.data_ptr(), n_pages * nkv * ps, hd, ps, 1 if values else 0) != 0:
        return None
    return (buf, aligned)


def tca_status() -> int:
    """0, or 1 when the tcgen05 attention kernel gave up waiting on a barrier since the library was loaded."""
    out = ctypes.c_int(0)
    library().pico_tca_status(ctypes.addressof(out))
    return out.value


def tma_status() -> int:
    """0, or 1 when a kernel gave up waiting for a TMA copy since the library was loaded."""
    out = ctypes.c_int(0)
    library().pico_tma_status(ctypes.addressof(out))
    return out.value


def check_kernel_status() -> None:
    """Raises KernelError when a kernel gave up a bounded wait (on a TMA copy or a tensor-core barrier)
    since the library was loaded: such a block leaves its part of the result unwritten, so the
    tokens computed since are not to be trusted.  Reads three status words from the device (a few
    synchronous 4-byte copies); does nothing before the library was first used."""
    if _lib is None:
        return
    bad = [name for name, word in (("paged_decode_tma (decode attention)", tma_status()),
                                   ("paged_prefill_tcgen05 (prompt attention)", tca_status()),
                                   ("gemm_tcgen05_pair (feed-forward product)", tc_status())) if word]
    if bad:
        raise KernelError("a bounded wait ran out in: " + ", ".join(bad) + "; results since then are invalid")


_PAIR_COUNTERS = {}


def _pair_counters(device: torch.device):
    """Zeroed int32 counters for the pairs of blocks that share a query tile in prompt attention (one per
    device; the kernel leaves them zero).  None while a graph is being recorded before they exist."""
    c = _PAIR_COUNTERS.get(device)
    if c is None:
        if torch.cuda.is_current_stream_capturing():
            return None
        c = _PAIR_COUNTERS[device] = torch.zeros(1 << 16, dtype=torch.int32, device=device)
    return c


def paged_attention_mma(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, out: torch.Tensor,
                        tok_seg: torch.Tensor, positions: torch.Tensor, block_table: torch.Tensor,
                        cu_q: torch.Tensor, prefill_segs: Optional[torch.Tensor], n_prefill_segs: int,
                        max_prefill_q: int, decode_tokens: Optional[torch.Tensor], n_decode_tokens: int,
                        n_heads: int, n_kv_heads: int, head_dim: int, page_size: int, window: Optional[int],
                        scale: float, n_splits: int = 1, scratch: Optional[torch.Tensor] = None,
                        k_map=None, v_map=None, k_map2d=None, v_map2d=None, pair_min_keys: int = 0,
                        softcap: Optional[float] = None, slopes: Optional[torch.Tensor] = None,
                        chunk: Optional[int] = None, sinks: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The same attention as :func:`paged_attention` for bfloat16 on tensor cores, in two launches:
    segments that bring two or more tokens (``prefill_segs`` int32 [n_prefill_segs], None = all
    segments; ``cu_q`` int32 [segments + 1]; ``max_prefill_q`` their longest) and single tokens
    (``decode_tokens`` int32 [n_decode_tokens], None = every token of the batch) whose key range is
    cut into ``n_splits`` parts.  Every token of the batch must be in exactly one of the two.
    With ``k_map`` / ``v_map`` (from :func:`make_kv_tensor_map` over these same pages) the single
    tokens run in the kernel that brings pages in by TMA; with ``k_map2d`` / ``v_map2d`` (from
    :func:`make_kv_tensor_map_2d`) the portions run on the tcgen05 tensor cores.
    ``slopes``, ``chunk`` and ``sinks`` as in :func:`paged_attention` (not together with ``softcap``); with them the
    single tokens run in the kernel that reads pages through the block table."""
    _cuda(q, k_pages, v_pages, out, tok_seg, positions, block_table, cu_q, prefill_segs, decode_tokens, scratch)
    T = q.shape[0]
    if not mma_attention_takes(q.dtype, n_heads, n_kv_heads, head_dim):
        raise KernelError(f"paged_attention_mma: bfloat16, head_dim multiple of 16 up to 256 and at most 16 query "
                          f"heads per kv head (got {q.dtype}, {head_dim}, {n_heads}/{n_kv_heads})")
    if q.stride(1) != 1 or q.shape[1] < n_heads * head_dim or out.shape != (T, n_heads * head_dim):
        raise KernelError("paged_attention_mma: bad q or out shape")
    if not (out.is_contiguous() and k_pages.is_contiguous() and v_pages.is_contiguous() and block_table.stride(1) == 1):
        raise KernelError("paged_attention_mma: out, pages and block_table rows must be contiguous")
    if tuple(k_pages.shape[1:]) != (n_kv_heads, page_size, head_dim) or k_pages.shape != v_pages.shape:
        raise KernelError("paged_attention_mma: pages must be [pages, kv_heads, page_size, head_dim]")
    if not (q.dtype == k_pages.dtype == v_pages.dtype == out.dtype):
        raise KernelError("paged_attention_mma: q, pages and out must share one dtype")
    for t in (tok_seg, positions, block_table, cu_q, prefill_segs, decode_tokens):
        if t is not None and t.dtype != torch.int32:
            raise KernelError("paged_attention_mma: index tensors must be int32")
    _cuda(slopes, sinks)
    for t in (slopes, sinks):
        if t is not None and (t.dtype != torch.float32 or t.shape != (n_heads,)):
            raise KernelError("paged_attention_mma: slopes and sinks must be float32 [n_heads]")
    lib = library()
    win = int(window) if window else 0
    cap = float(softcap) if softcap else 0.0
    chunk = int(chunk) if chunk else 0
    extra = slopes is not None or sinks is not None or chunk > 0
    if extra and cap > 0.0:
        raise KernelError("paged_attention_mma: a distance bias, chunks or a sink are not built together with a soft cap")
    if extra:
        k_map = v_map = None
    if n_prefill_segs > 0 and k_map2d is not None and v_map2d is not None:
        # pair_min_keys > 0 (and scratch for two partial results per (token, head)): every query tile gets two
        # blocks, which share it when it sees at least that many keys; the pairs' counters are zero between launches
        T = q.shape[0]
        counters = _pair_counters(q.device) if pair_min_keys > 0 else None
        split = (counters is not None and scratch is not None and scratch.dtype == torch.float32
                 and scratch.numel() >= 2 * T * n_heads * (head_dim + 2))
        _check(lib.pico_paged_prefill_tcgen05(k_map2d[1], v_map2d[1], _ptr(q), q.stride(0), _ptr(out),
                                              _ptr(prefill_segs), n_prefill_segs, _ptr(cu_q), max_prefill_q,
                                              _ptr(positions), _ptr(block_table), block_table.stride(0), n_heads,
                                              n_kv_heads, head_dim, page_size, win, float(scale),
                                              int(pair_min_keys) if split else 0, _ptr(scratch) if split else None, T,
                                              _ptr(counters) if split else None, counters.numel() if split else 0,
                                              cap, _ptr(slopes), chunk, _ptr(sinks), _stream()),
               f"paged_prefill_tcgen05 (head_dim {head_dim})")
        _count()
    elif n_prefill_segs > 0:
        _check(lib.pico_paged_prefill_mma(_ptr(q), q.stride(0), _ptr(k_pages), _ptr(v_pages), _ptr(out),
                                          _ptr(prefill_segs), n_prefill_segs, _ptr(cu_q), max_prefill_q,
                                          _ptr(positions), _ptr(block_table), block_table.stride(0), n_heads,
                                          n_kv_heads, head_dim, page_size, win, float(scale), cap, _ptr(slopes), chunk,
                                          _ptr(sinks), _stream()),
               f"paged_prefill_mma (head_dim {head_dim})")
        _count()
    if n_decode_tokens > 0:
        part_o = part_ml = None
        if n_splits > 1:
            need = attention_scratch_floats(T, n_heads, head_dim, n_splits)
            if scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need:
                raise KernelError(f"paged_attention_mma: n_splits={n_splits} needs {need} float32 of scratch")
            part_o = scratch.data_ptr()
            part_ml = part_o + 4 * T * n_heads * n_splits * head_dim
        if k_map is not None and v_map is not None:
            _check(lib.pico_paged_decode_tma(k_map[1], v_map[1], _ptr(q), q.stride(0), _ptr(out), part_o, part_ml,
                                             _ptr(decode_tokens), n_decode_tokens, _ptr(tok_seg), _ptr(positions),
                                             _ptr(block_table), block_table.stride(0), n_heads, n_kv_heads,
                                             head_dim, page_size, win, float(scale), n_splits,
                                             1 if k_pages.data_ptr() == v_pages.data_ptr() else 0, cap, _stream()),
                   f"paged_decode_tma (head_dim {head_dim})")
        else:
            _check(lib.pico_paged_decode_mma(_ptr(q), q.stride(0), _ptr(k_pages), _ptr(v_pages), _ptr(out), part_o,
                                             part_ml, _ptr(decode_tokens), n_decode_tokens, _ptr(tok_seg),
                                             _ptr(positions), _ptr(block_table), block_table.stride(0), n_heads,
                                             n_kv_heads, head_dim, page_size, win, float(scale), n_splits, cap,
                                             _ptr(slopes), chunk, _ptr(sinks), _stream()),
                   f"paged_decode_mma (head_dim {head_dim})")
        clustered = k_map is not None and v_map is not None and n_splits in (2, 4, 8, 16)
        _count(2 if n_splits > 1 and not clustered else 1)
    return out


# ------------------------------------------------------------------------------------------
# Products for a handful of tokens (decode): own kernels that stream the weights once and fuse
# what follows the product.  ``skinny_takes`` says whether the sizes fit; callers fall back to
# ``linear`` + the separate kernels otherwise.
SKINNY_MAX_TOKENS = 16


def skinny_takes(x: torch.Tensor, weight: torch.Tensor, n_multiple: int = 16) -> bool:
    return (x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
            and 1 <= x.shape[0] <= SKINNY_MAX_TOKENS and x.shape[1] % 16 == 0 and x.shape[1] >= 16
            and weight.shape[0] % n_multiple == 0 and weight.shape[0] >= 16
            and x.stride(1) == 1 and x.stride(0) % 8 == 0 and weight.is_contiguous())


def skinny_norm_takes(x: torch.Tensor, weight: torch.Tensor, n_rows: Optional[int] = None) -> bool:
    """True when the small-batch kernels can take the float32 residual stream ``x`` [*, K] itself and
    RMS-norm it on the way in (``n_rows`` rows of it, default all), instead of normed activations."""
    M = x.shape[0] if n_rows is None else n_rows
    return (x.is_cuda and x.dtype == torch.float32 and x.is_contiguous() and weight.dtype == torch.bfloat16
            and weight.is_contiguous() and weight.shape[0] % 16 == 0 and weight.shape[0] >= 16
            and weight.shape[1] == x.shape[1] and 1 <= M <= SKINNY_MAX_TOKENS
            and library().pico_skinny_norm_fits(M, x.shape[1]) == 1)


def _norm_args(x, norm_weight, what):
    if norm_weight is None:
        return None
    if x.dtype != torch.float32 or not x.is_contiguous() or norm_weight.dtype != torch.float32 \
            or norm_weight.shape != (x.shape[1],):
        raise KernelError(f"{what}: with a norm weight, x must be the contiguous float32 residual stream")
    return norm_weight


def skinny_linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
                  out_dtype: torch.dtype = torch.bfloat16, norm_weight: Optional[torch.Tensor] = None,
                  eps: float = 0.0, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [M<=16, K] times weight[N, K] transposed (+ bias), bfloat16 in, out bfloat16 or float32.
    With ``norm_weight``: x is the float32 residual stream and is RMS-normed on the way in
    (``rows`` int32 picks the rows to use)."""
    _cuda(x, weight, bias, norm_weight, rows)
    if _norm_args(x, norm_weight, "skinny_linear") is not None:
        M = rows.shape[0] if rows is not None else x.shape[0]
        if not skinny_norm_takes(x, weight, M) or (rows is not None and rows.dtype != torch.int32):
            raise KernelError("skinny_linear: sizes not taken with a fused norm")
    else:
        if not skinny_takes(x, weight):
            raise KernelError("skinny_linear: needs bfloat16, at most 16 tokens, K and N multiples of 16")
        M = x.shape[0]
    K = x.shape[1]
    N = weight.shape[0]
    out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    _check(library().pico_skinny_linear(_ptr(x), x.stride(0), _ptr(weight), _ptr(bias), _ptr(out), N,
                                        1 if out_dtype == torch.float32 else 0, M, N, K, _ptr(norm_weight),
                                        float(eps), _ptr(rows), _stream()), "skinny_linear")
    _count()
    return out


def skinny_argmax(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, norm_weight: Optional[torch.Tensor] = None,
                  eps: float = 0.0, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[m] = the first n with the largest (x weight^T)[m, n]: the greedy choice of an output head in the
    product's own epilogue, without writing the [M, N] logits.  x [M <= 16, K] bfloat16, or with ``norm_weight``
    the float32 residual stream, RMS-normed on the way in (``rows`` int32 picks its rows); out int32, at least M
    long.  Calls must follow one another on one stream (they share a table of partial results)."""
    _cuda(x, weight, out, norm_weight, rows)
    if _norm_args(x, norm_weight, "skinny_argmax") is not None:
        M = rows.shape[0] if rows is not None else x.shape[0]
        if not skinny_norm_takes(x, weight, M) or (rows is not None and rows.dtype != torch.int32):
            raise KernelError("skinny_argmax: sizes not taken with a fused norm")
    else:
        if not skinny_takes(x, weight):
            raise KernelError("skinny_argmax: needs bfloat16, at most 16 tokens, K and N multiples of 16")
        M = x.shape[0]
    if out.dtype != torch.int32 or out.dim() != 1 or out.shape[0] < M or not out.is_contiguous():
        raise KernelError("skinny_argmax: out must be int32 with room for one token per row")
    _check(library().pico_skinny_argmax(_ptr(x), x.stride(0), _ptr(weight), _ptr(out), M, weight.shape[0], x.shape[1],
                                        _ptr(norm_weight), float(eps), _ptr(rows), _stream()), "skinny_argmax")
    _count()
    return out


def skinny_linear_residual(x: torch.Tensor, weight: torch.Tensor, residual: torch.Tensor) -> None:
    """residual [M, N] float32 += x [M<=16, K] times weight[N, K] transposed, in one kernel."""
    _cuda(x, weight, residual)
    M, K = x.shape
    N = weight.shape[0]
    if not skinny_takes(x, weight) or residual.dtype != torch.float32 or residual.shape != (M, N) \
            or not residual.is_contiguous():
        raise KernelError("skinny_linear_residual: needs bfloat16 x and weight, float32 contiguous residual [M, N]")
    _check(library().pico_skinny_linear_residual(_ptr(x), x.stride(0), _ptr(weight), _ptr(residual), M, N, K,
                                                 _stream()), "skinny_linear_residual")
    _count()


def skinny_gate_up_swiglu(x: torch.Tensor, gate_up_weight: torch.Tensor, norm_weight: Optional[torch.Tensor] = None,
                          eps: float = 0.0) -> torch.Tensor:
    """silu(x wg^T) * (x wu^T) for gate_up_weight = [wg; wu] ([2I, K]); returns [M, I] bfloat16.
    With ``norm_weight``: x is the float32 residual stream and is RMS-normed on the way in."""
    _cuda(x, gate_up_weight, norm_weight)
    if _norm_args(x, norm_weight, "skinny_gate_up_swiglu") is not None:
        if not skinny_norm_takes(x, gate_up_weight):
            raise KernelError("skinny_gate_up_swiglu: sizes not taken with a fused norm")
    elif not skinny_takes(x, gate_up_weight):
        raise KernelError("skinny_gate_up_swiglu: needs bfloat16, at most 16 tokens, K and 2I multiples of 16")
    M, K = x.shape
    I = gate_up_weight.shape[0] // 2
    out = torch.empty((M, I), dtype=torch.bfloat16, device=x.device)
    _check(library().pico_skinny_gate_up_swiglu(_ptr(x), x.stride(0), _ptr(gate_up_weight), _ptr(out), M, I, K,
                                                _ptr(norm_weight), float(eps), _stream()), "skinny_gate_up_swiglu")
    _count()
    return out


def skinny_qkv_rope_store(x: torch.Tensor, qkv_weight: torch.Tensor, bias: Optional[torch.Tensor],
                          positions: torch.Tensor, inv_freq: torch.Tensor, slots: Optional[torch.Tensor],
                          k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor], n_heads: int,
                          n_kv_heads: int, head_dim: int, page_size: int,
                          norm_weight: Optional[torch.Tensor] = None, eps: float = 0.0,
                          pairing: str = "half") -> torch.Tensor:
    """qkv projection, bias, rotary encoding and cache store in one kernel; returns the rotated
    queries [M, n_heads * head_dim] bfloat16.  Same meaning as ``linear`` + ``rope_store``.
    With ``norm_weight``: x is the float32 residual stream and is RMS-normed on the way in."""
    _cuda(x, qkv_weight, bias, positions, inv_freq, slots, k_pages, v_pages, norm_weight)
    _check_pairing(pairing, "skinny_qkv_rope_store")
    M, K = x.shape
    takes = skinny_norm_takes(x, qkv_weight) if _norm_args(x, norm_weight, "skinny_qkv_rope_store") is not None \
        else skinny_takes(x, qkv_weight)
    if not takes or head_dim % 16 != 0 \
            or qkv_weight.shape[0] != (n_heads + 2 * n_kv_heads) * head_dim:
        raise KernelError("skinny_qkv_rope_store: sizes not taken")
    if bias is not None and (bias.dtype != torch.float32 or bias.shape != (qkv_weight.shape[0],)):
        raise KernelError("skinny_qkv_rope_store: bias must be float32 of the qkv width")
    if positions.dtype != torch.int32 or inv_freq.dtype != torch.float32:
        raise KernelError("skinny_qkv_rope_store: positions int32, inv_freq float32")
    if slots is not None:
        if slots.dtype != torch.int32 or k_pages is None or v_pages is None:
            raise KernelError("skinny_qkv_rope_store: slots must be int32 and come with pages")
        for pg in (k_pages, v_pages):
            if pg.dtype != torch.bfloat16 or not pg.is_contiguous() or tuple(pg.shape[1:]) != (n_kv_heads, page_size, head_dim):
                raise KernelError("skinny_qkv_rope_store: pages must be contiguous bfloat16 [pages, kv_heads, page_size, head_dim]")
    q = torch.empty((M, n_heads * head_dim), dtype=torch.bfloat16, device=x.device)
    _check(library().pico_skinny_qkv_rope_store(_ptr(x), x.stride(0), _ptr(qkv_weight), _ptr(bias), _ptr(q),
                                                _ptr(positions), _ptr(inv_freq), 2 * inv_freq.shape[0], _ptr(slots),
                                                _ptr(k_pages), _ptr(v_pages), M, K, n_heads, n_kv_heads, head_dim,
                                                page_size, _ptr(norm_weight), float(eps), _stream()),
           "skinny_qkv_rope_store")
    _count()
    return q


# ------------------------------------------------------------------------------------------
# Products for many tokens on the tcgen05 tensor cores (TMA-fed, accumulator in tensor memory, two SMs per tile).
# Measured for gate_up + SwiGLU at 17920 x 1536: the library product followed by the SwiGLU kernel takes 13.8 us at
# 64 tokens, 15.0 at 128, 17.1 at 200, 18.6 at 256; this kernel 17.1 us anywhere up to 256 tokens.  So the model's
# feed-forward takes the tcgen05 path from TC_PAIR_MIN_TOKENS = 200 tokens on; TC_MIN_TOKENS is what the kernel takes.
TC_MIN_TOKENS = 128


def tc_takes(x: torch.Tensor, weight: torch.Tensor) -> bool:
    return (x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.shape[0] >= TC_MIN_TOKENS
            and x.shape[1] % 8 == 0 and x.shape[1] >= 64 and weight.shape[0] % 16 == 0 and x.stride(1) == 1
            and x.stride(0) % 8 == 0 and weight.is_contiguous() and weight.shape[1] == x.shape[1])


def tc_status() -> int:
    """0, or 1 when the tcgen05 product kernel gave up waiting on a barrier since the library was loaded."""
    out = ctypes.c_int(0)
    library().pico_tp_status(ctypes.addressof(out))
    return out.value


TC_PAIR_MIN_TOKENS = 200      # from here on the tcgen05 path pays


def _tc_gemm(x, weight, out, residual, M, N, K, epi, rows, what):
    """The tcgen05 product kernel: a tile per pair of blocks (``tcgen05.mma.cta_group::2``).  ``rows``: None = the
    kernel picks its tile; 256 or 512 = that many rows of x per pair."""
    _check(library().pico_gemm_tcgen05_pair(_ptr(x), x.stride(0), _ptr(weight), _ptr(out), _ptr(residual), M, N, K,
                                            epi, int(rows or 0), _stream()), "gemm_tcgen05_pair" + what)
    _count()


def tc_linear(x: torch.Tensor, weight: torch.Tensor, rows=None) -> torch.Tensor:
    """x [M, K] times weight[N, K] transposed on the tcgen05 tensor cores; bfloat16 out."""
    _cuda(x, weight)
    if not tc_takes(x, weight):
        raise KernelError("tc_linear: needs bfloat16, at least 128 tokens, K a multiple of 8, N a multiple of 16")
    M, K = x.shape
    N = weight.shape[0]
    out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    _tc_gemm(x, weight, out, None, M, N, K, 0, rows, "")
    return out


def tc_linear_residual(x: torch.Tensor, weight: torch.Tensor, residual: torch.Tensor, rows=None) -> None:
    """residual [M, N] float32 += x [M, K] times weight[N, K] transposed."""
    _cuda(x, weight, residual)
    M, K = x.shape
    N = weight.shape[0]
    if not tc_takes(x, weight) or residual.dtype != torch.float32 or residual.shape != (M, N) \
            or not residual.is_contiguous():
        raise KernelError("tc_linear_residual: sizes not taken")
    _tc_gemm(x, weight, None, residual, M, N, K, 1, rows, " (residual)")


def tc_gate_up_swiglu(x: torch.Tensor, gate_up_weight: torch.Tensor, rows=None) -> torch.Tensor:
    """silu(x wg^T) * (x wu^T) for gate_up_weight = [wg; wu]; returns [M, I] bfloat16."""
    _cuda(x, gate_up_weight)
    if not tc_takes(x, gate_up_weight):
        raise KernelError("tc_gate_up_swiglu: sizes not taken")
    M, K = x.shape
    I = gate_up_weight.shape[0] // 2
    out = torch.empty((M, I), dtype=torch.bfloat16, device=x.device)
    _tc_gemm(x, gate_up_weight, out, None, M, 2 * I, K, 2, rows, " (swiglu)")
    return out


def linear(x: torch.Tensor, weight: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [T, K] times weight[N, K] transposed, a library matrix product (cuBLAS through torch).

    A weight kept in float32 beside bfloat16 activations is multiplied in float32 and the result
    rounded to bfloat16.  float32 products never use a reduced-precision (TF32) mode.
    """
    _cuda(x, weight)
    if x.dtype == weight.dtype:
        if out is None:
            return torch.mm(x, weight.t())
        return torch.mm(x, weight.t(), out=out)
    if weight.dtype == torch.float32 and x.dtype == torch.bfloat16:
        y = torch.mm(x.float(), weight.t()).to(torch.bfloat16)
        if out is not None:
            out.copy_(y)
            return out
        return y
    raise KernelError(f"linear: activations {x.dtype} with weights {weight.dtype} is not supported")


def logits_linear(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """Float32 logits x [R, K] times weight[V, K] transposed (library matrix product)."""
    _cuda(x, weight)
    if x.dtype == torch.float32 and weight.dtype == torch.float32:
        return torch.mm(x, weight.t())
    if skinny_takes(x, weight):
        return skinny_linear(x, weight, None, torch.float32)
    if x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16:
        return torch.mm(x, weight.t(), out_dtype=torch.float32)
    if x.dtype == torch.bfloat16 and weight.dtype == torch.float32:
        return torch.mm(x.float(), weight.t())
    raise KernelError(f"logits_linear: activations {x.dtype} with weights {weight.dtype} is not supported")


def sample(logits: torch.Tensor, temperature: Optional[torch.Tensor], top_p: Optional[torch.Tensor],
           uniform: Optional[torch.Tensor], out: torch.Tensor) -> torch.Tensor:
    """Chooses one token per row of float32 logits [R, V]: argmax where temperature is 0 (or
    temperature is None), else inverse-CDF sampling of softmax(logits / temperature) restricted
    to the top-p set, with the row's uniform number in [0, 1).  out int32 [R]."""
    _cuda(logits, temperature, top_p, uniform, out)
    R, V = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1 or out.dtype != torch.int32 or out.shape != (R,):
        raise KernelError("sample: logits float32 [R, V], out int32 [R]")
    for t in (temperature, top_p, uniform):
        if t is not None and (t.dtype != torch.float32 or t.shape != (R,)):
            raise KernelError("sample: temperature, top_p and uniform must be float32 [R]")
    if temperature is not None and uniform is None:
        raise KernelError("sample: sampling needs uniform numbers")
    _check(library().pico_sample(_ptr(logits), logits.stride(0), R, V, _ptr(temperature), _ptr(top_p),
                                 _ptr(uniform), _ptr(out), _stream()), "sample")
    _count()
    return out


# ------------------------------------------------------------------------------------------
# Norm of a sublayer's output, residual add and the next norm in one kernel.
def post_add_norm(x: torch.Tensor, delta: Optional[torch.Tensor], post_weight: Optional[torch.Tensor], post_kind: int,
                  post_eps: float, weight: Optional[torch.Tensor], kind: int, eps: float, out: Optional[torch.Tensor],
                  rows: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """x float32 [T, H] += N_post(delta) (written back unless ``rows`` picks rows), out = N(x).

    ``post_kind`` / ``kind``: NORM_NONE, NORM_RMS (u / sqrt(mean u^2 + eps) * w) or NORM_CENTRED ((u - mean u) /
    sqrt(mean (u - mean u)^2 + eps) * w); weights float32 [H].  delta (or None) and out are in the activation
    type; with ``rows`` (int32 [R]) out[r] is computed from row rows[r] and x is left alone; ``out`` None: the add
    alone."""
    _cuda(x, delta, post_weight, weight, out, rows)
    H = x.shape[1]
    R = rows.shape[0] if rows is not None else x.shape[0]
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise KernelError("post_add_norm: x must be contiguous float32 [T, H]")
    for w, k, what in ((post_weight, post_kind, "post_weight"), (weight, kind, "weight")):
        if k not in (NORM_NONE, NORM_RMS, NORM_CENTRED) and not (k == NORM_COPY and what == "weight"):
            raise KernelError(f"post_add_norm: unknown kind of norm {k}")
        if w is not None and (w.dtype != torch.float32 or w.shape != (H,)):
            raise KernelError(f"post_add_norm: {what} must be float32 [H]")
    if out is None and delta is None:
        return None
    like = out if out is not None else delta
    if delta is not None and (delta.shape != x.shape or delta.dtype != like.dtype or not delta.is_contiguous()):
        raise KernelError("post_add_norm: delta must be contiguous, shaped like x, in the activation type")
    if out is not None and (out.shape != (R, H) or not out.is_contiguous()):
        raise KernelError("post_add_norm: out must be contiguous [rows, H]")
    if rows is not None and rows.dtype != torch.int32:
        raise KernelError("post_add_norm: rows must be int32")
    _check(library().pico_post_add_norm(_ptr(x), _ptr(delta), _ptr(post_weight), int(post_kind), float(post_eps),
                                        _ptr(weight), int(kind) if out is not None else NORM_NONE, float(eps), _ptr(out),
                                        _ptr(rows), R, H, _dtype_code(like), _stream()), f"post_add_norm (width {H})")
    _count()
    return out


def scale_softcap(logits: torch.Tensor, scale: float, cap: Optional[float]) -> torch.Tensor:
    """In place on float32 logits [R, V]: y = y * scale, then y = cap * tanh(y / cap) when ``cap`` is given."""
    _cuda(logits)
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("scale_softcap: logits must be float32 [R, V] with contiguous rows")
    _check(library().pico_scale_softcap(_ptr(logits), logits.shape[0], logits.shape[1], logits.stride(0), float(scale),
                                        float(cap) if cap else 0.0, _stream()), "scale_softcap")
    _count()
    return logits


# ------------------------------------------------------------------------------------------
# Latent attention: what stands between its matrix products.
def latent_norm_store(proj: torch.Tensor, q_off: int, q_rank: int, q_weight: Optional[torch.Tensor], kv_off: int, kv_rank: int,
                      kv_weight: Optional[torch.Tensor], slots: Optional[torch.Tensor], cache: Optional[torch.Tensor],
                      g_off: int, heads: int, eps: float):
    """From a token's down projection row ``proj[t]`` (query latent at q_off, key/value latent at kv_off, one gate
    logit per head at g_off): the RMS-normed query latent [T, q_rank], the RMS-normed key/value latent into cache
    row ``slots[t]`` (``cache`` [..., row width >= kv_rank], zero beyond kv_rank; nothing for a slot of -1;
    kv_rank 0: no key/value part), and sigmoid of the gate logits (float32 [T, heads]).  ``q_rank`` 0: no query latent,
    ``heads`` 0: no gate; the part that is absent comes back as None.  Returns (cq, gate)."""
    _cuda(proj, q_weight, kv_weight, slots, cache)
    T = proj.shape[0]
    if proj.stride(1) != 1 or max(q_off + q_rank, kv_off + kv_rank, g_off + heads) > proj.shape[1]:
        raise KernelError("latent_norm_store: the projection row is narrower than its parts")
    if q_rank > 0 and (q_weight is None or q_weight.dtype != torch.float32 or q_weight.shape != (q_rank,)):
        raise KernelError("latent_norm_store: q_weight must be float32 [q_rank]")
    row = 0
    if kv_rank > 0:
        if kv_weight is None or kv_weight.dtype != torch.float32 or kv_weight.shape != (kv_rank,):
            raise KernelError("latent_norm_store: kv_weight must be float32 [kv_rank]")
        if slots is None or slots.dtype != torch.int32 or slots.shape[0] != T or cache is None \
                or cache.dtype != proj.dtype or not cache.is_contiguous() or cache.shape[-1] < kv_rank:
            raise KernelError("latent_norm_store: needs int32 slots and a contiguous cache of the activation type")
        row = cache.shape[-1]
    cq = torch.empty((T, q_rank), dtype=proj.dtype, device=proj.device) if q_rank > 0 else None
    gate = torch.empty((T, heads), dtype=torch.float32, device=proj.device) if heads > 0 else None
    _check(library().pico_latent_norm_store(_ptr(proj), proj.stride(0), q_off, q_rank, _ptr(q_weight), _ptr(cq), kv_off,
                                            kv_rank, _ptr(kv_weight), _ptr(slots), _ptr(cache) if kv_rank > 0 else None,
                                            row, g_off, heads, _ptr(gate), float(eps), T, _dtype_code(proj), _stream()),
           "latent_norm_store")
    _count()
    return cq, gate


def head_linear(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Per-head product: out[t, a, :] = gate[t, a] * (x[t, a, :] @ weight[a]) for x [T, H * K], weight [H, K, N], out
    [T, H * N]; ``gate`` float32 [T, H] or None: a strided batched library product over the heads, written straight
    into ``out``'s layout, and the gate kernel.  (A kernel of this package's own for up to 16 tokens, a thread per
    output feature with the gate in its epilogue, took 25 to 60 us a launch against 4 + 4 + 3 us and was dropped.)"""
    _cuda(x, weight, out, gate)
    T = x.shape[0]
    H, K, N = weight.shape
    if x.shape != (T, H * K) or out.shape != (T, H * N) or not (x.is_contiguous() and out.is_contiguous()
                                                                and weight.is_contiguous()):
        raise KernelError("head_linear: x [T, H K], weight [H, K, N] and out [T, H N] must be contiguous")
    if not (x.dtype == weight.dtype == out.dtype):
        raise KernelError("head_linear: x, weight and out must share one dtype")
    if gate is not None and (gate.dtype != torch.float32 or gate.shape != (T, H) or not gate.is_contiguous()):
        raise KernelError("head_linear: gate must be contiguous float32 [T, H]")
    torch.bmm(x.view(T, H, K).transpose(0, 1), weight, out=out.view(T, H, N).transpose(0, 1))
    if gate is not None:
        head_scale(out, gate, H)
    return out


def head_scale(o: torch.Tensor, gate: torch.Tensor, heads: int) -> torch.Tensor:
    """In place: o[t, h, :] *= gate[t, h] for o [T, heads * w] contiguous and gate float32 [T, heads]."""
    _cuda(o, gate)
    T = o.shape[0]
    if not o.is_contiguous() or o.shape[1] % heads or gate.dtype != torch.float32 or gate.shape != (T, heads) \
            or not gate.is_contiguous():
        raise KernelError("head_scale: o must be contiguous [T, heads * w] and gate float32 [T, heads]")
    _check(library().pico_head_scale(_ptr(o), _ptr(gate), T, heads, o.shape[1] // heads, _dtype_code(o), _stream()),
           "head_scale")
    _count()
    return o


# ------------------------------------------------------------------------------------------
# Routed experts.
MOE_SCORE_SOFTMAX_CHOSEN, MOE_SCORE_SIGMOID, MOE_SCORE_SOFTMAX_ALL = 0, 1, 2
MOE_ACT_SILU, MOE_ACT_RELU2, MOE_ACT_CAPPED = 0, 1, 2


def moe_route(h: torch.Tensor, router_weight: torch.Tensor, router_bias: Optional[torch.Tensor], top: int,
              scoring: int = MOE_SCORE_SOFTMAX_CHOSEN, choice_bias: Optional[torch.Tensor] = None, weight_scale: float = 1.0,
              groups: int = 1, groups_keep: int = 1, renorm: bool = False):
    """Router logits z = h W^T + b in float32, the ``top`` largest per token and the softmax over those alone
    (``scoring`` MOE_SCORE_SIGMOID: each chosen expert's weight is sigmoid(z) of its own logit, not renormalised;
    MOE_SCORE_SOFTMAX_ALL: an expert's score is its share of the softmax over all E logits, the ``top`` largest of score +
    ``choice_bias`` (float32 [E]) are chosen, and the weight is the score itself times ``weight_scale``, not renormalised -
    or, with ``renorm``, the score divided by the sum of the chosen scores (+ 1e-20) times ``weight_scale``; with ``groups`` > 1
    the experts form that many equal runs of neighbours and only the experts of the ``groups_keep`` runs whose largest
    score + choice_bias is largest can be chosen).
    h [T, D]; router_weight float32 [E, D]; router_bias float32 [E] or None.  Returns (idx int32 [T, top],
    weights float32 [T, top])."""
    _cuda(h, router_weight, router_bias)
    T, D = h.shape
    E = router_weight.shape[0]
    if not h.is_contiguous() or router_weight.dtype != torch.float32 or router_weight.shape != (E, D) \
            or not router_weight.is_contiguous():
        raise KernelError("moe_route: h must be contiguous [T, D] and the router weight float32 [E, D]")
    if router_bias is not None and (router_bias.dtype != torch.float32 or router_bias.shape != (E,)):
        raise KernelError("moe_route: the router bias must be float32 [E]")
    if choice_bias is not None and (choice_bias.dtype != torch.float32 or choice_bias.shape != (E,) or not choice_bias.is_cuda):
        raise KernelError("moe_route: the choice bias must be float32 [E]")
    if groups < 1 or E % groups or not 1 <= groups_keep <= groups or top > E // groups * groups_keep:
        raise KernelError(f"moe_route: {E} experts in {groups} groups of which {groups_keep} stay cannot give {top} choices")
    if (groups > 1 or renorm) and scoring != MOE_SCORE_SOFTMAX_ALL:
        raise KernelError("moe_route: groups and renormalised weights are built for the softmax over all experts")
    idx = torch.empty((T, top), dtype=torch.int32, device=h.device)
    wgt = torch.empty((T, top), dtype=torch.float32, device=h.device)
    _check(library().pico_moe_route(_ptr(h), _ptr(router_weight), _ptr(router_bias), T, D, E, top, int(scoring), _ptr(idx), _ptr(wgt),
                                    _dtype_code(h), _ptr(choice_bias), float(weight_scale), int(groups), int(groups_keep),
                                    1 if renorm else 0, _stream()),
           f"moe_route ({E} experts, top {top})")
    _count()
    return idx, wgt


def moe_experts(h: torch.Tensor, idx: torch.Tensor, wgt: torch.Tensor, gate_up_weight: torch.Tensor,
                down_weight: torch.Tensor, gated: bool = True, act: int = MOE_ACT_SILU, weight_on_input: bool = False,
                base: Optional[torch.Tensor] = None, identity: int = 0, limit: float = 0.0) -> torch.Tensor:
    """The routed experts' sum.  With e = idx[t, j]:

    gated, weight on the output (the default):  sum_j wgt[t, j] * down[e] (silu(gate[e] h_t) * (up[e] h_t)),
    gate_up_weight [E, 2 ff, D] (gate rows, then up rows);
    not gated:  sum_j down[e] act(up[e] (wgt[t, j] h_t)) with ``weight_on_input`` (the weight multiplies the float32
    result of the up product, which is the product of the weighted input), or sum_j wgt[t, j] * down[e] act(up[e] h_t)
    without; gate_up_weight is then the up matrices [E, ff, D]; ``act`` MOE_ACT_SILU or MOE_ACT_RELU2 (relu squared).

    The (token, j) entries are listed per expert on the device, the two products run as grouped products over those
    lists, and the sum is taken in float32; ``base`` [T, D] (a shared expert's output) is added in the same kernel.
    down_weight [E, D, ff]; all in h's type.  ``identity`` n: idx may also name E .. E + n - 1, experts without tensors whose
    output is their input (wgt[t, j] * h_t; weight on the output only).  ``act`` MOE_ACT_CAPPED (gated experts): with
    g' = min(gate h, limit) and u' = clamp(up h, -limit, limit) the expert is down (g' sigmoid(1.702 g') (u' + 1)).
    Returns [T, D] in h's type."""
    _cuda(h, idx, wgt, gate_up_weight, down_weight, base)
    T, D = h.shape
    top = idx.shape[1]
    E, ff_rows, _ = gate_up_weight.shape
    ff = ff_rows // 2 if gated else ff_rows
    if not (h.is_contiguous() and gate_up_weight.is_contiguous() and down_weight.is_contiguous()) \
            or gate_up_weight.shape != (E, (2 if gated else 1) * ff, D) or down_weight.shape != (E, D, ff) \
            or not (h.dtype == gate_up_weight.dtype == down_weight.dtype):
        raise KernelError("moe_experts: needs contiguous h [T, D], gate_up [E, 2 ff, D] (or up [E, ff, D]) and down [E, D, ff] "
                          "of one type")
    if idx.dtype != torch.int32 or wgt.dtype != torch.float32 or idx.shape != (T, top) or wgt.shape != (T, top) \
            or not (idx.is_contiguous() and wgt.is_contiguous()):
        raise KernelError("moe_experts: idx int32 [T, top] and wgt float32 [T, top]")
    if gated and (act not in (MOE_ACT_SILU, MOE_ACT_CAPPED) or weight_on_input):
        raise KernelError("moe_experts: gated experts are built with silu or the capped form and the weight on the output only")
    if act == MOE_ACT_CAPPED and not (gated and limit > 0.0):
        raise KernelError("moe_experts: the capped form is for gated experts and needs a positive limit")
    if base is not None and (base.shape != (T, D) or base.dtype != h.dtype or not base.is_contiguous()):
        raise KernelError("moe_experts: base must be contiguous [T, D] in h's type")
    if identity and (weight_on_input or identity < 0):
        raise KernelError("moe_experts: experts that pass their input on are built with the weight on the output only")
    n = T * top
    lib, code, st = library(), _dtype_code(h), _stream()
    grouped = moe_library_takes(h, n, D, ff)
    # entries are listed for the E real experts and, after them, for the ones that pass their input on: the products
    # below see the first E lists only (offsets[E] and tile_start[E] end the real entries), the sum reads h for the rest
    Et = E + identity
    meta = torch.empty(2 * (Et + 1) + 2 * n, dtype=torch.int32, device=h.device)
    offsets, tile_start = meta[:Et + 1], meta[Et + 1:2 * (Et + 1)]
    perm, place = meta[2 * (Et + 1):2 * (Et + 1) + n], meta[2 * (Et + 1) + n:]
    bm = lib.pico_moe_tile_rows(n, E, code, D, ff)      # rows per tile of this package's grouped kernels
    _check(lib.pico_moe_group(_ptr(idx), n, Et, bm, _ptr(offsets), _ptr(tile_start), _ptr(perm),
                              _ptr(place) if grouped else None, st), "moe_group")
    eidx, hsrc = (idx, h) if identity else (None, None)
    y = torch.empty((T, D), dtype=h.dtype, device=h.device)
    in_w = wgt if (not gated and weight_on_input) else None         # the weight inside the activation ...
    out_w = None if (not gated and weight_on_input) else wgt        # ... or on the expert's output
    if grouped:
        # many tokens: rows in expert order, the library's grouped products (their group ends are read on the device),
        # the activation kernel between them.  A shape the library refuses goes to this package's kernels below.
        try:
            xs = torch.empty((n, D), dtype=h.dtype, device=h.device)
            _check(lib.pico_moe_gather(_ptr(h), _ptr(perm), n, top, D * h.element_size(), _ptr(xs), st), "moe_gather")
            ends = offsets[1:E + 1]
            gu = torch._grouped_mm(xs, gate_up_weight.transpose(1, 2), offs=ends)
            if gated:
                if act == MOE_ACT_CAPPED:
                    a = capped_glu(gu, ff, limit)
                else:
                    a = torch.empty((n, ff), dtype=h.dtype, device=h.device)
                    swiglu(gu, a)
            else:
                a = gu
                _check(lib.pico_moe_scaled_act(_ptr(gu), _ptr(perm), _ptr(in_w), n, ff, int(act), _ptr(a), code, st),
                       "moe_scaled_act")
            ys = torch._grouped_mm(a, down_weight.transpose(1, 2), offs=ends)
            _check(lib.pico_moe_combine_placed(_ptr(ys), _ptr(place), _ptr(out_w), T, top, D, _ptr(y), _ptr(base), code, _ptr(eidx), E,
                                               _ptr(hsrc), st), "moe_combine_placed")
            _count(3)
            return y
        except (RuntimeError, NotImplementedError):
            if torch.cuda.is_current_stream_capturing():
                raise
    a = torch.empty((n, ff), dtype=h.dtype, device=h.device)
    _check(lib.pico_moe_gemm(_ptr(h), _ptr(gate_up_weight), _ptr(offsets), _ptr(tile_start), _ptr(perm), n, E, top, ff, D,
                             0 if gated else 2, bm, _ptr(a), None, _ptr(in_w), int(act), float(limit), code, st), "moe_gemm (up)")
    out2 = torch.empty((n, D), dtype=torch.float32, device=h.device)
    _check(lib.pico_moe_gemm(_ptr(a), _ptr(down_weight), _ptr(offsets), _ptr(tile_start), _ptr(perm), n, E, top, D, ff,
                             1, bm, None, _ptr(out2), None, 0, 0.0, code, st), "moe_gemm (down)")
    _check(lib.pico_moe_combine(_ptr(out2), _ptr(out_w), T, top, D, _ptr(y), _ptr(base), code, _ptr(eidx), E, _ptr(hsrc), st),
           "moe_combine")
    _count(4)
    return y


def activation(u: torch.Tensor, act: int) -> torch.Tensor:
    """In place on [n, ff]: silu (MOE_ACT_SILU) or relu squared (MOE_ACT_RELU2), float32 inside."""
    _cuda(u)
    if u.dim() != 2 or not u.is_contiguous():
        raise KernelError("activation: u must be contiguous [n, ff]")
    _check(library().pico_moe_scaled_act(_ptr(u), None, None, u.shape[0], u.shape[1], int(act), _ptr(u), _dtype_code(u),
                                         _stream()), "activation")
    _count()
    return u


# ------------------------------------------------------------------------------------------
# Attention with normed queries and keys; linear attention with a state.
def qk_norm_rope_store(qkv: torch.Tensor, bias: Optional[torch.Tensor], positions: torch.Tensor, inv_freq: torch.Tensor,
                       mult: float, q_norm: Optional[torch.Tensor], k_norm: Optional[torch.Tensor], eps: float,
                       slots: Optional[torch.Tensor], k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor],
                       n_heads: int, n_kv_heads: int, head_dim: int, page_size: int, values_from_keys: bool,
                       norm_dim: Optional[int] = None) -> None:
    """Per token row [q heads | k heads | v heads (absent with ``values_from_keys``) | anything]: adds the bias, stores the
    values (with ``values_from_keys``: the biased keys before norm and rotation), RMS-norms every q and k head over
    head_dim with the weights q_norm / k_norm (float32 [head_dim], shared by the heads; None: no norm), rotates the first
    2 * len(inv_freq) dims of each head (dim i with i + len(inv_freq)) by position * inv_freq with cos and sin times
    ``mult``, writes q back in place and k into its page.  float32 inside.  ``slots`` None: only q is treated.
    ``norm_dim``: the number of elements the norm's mean is taken over (heads padded with zeros up to head_dim)."""
    _cuda(qkv, bias, positions, inv_freq, q_norm, k_norm, slots, k_pages, v_pages)
    T = qkv.shape[0]
    cols = (n_heads + n_kv_heads * (1 if values_from_keys else 2)) * head_dim
    if qkv.dim() != 2 or qkv.shape[1] < cols or qkv.stride(1) != 1:
        raise KernelError(f"qk_norm_rope_store: rows must have at least {cols} contiguous columns")
    if bias is not None and (bias.dtype != torch.float32 or bias.shape[0] < cols or not bias.is_contiguous()):
        raise KernelError("qk_norm_rope_store: bias must be float32 over the q, k (and v) columns")
    for w in (q_norm, k_norm):
        if w is not None and (w.dtype != torch.float32 or w.shape != (head_dim,)):
            raise KernelError("qk_norm_rope_store: norm weights must be float32 [head_dim]")
    if positions.dtype != torch.int32 or inv_freq.dtype != torch.float32 or 2 * inv_freq.shape[0] > head_dim:
        raise KernelError("qk_norm_rope_store: positions int32, inv_freq float32 [<= head_dim / 2]")
    if slots is not None:
        if slots.dtype != torch.int32 or k_pages is None or v_pages is None:
            raise KernelError("qk_norm_rope_store: slots must be int32 and come with pages")
        for p in (k_pages, v_pages):
            if p.dtype != qkv.dtype or not p.is_contiguous() or tuple(p.shape[1:]) != (n_kv_heads, page_size, head_dim):
                raise KernelError("qk_norm_rope_store: pages must be contiguous [pages, kv_heads, page_size, head_dim] in qkv's dtype")
    _check(library().pico_qk_norm_rope_store(_ptr(qkv), qkv.stride(0), _ptr(bias), _ptr(positions), _ptr(inv_freq),
                                             float(mult), _ptr(q_norm), _ptr(k_norm), float(eps), _ptr(slots), _ptr(k_pages),
                                             _ptr(v_pages), T, n_heads, n_kv_heads if slots is not None else 0, head_dim,
                                             int(norm_dim or head_dim), 2 * inv_freq.shape[0], page_size, 1 if values_from_keys else 0,
                                             _dtype_code(qkv), _stream()), f"qk_norm_rope_store (head_dim {head_dim})")
    _count()


def sigmoid_gate(o: torch.Tensor, gate_logits: torch.Tensor) -> torch.Tensor:
    """In place: o[t, c] *= sigmoid(gate_logits[t, c]); gate_logits may be a column slice of a wider buffer."""
    _cuda(o, gate_logits)
    if o.dim() != 2 or not o.is_contiguous() or gate_logits.shape != o.shape or gate_logits.dtype != o.dtype \
            or gate_logits.stride(1) != 1:
        raise KernelError("sigmoid_gate: o contiguous [T, n], gate logits [T, n] of the same type with contiguous rows")
    _check(library().pico_sigmoid_gate(_ptr(o), _ptr(gate_logits), gate_logits.stride(0), o.shape[0], o.shape[1],
                                       _dtype_code(o), _stream()), "sigmoid_gate")
    _count()
    return o


def decay_linear_attention(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, decay: torch.Tensor,
                           state: torch.Tensor, seg_slots: torch.Tensor, cu_q: torch.Tensor, positions: torch.Tensor,
                           heads: int, dim: int, vdim: int, act: int = 1, max_q_len: int = 1,
                           chunk: Optional[int] = None) -> torch.Tensor:
    """Linear attention with a decay per head: per head S <- decay * S + k_t v_t^T, o_t = S^T q_t, token by token in
    the order of each segment, from and into ``state`` float32 [slots, heads, vdim, dim] (row ``seg_slots[s]`` for
    segment s; S stored transposed).  q, k, v of a token lie in its row of ``proj`` at q_off + h * dim, k_off + h * dim,
    v_off + h * vdim and pass through silu (``act`` 1) or nothing (0) in float32.  A segment whose first position is
    negative is padding.  Returns o float32 [T, heads * vdim].

    ``max_q_len``: the longest segment.  From LINEAR_CHUNK_MIN_TOKENS on the segments are cut into chunks of LINEAR_CHUNK
    tokens that run side by side (local states, a scan over the chunks, then the outputs); ``chunk`` overrides that
    policy (0: never)."""
    _cuda(proj, decay, state, seg_slots, cu_q, positions)
    T = proj.shape[0]
    S = seg_slots.shape[0]
    if proj.dim() != 2 or proj.stride(1) != 1 or max(q_off + heads * dim, k_off + heads * dim, v_off + heads * vdim) > proj.shape[1]:
        raise KernelError("decay_linear_attention: the projection row is narrower than its parts")
    if decay.dtype != torch.float32 or decay.shape != (heads,):
        raise KernelError("decay_linear_attention: decay must be float32 [heads]")
    if state.dtype != torch.float32 or not state.is_contiguous() or tuple(state.shape[1:]) != (heads, vdim, dim):
        raise KernelError("decay_linear_attention: state must be contiguous float32 [slots, heads, vdim, dim]")
    for t in (seg_slots, cu_q, positions):
        if t.dtype != torch.int32:
            raise KernelError("decay_linear_attention: index tensors must be int32")
    if cu_q.shape[0] != S + 1 or positions.shape[0] != T:
        raise KernelError("decay_linear_attention: cu_q must have one more entry than seg_slots, positions one per token")
    out = torch.empty((T, heads * vdim), dtype=torch.float32, device=proj.device)
    if chunk is None:
        chunk = LINEAR_CHUNK if max_q_len >= LINEAR_CHUNK_MIN_TOKENS else 0
    chunk_state = prepared = None
    if chunk > 0:
        chunk_state = torch.empty((T // chunk + S) * heads * vdim * dim, dtype=torch.float32, device=proj.device)
        prepared = torch.empty(T * heads * (2 * dim + vdim), dtype=torch.float32, device=proj.device)
    _check(library().pico_decay_linear_attention(_ptr(proj), proj.stride(0), q_off, k_off, v_off, _ptr(decay), _ptr(state),
                                                 _ptr(seg_slots), _ptr(cu_q), _ptr(positions), _ptr(out), S, heads, dim,
                                                 vdim, int(act), int(chunk), int(max(max_q_len, 1)), _ptr(chunk_state),
                                                 _ptr(prepared), T, _dtype_code(proj), _stream()),
           f"decay_linear_attention (dim {dim})")
    _count(4 if chunk > 0 else 1)
    return out


LINEAR_CHUNK = 64                  # tokens per chunk of the chunked form of decay_linear_attention
LINEAR_CHUNK_MIN_TOKENS = 256      # the longest segment of a step from which the chunked form is used


def gated_rms_norm(x: torch.Tensor, weight: Optional[torch.Tensor], gate_logits: Optional[torch.Tensor], eps: float,
                   out_dtype: torch.dtype) -> torch.Tensor:
    """y = x / sqrt(mean(x^2) + eps) * weight * sigmoid(gate_logits) over whole rows; x float32 [T, N]; weight float32
    [N] or None; gate_logits [T, N] in ``out_dtype`` (may be a column slice) or None.  Returns [T, N] in ``out_dtype``."""
    _cuda(x, weight, gate_logits)
    T, N = x.shape
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise KernelError("gated_rms_norm: x must be contiguous float32 [T, N]")
    if weight is not None and (weight.dtype != torch.float32 or weight.shape != (N,)):
        raise KernelError("gated_rms_norm: weight must be float32 [N]")
    if gate_logits is not None and (gate_logits.shape != (T, N) or gate_logits.dtype != out_dtype or gate_logits.stride(1) != 1):
        raise KernelError("gated_rms_norm: gate logits must be [T, N] in the output type with contiguous rows")
    y = torch.empty((T, N), dtype=out_dtype, device=x.device)
    _check(library().pico_gated_rms_norm(_ptr(x), _ptr(weight), _ptr(gate_logits),
                                         gate_logits.stride(0) if gate_logits is not None else 0, float(eps), _ptr(y), T, N,
                                         _dtype_code(y), _stream()), "gated_rms_norm")
    _count()
    return y


MOE_LIBRARY_MIN_ROWS = 1024       # (token, expert) pairs from which the library's grouped product is used


def moe_library_takes(h: torch.Tensor, n: int, D: int, ff: int) -> bool:
    """Whether the experts' products go to the library's grouped matrix product (bfloat16, many rows, row sizes
    that are multiples of 16 bytes) instead of this package's grouped kernels."""
    return (h.dtype == torch.bfloat16 and n >= MOE_LIBRARY_MIN_ROWS and D % 8 == 0 and ff % 8 == 0
            and hasattr(torch, "_grouped_mm"))


# ------------------------------------------------------------------------------------------ several residual streams
def hyper_expand(x: torch.Tensor, streams: int) -> torch.Tensor:
    """[T, D] float32 -> [T, streams, D]: every stream starts as a copy of the embedding stage's output."""
    _cuda(x)
    if x.dtype != torch.float32 or x.dim() != 2 or not x.is_contiguous() or streams < 1:
        raise KernelError("hyper_expand: x must be contiguous float32 [T, D]")
    T, D = x.shape
    out = torch.empty((T, streams, D), dtype=torch.float32, device=x.device)
    _check(library().pico_hyper_expand(_ptr(x), _ptr(out), T, streams, D, _stream()), "hyper_expand")
    _count()
    return out


def hyper_step(x: torch.Tensor, y: Optional[torch.Tensor], mix: Optional[torch.Tensor], out_w: Optional[torch.Tensor],
               in_w: Optional[torch.Tensor], norm_w: Optional[torch.Tensor], eps: float, out_dtype: torch.dtype,
               rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One pass over a token's residual streams x float32 [T, S, D]: first the write of the sublayer whose output ``y``
    [T, D] is still pending,  x_t <- sum_s mix[s, t] x_s + out_w[t] y  (all t from the old streams; skipped when y is
    None), then the read of the next one,  u = sum_s in_w[s] x_s  (``in_w`` None: the plain sum), RMS-normed with the
    weight ``norm_w`` float32 [D] and returned [T, D] in ``out_dtype``.  With ``rows`` (int32) only those tokens are read
    and x is not written."""
    _cuda(x, y, mix, out_w, in_w, norm_w, rows)
    if x.dtype != torch.float32 or x.dim() != 3 or not x.is_contiguous():
        raise KernelError("hyper_step: the streams must be contiguous float32 [T, S, D]")
    T, S, D = x.shape
    if y is not None and (y.shape != (T, D) or not y.is_contiguous() or y.dtype != out_dtype or mix is None or out_w is None):
        raise KernelError("hyper_step: the pending output must be contiguous [T, D] in the activation type, with its mix and out weights")
    for t, shape in ((mix, (S, S)), (out_w, (S,)), (in_w, (S,)), (norm_w, (D,))):
        if t is not None and (t.dtype != torch.float32 or tuple(t.shape) != shape or not t.is_contiguous()):
            raise KernelError(f"hyper_step: a weight must be contiguous float32 {list(shape)}")
    if rows is not None and rows.dtype != torch.int32:
        raise KernelError("hyper_step: rows must be int32")
    R = T if rows is None else rows.shape[0]
    h = torch.empty((R, D), dtype=out_dtype, device=x.device)
    _check(library().pico_hyper_step(_ptr(x), _ptr(y), _ptr(mix), _ptr(out_w), _ptr(in_w), _ptr(norm_w), float(eps), _ptr(h),
                                     _ptr(rows), None, R, S, D, _dtype_code(h), _stream()), f"hyper_step ({S} streams)")
    _count()
    return h


def scale_add_rows(x: torch.Tensor, scale: float, table: Optional[torch.Tensor], positions: Optional[torch.Tensor]) -> torch.Tensor:
    """x[t] <- x[t] * scale + table[positions[t]] in place on the float32 stream x [T, D] (a negative position gets no
    row; ``table`` None: the scale alone)."""
    _cuda(x, table, positions)
    if x.dtype != torch.float32 or x.dim() != 2 or not x.is_contiguous():
        raise KernelError("scale_add_rows: x must be contiguous float32 [T, D]")
    T, D = x.shape
    if table is not None and (table.dim() != 2 or table.shape[1] != D or not table.is_contiguous() or positions is None
                              or positions.dtype != torch.int32 or positions.shape[0] != T):
        raise KernelError("scale_add_rows: the table must be contiguous [rows, D] and positions int32 [T]")
    _check(library().pico_scale_add_rows(_ptr(x), float(scale), _ptr(table), _ptr(positions), T, D,
                                         _dtype_code(table) if table is not None else _F32, _stream()), "scale_add_rows")
    _count()
    return x


def scaled_sum(a: torch.Tensor, sa: float, b: torch.Tensor, sb: float) -> torch.Tensor:
    """sa * a + sb * b in float32, returned in the tensors' own type."""
    _cuda(a, b)
    if a.shape != b.shape or a.dtype != b.dtype or not a.is_contiguous() or not b.is_contiguous():
        raise KernelError("scaled_sum: two contiguous tensors of one shape and type")
    out = torch.empty_like(a)
    _check(library().pico_scaled_sum(_ptr(a), float(sa), _ptr(b), float(sb), _ptr(out), a.numel(), _dtype_code(a), _stream()),
           "scaled_sum")
    _count()
    return out


# ------------------------------------------------------------------------------------------ recurrences with gates per token
def _f32_rows(t: torch.Tensor, what: str) -> None:
    if t.dtype != torch.float32 or t.dim() != 2 or t.stride(1) != 1:
        raise KernelError(f"{what} must be float32 rows with contiguous columns")


def gated_linear_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, gate: torch.Tensor, per_row: bool,
                           state: torch.Tensor, seg_slots: torch.Tensor, cu_q: torch.Tensor, positions: torch.Tensor,
                           heads: int, qk_rep: int, dim: int, vdim: int, max_q_len: int = 1,
                           chunk: Optional[int] = None) -> torch.Tensor:
    """Per head h:  S <- diag(a_t) S + k_t v_t^T,  o_t = S^T q_t  (S [dim, vdim]), token by token in the order of each
    segment, from and into ``state`` float32 [slots, heads, vdim, dim] (S transposed; row ``seg_slots[s]``).  q, k, v and
    gate are float32 rows (column slices are fine): head h reads q and k at (h // qk_rep) * dim (``qk_rep`` heads share a
    query and key), v at h * vdim, and its gate a_t at h (one number a head, ``per_row`` False) or at h * dim .. (one a
    row of S).  A segment whose first position is negative is padding.  Returns o float32 [T, heads * vdim].
    Long segments (``max_q_len`` from LINEAR_CHUNK_MIN_TOKENS on, or ``chunk`` > 0) run as chunks side by side: local
    states and gate products, a scan, then the outputs."""
    _cuda(q, k, v, gate, state, seg_slots, cu_q, positions)
    for t, what in ((q, "q"), (k, "k"), (v, "v"), (gate, "gate")):
        _f32_rows(t, f"gated_linear_attention: {what}")
    T, S = q.shape[0], seg_slots.shape[0]
    groups = heads // max(qk_rep, 1)
    if qk_rep < 1 or heads % qk_rep or q.shape[1] < groups * dim or k.shape[1] < groups * dim or v.shape[1] < heads * vdim \
            or gate.shape[1] < heads * (dim if per_row else 1) or not (k.shape[0] == v.shape[0] == gate.shape[0] == T):
        raise KernelError("gated_linear_attention: a row is narrower than its heads")
    if state.dtype != torch.float32 or not state.is_contiguous() or tuple(state.shape[1:]) != (heads, vdim, dim):
        raise KernelError("gated_linear_attention: state must be contiguous float32 [slots, heads, vdim, dim]")
    for t in (seg_slots, cu_q, positions):
        if t.dtype != torch.int32:
            raise KernelError("gated_linear_attention: index tensors must be int32")
    if cu_q.shape[0] != S + 1 or positions.shape[0] != T:
        raise KernelError("gated_linear_attention: cu_q must have one more entry than seg_slots, positions one per token")
    out = torch.empty((T, heads * vdim), dtype=torch.float32, device=q.device)
    if chunk is None:
        chunk = LINEAR_CHUNK if max_q_len >= LINEAR_CHUNK_MIN_TOKENS else 0
    chunk_state = chunk_gate = None
    if chunk > 0:
        n = T // chunk + S
        chunk_state = torch.empty(n * heads * vdim * dim, dtype=torch.float32, device=q.device)
        chunk_gate = torch.empty(n * heads * dim, dtype=torch.float32, device=q.device)
    _check(library().pico_gated_linear_attention(
        _ptr(q), q.stride(0), _ptr(k), k.stride(0), _ptr(v), v.stride(0), _ptr(gate), gate.stride(0), 2 if per_row else 1,
        _ptr(state), _ptr(seg_slots), _ptr(cu_q), _ptr(positions), _ptr(out), out.stride(0), S, heads, qk_rep, dim, vdim,
        int(chunk), int(max(max_q_len, 1)), _ptr(chunk_state), _ptr(chunk_gate), _stream()),
        f"gated_linear_attention (dim {dim})")
    _count(3 if chunk > 0 else 1)
    return out


def mlstm_prepare(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, i_off: int, f_off: int,
                  i_bias: Optional[torch.Tensor], f_bias: Optional[torch.Tensor], cap: float, q_scale: float,
                  m_state: torch.Tensor, seg_slots: torch.Tensor, cu_q: torch.Tensor, positions: torch.Tensor,
                  heads: int, dim: int, vdim: int):
    """The gates of a matrix memory with exponential gating, kept finite by a running maximum m per head (``m_state``
    float32 [slots, heads], carried on):  i = cap tanh((z_i + b_i) / cap),  f = logsigmoid(cap tanh((z_f + b_f) / cap)),
    m_t = max(f + m_(t-1), i).  Returns (keep [T, heads] = exp(f + m_(t-1) - m_t), floor [T, heads] = exp(-m_t), prepared
    float32 [T, q: heads*dim | k: heads*dim | v: heads*(vdim+1)] with q * q_scale, k * exp(i - m_t), and one more column of
    ones after each head's values, whose row of the memory is the normaliser)."""
    _cuda(proj, i_bias, f_bias, m_state, seg_slots, cu_q, positions)
    T, S = proj.shape[0], seg_slots.shape[0]
    if proj.dim() != 2 or proj.stride(1) != 1 or max(q_off + heads * dim, k_off + heads * dim, v_off + heads * vdim,
                                                     i_off + heads, f_off + heads) > proj.shape[1]:
        raise KernelError("mlstm_prepare: the projection row is narrower than its parts")
    if m_state.dtype != torch.float32 or not m_state.is_contiguous() or tuple(m_state.shape[1:]) != (heads,):
        raise KernelError("mlstm_prepare: the running maximum must be contiguous float32 [slots, heads]")
    for t in (i_bias, f_bias):
        if t is not None and (t.dtype != torch.float32 or t.shape != (heads,)):
            raise KernelError("mlstm_prepare: gate biases must be float32 [heads]")
    dev = proj.device
    gates = torch.empty((3, T, heads), dtype=torch.float32, device=dev)
    prepared = torch.empty((T, 2 * heads * dim + heads * (vdim + 1)), dtype=torch.float32, device=dev)
    _check(library().pico_mlstm_prepare(_ptr(proj), proj.stride(0), q_off, k_off, v_off, i_off, f_off, _ptr(i_bias), _ptr(f_bias),
                                        float(cap), float(q_scale), _ptr(m_state), _ptr(seg_slots), _ptr(cu_q), _ptr(positions),
                                        _ptr(gates[0]), _ptr(gates[1]), _ptr(gates[2]), _ptr(prepared), T, S, heads, dim, vdim,
                                        _dtype_code(proj), _stream()), "mlstm_prepare")
    _count(2)
    return gates[0], gates[2], prepared


def hgrn2_prepare(proj: torch.Tensor, q_off: int, f_off: int, v_off: int, f_bias: Optional[torch.Tensor],
                  lower: Optional[torch.Tensor], nqk: int, nv: int) -> torch.Tensor:
    """float32 [T, q: nqk | k: nqk | f: nqk | v: nv] with q = silu(z_q), f = lower + (1 - lower) sigmoid(z_f + b_f) and
    k = 1 - f: a forget gate that also decides what is written."""
    _cuda(proj, f_bias, lower)
    T = proj.shape[0]
    if proj.dim() != 2 or proj.stride(1) != 1 or max(q_off + nqk, f_off + nqk, v_off + nv) > proj.shape[1]:
        raise KernelError("hgrn2_prepare: the projection row is narrower than its parts")
    for t in (f_bias, lower):
        if t is not None and (t.dtype != torch.float32 or t.shape != (nqk,)):
            raise KernelError("hgrn2_prepare: the gate's bias and lower bound must be float32 [heads * dim]")
    prepared = torch.empty((T, 3 * nqk + nv), dtype=torch.float32, device=proj.device)
    _check(library().pico_hgrn2_prepare(_ptr(proj), proj.stride(0), q_off, f_off, v_off, _ptr(f_bias), _ptr(lower), _ptr(prepared),
                                        T, nqk, nv, _dtype_code(proj), _stream()), "hgrn2_prepare")
    _count()
    return prepared


def causal_conv_silu(proj: torch.Tensor, c_off: int, weight: torch.Tensor, bias: Optional[torch.Tensor],
                     conv_state: torch.Tensor, tok_seg: torch.Tensor, seg_slots: torch.Tensor, cu_q: torch.Tensor,
                     positions: torch.Tensor, act: bool = True) -> torch.Tensor:
    """silu of a causal convolution per channel over the tokens of each segment: out[t, c] = silu(b[c] + sum_j w[c, j] *
    in(t - (taps - 1) + j, c)), the last tap on the token itself.  The channels are columns c_off .. of ``proj``; inputs from
    before the segment come from ``conv_state`` float32 [slots, taps - 1, C] (zero at a request's start), which afterwards
    holds the segment's last taps - 1 inputs.  ``act`` False: the convolution alone, no silu.  Returns float32 [T, C]."""
    _cuda(proj, weight, bias, conv_state, tok_seg, seg_slots, cu_q, positions)
    T, S = proj.shape[0], seg_slots.shape[0]
    C, taps = weight.shape
    if proj.dim() != 2 or proj.stride(1) != 1 or c_off + C > proj.shape[1]:
        raise KernelError("causal_conv_silu: the projection row is narrower than the channels")
    if weight.dtype != torch.float32 or not weight.is_contiguous() or (bias is not None and (bias.dtype != torch.float32 or bias.shape != (C,))):
        raise KernelError("causal_conv_silu: weight float32 [C, taps], bias float32 [C]")
    if conv_state.dtype != torch.float32 or not conv_state.is_contiguous() or tuple(conv_state.shape[1:]) != (taps - 1, C):
        raise KernelError("causal_conv_silu: the state must be contiguous float32 [slots, taps - 1, C]")
    out = torch.empty((T, C), dtype=torch.float32, device=proj.device)
    _check(library().pico_causal_conv_silu(_ptr(proj), proj.stride(0), c_off, _ptr(weight), _ptr(bias), _ptr(conv_state),
                                           _ptr(tok_seg), _ptr(seg_slots), _ptr(cu_q), _ptr(positions), _ptr(out), T, S, C, taps,
                                           _dtype_code(proj), 1 if act else 0, _stream()), f"causal_conv_silu ({taps} taps)")
    _count(2 if taps > 1 else 1)
    return out


def mamba2_prepare(proj: torch.Tensor, dt_off: int, dt_bias: Optional[torch.Tensor], a_log: torch.Tensor, x: torch.Tensor,
                   heads: int, vdim: int):
    """Step size and decay of a state-space layer: dt = softplus(z_dt + dt_bias) (no clamp), keep [T, heads] =
    exp(-exp(a_log) dt), vdt [T, heads * vdim] = dt * x.  x: float32 rows (a column slice is fine)."""
    _cuda(proj, dt_bias, a_log, x)
    T = proj.shape[0]
    _f32_rows(x, "mamba2_prepare: x")
    if proj.dim() != 2 or proj.stride(1) != 1 or dt_off + heads > proj.shape[1] or x.shape[1] < heads * vdim or x.shape[0] != T:
        raise KernelError("mamba2_prepare: a row is narrower than its heads")
    for t in (dt_bias, a_log):
        if t is not None and (t.dtype != torch.float32 or t.shape != (heads,)):
            raise KernelError("mamba2_prepare: dt_bias and a_log must be float32 [heads]")
    keep = torch.empty((T, heads), dtype=torch.float32, device=proj.device)
    vdt = torch.empty((T, heads * vdim), dtype=torch.float32, device=proj.device)
    _check(library().pico_mamba2_prepare(_ptr(proj), proj.stride(0), dt_off, _ptr(dt_bias), _ptr(a_log), _ptr(x), x.stride(0),
                                         _ptr(keep), _ptr(vdt), T, heads, vdim, _dtype_code(proj), _stream()), "mamba2_prepare")
    _count()
    return keep, vdt


def group_rms_norm(x: torch.Tensor, groups: int, n: int, group_stride: int, weight: Optional[torch.Tensor], eps: float,
                   out_dtype: torch.dtype, den_floor: Optional[torch.Tensor] = None, skip: Optional[torch.Tensor] = None,
                   skip_w: Optional[torch.Tensor] = None, skip_head: int = 1, pre_gate: Optional[torch.Tensor] = None,
                   post_gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The norm that finishes a recurrent mixer, a root mean square per group of ``n`` columns (group g starts at column
    g * group_stride of x, float32 rows).  For column j of group g, col = g * n + j, in this order:
      ``den_floor`` [T, groups]: val /= max(|x[t, g * group_stride + n]|, den_floor[t, g]) + 1e-6 (a normaliser that rides
      as column n of its group);  ``skip`` (float32 rows) with ``skip_w``: val += skip_w[col // skip_head] * skip[t, col];
      ``pre_gate``: val *= silu(pre_gate[t, col]);  y = val / sqrt(mean_j val^2 + eps) * weight[col];
      ``post_gate``: y *= sigmoid(post_gate[t, col]).  Gates are in ``out_dtype`` (column slices are fine).
    Returns [T, groups * n] in ``out_dtype``."""
    _cuda(x, weight, den_floor, skip, skip_w, pre_gate, post_gate)
    _f32_rows(x, "group_rms_norm: x")
    T, N = x.shape[0], groups * n
    if x.shape[1] < (groups - 1) * group_stride + n + (1 if den_floor is not None else 0):
        raise KernelError("group_rms_norm: x is narrower than its groups")
    if weight is not None and (weight.dtype != torch.float32 or weight.shape != (N,)):
        raise KernelError("group_rms_norm: weight must be float32 [groups * n]")
    if den_floor is not None and (den_floor.dtype != torch.float32 or den_floor.shape != (T, groups) or not den_floor.is_contiguous()):
        raise KernelError("group_rms_norm: den_floor must be contiguous float32 [T, groups]")
    if skip is not None:
        _f32_rows(skip, "group_rms_norm: skip")
        if skip.shape[1] < N or skip_w is None or skip_w.dtype != torch.float32 or skip_w.numel() * skip_head < N:
            raise KernelError("group_rms_norm: skip needs float32 weights, one per skip_head columns")
    for g in (pre_gate, post_gate):
        if g is not None and (g.dtype != out_dtype or g.dim() != 2 or g.stride(1) != 1 or g.shape[0] != T or g.shape[1] < N):
            raise KernelError("group_rms_norm: gates must be rows in the output type")
    y = torch.empty((T, N), dtype=out_dtype, device=x.device)
    _check(library().pico_group_rms_norm(_ptr(x), x.stride(0), group_stride, groups, n, _ptr(weight), float(eps), _ptr(den_floor),
                                         _ptr(skip), skip.stride(0) if skip is not None else 0, _ptr(skip_w), int(skip_head),
                                         _ptr(pre_gate), pre_gate.stride(0) if pre_gate is not None else 0, _ptr(post_gate),
                                         post_gate.stride(0) if post_gate is not None else 0, _ptr(y), T, _dtype_code(y), _stream()),
           "group_rms_norm")
    _count()
    return y


def whole_norm_store(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, q_w: Optional[torch.Tensor],
                     k_w: Optional[torch.Tensor], eps: float, v_norm: bool, slots: Optional[torch.Tensor],
                     k_pages: torch.Tensor, v_pages: torch.Tensor, heads: int, kv_heads: int, dim: int, vdim: int, row: int,
                     page_size: int) -> torch.Tensor:
    """Queries and keys RMS-normed over their whole projection (all heads of a token at once; weights ``q_w`` float32
    [heads * dim], ``k_w`` [kv_heads * dim]; None: no norm), values divided by their root mean square per head (``v_norm``),
    keys and values written to the token's place in the pages [pages, kv_heads, page_size, row] (``slots`` int32; -1 or None:
    not stored).  Heads are padded with zeros to ``row`` elements.  Returns the queries [T, heads * row]."""
    _cuda(proj, q_w, k_w, slots, k_pages, v_pages)
    T = proj.shape[0]
    if proj.dim() != 2 or proj.stride(1) != 1 or max(q_off + heads * dim, k_off + kv_heads * dim, v_off + kv_heads * vdim) > proj.shape[1]:
        raise KernelError("whole_norm_store: the projection row is narrower than its parts")
    for t, n in ((q_w, heads * dim), (k_w, kv_heads * dim)):
        if t is not None and (t.dtype != torch.float32 or t.shape != (n,)):
            raise KernelError("whole_norm_store: norm weights must be float32 over the whole projection")
    for t in (k_pages, v_pages):
        if t.dtype != proj.dtype or t.dim() != 4 or tuple(t.shape[1:]) != (kv_heads, page_size, row) or not t.is_contiguous():
            raise KernelError("whole_norm_store: pages must be contiguous [pages, kv_heads, page_size, row] in the activation type")
    if slots is not None and (slots.dtype != torch.int32 or slots.shape[0] != T):
        raise KernelError("whole_norm_store: slots must be int32 [T]")
    q_out = torch.empty((T, heads * row), dtype=proj.dtype, device=proj.device)
    _check(library().pico_whole_norm_store(_ptr(proj), proj.stride(0), q_off, k_off, v_off, _ptr(q_w), _ptr(k_w), float(eps),
                                           1 if v_norm else 0, _ptr(slots), _ptr(k_pages), _ptr(v_pages), _ptr(q_out), T, heads,
                                           kv_heads, dim, vdim, row, page_size, _dtype_code(proj), _stream()), "whole_norm_store")
    _count()
    return q_out


# ------------------------------------------------------------------------------------------ the delta rule; neighbours that turn together
def delta_prepare(xc: torch.Tensor, q_off: int, k_off: int, proj: torch.Tensor, b_off: int, dt: torch.Tensor,
                  dt_bias: Optional[torch.Tensor], a_log: torch.Tensor, heads: int, kv_heads: int, dim: int,
                  unit_eps: float = 1e-6) -> torch.Tensor:
    """The float32 inputs of the gated delta rule.  ``xc`` float32 rows hold ``kv_heads`` query heads at q_off and as many key
    heads at k_off (``dim`` each); ``proj`` (activation type) one logit per head at b_off; ``dt`` [T, heads * dim] (activation
    type) the decay's argument, ``dt_bias`` float32 [heads * dim], ``a_log`` float32 [heads].  Returns float32 [T, P],
    P = 2 G d + H d + H + G:  q / sqrt(|q|^2 + unit_eps) * d^-1/2  |  k / sqrt(|k|^2 + unit_eps)  |
    exp(-exp(a_log) softplus(dt + dt_bias))  |  sigmoid(logit)  |  k . q."""
    _cuda(xc, proj, dt, dt_bias, a_log)
    T = xc.shape[0]
    _f32_rows(xc, "delta_prepare: xc")
    H, G, d = heads, kv_heads, dim
    if H % G or max(q_off, k_off) + G * d > xc.shape[1] or proj.dim() != 2 or proj.stride(1) != 1 or b_off + H > proj.shape[1] \
            or dt.dim() != 2 or dt.stride(1) != 1 or dt.shape != (T, H * d) or dt.dtype != proj.dtype or proj.shape[0] != T:
        raise KernelError("delta_prepare: a row is narrower than its heads")
    if a_log.dtype != torch.float32 or a_log.shape != (H,) or (dt_bias is not None and (dt_bias.dtype != torch.float32 or dt_bias.shape != (H * d,))):
        raise KernelError("delta_prepare: a_log float32 [heads], dt_bias float32 [heads * dim]")
    prep = torch.empty((T, 2 * G * d + H * d + H + G), dtype=torch.float32, device=xc.device)
    _check(library().pico_delta_prepare(_ptr(xc), xc.stride(0), q_off, k_off, _ptr(proj), proj.stride(0), b_off, _ptr(dt),
                                        dt.stride(0), _ptr(dt_bias), _ptr(a_log), _ptr(prep), T, H, G, d, float(d) ** -0.5,
                                        float(unit_eps), _dtype_code(proj), _stream()), "delta_prepare")
    _count()
    return prep


def gated_delta_rule(prep: torch.Tensor, v: torch.Tensor, state: torch.Tensor, seg_slots: torch.Tensor, cu_q: torch.Tensor,
                     positions: torch.Tensor, heads: int, kv_heads: int, dim: int, vdim: int) -> torch.Tensor:
    """Per head h, token by token in the order of each segment, from and into ``state`` float32 [slots, heads, vdim, dim] (S
    transposed; row ``seg_slots[s]``):  S <- diag(a) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q.  ``prep``: the rows
    :func:`delta_prepare` made (head h reads query and key head h // (heads / kv_heads)); ``v`` float32 rows with head h's values
    at h * vdim (a column slice is fine).  A segment whose first position is negative is padding.  Returns o float32
    [T, heads * vdim]."""
    _cuda(prep, v, state, seg_slots, cu_q, positions)
    _f32_rows(v, "gated_delta_rule: v")
    T, S = prep.shape[0], seg_slots.shape[0]
    H, G, d = heads, kv_heads, dim
    if prep.dtype != torch.float32 or not prep.is_contiguous() or prep.shape[1] != 2 * G * d + H * d + H + G or v.shape[0] != T \
            or v.shape[1] < H * vdim:
        raise KernelError("gated_delta_rule: prep must be what delta_prepare returns and v hold every head's values")
    if state.dtype != torch.float32 or not state.is_contiguous() or tuple(state.shape[1:]) != (H, vdim, d):
        raise KernelError("gated_delta_rule: state must be contiguous float32 [slots, heads, vdim, dim]")
    if d > 256:
        raise KernelError(f"gated_delta_rule: key size {d} above 256 is not built")
    for t in (seg_slots, cu_q, positions):
        if t.dtype != torch.int32:
            raise KernelError("gated_delta_rule: index tensors must be int32")
    if cu_q.shape[0] != S + 1 or positions.shape[0] != T:
        raise KernelError("gated_delta_rule: cu_q must have one more entry than seg_slots, positions one per token")
    out = torch.empty((T, H * vdim), dtype=torch.float32, device=prep.device)
    _check(library().pico_gated_delta_rule(_ptr(prep), _ptr(v), v.stride(0), _ptr(state), _ptr(seg_slots), _ptr(cu_q),
                                           _ptr(positions), _ptr(out), out.stride(0), S, H, G, d, vdim, _stream()),
           f"gated_delta_rule (dim {d})")
    _count()
    return out


def pair_rope_norm_store(x: torch.Tensor, q_off: int, k_off: int, v_off: int, positions: torch.Tensor,
                         inv_freq: Optional[torch.Tensor], norm: bool, q_w: Optional[torch.Tensor], k_w: Optional[torch.Tensor],
                         eps: float, slots: Optional[torch.Tensor], k_pages: torch.Tensor, v_pages: torch.Tensor, heads: int,
                         kv_heads: int, dim: int, vdim: int, row: int, page_size: int, out_dtype: torch.dtype) -> torch.Tensor:
    """From float32 rows ``x`` (queries at q_off, keys at k_off, values at v_off): every query and key head turned in its
    first 2 * len(inv_freq) dimensions, dimension 2i with 2i + 1 by position * inv_freq[i], then (``norm``) divided by its root
    mean square over ``dim`` (eps inside the root) and multiplied by ``q_w`` / ``k_w`` (float32 [dim]; None: no weight); keys
    and untouched values written to the token's place in the pages [pages, kv_heads, page_size, row] (``slots`` int32; -1 or
    None: not stored), heads padded with zeros to ``row``.  Returns the queries [T, heads * row] in ``out_dtype``."""
    _cuda(x, positions, inv_freq, q_w, k_w, slots, k_pages, v_pages)
    _f32_rows(x, "pair_rope_norm_store: x")
    T = x.shape[0]
    if max(q_off + heads * dim, k_off + kv_heads * dim, v_off + kv_heads * vdim) > x.shape[1]:
        raise KernelError("pair_rope_norm_store: a row is narrower than its heads")
    rot = 0 if inv_freq is None else 2 * inv_freq.shape[0]
    if positions.dtype != torch.int32 or (inv_freq is not None and inv_freq.dtype != torch.float32) or rot > dim:
        raise KernelError("pair_rope_norm_store: positions int32, inv_freq float32 [<= dim / 2]")
    for w in (q_w, k_w):
        if w is not None and (w.dtype != torch.float32 or w.shape != (dim,)):
            raise KernelError("pair_rope_norm_store: norm weights must be float32 [dim]")
    for t in (k_pages, v_pages):
        if t.dtype != out_dtype or t.dim() != 4 or tuple(t.shape[1:]) != (kv_heads, page_size, row) or not t.is_contiguous():
            raise KernelError("pair_rope_norm_store: pages must be contiguous [pages, kv_heads, page_size, row] in the activation type")
    if slots is not None and (slots.dtype != torch.int32 or slots.shape[0] != T):
        raise KernelError("pair_rope_norm_store: slots must be int32 [T]")
    q_out = torch.empty((T, heads * row), dtype=out_dtype, device=x.device)
    _check(library().pico_pair_rope_norm_store(_ptr(x), x.stride(0), q_off, k_off, v_off, _ptr(positions), _ptr(inv_freq), rot,
                                               1 if norm else 0, _ptr(q_w), _ptr(k_w), float(eps), _ptr(slots), _ptr(k_pages),
                                               _ptr(v_pages), _ptr(q_out), T, heads, kv_heads, dim, vdim, row, page_size,
                                               _dtype_code(q_out), _stream()), "pair_rope_norm_store")
    _count()
    return q_out


# ------------------------------------------------------------------------------------------ several outputs into the stream at once
def sum_add_norm(x: torch.Tensor, terms, weight: Optional[torch.Tensor], kind: int, eps: float, out: Optional[torch.Tensor],
                 rows: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """x float32 [T, H] += sum over ``terms`` (up to three) of scale * N(delta), each term a tuple (delta [T, H] in the
    activation type, norm weight float32 [H] or None, norm kind NORM_NONE or NORM_RMS, eps, scale); then out = N(x) with
    ``kind`` NORM_RMS (weight float32 [H]), NORM_COPY (x in the activation type) or NORM_NONE / ``out`` None (nothing).  With
    ``rows`` (int32 [R]) out[r] is made from row rows[r] and x is left alone."""
    terms = list(terms)
    if len(terms) > 3:
        raise KernelError("sum_add_norm: at most three terms")
    H = x.shape[1]
    R = rows.shape[0] if rows is not None else x.shape[0]
    if x.dtype != torch.float32 or x.dim() != 2 or not x.is_contiguous():
        raise KernelError("sum_add_norm: x must be contiguous float32 [T, H]")
    like = out if out is not None else (terms[0][0] if terms else None)
    if like is None:
        return None
    flat = []
    for delta, w, k, e, s in terms:
        _cuda(delta, w)
        if delta.shape != x.shape or delta.dtype != like.dtype or not delta.is_contiguous():
            raise KernelError("sum_add_norm: every term must be contiguous, shaped like x, in the activation type")
        if k not in (NORM_NONE, NORM_RMS) or (w is not None and (w.dtype != torch.float32 or w.shape != (H,))):
            raise KernelError("sum_add_norm: a term's norm is none or RMS with a float32 [H] weight")
        flat += [_ptr(delta), _ptr(w), int(k), float(e), float(s)]
    flat += [None, None, 0, 0.0, 0.0] * (3 - len(terms))
    _cuda(x, weight, out, rows)
    if weight is not None and (weight.dtype != torch.float32 or weight.shape != (H,)):
        raise KernelError("sum_add_norm: weight must be float32 [H]")
    if out is not None and (out.shape != (R, H) or not out.is_contiguous()):
        raise KernelError("sum_add_norm: out must be contiguous [rows, H]")
    if rows is not None and rows.dtype != torch.int32:
        raise KernelError("sum_add_norm: rows must be int32")
    _check(library().pico_sum_add_norm(_ptr(x), *flat, _ptr(weight), int(kind) if out is not None else NORM_NONE, float(eps),
                                       _ptr(out), _ptr(rows), R, H, _dtype_code(like), _stream()), f"sum_add_norm (width {H})")
    _count()
    return out


def gelu_gate_rows(z: torch.Tensor, table: torch.Tensor, off: int, tokens: torch.Tensor,
                   feedback: Optional[torch.Tensor] = None) -> torch.Tensor:
    """g[t, j] = gelu_tanh(z[t, j]) * table[tokens[t], off + j] for z [T, n] (float32 inside; gelu_tanh(a) = a / 2 * (1 +
    tanh(sqrt(2 / pi) (a + 0.044715 a^3)))).  A token id -(j + 1) names feedback[j], as in :func:`embedding`."""
    _cuda(z, table, tokens, feedback)
    T, n = z.shape
    if not z.is_contiguous() or table.dim() != 2 or table.dtype != z.dtype or not table.is_contiguous() or off + n > table.shape[1]:
        raise KernelError("gelu_gate_rows: z contiguous [T, n], table contiguous [V, >= off + n] of the same type")
    if tokens.dtype != torch.int32 or tokens.shape[0] != T or (feedback is not None and feedback.dtype != torch.int32):
        raise KernelError("gelu_gate_rows: tokens (and feedback) must be int32")
    g = torch.empty_like(z)
    _check(library().pico_gelu_gate_rows(_ptr(z), _ptr(table), table.stride(0), off, _ptr(tokens), _ptr(feedback), table.shape[0],
                                         T, n, _ptr(g), _dtype_code(z), _stream()), "gelu_gate_rows")
    _count()
    return g


def capped_glu(gu: torch.Tensor, ff: int, limit: float, row_gate_col: Optional[int] = None, alpha: float = 1.702) -> torch.Tensor:
    """From rows [gate: ff | up: ff | ...]:  y = g' sigmoid(alpha g') (u' + 1) with g' = min(g, limit), u' = clamp(u, -limit,
    limit), float32 inside; with ``row_gate_col`` the whole row is also multiplied by sigmoid of that column.  Returns [n, ff]."""
    _cuda(gu)
    if gu.dim() != 2 or gu.stride(1) != 1 or gu.shape[1] < 2 * ff or (row_gate_col is not None and not 0 <= row_gate_col < gu.shape[1]):
        raise KernelError("capped_glu: rows must hold gate and up (and the row gate's column)")
    out = torch.empty((gu.shape[0], ff), dtype=gu.dtype, device=gu.device)
    _check(library().pico_capped_glu(_ptr(gu), gu.stride(0), gu.shape[0], ff, float(limit), float(alpha),
                                     -1 if row_gate_col is None else int(row_gate_col), _ptr(out), _dtype_code(gu), _stream()),
           "capped_glu")
    _count()
    return out
