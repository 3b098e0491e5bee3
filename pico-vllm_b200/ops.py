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
                                         i32, i32, f32, i32, i32, vp],
        "pico_paged_prefill_mma": [vp, i32, vp, vp, vp, vp, i32, vp, i32, vp, vp, i32, i32, i32, i32, i32, i32, f32, vp],
        "pico_paged_decode_mma": [vp, i32, vp, vp, vp, vp, vp, vp, i32, vp, vp, vp, i32, i32, i32, i32, i32, i32,
                                  f32, i32, vp],
        "pico_skinny_linear": [vp, i32, vp, vp, vp, i32, i32, i32, i32, i32, vp, f32, vp, vp],
        "pico_skinny_argmax": [vp, i32, vp, vp, i32, i32, i32, vp, f32, vp, vp],
        "pico_skinny_norm_fits": [i32, i32],
        "pico_skinny_linear_residual": [vp, i32, vp, vp, i32, i32, i32, vp],
        "pico_skinny_gate_up_swiglu": [vp, i32, vp, vp, i32, i32, i32, vp, f32, vp],
        "pico_skinny_qkv_rope_store": [vp, i32, vp, vp, vp, vp, vp, i32, vp, vp, vp, i32, i32, i32, i32, i32, i32, vp, f32,
                                       vp],
        "pico_make_kv_tensor_map": [vp, vp, i64, i32, i32],
        "pico_paged_decode_tma": [vp, vp, vp, i32, vp, vp, vp, vp, i32, vp, vp, vp, i32, i32, i32, i32, i32, i32,
                                  f32, i32, vp],
        "pico_tma_status": [vp],
        "pico_make_kv_tensor_map_2d": [vp, vp, i64, i32, i32, i32],
        "pico_paged_prefill_tcgen05": [vp, vp, vp, i32, vp, vp, i32, vp, i32, vp, vp, i32, i32, i32, i32, i32, i32, f32, i32,
                                       vp, i32, vp, i32, vp],
        "pico_tca_status": [vp],
        "pico_gemm_tcgen05_pair": [vp, i32, vp, vp, vp, i32, i32, i32, i32, i32, vp],
        "pico_tp_status": [vp],
        "pico_sample": [vp, i32, i32, i32, vp, vp, vp, vp, vp],
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
                    scale: float, n_splits: int = 1, scratch: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal attention of every token of the batch over its request's cache pages.

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
        int(window) if window else 0, float(scale), n_splits, _dtype_code(q), _stream()),
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
                        k_map=None, v_map=None, k_map2d=None, v_map2d=None, pair_min_keys: int = 0) -> torch.Tensor:
    """The same attention as :func:`paged_attention` for bfloat16 on tensor cores, in two launches:
    segments that bring two or more tokens (``prefill_segs`` int32 [n_prefill_segs], None = all
    segments; ``cu_q`` int32 [segments + 1]; ``max_prefill_q`` their longest) and single tokens
    (``decode_tokens`` int32 [n_decode_tokens], None = every token of the batch) whose key range is
    cut into ``n_splits`` parts.  Every token of the batch must be in exactly one of the two.
    With ``k_map`` / ``v_map`` (from :func:`make_kv_tensor_map` over these same pages) the single
    tokens run in the kernel that brings pages in by TMA; with ``k_map2d`` / ``v_map2d`` (from
    :func:`make_kv_tensor_map_2d`) the portions run on the tcgen05 tensor cores."""
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
    lib = library()
    win = int(window) if window else 0
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
                                              _stream()),
               f"paged_prefill_tcgen05 (head_dim {head_dim})")
        _count()
    elif n_prefill_segs > 0:
        _check(lib.pico_paged_prefill_mma(_ptr(q), q.stride(0), _ptr(k_pages), _ptr(v_pages), _ptr(out),
                                          _ptr(prefill_segs), n_prefill_segs, _ptr(cu_q), max_prefill_q,
                                          _ptr(positions), _ptr(block_table), block_table.stride(0), n_heads,
                                          n_kv_heads, head_dim, page_size, win, float(scale), _stream()),
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
                                             head_dim, page_size, win, float(scale), n_splits, _stream()),
                   f"paged_decode_tma (head_dim {head_dim})")
        else:
            _check(lib.pico_paged_decode_mma(_ptr(q), q.stride(0), _ptr(k_pages), _ptr(v_pages), _ptr(out), part_o,
                                             part_ml, _ptr(decode_tokens), n_decode_tokens, _ptr(tok_seg),
                                             _ptr(positions), _ptr(block_table), block_table.stride(0), n_heads,
                                             n_kv_heads, head_dim, page_size, win, float(scale), n_splits,
                                             _stream()),
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
