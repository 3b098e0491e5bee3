"""Test doubles of the CUDA kernels in plain torch, for tests of host-side logic on the CPU.

``install(monkeypatch)`` replaces the functions of ``pico_vllm_b200.ops`` so that the step
function, the cache and the scheduler can be driven without a GPU.  These doubles also serve
as the plain reference of each kernel in the GPU tests (same signatures, float32 arithmetic).
They are not part of the product: the package itself has no CPU path.
"""
import math

import torch

import plain_qwen2 as plain


def embedding(ids, table, out, feedback=None):
    ids = ids.long()
    if feedback is not None:
        ids = torch.where(ids < 0, feedback.long()[(-ids - 1).clamp(min=0)], ids)
    out.copy_(table[ids].float())
    return out


def add_rmsnorm(x, delta, weight, eps, out, rows=None):
    if rows is None:
        if delta is not None:
            x.add_(delta.float())
        src = x
    else:
        src = x[rows.long()]
        if delta is not None:
            src = src + delta[rows.long()].float()
    out.copy_(plain.rms_norm(src, weight, eps).to(out.dtype))
    return out


def swiglu(gate_up, out):
    I = out.shape[1]
    g, u = gate_up[:, :I].float(), gate_up[:, I:].float()
    out.copy_((g * torch.sigmoid(g) * u).to(out.dtype))
    return out


def rope_store(qkv, bias, positions, inv_freq, slots, k_pages, v_pages, n_heads, n_kv_heads, head_dim,
               page_size, pairing="half"):
    T = qkv.shape[0]
    x = qkv.float()
    if bias is not None:
        x = x + bias
    nq, nk = n_heads * head_dim, n_kv_heads * head_dim
    q = x[:, :nq].view(T, n_heads, head_dim)
    k = x[:, nq:nq + nk].view(T, n_kv_heads, head_dim)
    v = x[:, nq + nk:].view(T, n_kv_heads, head_dim)
    ang = positions.float()[:, None] * inv_freq[None, :]
    cos, sin = ang.cos(), ang.sin()
    r = inv_freq.shape[0]
    half = head_dim // 2

    def rot(t):
        t = t.clone()
        x1, x2 = t[..., :r].clone(), t[..., half:half + r].clone()
        t[..., :r] = x1 * cos[:, None, :] - x2 * sin[:, None, :]
        t[..., half:half + r] = x2 * cos[:, None, :] + x1 * sin[:, None, :]
        return t
    qkv[:, :nq] = rot(q).reshape(T, nq).to(qkv.dtype)
    if slots is not None:
        kr = rot(k)
        keep = slots >= 0
        s = slots[keep].long()
        page, off = s // page_size, s % page_size
        k_pages[page, :, off, :] = kr[keep].to(k_pages.dtype)
        v_pages[page, :, off, :] = v[keep].to(v_pages.dtype)


def attention_scratch_floats(T, n_heads, head_dim, n_splits):
    return 0 if n_splits <= 1 else T * n_heads * n_splits * (head_dim + 2)


def paged_attention(q, k_pages, v_pages, out, tok_seg, positions, block_table, n_heads, n_kv_heads,
                    head_dim, page_size, window, scale, n_splits=1, scratch=None):
    T = q.shape[0]
    g = n_heads // n_kv_heads
    for t in range(T):
        p = int(positions[t])
        if p < 0:
            out[t] = 0
            continue
        lo = max(0, p + 1 - window) if window else 0
        n = torch.arange(lo, p + 1)
        pages = block_table[int(tok_seg[t])].long()[n // page_size]
        k = k_pages[pages, :, n % page_size, :].float()    # [keys, kv_heads, hd]
        v = v_pages[pages, :, n % page_size, :].float()
        qt = q[t, :n_heads * head_dim].float().view(n_heads, head_dim)
        for h in range(n_heads):
            s = (k[:, h // g, :] @ qt[h]) * scale
            pr = torch.softmax(s, dim=0)
            out[t, h * head_dim:(h + 1) * head_dim] = (pr @ v[:, h // g, :]).to(out.dtype)
    return out


def mma_attention_takes(dtype, n_heads, n_kv_heads, head_dim):
    return (dtype == torch.bfloat16 and head_dim % 16 == 0 and 16 <= head_dim <= 256
            and n_heads % n_kv_heads == 0 and n_heads // n_kv_heads <= 16)


def paged_attention_mma(q, k_pages, v_pages, out, tok_seg, positions, block_table, cu_q, prefill_segs,
                        n_prefill_segs, max_prefill_q, decode_tokens, n_decode_tokens, n_heads, n_kv_heads, head_dim,
                        page_size, window, scale, n_splits=1, scratch=None, k_map=None, v_map=None, k_map2d=None,
                        v_map2d=None, pair_min_keys=0):
    return paged_attention(q, k_pages, v_pages, out, tok_seg, positions, block_table, n_heads, n_kv_heads, head_dim,
                           page_size, window, scale)


SKINNY_MAX_TOKENS = 16


def skinny_takes(x, weight, n_multiple=16):
    return (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and 1 <= x.shape[0] <= 16
            and x.shape[1] % 16 == 0 and weight.shape[0] % n_multiple == 0 and weight.shape[0] >= 16)


def skinny_norm_takes(x, weight, n_rows=None):
    M = x.shape[0] if n_rows is None else n_rows
    return x.dtype == torch.float32 and weight.dtype == torch.bfloat16 and 1 <= M <= 16 and x.shape[1] % 16 == 0 \
        and weight.shape[0] % 16 == 0 and x.shape[1] <= 2000


def _normed(x, norm_weight, eps, rows=None):
    if norm_weight is None:
        return x
    if rows is not None:
        x = x[rows.long()]
    return plain.rms_norm(x.float(), norm_weight, eps).to(torch.bfloat16)


def skinny_linear(x, weight, bias=None, out_dtype=torch.bfloat16, norm_weight=None, eps=0.0, rows=None):
    x = _normed(x, norm_weight, eps, rows)
    y = x.float() @ weight.float().t()
    if bias is not None:
        y = y + bias
    return y.to(out_dtype)


def skinny_argmax(x, weight, out, norm_weight=None, eps=0.0, rows=None):
    logits = skinny_linear(x, weight, None, torch.float32, norm_weight, eps, rows)
    out[:logits.shape[0]] = logits.argmax(-1).to(out.dtype)
    return out


def skinny_linear_residual(x, weight, residual):
    residual.add_(x.float() @ weight.float().t())


def skinny_gate_up_swiglu(x, gate_up_weight, norm_weight=None, eps=0.0):
    x = _normed(x, norm_weight, eps)
    gu = x.float() @ gate_up_weight.float().t()
    I = gu.shape[1] // 2
    g, u = gu[:, :I], gu[:, I:]
    return (g * torch.sigmoid(g) * u).to(torch.bfloat16)


def skinny_qkv_rope_store(x, qkv_weight, bias, positions, inv_freq, slots, k_pages, v_pages, n_heads, n_kv_heads,
                          head_dim, page_size, norm_weight=None, eps=0.0, pairing="half"):
    x = _normed(x, norm_weight, eps)
    qkv = x.float() @ qkv_weight.float().t()          # float32 until after the rotation, like the kernel
    rope_store(qkv, bias, positions, inv_freq, slots, k_pages, v_pages, n_heads, n_kv_heads, head_dim, page_size)
    return qkv[:, :n_heads * head_dim].to(torch.bfloat16)


def make_kv_tensor_map(pages):
    return None


def make_kv_tensor_map_2d(pages, values=False):
    return None


def tc_takes(x, weight):
    return False


def linear(x, weight, out=None):
    y = (x.float() @ weight.float().t()).to(x.dtype)
    if out is not None:
        out.copy_(y)
        return out
    return y


def logits_linear(x, weight):
    return x.float() @ weight.float().t()


def sample(logits, temperature, top_p, uniform, out):
    R, V = logits.shape
    for r in range(R):
        t = 0.0 if temperature is None else float(temperature[r])
        if t <= 0:
            out[r] = int(torch.argmax(logits[r]))
            continue
        probs = plain.softmax_temperature(logits[r].double(), t)
        tp = 1.0 if top_p is None else float(top_p[r])
        if tp < 1.0:
            probs = plain.top_p_filter(probs[None], tp)[0]
        cum = torch.cumsum(probs, 0)
        idx = int(torch.searchsorted(cum, torch.tensor(float(uniform[r]) * float(cum[-1]), dtype=cum.dtype),
                                     right=True))
        out[r] = min(idx, V - 1)
    return out


NAMES = ["embedding", "add_rmsnorm", "swiglu", "rope_store", "attention_scratch_floats", "paged_attention",
         "mma_attention_takes", "paged_attention_mma", "make_kv_tensor_map", "make_kv_tensor_map_2d", "tc_takes", "skinny_takes", "skinny_norm_takes", "skinny_linear", "skinny_linear_residual",
         "skinny_gate_up_swiglu", "skinny_qkv_rope_store",
         "linear", "logits_linear", "sample"]


def install(monkeypatch):
    """Replaces the kernels of pico_vllm_b200.ops with the doubles above."""
    import pico_vllm_b200.ops as ops
    for name in NAMES:
        monkeypatch.setattr(ops, name, globals()[name])
