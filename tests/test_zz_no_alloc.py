"""The entry point that allocates nothing, called through its exported C symbol.

Some users of the kernel library cannot allocate device memory when they call it - a serving
loop with a fixed memory plan, a process whose memory pool belongs to someone else, a callback
in which cudaMalloc would stall the device.  For them the library has
``pico_paged_attention_noalloc``: split-key paged attention whose scratch is a fixed 8 MiB
array inside the library.  This test calls it twice in a row, with different inputs, and checks
each result against the ordinary entry point (which gets its scratch from the caller), within
the tolerance of the other kernel tests.  It also checks that a request beyond the built-in
scratch is refused with a message.  The file name sorts last so that a run that stops at the
first failure has already run every other test.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _entry():
    from pico_vllm_b200 import ops
    lib = ops.library()
    fn = lib.pico_paged_attention_noalloc
    vp, i32, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn.argtypes = [vp, i32, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, f32, i32, i32, vp,
                   ctypes.c_char_p, i32]
    fn.restype = ctypes.c_int
    return fn


def _case(seed, dtype, nh=6, nkv=2, hd=64, ps=16, lens=(700, 333, 40, 3), window=None):
    g = torch.Generator().manual_seed(seed)
    S = len(lens)
    blocks = [-(-n // ps) for n in lens]
    pages = sum(blocks) + 2
    perm = torch.randperm(pages, generator=g).tolist()
    table = torch.zeros(S, max(blocks), dtype=torch.int32)
    at = 0
    for s, b in enumerate(blocks):
        table[s, :b] = torch.tensor(perm[at:at + b], dtype=torch.int32)
        at += b
    k = torch.randn(pages, nkv, ps, hd, generator=g).to(dtype).to(DEV)
    v = torch.randn(pages, nkv, ps, hd, generator=g).to(dtype).to(DEV)
    q = torch.randn(S, nh * hd, generator=g).to(dtype).to(DEV)
    seg = torch.arange(S, dtype=torch.int32, device=DEV)
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV)
    return dict(q=q, k=k, v=v, seg=seg, pos=pos, table=table.to(DEV), nh=nh, nkv=nkv, hd=hd, ps=ps, window=window)


def _call_noalloc(fn, c, splits):
    out = torch.empty(c["q"].shape[0], c["nh"] * c["hd"], dtype=c["q"].dtype, device=DEV)
    err = ctypes.create_string_buffer(256)
    rc = fn(c["q"].data_ptr(), c["q"].stride(0), c["k"].data_ptr(), c["v"].data_ptr(), out.data_ptr(),
            c["seg"].data_ptr(), c["pos"].data_ptr(), c["table"].data_ptr(), c["table"].stride(0),
            c["q"].shape[0], c["nh"], c["nkv"], c["hd"], c["ps"], c["window"] or 0, 1.0 / math.sqrt(c["hd"]),
            splits, 0 if c["q"].dtype == torch.float32 else 1, torch.cuda.current_stream().cuda_stream, err, 256)
    return rc, out, err.value.decode()


def _call_ordinary(c, splits):
    from pico_vllm_b200 import ops
    T = c["q"].shape[0]
    out = torch.empty(T, c["nh"] * c["hd"], dtype=c["q"].dtype, device=DEV)
    scratch = torch.empty(ops.attention_scratch_floats(T, c["nh"], c["hd"], splits), dtype=torch.float32, device=DEV)
    ops.paged_attention(c["q"], c["k"], c["v"], out, c["seg"], c["pos"], c["table"], c["nh"], c["nkv"], c["hd"],
                        c["ps"], c["window"], 1.0 / math.sqrt(c["hd"]), splits, scratch)
    return out


def _plain(c):
    """The same attention by the plain double of the kernels, on the CPU."""
    import fake_ops
    T = c["q"].shape[0]
    out = torch.empty(T, c["nh"] * c["hd"], dtype=c["q"].dtype)
    fake_ops.paged_attention(c["q"].cpu(), c["k"].cpu(), c["v"].cpu(), out, c["seg"].cpu(), c["pos"].cpu(),
                             c["table"].cpu(), c["nh"], c["nkv"], c["hd"], c["ps"], c["window"],
                             1.0 / math.sqrt(c["hd"]))
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_no_alloc_entry_point_matches_the_ordinary_one_twice_in_a_row(dtype):
    fn = _entry()
    tol = dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
    # two calls in a row with different inputs and split counts: the second finds the first's leftovers
    for seed, splits, window in ((1, 8, None), (2, 5, 100)):
        c = _case(seed, dtype, window=window)
        rc, got, msg = _call_noalloc(fn, c, splits)
        assert rc == 0, msg
        want = _call_ordinary(c, splits)
        torch.cuda.synchronize()
        assert torch.allclose(got.float(), want.float(), **tol)
        assert torch.allclose(got.float().cpu(), _plain(c).float(), **tol)      # and the plain attention, directly


def test_no_alloc_entry_point_refuses_more_scratch_than_it_has():
    fn = _entry()
    c = _case(3, torch.float32, nh=32, nkv=4, hd=128, lens=tuple([50] * 64))
    rc, _, msg = _call_noalloc(fn, c, 64)        # 64 * 32 * 64 * 130 floats > 2 Mi
    assert rc == -5
    assert "scratch" in msg and "2097152" in msg


def test_no_alloc_entry_point_takes_any_number_of_tokens_with_one_part():
    """With one part per token the kernels use no scratch, so the limit does not apply: 2,048 tokens of 12
    heads of 128 would need 3.2 Mi floats per part if they did."""
    fn = _entry()
    c = _case(4, torch.bfloat16, nh=12, nkv=2, hd=128, lens=tuple([37] * 2048))
    rc, got, msg = _call_noalloc(fn, c, 1)
    assert rc == 0, msg
    want = _call_ordinary(c, 1)
    torch.cuda.synchronize()
    assert torch.allclose(got.float(), want.float(), atol=2e-2, rtol=2e-2)
    rc, _, msg = _call_noalloc(fn, c, 2)
    assert rc == -5 and "scratch" in msg
