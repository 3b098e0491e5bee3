"""Each CUDA kernel alone against its plain float32 reference (tests/fake_ops.py), at sizes
other than the engine's tiny and benchmark configurations."""
import math

import pytest
import torch

import fake_ops

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)


def gen(seed):
    return torch.Generator().manual_seed(seed)


@pytest.mark.parametrize("tdtype", DTYPES)
@pytest.mark.parametrize("T,H,V", [(1, 16, 7), (37, 200, 331), (5, 1000, 50)])
def test_embedding(tdtype, T, H, V):
    from pico_vllm_b200 import ops
    table = torch.randn(V, H, generator=gen(1)).to(tdtype)
    ids = torch.randint(0, V, (T,), generator=gen(2), dtype=torch.int32)
    out = torch.empty(T, H, dtype=torch.float32, device=DEV)
    ops.embedding(ids.to(DEV), table.to(DEV), out)
    want = fake_ops.embedding(ids, table, torch.empty(T, H))
    assert torch.equal(out.cpu(), want)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,H,eps", [(1, 16, 1e-6), (9, 200, 1e-5), (4, 1000, 1e-3), (3, 5000, 1e-6),
                                     (70, 200, 1e-5), (131, 1536, 1e-6), (65, 3584, 1e-6), (64, 4100, 1e-6), (77, 1100, 1e-4)])
@pytest.mark.parametrize("with_delta", [False, True])
def test_add_rmsnorm(dtype, T, H, eps, with_delta):
    from pico_vllm_b200 import ops
    x = torch.randn(T, H, generator=gen(3)) * 3
    d = (torch.randn(T, H, generator=gen(4))).to(dtype) if with_delta else None
    w = 1 + 0.1 * torch.randn(H, generator=gen(5))
    xg = x.to(DEV)
    out = torch.empty(T, H, dtype=dtype, device=DEV)
    ops.add_rmsnorm(xg, None if d is None else d.to(DEV), w.to(DEV), eps, out)
    xr = x.clone()
    want = fake_ops.add_rmsnorm(xr, d, w, eps, torch.empty(T, H, dtype=dtype))
    assert torch.allclose(out.cpu().float(), want.float(), **tol(dtype))
    assert torch.allclose(xg.cpu(), xr, atol=1e-6)            # the residual stream was updated in place
    # rows: norm of chosen rows, residual untouched
    rows = torch.tensor([T - 1, 0], dtype=torch.int32)
    x2 = x.to(DEV)
    out2 = torch.empty(2, H, dtype=dtype, device=DEV)
    ops.add_rmsnorm(x2, None if d is None else d.to(DEV), w.to(DEV), eps, out2, rows.to(DEV))
    want2 = fake_ops.add_rmsnorm(x.clone(), d, w, eps, torch.empty(2, H, dtype=dtype), rows)
    assert torch.allclose(out2.cpu().float(), want2.float(), **tol(dtype))
    assert torch.equal(x2.cpu(), x)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,I", [(1, 8), (7, 176), (33, 1000)])
def test_swiglu(dtype, T, I):
    from pico_vllm_b200 import ops
    gu = (torch.randn(T, 2 * I, generator=gen(6)) * 4).to(dtype)
    out = torch.empty(T, I, dtype=dtype, device=DEV)
    ops.swiglu(gu.to(DEV), out)
    want = fake_ops.swiglu(gu, torch.empty(T, I, dtype=dtype))
    assert torch.allclose(out.cpu().float(), want.float(), **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd,ps,rot", [(4, 2, 16, 16, 16), (6, 3, 32, 8, 32), (5, 1, 48, 4, 48),
                                              (3, 3, 80, 16, 40), (2, 1, 128, 32, 0)])
def test_rope_store(dtype, nh, nkv, hd, ps, rot):
    from pico_vllm_b200 import ops
    T, pages = 19, 12
    width = (nh + 2 * nkv) * hd
    qkv = torch.randn(T, width, generator=gen(7)).to(dtype)
    bias = 0.5 * torch.randn(width, generator=gen(8))
    pos = torch.randint(0, 5000, (T,), generator=gen(9), dtype=torch.int32)
    inv = 1.0 / (10000.0 ** (torch.arange(0, rot, 2).float() / max(rot, 1))) if rot else torch.zeros(0)
    slots = torch.randperm(pages * ps, generator=gen(10))[:T].to(torch.int32)
    slots[3] = -1
    k0 = torch.randn(pages, nkv, ps, hd, generator=gen(11)).to(dtype)
    v0 = torch.randn(pages, nkv, ps, hd, generator=gen(12)).to(dtype)
    qg, kg, vg = qkv.to(DEV), k0.to(DEV), v0.to(DEV)
    ops.rope_store(qg, bias.to(DEV), pos.to(DEV), inv.to(DEV), slots.to(DEV), kg, vg, nh, nkv, hd, ps)
    qr, kr, vr = qkv.clone(), k0.clone(), v0.clone()
    fake_ops.rope_store(qr, bias, pos, inv, slots, kr, vr, nh, nkv, hd, ps)
    t = dict(atol=3e-4, rtol=1e-4) if dtype == torch.float32 else tol(dtype)   # angles up to 5000 rad
    assert torch.allclose(qg.cpu().float()[:, :nh * hd], qr.float()[:, :nh * hd], **t)
    assert torch.allclose(kg.cpu().float(), kr.float(), **t)
    assert torch.allclose(vg.cpu().float(), vr.float(), **t)
    # without slots only q is rotated and the pages stay as they were
    qg2, kg2 = qkv.to(DEV), k0.to(DEV)
    ops.rope_store(qg2, bias.to(DEV), pos.to(DEV), inv.to(DEV), None, None, None, nh, nkv, hd, ps)
    assert torch.allclose(qg2.cpu().float()[:, :nh * hd], qr.float()[:, :nh * hd], **t)


def _attention_case(dtype, nh, nkv, hd, ps, window, seg_lens, q_lens, splits, seed=0, spike=False, mma=False,
                    tma=False, poison=False, tc=False, pair=False):
    """Segments with kv lengths seg_lens, of which the last q_lens are this step's queries."""
    from pico_vllm_b200 import ops
    g = gen(20 + seed)
    S = len(seg_lens)
    blocks = [-(-n // ps) for n in seg_lens]
    pages = sum(blocks) + 3
    perm = torch.randperm(pages, generator=g).tolist()
    W = max(blocks) + 1
    table = torch.zeros(S, W, dtype=torch.int32)
    at = 0
    for s, b in enumerate(blocks):
        table[s, :b] = torch.tensor(perm[at:at + b], dtype=torch.int32)
        at += b
    k = torch.randn(pages, nkv, ps, hd, generator=g).to(dtype)
    v = torch.randn(pages, nkv, ps, hd, generator=g).to(dtype)
    T = sum(q_lens)
    q = torch.randn(T, (nh + 2 * nkv) * hd, generator=g).to(dtype)
    tok_seg = torch.cat([torch.full((n,), s, dtype=torch.int32) for s, n in enumerate(q_lens)])
    pos = torch.cat([torch.arange(L - n, L, dtype=torch.int32) for L, n in zip(seg_lens, q_lens)])
    if spike:
        # one far key gets a score that dwarfs the rest: a kernel that skips it, or reads the wrong
        # page for it, gives a visibly different output
        for s, L in enumerate(seg_lens):
            far = 1 if window is None else max(0, L - window)       # first visible key of the last query
            pg, off = table[s, far // ps], far % ps
            t_last = int((tok_seg == s).nonzero()[-1])
            qv = q[t_last, :hd].float()
            k[pg, 0, off, :] = (qv / qv.norm() * 30).to(dtype)
            q[t_last, :hd] = (qv / qv.norm() * 6).to(dtype)
    out = torch.empty(T, nh * hd, dtype=dtype, device=DEV)
    scratch = None
    if splits > 1 or pair:
        # pair (a number of keys): room for two partial results per (token, head), with which the tcgen05 prompt
        # kernel lets two blocks share a query tile that sees at least that many keys
        scratch = torch.full((ops.attention_scratch_floats(T, nh, hd, max(splits, 2)),), float("nan"), dtype=torch.float32,
                             device=DEV)
    scale = 1.0 / math.sqrt(hd)
    if mma:
        cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32)
        pf = torch.tensor([i for i, n in enumerate(q_lens) if n > 1], dtype=torch.int32)
        dec = torch.tensor([int(cu[i]) for i, n in enumerate(q_lens) if n == 1], dtype=torch.int32)
        out.fill_(float("nan"))
        kd, vd = k.to(DEV), v.to(DEV)
        if poison:
            # what lies beyond a request's last token inside its last page, and pages it does not hold,
            # is not-a-number: nothing of it may reach the result
            held = torch.zeros(pages, ps, dtype=torch.bool)
            for sgi, L in enumerate(seg_lens):
                for n in range(L):
                    held[table[sgi, n // ps], n % ps] = True
            kd[~held.to(DEV)[:, None, :].expand(-1, nkv, -1)] = float("nan")
            vd[~held.to(DEV)[:, None, :].expand(-1, nkv, -1)] = float("nan")
        maps = (ops.make_kv_tensor_map(kd), ops.make_kv_tensor_map(vd)) if tma else (None, None)
        if tma:
            assert maps[0] is not None and maps[1] is not None
        if tc:
            maps = maps + (ops.make_kv_tensor_map_2d(kd), ops.make_kv_tensor_map_2d(vd, values=True))
            assert maps[2] is not None and maps[3] is not None
        ops.paged_attention_mma(q.to(DEV), kd, vd, out, tok_seg.to(DEV), pos.to(DEV), table.to(DEV),
                                cu.to(DEV), pf.to(DEV), len(pf), max([n for n in q_lens if n > 1], default=0),
                                dec.to(DEV), len(dec), nh, nkv, hd, ps, window, scale, splits, scratch, *maps,
                                **({"pair_min_keys": pair} if pair else {}))
        if tma:
            torch.cuda.synchronize()
            assert ops.tma_status() == 0
        if tc:
            assert ops.tca_status() == 0
    else:
        ops.paged_attention(q.to(DEV), k.to(DEV), v.to(DEV), out, tok_seg.to(DEV), pos.to(DEV), table.to(DEV),
                            nh, nkv, hd, ps, window, scale, splits, scratch)
    want = torch.empty(T, nh * hd, dtype=dtype)
    fake_ops.paged_attention(q, k, v, want, tok_seg, pos, table, nh, nkv, hd, ps, window, scale)
    return out.cpu().float(), want.float()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd,ps", [(4, 2, 16, 16), (6, 3, 32, 8), (5, 1, 48, 4), (12, 2, 128, 16),
                                          (3, 3, 80, 16), (8, 1, 256, 32)])
@pytest.mark.parametrize("window", [None, 24])
def test_paged_attention_mixed_segments(dtype, nh, nkv, hd, ps, window):
    # a long prompt portion, a decode token with a long context, a short one, a first token
    got, want = _attention_case(dtype, nh, nkv, hd, ps, window, seg_lens=[70, 133, 9, 1], q_lens=[33, 1, 2, 1],
                                splits=1)
    assert torch.allclose(got, want, **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("splits", [2, 5, 16])
@pytest.mark.parametrize("window", [None, 100])
def test_paged_attention_split_keys(dtype, splits, window):
    got, want = _attention_case(dtype, 6, 2, 64, 16, window, seg_lens=[700, 333, 40, 3], q_lens=[1, 1, 1, 1],
                                splits=splits, seed=3)
    assert torch.allclose(got, want, **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window,splits", [(None, 1), (None, 8), (64, 1), (64, 4)])
def test_paged_attention_far_key_and_window_edge(dtype, window, splits):
    got, want = _attention_case(dtype, 4, 2, 32, 8, window, seg_lens=[517, 300], q_lens=[1, 2], splits=splits,
                                seed=5, spike=True)
    assert torch.allclose(got, want, **tol(dtype))


MMA_TOL = dict(atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("nh,nkv,hd,ps", [(4, 2, 16, 16), (6, 3, 32, 8), (5, 1, 48, 4), (12, 2, 128, 16), (3, 3, 80, 16),
                                          (8, 1, 256, 32), (28, 4, 128, 16), (16, 1, 64, 16), (4, 4, 112, 2)])
@pytest.mark.parametrize("window", [None, 24, 200])
def test_mma_attention_mixed_segments(nh, nkv, hd, ps, window):
    # long portions (several 64-row tiles), short ones, single tokens with long and short contexts
    got, want = _attention_case(torch.bfloat16, nh, nkv, hd, ps, window, seg_lens=[300, 133, 9, 1, 70, 2, 64],
                                q_lens=[257, 1, 2, 1, 33, 2, 1], splits=1, mma=True)
    assert torch.isfinite(got).all()
    assert torch.allclose(got, want, **MMA_TOL)


@pytest.mark.parametrize("splits", [1, 2, 5, 16])
@pytest.mark.parametrize("window", [None, 100])
@pytest.mark.parametrize("nh,nkv,hd", [(6, 2, 64), (12, 2, 128), (7, 1, 96)])
def test_mma_decode_split_keys(splits, window, nh, nkv, hd):
    got, want = _attention_case(torch.bfloat16, nh, nkv, hd, 16, window, seg_lens=[700, 333, 40, 3, 64, 65, 1],
                                q_lens=[1, 1, 1, 1, 1, 1, 1], splits=splits, seed=3, mma=True)
    assert torch.isfinite(got).all()
    assert torch.allclose(got, want, **MMA_TOL)


@pytest.mark.parametrize("splits", [1, 2, 5, 16])
@pytest.mark.parametrize("window", [None, 100, 37])
@pytest.mark.parametrize("nh,nkv,hd,ps", [(6, 2, 64, 16), (12, 2, 128, 16), (7, 1, 128, 8), (16, 1, 64, 32), (4, 4, 128, 64)])
def test_tma_decode_split_keys(splits, window, nh, nkv, hd, ps):
    got, want = _attention_case(torch.bfloat16, nh, nkv, hd, ps, window, seg_lens=[700, 333, 40, 3, 64, 65, 1, 128],
                                q_lens=[1, 1, 1, 1, 1, 1, 1, 1], splits=splits, seed=3, mma=True, tma=True, poison=True)
    assert torch.isfinite(got).all()
    assert torch.allclose(got, want, **MMA_TOL)


@pytest.mark.parametrize("nh,nkv,hd,ps", [(6, 2, 64, 16), (12, 2, 128, 16), (7, 1, 128, 8), (16, 1, 64, 32), (4, 4, 128, 64),
                                          (28, 4, 128, 16)])
@pytest.mark.parametrize("window", [None, 24, 200])
def test_tma_attention_mixed_segments(nh, nkv, hd, ps, window):
    got, want = _attention_case(torch.bfloat16, nh, nkv, hd, ps, window, seg_lens=[300, 133, 9, 1, 70, 2, 64, 190],
                                q_lens=[257, 1, 2, 1, 33, 2, 1, 64], splits=1, mma=True, tma=True, poison=True)
    assert torch.isfinite(got).all()
    assert torch.allclose(got, want, **MMA_TOL)


@pytest.mark.parametrize("nh,nkv,hd,ps", [(6, 2, 64, 16), (12, 2, 128, 16), (7, 1, 128, 8), (16, 1, 64, 32), (4, 4, 128, 64),
                                          (28, 4, 128, 16), (3, 3, 64, 8)])
@pytest.mark.parametrize("window", [None, 24, 200])
@pytest.mark.parametrize("pair", [0, 128, 512])
def test_tcgen05_attention_mixed_segments(nh, nkv, hd, ps, window, pair):
    got, want = _attention_case(torch.bfloat16, nh, nkv, hd, ps, window, seg_lens=[300, 133, 9, 1, 70, 2, 64, 190, 1000],
                                q_lens=[257, 1, 2, 1, 33, 2, 1, 64, 700], splits=1, mma=True, tma=True, poison=True, tc=True,
                                pair=pair)
    assert torch.isfinite(got).all()
    assert torch.allclose(got, want, **MMA_TOL)


@pytest.mark.parametrize("window", [None, 5000])
@pytest.mark.parametrize("pair", [0, 4096])
def test_long_contexts_beyond_the_block_table_cache(window, pair):
    """Contexts whose block tables are longer than what a block keeps in shared memory (256 entries in
    the decode kernel, 1024 in the prompt kernel): the entries beyond come straight from global memory."""
    got, want = _attention_case(torch.bfloat16, 4, 2, 64, 8, window, seg_lens=[9100, 6000, 2100], q_lens=[300, 1, 1], splits=1,
                                seed=7, spike=True, mma=True, tma=True, poison=True, tc=True, pair=pair)
    assert torch.isfinite(got).all()
    assert torch.allclose(got, want, **MMA_TOL)


@pytest.mark.parametrize("window,q_lens", [(None, [200, 150]), (64, [200, 150]), (None, [2, 300]), (100, [517, 64])])
@pytest.mark.parametrize("pair", [0, 128])
def test_tcgen05_prefill_far_key_and_window_edge(window, q_lens, pair):
    got, want = _attention_case(torch.bfloat16, 4, 2, 64, 8, window, seg_lens=[517, 300], q_lens=q_lens, splits=1,
                                seed=5, spike=True, mma=True, tma=True, poison=True, tc=True, pair=pair)
    assert torch.allclose(got, want, **MMA_TOL)


@pytest.mark.parametrize("nh,nkv,hd,ps", [(12, 2, 128, 16), (6, 3, 64, 32)])
@pytest.mark.parametrize("window,seg_lens,q_lens", [(None, [2048], [2048]), (None, [6000, 700], [512, 700]),
                                                    (1500, [3000], [1024]), (None, [513, 511, 2000], [513, 2, 1100])])
def test_tcgen05_prefill_query_tiles_shared_by_two_blocks(nh, nkv, hd, ps, window, seg_lens, q_lens):
    """Query tiles that see 512 keys or more are computed by two blocks, half of the keys each, and the block that
    finishes last adds the two partial results: prompts around that size, portions late in a long context, a
    window, several requests; twice, since the pairs' counters have to be zero again after a launch."""
    for seed in (3, 4):
        got, want = _attention_case(torch.bfloat16, nh, nkv, hd, ps, window, seg_lens=seg_lens, q_lens=q_lens, splits=1,
                                    seed=seed, spike=True, mma=True, tma=True, poison=True, tc=True, pair=512)
        assert torch.isfinite(got).all()
        assert torch.allclose(got, want, **MMA_TOL)


@pytest.mark.parametrize("window,splits", [(None, 1), (None, 8), (64, 1), (64, 4)])
def test_tma_decode_far_key_and_window_edge(window, splits):
    got, want = _attention_case(torch.bfloat16, 4, 2, 64, 8, window, seg_lens=[517, 300], q_lens=[1, 1], splits=splits,
                                seed=5, spike=True, mma=True, tma=True, poison=True)
    assert torch.allclose(got, want, **MMA_TOL)


@pytest.mark.parametrize("window,splits,q_lens", [(None, 1, [1, 2]), (None, 8, [1, 1]), (64, 1, [1, 2]), (64, 4, [1, 1]),
                                                  (None, 1, [200, 150]), (64, 1, [200, 150])])
def test_mma_attention_far_key_and_window_edge(window, splits, q_lens):
    got, want = _attention_case(torch.bfloat16, 4, 2, 32, 8, window, seg_lens=[517, 300], q_lens=q_lens, splits=splits,
                                seed=5, spike=True, mma=True)
    assert torch.allclose(got, want, **MMA_TOL)


@pytest.mark.parametrize("M", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("N,K", [(64, 64), (176, 80), (2048, 1536), (1536, 8960), (512, 272)])
def test_skinny_linear_store_and_residual(M, N, K):
    from pico_vllm_b200 import ops
    x = torch.randn(M, K, generator=gen(60)).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=gen(61)) / math.sqrt(K)).to(torch.bfloat16)
    bias = torch.randn(N, generator=gen(62))
    want = x.float() @ w.float().t()
    got = ops.skinny_linear(x.to(DEV), w.to(DEV), bias.to(DEV), torch.float32).cpu()
    assert torch.allclose(got, want + bias, atol=2e-3, rtol=2e-3)
    got16 = ops.skinny_linear(x.to(DEV), w.to(DEV)).cpu()
    assert got16.dtype == torch.bfloat16 and torch.allclose(got16.float(), want, atol=2e-2, rtol=2e-2)
    res = torch.randn(M, N, generator=gen(63))
    rg = res.to(DEV)
    ops.skinny_linear_residual(x.to(DEV), w.to(DEV), rg)
    assert torch.allclose(rg.cpu(), res + want, atol=2e-3, rtol=2e-3)
    assert torch.allclose(ops.logits_linear(x.to(DEV), w.to(DEV)).cpu(), want, atol=2e-3, rtol=2e-3)


@pytest.mark.parametrize("M", [1, 8, 13])
@pytest.mark.parametrize("I,K", [(128, 64), (176, 80), (8960, 1536), (320, 192)])
def test_skinny_gate_up_swiglu(M, I, K):
    from pico_vllm_b200 import ops
    x = torch.randn(M, K, generator=gen(64)).to(torch.bfloat16)
    w = (torch.randn(2 * I, K, generator=gen(65)) * 2 / math.sqrt(K)).to(torch.bfloat16)
    got = ops.skinny_gate_up_swiglu(x.to(DEV), w.to(DEV)).cpu().float()
    want = fake_ops.skinny_gate_up_swiglu(x, w).float()
    assert torch.allclose(got, want, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("M", [1, 8, 16])
@pytest.mark.parametrize("nh,nkv,hd,ps,rot,K", [(4, 2, 16, 16, 16, 64), (6, 3, 32, 8, 32, 192), (5, 1, 48, 4, 48, 80),
                                                (12, 2, 128, 16, 128, 1536), (3, 3, 80, 16, 40, 96), (2, 1, 128, 32, 0, 64)])
def test_skinny_qkv_rope_store(M, nh, nkv, hd, ps, rot, K):
    from pico_vllm_b200 import ops
    pages = 12
    N = (nh + 2 * nkv) * hd
    x = torch.randn(M, K, generator=gen(66)).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=gen(67)) / math.sqrt(K)).to(torch.bfloat16)
    bias = 0.5 * torch.randn(N, generator=gen(68))
    pos = torch.randint(0, 5000, (M,), generator=gen(69), dtype=torch.int32)
    inv = 1.0 / (10000.0 ** (torch.arange(0, rot, 2).float() / max(rot, 1))) if rot else torch.zeros(0)
    slots = torch.randperm(pages * ps, generator=gen(70))[:M].to(torch.int32)
    if M > 2:
        slots[1] = -1
    k0 = torch.randn(pages, nkv, ps, hd, generator=gen(71)).to(torch.bfloat16)
    v0 = torch.randn(pages, nkv, ps, hd, generator=gen(72)).to(torch.bfloat16)
    kg, vg = k0.to(DEV), v0.to(DEV)
    qg = ops.skinny_qkv_rope_store(x.to(DEV), w.to(DEV), bias.to(DEV), pos.to(DEV), inv.to(DEV), slots.to(DEV), kg, vg,
                                   nh, nkv, hd, ps)
    kr, vr = k0.clone(), v0.clone()
    qr = fake_ops.skinny_qkv_rope_store(x, w, bias, pos, inv, slots, kr, vr, nh, nkv, hd, ps)
    t = dict(atol=3e-2, rtol=2e-2)
    assert torch.allclose(qg.cpu().float(), qr.float(), **t)
    assert torch.allclose(kg.cpu().float(), kr.float(), **t)
    assert torch.allclose(vg.cpu().float(), vr.float(), **t)
    # without slots only the queries are produced and the pages stay as they were
    kg2 = k0.to(DEV)
    q2 = ops.skinny_qkv_rope_store(x.to(DEV), w.to(DEV), bias.to(DEV), pos.to(DEV), inv.to(DEV), None, None, None,
                                   nh, nkv, hd, ps)
    assert torch.allclose(q2.cpu().float(), qr.float(), **t) and torch.equal(kg2.cpu(), k0)


@pytest.mark.parametrize("M", [1, 8, 11, 16])
@pytest.mark.parametrize("K,eps", [(64, 1e-6), (1536, 1e-6), (192, 1e-5), (80, 1e-3), (2048, 1e-6), (2096, 1e-5)])
def test_skinny_kernels_with_the_norm_inside(M, K, eps):
    """The residual stream goes in as float32 and is RMS-normed inside the product kernels.  Rows up to
    1536 wide are kept in registers between the two passes of the norm; wider rows (2048, 2096: taken at up
    to 8 tokens) are read twice."""
    from pico_vllm_b200 import ops
    T = M + 3
    x = torch.randn(T, K, generator=gen(80)) * 2
    nw = 1 + 0.1 * torch.randn(K, generator=gen(81))
    rows = torch.randperm(T, generator=gen(82))[:M].to(torch.int32)
    # head: chosen rows, float32 logits
    N = 272
    w = (torch.randn(N, K, generator=gen(83)) / math.sqrt(K)).to(torch.bfloat16)
    if not ops.skinny_norm_takes(x.to(DEV), w.to(DEV), M):
        assert M > 8 and K > 1000
        return
    got = ops.skinny_linear(x.to(DEV), w.to(DEV), None, torch.float32, nw.to(DEV), eps, rows.to(DEV)).cpu()
    want = fake_ops.skinny_linear(x, w, None, torch.float32, nw, eps, rows)
    assert torch.allclose(got, want, atol=3e-2, rtol=2e-2)
    # gate_up + swiglu on the first M rows
    I = 176
    wgu = (torch.randn(2 * I, K, generator=gen(84)) * 2 / math.sqrt(K)).to(torch.bfloat16)
    got = ops.skinny_gate_up_swiglu(x[:M].contiguous().to(DEV), wgu.to(DEV), nw.to(DEV), eps).cpu().float()
    want = fake_ops.skinny_gate_up_swiglu(x[:M], wgu, nw, eps).float()
    assert torch.allclose(got, want, atol=3e-2, rtol=3e-2)
    # qkv + rope + store
    nh, nkv, hd, ps, pages = 4, 2, 16, 8, 6
    wq = (torch.randn((nh + 2 * nkv) * hd, K, generator=gen(85)) / math.sqrt(K)).to(torch.bfloat16)
    bias = 0.3 * torch.randn((nh + 2 * nkv) * hd, generator=gen(86))
    pos = torch.randint(0, 900, (M,), generator=gen(87), dtype=torch.int32)
    inv = 1.0 / (10000.0 ** (torch.arange(0, hd, 2).float() / hd))
    slots = torch.randperm(pages * ps, generator=gen(88))[:M].to(torch.int32)
    k0 = torch.zeros(pages, nkv, ps, hd, dtype=torch.bfloat16)
    kg, vg = k0.to(DEV), k0.to(DEV)
    qg = ops.skinny_qkv_rope_store(x[:M].contiguous().to(DEV), wq.to(DEV), bias.to(DEV), pos.to(DEV), inv.to(DEV),
                                   slots.to(DEV), kg, vg, nh, nkv, hd, ps, nw.to(DEV), eps)
    kr, vr = k0.clone(), k0.clone()
    qr = fake_ops.skinny_qkv_rope_store(x[:M], wq, bias, pos, inv, slots, kr, vr, nh, nkv, hd, ps, nw, eps)
    t = dict(atol=3e-2, rtol=2e-2)
    assert torch.allclose(qg.cpu().float(), qr.float(), **t)
    assert torch.allclose(kg.cpu().float(), kr.float(), **t) and torch.allclose(vg.cpu().float(), vr.float(), **t)


@pytest.mark.parametrize("rows", [None, 256, 512])
@pytest.mark.parametrize("M", [128, 200, 2048, 777])
@pytest.mark.parametrize("N,K", [(256, 64), (2048, 1536), (1536, 1536), (1536, 8960), (272, 200), (512, 192)])
def test_tcgen05_linear_store_and_residual(M, N, K, rows):
    from pico_vllm_b200 import ops
    x = torch.randn(M, K, generator=gen(90)).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=gen(91)) / math.sqrt(K)).to(torch.bfloat16)
    want = x.float() @ w.float().t()
    got = ops.tc_linear(x.to(DEV), w.to(DEV), rows=rows).cpu().float()
    assert torch.allclose(got, want, atol=3e-2, rtol=2e-2)
    res = torch.randn(M, N, generator=gen(92))
    rg = res.to(DEV)
    ops.tc_linear_residual(x.to(DEV), w.to(DEV), rg, rows=rows)
    assert torch.allclose(rg.cpu(), res + want, atol=5e-3, rtol=5e-3)
    torch.cuda.synchronize()
    assert ops.tc_status() == 0


@pytest.mark.parametrize("rows", [None, 256, 512])
@pytest.mark.parametrize("M", [128, 333, 2048])
@pytest.mark.parametrize("I,K", [(128, 64), (8960, 1536), (320, 192), (176, 80)])
def test_tcgen05_gate_up_swiglu(M, I, K, rows):
    from pico_vllm_b200 import ops
    x = torch.randn(M, K, generator=gen(93)).to(torch.bfloat16)
    w = (torch.randn(2 * I, K, generator=gen(94)) * 2 / math.sqrt(K)).to(torch.bfloat16)
    got = ops.tc_gate_up_swiglu(x.to(DEV), w.to(DEV), rows=rows).cpu().float()
    want = fake_ops.skinny_gate_up_swiglu(x, w).float()
    assert torch.allclose(got, want, atol=3e-2, rtol=3e-2)
    torch.cuda.synchronize()
    assert ops.tc_status() == 0


def test_refuses_head_sizes_it_does_not_take():
    from pico_vllm_b200 import ops
    from pico_vllm_b200.errors import KernelError
    q = torch.zeros(1, 3 * 24, device=DEV)
    kv = torch.zeros(2, 1, 4, 24, device=DEV)
    i = torch.zeros(1, dtype=torch.int32, device=DEV)
    with pytest.raises(KernelError):
        ops.paged_attention(q, kv, kv, torch.zeros(1, 24, device=DEV), i, i, torch.zeros(1, 2, dtype=torch.int32,
                            device=DEV), 1, 1, 24, 4, None, 1.0)
    with pytest.raises(KernelError):
        ops.embedding(torch.zeros(1, dtype=torch.int32), torch.zeros(2, 2), torch.zeros(1, 2))   # CPU tensors


@pytest.mark.parametrize("V", [50, 331, 5000, 151936])
def test_sample_greedy_and_temperature(V):
    from pico_vllm_b200 import ops
    R = 6
    logits = torch.randn(R, V, generator=gen(30)) * 3
    logits[1, V // 2] = logits[1].max() + 1      # a clear winner
    logits[2, 3] = logits[2, 7] = logits[2].max() + 1   # a tie: the lower index wins
    out = torch.empty(R, dtype=torch.int32, device=DEV)
    ops.sample(logits.to(DEV), None, None, None, out)
    want = torch.empty(R, dtype=torch.int32)
    fake_ops.sample(logits, None, None, None, want)
    assert out.cpu().tolist() == want.tolist()
    assert out[2].item() == 3
    # temperature / top-p rows mixed with a greedy row
    temp = torch.tensor([0.0, 0.7, 1.0, 1.3, 0.8, 2.0])
    topp = torch.tensor([1.0, 1.0, 0.9, 0.5, 0.2, 1.0])
    for trial in range(4):
        u = torch.rand(R, generator=gen(40 + trial))
        ops.sample(logits.to(DEV), temp.to(DEV), topp.to(DEV), u.to(DEV), out)
        got = out.cpu().tolist()
        for r in range(R):
            if temp[r] == 0:
                assert got[r] == int(torch.argmax(logits[r]))
                continue
            probs = torch.softmax(logits[r].double() / float(temp[r]), 0)
            if topp[r] < 1:
                import plain_qwen2 as plain
                probs = plain.top_p_filter(probs[None], float(topp[r]))[0]
            assert probs[got[r]] > 0, "a token outside the top-p set was drawn"
            cum = torch.cumsum(probs, 0)
            lo = float(cum[got[r]] - probs[got[r]])
            hi = float(cum[got[r]])
            target = float(u[r]) * float(cum[-1])
            assert lo - 1e-4 <= target <= hi + 1e-4, (r, lo, target, hi)


def test_sample_distribution():
    from pico_vllm_b200 import ops
    V, N = 7, 4000
    logits = torch.tensor([[0.0, 1.0, 2.0, -1.0, 0.5, 3.0, -5.0]]).repeat(N, 1)
    u = torch.rand(N, generator=gen(50))
    out = torch.empty(N, dtype=torch.int32, device=DEV)
    ops.sample(logits.to(DEV), torch.full((N,), 1.5).to(DEV), torch.ones(N).to(DEV), u.to(DEV), out)
    freq = torch.bincount(out.cpu().long(), minlength=V).double() / N
    probs = torch.softmax(logits[0].double() / 1.5, 0)
    assert float((freq - probs).abs().max()) < 0.03


@pytest.mark.parametrize("M", [1, 8, 13, 16])
@pytest.mark.parametrize("N,K", [(336, 80), (4096, 1536), (151936, 1536)])
@pytest.mark.parametrize("normed", [False, True])
def test_skinny_argmax_is_the_first_largest_logit(M, N, K, normed):
    """The greedy head: the token is chosen in the product's epilogue.  It must be the argmax of the logits the
    same kernel family writes (the sums are the same), and the first of equal logits: rows 5 and N - 7 of the
    weights are made equal and dominant for token 0."""
    from pico_vllm_b200 import ops
    T = M + 2
    xf = torch.randn(T, K, generator=gen(140)) * 2
    w = (torch.randn(N, K, generator=gen(141)) / math.sqrt(K)).to(torch.bfloat16)
    nw = 1 + 0.1 * torch.randn(K, generator=gen(142))
    rows = torch.randperm(T, generator=gen(143))[:M].to(torch.int32)
    if normed:
        if not ops.skinny_norm_takes(xf.to(DEV), w.to(DEV), M):
            pytest.skip("the fused norm does not take this many rows of this width")
        x_eff = fake_ops._normed(xf, nw, 1e-5)[rows.long()]
    else:
        x_eff = xf[:M].to(torch.bfloat16)
    big = (x_eff[0].float() / x_eff[0].float().norm() * 3).to(torch.bfloat16)
    w[5] = big
    w[N - 7] = big
    out = torch.full((M + 3,), -1, dtype=torch.int32, device=DEV)
    if normed:
        ops.skinny_argmax(xf.to(DEV), w.to(DEV), out, nw.to(DEV), 1e-5, rows.to(DEV))
        logits = ops.skinny_linear(xf.to(DEV), w.to(DEV), None, torch.float32, nw.to(DEV), 1e-5, rows.to(DEV))
    else:
        ops.skinny_argmax(x_eff.to(DEV), w.to(DEV), out)
        logits = ops.skinny_linear(x_eff.to(DEV), w.to(DEV), None, torch.float32)
    got = out.cpu()
    assert got[M:].tolist() == [-1, -1, -1]                         # nothing written past the rows
    assert got[:M].tolist() == logits.cpu().argmax(-1).tolist()     # on the CPU torch's argmax returns the first of equals
    assert got[0] == 5
    # and against the plain product: the chosen logit is (nearly) the largest
    ref = x_eff.float() @ w.float().t()
    picked = ref[torch.arange(M), got[:M].long()]
    assert float((ref.max(-1).values - picked).max()) <= 2e-2 * float(ref.abs().max())
    # twice in a row: the second launch finds the first one's counters cleared
    out2 = torch.full((M,), -1, dtype=torch.int32, device=DEV)
    if normed:
        ops.skinny_argmax(xf.to(DEV), w.to(DEV), out2, nw.to(DEV), 1e-5, rows.to(DEV))
    else:
        ops.skinny_argmax(x_eff.to(DEV), w.to(DEV), out2)
    assert out2.cpu().tolist() == got[:M].tolist()
