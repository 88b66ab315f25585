"""Each kernel alone against a plain float32 torch statement of the same operation, at sizes the
engine's tiny models do not use (needs a GPU)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


@pytest.fixture(scope="module")
def ops():
    from sharpinference_b200.kernels import ops as _ops
    return _ops


def rnd(*shape, dtype=torch.float32, scale=1.0, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


# ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed_gather(ops, dtype):
    table = rnd(1000, 200, dtype=dtype)
    ids = torch.tensor([0, 999, 5, 5, 731], dtype=torch.int32, device=DEV)
    out = ops.embed_gather(ids, table)
    assert out.dtype == torch.float32 and torch.equal(out, table[ids.long()].float())


@pytest.mark.parametrize("H", [8, 1000, 5120, 8192, 9000, 20000])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_add_rmsnorm(ops, H, out_dtype):
    T, eps = 37, 1e-5
    x, delta, w = rnd(T, H, seed=1), rnd(T, H, seed=2), 1 + 0.1 * rnd(H, seed=3)
    ref_x = x + delta
    ref = ref_x * torch.rsqrt((ref_x.double() ** 2).mean(-1, keepdim=True) + eps).float() * w
    x1 = x.clone()
    out, out32 = ops.add_rmsnorm(x1, delta, w, eps, out_dtype, want_fp32=True)
    assert torch.equal(x1, ref_x)                                            # the residual stream got the sum
    assert torch.allclose(out32, ref, rtol=2e-6, atol=1e-6)
    assert torch.allclose(out.float(), ref.to(out_dtype).float(), rtol=1e-2 if out_dtype == torch.bfloat16 else 2e-6, atol=1e-6)
    # no delta; and the gathered form leaves x alone
    x2 = x.clone()
    out_nd, _ = ops.add_rmsnorm(x2, None, w, eps, torch.float32)
    assert torch.equal(x2, x)
    assert torch.allclose(out_nd, x * torch.rsqrt((x.double() ** 2).mean(-1, keepdim=True) + eps).float() * w, rtol=2e-6, atol=1e-6)
    rows = torch.tensor([36, 0, 7], dtype=torch.int32, device=DEV)
    x3 = x.clone()
    out_rows, _ = ops.add_rmsnorm(x3, delta, w, eps, torch.float32, rows=rows)
    assert torch.equal(x3, x) and torch.allclose(out_rows, ref[rows.long()], rtol=2e-6, atol=1e-6)


@pytest.mark.parametrize("H", [777, 5120, 8192, 9000])
def test_rmsnorm_rows_do_not_depend_on_the_batch(ops, H):
    """Steps of few rows take a kernel built for latency, steps of many rows one built for bandwidth; both add a
    row's squares in the same order, so a row alone, among 64 and among 300 gives the same bits."""
    x, w = rnd(300, H, seed=4), 1 + 0.1 * rnd(H, seed=5)
    full, _ = ops.add_rmsnorm(x.clone(), None, w, 1e-6, torch.float32)
    some, _ = ops.add_rmsnorm(x[:64].clone(), None, w, 1e-6, torch.float32)
    one, _ = ops.add_rmsnorm(x[13:14].clone(), None, w, 1e-6, torch.float32)
    assert torch.equal(full[13:14], one) and torch.equal(full[:64], some)


def test_swiglu_scales_before_the_nonlinearity(ops):
    M, I = 9, 300
    gu = rnd(M, 2 * I, seed=6)
    scale = torch.rand(20, device=DEV) + 0.1
    rows = torch.randint(0, 20, (M,), device=DEV, dtype=torch.int32)
    out = ops.swiglu(gu, torch.float32, row_scale=scale, scale_rows=rows)
    s = scale[rows.long()][:, None]
    g, u = gu[:, :I] * s, gu[:, I:] * s
    assert torch.allclose(out, g / (1 + torch.exp(-g)) * u, rtol=1e-5, atol=1e-6)
    plain_out = ops.swiglu(gu, torch.bfloat16)
    g, u = gu[:, :I], gu[:, I:]
    assert torch.allclose(plain_out.float(), (g / (1 + torch.exp(-g)) * u), rtol=1e-2, atol=1e-3)


# ---------------------------------------------------------------------------------------
def rope_ref(x, pos, inv_freq, pairing):
    ang = pos.float()[:, None] * inv_freq[None, :]
    cos, sin = torch.cos(ang.double())[:, None, :], torch.sin(ang.double())[:, None, :]
    x = x.double()
    out = torch.empty_like(x)
    if pairing == "interleaved":
        a, b = x[..., 0::2], x[..., 1::2]
        out[..., 0::2], out[..., 1::2] = a * cos - b * sin, a * sin + b * cos
    else:
        h = x.shape[-1] // 2
        a, b = x[..., :h], x[..., h:]
        out[..., :h], out[..., h:] = a * cos - b * sin, a * sin + b * cos
    return out


@pytest.mark.parametrize("nq,nkv,d", [(6, 2, 48), (5, 5, 16), (8, 1, 128), (2, 1, 272), (3, 1, 512), (2, 2, 6), (1, 1, 500)])
@pytest.mark.parametrize("variant", ["rope+l2", "halves", "nope+temp", "bare"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_qkv_post(ops, nq, nkv, d, variant, dtype):
    ps, pages, B = 8, 12, 2
    lens = [11, 5]
    starts = [3, 40]
    T = sum(lens)
    positions = torch.tensor([s + i for s, n in zip(starts, lens) for i in range(n)], dtype=torch.int32, device=DEV)
    row_req = torch.tensor([b for b, n in enumerate(lens) for _ in range(n)], dtype=torch.int32, device=DEV)
    table = torch.full((B, 8), -1, dtype=torch.int32, device=DEV)
    table[0, 0], table[0, 1] = 7, 2                    # positions 3..13 -> blocks 0, 1
    table[1, 5] = 9                                     # positions 40..44 -> block 5
    qkv = rnd(T, (nq + 2 * nkv) * d, seed=8)
    inv_freq = (1.0 / (10000.0 ** (torch.arange(0, d, 2).float() / d))).to(DEV)
    kv = torch.full((pages, 2, nkv, ps, d), 99.0, dtype=dtype, device=DEV)
    q_out = torch.empty(T, nq, d, dtype=dtype, device=DEV)
    use_rope = variant in ("rope+l2", "halves")
    pairing = {"rope+l2": ops.ROPE_INTERLEAVED, "halves": ops.ROPE_HALVES}.get(variant, ops.ROPE_NONE)
    l2 = 1e-6 if variant == "rope+l2" else -1.0
    temp = (0.1, 8.0) if variant == "nope+temp" else (0.0, 0.0)
    ops.qkv_post(qkv, positions, row_req, table, inv_freq if use_rope else None, q_out, kv, nq=nq, nkv=nkv, d=d,
                 page_size=ps, pairing=pairing, l2_eps=l2, temp_attn_scale=temp[0], temp_floor_scale=temp[1],
                 write_kv=True)
    q = qkv[:, :nq * d].view(T, nq, d).double()
    k = qkv[:, nq * d:(nq + nkv) * d].view(T, nkv, d).double()
    v = qkv[:, (nq + nkv) * d:].view(T, nkv, d).double()
    if use_rope:
        name = "interleaved" if variant == "rope+l2" else "halves"
        q, k = rope_ref(q, positions, inv_freq, name), rope_ref(k, positions, inv_freq, name)
    if l2 >= 0:
        q = q / torch.sqrt((q * q).mean(-1, keepdim=True) + l2)
        k = k / torch.sqrt((k * k).mean(-1, keepdim=True) + l2)
    if temp[1] > 0:
        q = q * (1 + temp[0] * torch.log1p(torch.floor((positions.double() + 1) / temp[1])))[:, None, None]
    tol = dict(rtol=2e-2, atol=2e-2) if dtype == torch.bfloat16 else dict(rtol=1e-5, atol=1e-5)
    assert torch.allclose(q_out.double(), q, **tol)
    for t in range(T):
        b, pos = int(row_req[t]), int(positions[t])
        page = int(table[b, pos // ps])
        assert torch.allclose(kv[page, 0, :, pos % ps, :].double(), k[t], **tol)
        assert torch.allclose(kv[page, 1, :, pos % ps, :].double(), v[t], **tol)
    written = {(int(table[int(row_req[t]), int(positions[t]) // ps]), int(positions[t]) % ps) for t in range(T)}
    untouched = [(p, o) for p in range(pages) for o in range(ps) if (p, o) not in written]
    p_idx = torch.tensor([p for p, _ in untouched], device=DEV)
    o_idx = torch.tensor([o for _, o in untouched], device=DEV)
    assert bool((kv[p_idx, :, :, o_idx, :] == 99.0).all())      # nothing else was written
    # a layer that borrows a cache writes q only
    kv2 = torch.full_like(kv, 5.0)
    ops.qkv_post(qkv, positions, row_req, table, None, q_out, kv2, nq=nq, nkv=nkv, d=d, page_size=ps,
                 pairing=ops.ROPE_NONE, l2_eps=-1.0, temp_attn_scale=0.0, temp_floor_scale=0.0, write_kv=False)
    assert bool((kv2 == 5.0).all())


# ---------------------------------------------------------------------------------------
def attention_ref(q, k_all, v_all, positions, row_req, lo_of, scale, nq, nkv):
    """q [T, nq, d]; k_all/v_all: per request [S, nkv, d] float64."""
    T, _, d = q.shape
    out = torch.zeros(T, nq, d, dtype=torch.float64)
    for t in range(T):
        b, pos = int(row_req[t]), int(positions[t])
        lo = lo_of(pos)
        for h in range(nq):
            kh = k_all[b][lo:pos + 1, h // (nq // nkv)]
            vh = v_all[b][lo:pos + 1, h // (nq // nkv)]
            p = torch.softmax((kh @ q[t, h].double()) * scale, dim=0)
            out[t, h] = p @ vh
    return out.reshape(T, nq * d)


def paged_setup(lens, nkv, d, ps, dtype, seed, shuffle=True):
    """Random K/V for requests of the given lengths, scattered over shuffled pages."""
    g = torch.Generator().manual_seed(seed)
    blocks = [(n + ps - 1) // ps for n in lens]
    pages = sum(blocks) + 3
    perm = torch.randperm(pages, generator=g).tolist() if shuffle else list(range(pages))
    table = torch.full((len(lens), max(blocks) + 1), -1, dtype=torch.int32)
    kv = torch.zeros(pages, 2, nkv, ps, d, dtype=dtype)
    ks, vs, at = [], [], 0
    for b, n in enumerate(lens):
        k = torch.randn(n, nkv, d, generator=g).to(dtype)
        v = torch.randn(n, nkv, d, generator=g).to(dtype)
        ks.append(k.double()); vs.append(v.double())
        for blk in range(blocks[b]):
            page = perm[at]; at += 1
            table[b, blk] = page
            n_in = min(ps, n - blk * ps)
            kv[page, 0, :, :n_in] = k[blk * ps: blk * ps + n_in].transpose(0, 1)
            kv[page, 1, :, :n_in] = v[blk * ps: blk * ps + n_in].transpose(0, 1)
    return kv.to(DEV), table.to(DEV), ks, vs


@pytest.mark.parametrize("nq,nkv,d,ps", [(4, 2, 16, 4), (6, 3, 48, 16), (5, 1, 128, 64), (2, 2, 256, 8), (40, 8, 128, 64)])
@pytest.mark.parametrize("mask", [("full", 0), ("chunk", 24), ("window", 9)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_paged_attention_generic(ops, nq, nkv, d, ps, mask, dtype):
    lens = [150, 37, 1]
    kv, table, ks, vs = paged_setup(lens, nkv, d, ps, dtype, seed=d + ps)
    # rows: a prompt portion of request 0 (positions 100..149), the last token of request 1, request 2's only token
    rows = [(0, p) for p in range(100, 150)] + [(1, 36), (2, 0)]
    positions = torch.tensor([p for _, p in rows], dtype=torch.int32, device=DEV)
    row_req = torch.tensor([b for b, _ in rows], dtype=torch.int32, device=DEV)
    q = rnd(len(rows), nq, d, dtype=dtype, seed=11)
    kind, span = mask
    code = {"full": ops.MASK_FULL, "chunk": ops.MASK_CHUNK, "window": ops.MASK_WINDOW}[kind]
    lo_of = {"full": lambda p: 0, "chunk": lambda p: p // span * span, "window": lambda p: max(0, p - span + 1)}[kind]
    scale = 1.0 / math.sqrt(d)
    out = ops.paged_attention_generic(q, kv, table, row_req, positions, nq=nq, nkv=nkv, d=d, page_size=ps,
                                      mask_kind=code, mask_span=max(span, 1), scale=scale)
    ref = attention_ref(q.cpu(), ks, vs, positions.cpu(), row_req.cpu(), lo_of, scale, nq, nkv)
    tol = dict(rtol=2e-2, atol=2e-2) if dtype == torch.bfloat16 else dict(rtol=1e-5, atol=1e-5)
    assert torch.allclose(out.double().cpu(), ref, **tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_finds_one_far_key_among_hundreds(ops, dtype):
    """One key far back is made to match the query; its value must dominate the output.  A kernel
    that loses a tile, a page or the first key of a chunk shows here where random data would hide it."""
    nq, nkv, d, ps = 4, 2, 32, 16
    n = 700
    for far in (0, 1, 15, 16, 127, 128, 129, 383, 384, 698, 699):
        kv, table, ks, vs = paged_setup([n], nkv, d, ps, dtype, seed=far)
        q = rnd(1, nq, d, dtype=dtype, seed=far + 1)
        page, off = int(table[0, far // ps]), far % ps
        for h in range(nkv):
            kv[page, 0, h, off] = (q[0, h * 2].float() * 8.0).to(dtype)          # q.k / sqrt(d) is far above the rest
        positions = torch.tensor([n - 1], dtype=torch.int32, device=DEV)
        row_req = torch.zeros(1, dtype=torch.int32, device=DEV)
        out = ops.paged_attention_generic(q, kv, table, row_req, positions, nq=nq, nkv=nkv, d=d, page_size=ps,
                                          mask_kind=ops.MASK_FULL, mask_span=1, scale=1 / math.sqrt(d))
        out = out.view(nq, d).float()
        for h in range(nkv):
            target = kv[page, 1, h, off].float()
            assert torch.allclose(out[h * 2], target, atol=5e-2), (far, h)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_chunk_and_window_edges(ops, dtype):
    """The key just outside a chunk or window is made overwhelmingly attractive: it must not be seen.
    The key just inside is made attractive next: it must be."""
    nq, nkv, d, ps, n = 2, 1, 16, 8, 100
    for kind, span, pos, outside, inside in (("chunk", 24, 50, 47, 48), ("chunk", 24, 48, 47, 48),
                                             ("window", 9, 60, 51, 52), ("window", 9, 8, None, 0)):
        code = {"chunk": 1, "window": 2}[kind]
        for which, key in (("outside", outside), ("inside", inside)):
            if key is None:
                continue
            kv, table, ks, vs = paged_setup([n], nkv, d, ps, dtype, seed=pos)
            q = rnd(1, nq, d, dtype=dtype, seed=3)
            page, off = int(table[0, key // ps]), key % ps
            kv[page, 0, 0, off] = (q[0, 0].float() * 10.0).to(dtype)
            kv[page, 1, 0, off] = 50.0
            positions = torch.tensor([pos], dtype=torch.int32, device=DEV)
            out = ops.paged_attention_generic(q, kv, table, torch.zeros(1, dtype=torch.int32, device=DEV), positions,
                                              nq=nq, nkv=nkv, d=d, page_size=ps, mask_kind=code, mask_span=span,
                                              scale=1 / math.sqrt(d)).float()
            if which == "outside":
                assert float(out[0, :d].abs().max()) < 10.0, (kind, pos, key)
            else:
                assert float(out[0, :d].min()) > 40.0, (kind, pos, key)


# ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("M,N,K", [(1, 1, 1), (37, 53, 71), (64, 64, 16), (130, 300, 257), (3, 2000, 96)])
@pytest.mark.parametrize("dt", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                (torch.float32, torch.bfloat16), (torch.bfloat16, torch.float32)])
def test_gemm_nt_dense(ops, M, N, K, dt):
    a, w = rnd(M, K, dtype=dt[0], seed=1), rnd(N, K, dtype=dt[1], seed=2)
    out = ops.gemm_nt(a, w)
    ref = (a.double() @ w.double().T)
    assert torch.allclose(out.double(), ref, rtol=1e-5, atol=1e-4)


def test_gemm_nt_rows_do_not_depend_on_the_batch(ops):
    a, w = rnd(200, 300, seed=3), rnd(77, 300, seed=4)
    full = ops.gemm_nt(a, w)
    assert torch.equal(full[131:132], ops.gemm_nt(a[131:132].contiguous(), w))
    assert torch.equal(full[:70], ops.gemm_nt(a[:70].contiguous(), w))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gemm_nt_grouped_gather_scatter_accumulate(ops, dtype):
    E, N, K, T = 5, 70, 90, 200
    w = rnd(E, N, K, dtype=dtype, seed=5)
    a = rnd(T, K, dtype=dtype, seed=6)
    expert = torch.randint(0, E, (T,), generator=torch.Generator().manual_seed(7))
    expert[expert == 3] = 1                                  # expert 3 gets no rows
    order = torch.argsort(expert, stable=True)
    counts = torch.bincount(expert, minlength=E)
    offsets = torch.cat([torch.zeros(1, dtype=torch.long), torch.cumsum(counts, 0)]).to(torch.int32).to(DEV)
    sorted_rows = order.to(torch.int32).to(DEV)
    ref = torch.stack([a[t].double() @ w[int(expert[t])].double().T for t in range(T)])
    gathered = ops.gemm_nt(a, w, group_offsets=offsets, a_rows=sorted_rows, rows=T)
    assert torch.allclose(gathered.double(), ref[order.to(DEV)], rtol=1e-5, atol=1e-4)
    base = rnd(T, N, seed=8)
    acc = base.clone()
    ops.gemm_nt(a[order.to(DEV)].contiguous(), w, group_offsets=offsets, out_rows=sorted_rows, rows=T, out=acc,
                accumulate=True)
    assert torch.allclose(acc.double(), base.double() + ref, rtol=1e-5, atol=1e-4)


# ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("T,H,E", [(1, 77, 5), (50, 5120, 16), (9, 5120, 128), (3, 20000, 7), (1100, 333, 6),
                                   (1029, 1280, 19), (40, 24, 3), (1030, 5120, 16), (1100, 8192, 5), (2050, 5120, 128),
                                   (1025, 2048, 7)])
def test_router_top1(ops, T, H, E):
    h, wr = rnd(T, H, seed=9), rnd(E, H, scale=0.05, seed=10)
    expert, weight, logits = ops.router_top1(h, wr, want_logits=True)
    ref = h.double() @ wr.double().T
    assert torch.allclose(logits.double(), ref, rtol=1e-4, atol=1e-4)
    p = torch.sigmoid(logits)
    assert torch.equal(expert.long(), torch.argmax(p, dim=1))
    assert torch.allclose(weight, p.max(dim=1).values, rtol=1e-6)


@pytest.mark.parametrize("T,E", [(1, 16), (8, 16), (32, 128), (7, 3), (33, 5), (1200, 16)])
def test_router_sorts_in_the_same_call(ops, T, E):
    """With sort=True the rows come back sorted by expert: from the router's own launch for up to 32 tokens
    (three calls in a row: the counters are left at zero), from the sort kernel otherwise."""
    for seed in range(3):
        h, wr = rnd(T, 640, seed=40 + seed), rnd(E, 640, scale=0.05, seed=50 + seed)
        expert, weight, _, offsets, rows = ops.router_top1(h, wr, sort=True)
        ref_offsets, ref_rows = ops.moe_sort(expert, E)
        assert torch.equal(offsets, ref_offsets) and torch.equal(rows, ref_rows)
        assert rows.cpu().tolist() == torch.argsort(expert.long().cpu(), stable=True).tolist()


def test_router_first_of_equal_experts_wins(ops):
    h = torch.ones(2, 16, device=DEV)
    wr = torch.zeros(6, 16, device=DEV)
    wr[2], wr[4] = 0.25, 0.25
    expert, weight, _ = ops.router_top1(h, wr)
    assert expert.tolist() == [2, 2] and float(weight[0]) == pytest.approx(1 / (1 + math.exp(-4.0)))


@pytest.mark.parametrize("T,E", [(0, 4), (1, 1), (33, 4), (1000, 16), (5000, 128), (77, 1000), (4096, 3), (9001, 40)])
def test_moe_sort_is_a_stable_counting_sort(ops, T, E):
    ids = torch.randint(0, E, (T,), generator=torch.Generator().manual_seed(T + E)).to(torch.int32).to(DEV)
    offsets, rows = ops.moe_sort(ids, E)
    counts = torch.bincount(ids.long().cpu(), minlength=E)
    assert offsets.cpu().tolist() == [0] + torch.cumsum(counts, 0).tolist()
    assert rows.cpu().tolist() == torch.argsort(ids.long().cpu(), stable=True).tolist()


# ---------------------------------------------------------------------------------------
def test_argmax_lowest_index_wins(ops):
    logits = rnd(5, 202048, seed=12)
    logits[0, 7] = logits[0, 150000] = 50.0
    logits[1, :] = 0.0
    logits[2, 202047] = 60.0
    logits[3, 0] = 60.0
    out = ops.argmax_rows(logits).tolist()
    assert out[:4] == [7, 0, 202047, 0] and out[4] == int(torch.argmax(logits[4]))


@pytest.mark.parametrize("R,V", [(1, 4097), (3, 202048), (16, 5000), (17, 5000), (70, 5000), (2, 100), (9, 32003)])
def test_argmax_sliced_and_whole_rows_agree_with_a_scan(ops, R, V):
    """Up to 16 rows of at least 4096 entries are cut over 32 blocks each; everything else takes a block per
    row.  Three calls in a row (the counters go back to zero), ties and rows without a finite entry."""
    for seed in range(3):
        logits = rnd(R, V, seed=60 + seed)
        logits[0, V // 3] = logits[0, V - 1] = 99.0                 # a tie across slices: the lower index
        if R > 1:
            logits[1, :] = float("-inf")                            # nothing finite: index 0
        out = ops.argmax_rows(logits).tolist()
        ref = [int(torch.argmax(logits[r])) for r in range(R)]
        ref[0] = V // 3
        if R > 1:
            ref[1] = 0
        assert out == ref


def test_sampling_follows_the_filtered_distribution(ops):
    import plain_llama4 as plain
    V, R = 1000, 256
    row = rnd(V, scale=2.0, seed=13)
    u = ((torch.arange(R, dtype=torch.float32) + 0.5) / R).to(DEV)
    for temp, k, p, mp in ((0.8, 0, 1.0, 0.0), (1.0, 40, 1.0, 0.0), (0.7, 0, 0.9, 0.0), (1.3, 0, 1.0, 0.05),
                           (0.7, 40, 0.95, 0.05)):
        dist = plain.sample_distribution(row.cpu(), temp, top_k=k, top_p=p, min_p=mp)
        got = ops.sample_rows(row.expand(R, V).contiguous(), torch.full((R,), temp, device=DEV),
                              torch.full((R,), k, dtype=torch.int32, device=DEV), torch.full((R,), p, device=DEV),
                              torch.full((R,), mp, device=DEV), u).tolist()
        want = [plain.draw(dist, float(x)) for x in u.tolist()]
        differ = sum(a != b for a, b in zip(got, want))
        assert differ <= 2, (temp, k, p, mp, differ)          # a draw may sit on a boundary of the cumulative sum
        assert all(dist[t] > 0 for t in got)                   # never a token outside the kept set
    greedy = ops.sample_rows(row.expand(3, V).contiguous(), torch.zeros(3, device=DEV),
                             torch.zeros(3, dtype=torch.int32, device=DEV), torch.ones(3, device=DEV),
                             torch.zeros(3, device=DEV), torch.rand(3, device=DEV)).tolist()
    assert greedy == [int(torch.argmax(row))] * 3


@pytest.mark.parametrize("V", [4096, 50021, 202048])
def test_sliced_sampler_follows_the_filtered_distribution(ops, V):
    """Large vocabularies: every row cut over 32 blocks, thresholds by radix selection, mass in fixed point.
    Against the plain statement, for every filter alone and all together."""
    import plain_llama4 as plain
    R = 128
    row = rnd(V, scale=2.5, seed=17)
    u = ((torch.arange(R, dtype=torch.float32) + 0.5) / R).to(DEV)
    for temp, k, p, mp in ((0.8, 0, 1.0, 0.0), (1.0, 40, 1.0, 0.0), (0.7, 0, 0.9, 0.0), (1.3, 0, 1.0, 0.05),
                           (0.7, 40, 0.95, 0.05), (1.0, 1, 1.0, 0.0), (0.9, 5000, 0.5, 0.0)):
        dist = plain.sample_distribution(row.cpu(), temp, top_k=k, top_p=p, min_p=mp)
        got = ops.sample_rows(row.expand(R, V).contiguous(), torch.full((R,), temp, device=DEV),
                              torch.full((R,), k, dtype=torch.int32, device=DEV), torch.full((R,), p, device=DEV),
                              torch.full((R,), mp, device=DEV), u, any_top_k=k > 0, any_top_p=p < 1.0).tolist()
        csum = torch.cumsum(dist, 0)                          # plain.draw, for all draws at once
        want = torch.searchsorted(csum, u.cpu().double()).clamp(max=V - 1).tolist()
        differ = sum(a != b for a, b in zip(got, want))
        assert differ <= 3, (temp, k, p, mp, differ)          # a draw may sit on a boundary of the cumulative sum
        assert all(dist[t] > 0 for t in got), (temp, k, p, mp)  # never a token outside the kept set


def test_sliced_sampler_rows_are_independent_and_repeatable(ops):
    """Rows with different settings in one call (greedy, plain temperature, top-k, top-p, both): each row gets
    what it gets alone, twice in a row, and ties at a threshold stay together."""
    V = 30011
    logits = rnd(6, V, scale=3.0, seed=23)
    logits[4, 100] = logits[4, 20000] = logits[4, 7] = 50.0              # a three-way tie at the top
    temp = torch.tensor([0.0, 0.9, 1.0, 0.7, 1.0, 0.8], device=DEV)
    k = torch.tensor([0, 0, 20, 0, 2, 50], dtype=torch.int32, device=DEV)
    p = torch.tensor([1.0, 1.0, 1.0, 0.8, 1.0, 0.9], device=DEV)
    mp = torch.tensor([0.0, 0.0, 0.0, 0.0, 0.0, 0.02], device=DEV)
    for u0 in (0.03, 0.5, 0.97):
        u = torch.full((6,), u0, device=DEV)
        both = ops.sample_rows(logits, temp, k, p, mp, u).tolist()
        again = ops.sample_rows(logits, temp, k, p, mp, u).tolist()
        alone = [ops.sample_rows(logits[r:r + 1].contiguous(), temp[r:r + 1], k[r:r + 1], p[r:r + 1], mp[r:r + 1],
                                 u[r:r + 1]).tolist()[0] for r in range(6)]
        assert both == again == alone
        assert both[0] == int(torch.argmax(logits[0]))
        assert both[4] in (7, 100, 20000)                   # top-k 2 with three equal leaders keeps all three
    picks = {ops.sample_rows(logits[4:5].contiguous(), temp[4:5], k[4:5], p[4:5], mp[4:5],
                             torch.tensor([x], device=DEV)).tolist()[0] for x in (0.1, 0.5, 0.9)}
    assert picks == {7, 100, 20000}


def test_penalties_and_bias(ops):
    logits = torch.tensor([[2.0, -1.0, 0.5, 3.0], [1.0, 1.0, 1.0, 1.0]], device=DEV)
    ops.add_logit_bias(logits, torch.tensor([0, 1], dtype=torch.int32, device=DEV),
                       torch.tensor([2, 3], dtype=torch.int32, device=DEV), torch.tensor([1.5, -4.0], device=DEV))
    assert logits.tolist() == [[2.0, -1.0, 2.0, 3.0], [1.0, 1.0, 1.0, -3.0]]
    ops.apply_penalties(logits, torch.tensor([0, 0, 1], dtype=torch.int32, device=DEV),
                        torch.tensor([0, 1, 3], dtype=torch.int32, device=DEV),
                        torch.tensor([1, 3, 2], dtype=torch.int32, device=DEV),
                        torch.tensor([2.0, 1.0], device=DEV), torch.tensor([0.0, 0.5], device=DEV),
                        torch.tensor([0.0, 0.25], device=DEV))
    # row 0: repetition 2 -> positive halves, negative doubles; row 1: -(2 * 0.5 + 0.25)
    assert logits.tolist() == [[1.0, -2.0, 2.0, 3.0], [1.0, 1.0, 1.0, -4.25]]


def test_no_cpu_path(ops):
    from sharpinference_b200.kernels.library import KernelError
    with pytest.raises(KernelError, match="CUDA"):
        ops.embed_gather(torch.zeros(2, dtype=torch.int32), torch.zeros(4, 4))
    with pytest.raises(KernelError):
        ops.paged_attention_generic(torch.zeros(1, 3, 16, device=DEV), torch.zeros(1, 2, 2, 4, 16, device=DEV),
                                    torch.zeros(1, 1, dtype=torch.int32, device=DEV),
                                    torch.zeros(1, dtype=torch.int32, device=DEV),
                                    torch.zeros(1, dtype=torch.int32, device=DEV), nq=3, nkv=2, d=16, page_size=4,
                                    mask_kind=0, mask_span=1, scale=1.0)


# ---------------------------------------------------------------------------------------
# tensor-core grouped product (tcgen05 / TMEM / TMA)
# ---------------------------------------------------------------------------------------
def grouped_case(T, E, K, seed, empty=()):
    g = torch.Generator().manual_seed(seed)
    expert = torch.randint(0, E, (T,), generator=g)
    for e in empty:
        expert[expert == e] = (e + 1) % E
    order = torch.argsort(expert, stable=True)
    counts = torch.bincount(expert, minlength=E)
    offsets = torch.cat([torch.zeros(1, dtype=torch.long), torch.cumsum(counts, 0)]).to(torch.int32).to(DEV)
    a = (torch.randn(T, K, generator=g)).to(torch.bfloat16)
    return expert, order, offsets, a


@pytest.mark.parametrize("T,E,N,K,row_tile", [(8, 4, 256, 128, 16), (5, 3, 200, 72, 16), (64, 16, 384, 512, 16),
                                              (300, 5, 136, 264, 64), (700, 3, 520, 128, 128), (70, 2, 128, 64, 32),
                                              (1500, 4, 256, 192, 256), (2100, 3, 520, 128, 128),
                                              (2500, 5, 136, 72, 128), (2048, 2, 256, 64, 256),
                                              (700, 3, 520, 128, 0), (2500, 5, 136, 72, 0), (1100, 40, 264, 192, 0)])
def test_tc_grouped_gemm_store(ops, T, E, N, K, row_tile):
    expert, order, offsets, a = grouped_case(T, E, K, seed=T + N, empty=(1,) if E > 2 else ())
    w = rnd(E, N, K, dtype=torch.bfloat16, scale=0.1, seed=3)
    a_sorted = a[order].contiguous().to(DEV)
    ref = torch.stack([a[t].double() @ w[int(expert[t])].double().cpu().T for t in range(T)])
    sorted_rows = order.to(torch.int32).to(DEV)
    out = ops.tc_grouped_gemm(a_sorted, w, offsets, mode=ops.TC_MODE_STORE, row_tile=row_tile)
    ops.check_status(DEV)
    assert torch.allclose(out.double().cpu(), ref[order], rtol=1e-4, atol=1e-3)
    base = rnd(T, N, seed=4)
    acc = base.clone()
    ops.tc_grouped_gemm(a_sorted, w, offsets, mode=ops.TC_MODE_STORE, out=acc, out_rows=sorted_rows, accumulate=True,
                        row_tile=row_tile)
    ops.check_status(DEV)
    assert torch.allclose(acc.double().cpu(), base.double().cpu() + ref, rtol=1e-4, atol=1e-3)


@pytest.mark.parametrize("T,E,I,K,row_tile", [(8, 4, 128, 128, 16), (7, 3, 40, 88, 16), (64, 16, 256, 320, 16),
                                              (300, 5, 72, 264, 64), (900, 3, 200, 128, 128), (600, 2, 136, 64, 256),
                                              (900, 3, 200, 128, 0), (2300, 7, 136, 320, 0), (2048, 128, 136, 128, 0), (64, 128, 72, 64, 16),
                                              (3000, 200, 40, 64, 0)])
def test_tc_grouped_gemm_swiglu(ops, T, E, I, K, row_tile):
    expert, order, offsets, a = grouped_case(T, E, K, seed=T + I, empty=(0,) if E > 2 else ())
    w = rnd(E, 2 * I, K, dtype=torch.bfloat16, scale=0.1, seed=5)
    scale = (torch.rand(T, generator=torch.Generator().manual_seed(6)) * 0.5 + 0.25)
    a_sorted = ops.gather_rows_bf16(a.to(DEV), order.to(torch.int32).to(DEV))
    assert torch.equal(a_sorted.cpu(), a[order])
    act = ops.tc_grouped_gemm(a_sorted, w, offsets, mode=ops.TC_MODE_SWIGLU, row_scale=scale.to(DEV),
                              scale_rows=order.to(torch.int32).to(DEV), row_tile=row_tile)
    ops.check_status(DEV)
    ref = []
    for t in order.tolist():
        gu = (a[t].double() @ w[int(expert[t])].double().cpu().T) * float(scale[t])
        g, u = gu[:I], gu[I:]
        ref.append(g / (1 + torch.exp(-g)) * u)
    ref = torch.stack(ref)
    assert act.dtype == torch.bfloat16 and act.shape == (T, I)
    assert torch.allclose(act.double().cpu(), ref, rtol=1e-2, atol=1e-2 * float(ref.abs().max()))


def test_tc_grouped_gemm_rows_do_not_depend_on_the_batch(ops):
    """A row alone, in a small batch and in a large one gives bit-identical results."""
    E, N, K = 4, 256, 320
    w = rnd(E, N, K, dtype=torch.bfloat16, scale=0.1, seed=7)
    a = rnd(400, K, dtype=torch.bfloat16, seed=8)
    expert = torch.arange(400) % E
    order = torch.argsort(expert, stable=True)
    offsets = torch.tensor([0, 100, 200, 300, 400], dtype=torch.int32, device=DEV)
    big = ops.tc_grouped_gemm(a[order.to(DEV)].contiguous(), w, offsets, mode=ops.TC_MODE_STORE, row_tile=128)
    t = 37                                                   # row 37 goes to expert 1, sorted position 100 + 9
    one = ops.tc_grouped_gemm(a[t:t + 1].contiguous(), w, torch.tensor([0, 0, 1, 1, 1], dtype=torch.int32, device=DEV),
                              mode=ops.TC_MODE_STORE, row_tile=16, k_split=1)
    ops.check_status(DEV)
    assert torch.equal(one[0], big[100 + 9])
    # from 2048 rows on a CTA takes two weight tiles beside one tile of rows: the same bits again
    a_many = torch.cat([a, rnd(2000, K, dtype=torch.bfloat16, seed=9)])
    expert_many = torch.arange(2400) % E
    order_many = torch.argsort(expert_many, stable=True)
    offsets_many = torch.tensor([0, 600, 1200, 1800, 2400], dtype=torch.int32, device=DEV)
    many = ops.tc_grouped_gemm(a_many[order_many.to(DEV)].contiguous(), w, offsets_many, mode=ops.TC_MODE_STORE,
                               row_tile=128)
    ops.check_status(DEV)
    assert torch.equal(one[0], many[600 + 9])
    # the persistent kernel (items of up to 256 rows, MMA extents cut to the rows there are): the same bits
    walked = ops.tc_grouped_gemm(a_many[order_many.to(DEV)].contiguous(), w, offsets_many, mode=ops.TC_MODE_STORE,
                                 row_tile=0)
    ops.check_status(DEV)
    assert torch.equal(walked, many)
    # with K cut over several CTAs the parts are added in another order: equal to rounding, not to the bit
    cut = ops.tc_grouped_gemm(a[t:t + 1].contiguous(), w, torch.tensor([0, 0, 1, 1, 1], dtype=torch.int32, device=DEV),
                              mode=ops.TC_MODE_STORE, row_tile=16, k_split=3)
    ops.check_status(DEV)
    assert torch.allclose(cut[0], big[100 + 9], rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("M,N,K", [(1, 7168, 5120), (8, 5120, 8192), (3, 40, 64), (7, 77, 136), (9, 264, 520),
                                   (16, 1000, 2048), (1, 8, 8), (5, 202048, 256)])
def test_dense_rows(ops, M, N, K):
    """The weight-streaming product of up to 16 rows: store (with and without bias), add-in, and for even N the
    SwiGLU epilogue; sizes that are no multiples of a tile, a piece of K, or the warps' stride."""
    a = rnd(M, K, dtype=torch.bfloat16, seed=M + K)
    w = rnd(N, K, dtype=torch.bfloat16, scale=0.05, seed=N)
    ref = a.double().cpu() @ w.double().cpu().T
    atol = 1e-4 * float(ref.abs().max()) + 1e-6
    out = ops.dense_rows(a, w)
    assert out.dtype == torch.float32 and torch.allclose(out.double().cpu(), ref, rtol=1e-4, atol=atol)
    bias = rnd(N, seed=3)
    out_b = ops.dense_rows(a, w, bias=bias)
    assert torch.allclose(out_b.double().cpu(), ref + bias.double().cpu(), rtol=1e-4, atol=atol)
    base = rnd(M, N, seed=4)
    acc = base.clone()
    ops.dense_rows(a, w, out=acc, accumulate=True)
    assert torch.allclose(acc.double().cpu(), base.double().cpu() + ref, rtol=1e-4, atol=atol)
    if N % 2 == 0:
        act = ops.dense_rows(a, w, swiglu=True)
        g, u = ref[:, :N // 2], ref[:, N // 2:]
        want = g / (1 + torch.exp(-g)) * u
        assert act.dtype == torch.bfloat16 and act.shape == (M, N // 2)
        assert torch.allclose(act.double().cpu(), want, rtol=1e-2, atol=1e-2 * float(want.abs().max()) + 1e-6)


def test_dense_rows_do_not_depend_on_the_batch(ops):
    """A row gives the same bits alone, among eight and among sixteen rows, at any place in the batch."""
    N, K = 520, 1288
    a = rnd(16, K, dtype=torch.bfloat16, seed=5)
    w = rnd(N, K, dtype=torch.bfloat16, scale=0.05, seed=6)
    all16 = ops.dense_rows(a, w)
    first8 = ops.dense_rows(a[:8].contiguous(), w)
    one = ops.dense_rows(a[11:12].contiguous(), w)
    assert torch.equal(all16[:8], first8) and torch.equal(all16[11:12], one)
    act16 = ops.dense_rows(a, w, swiglu=True)
    act1 = ops.dense_rows(a[5:6].contiguous(), w, swiglu=True)
    assert torch.equal(act16[5:6], act1)


def test_dense_rows_refuses_what_it_does_not_take(ops):
    w = rnd(64, 128, dtype=torch.bfloat16, seed=1)
    with pytest.raises(Exception, match="16 rows"):
        ops.dense_rows(rnd(17, 128, dtype=torch.bfloat16, seed=2), w)
    with pytest.raises(Exception):
        ops.dense_rows(rnd(2, 132, dtype=torch.bfloat16, seed=2), rnd(64, 132, dtype=torch.bfloat16, seed=1))   # K % 8
    with pytest.raises(Exception, match="width"):
        ops.dense_rows(rnd(2, 64, dtype=torch.bfloat16, seed=2), w)


@pytest.mark.parametrize("k_split", [2, 4, 7])
def test_tc_grouped_gemm_k_split(ops, k_split):
    """Few rows: K is cut over several CTAs per tile; the last of them adds the parts and applies the epilogue."""
    T, E, I, K = 5, 4, 136, 328
    expert, order, offsets, a = grouped_case(T, E, K, seed=31)
    w_gu = rnd(E, 2 * I, K, dtype=torch.bfloat16, scale=0.1, seed=32)
    scale = torch.rand(T, generator=torch.Generator().manual_seed(33)) * 0.5 + 0.25
    a_sorted = a[order].contiguous().to(DEV)
    sorted_rows = order.to(torch.int32).to(DEV)
    act = ops.tc_grouped_gemm(a_sorted, w_gu, offsets, mode=ops.TC_MODE_SWIGLU, row_scale=scale.to(DEV),
                              scale_rows=sorted_rows, k_split=k_split)
    ops.check_status(DEV)
    ref = []
    for t in order.tolist():
        gu = (a[t].double() @ w_gu[int(expert[t])].double().cpu().T) * float(scale[t])
        ref.append(gu[:I] / (1 + torch.exp(-gu[:I])) * gu[I:])
    ref = torch.stack(ref)
    assert torch.allclose(act.double().cpu(), ref, rtol=1e-2, atol=1e-2 * float(ref.abs().max()))
    w_d = rnd(E, 200, K, dtype=torch.bfloat16, scale=0.1, seed=34)
    base = rnd(T, 200, seed=35)
    acc = base.clone()
    ops.tc_grouped_gemm(a_sorted, w_d, offsets, mode=ops.TC_MODE_STORE, out=acc, out_rows=sorted_rows, accumulate=True,
                        k_split=k_split)
    ops.check_status(DEV)
    ref_d = torch.stack([a[t].double() @ w_d[int(expert[t])].double().cpu().T for t in range(T)])
    assert torch.allclose(acc.double().cpu(), base.double().cpu() + ref_d, rtol=1e-4, atol=1e-3)


# ---------------------------------------------------------------------------------------
# tensor-core attention kernels (bfloat16): single rows split over their keys, and tiles of rows
# ---------------------------------------------------------------------------------------
MASKS = {"full": (0, lambda span: (lambda p: 0)), "chunk": (1, lambda span: (lambda p: p // span * span)),
         "window": (2, lambda span: (lambda p: max(0, p - span + 1)))}


@pytest.mark.parametrize("nq,nkv,d,ps", [(4, 2, 16, 4), (6, 3, 48, 16), (5, 1, 128, 64), (40, 8, 128, 64), (34, 2, 64, 32),
                                         (3, 3, 112, 16)])
@pytest.mark.parametrize("mask", [("full", 0), ("chunk", 300), ("chunk", 256), ("window", 100), ("window", 700)])
def test_attention_decode_rows(ops, nq, nkv, d, ps, mask):
    lens = [1000, 37, 1, 513, 256, 257]
    kv, table, ks, vs = paged_setup(lens, nkv, d, ps, torch.bfloat16, seed=d + ps + nq)
    rows = [(0, 999), (1, 36), (2, 0), (3, 512), (4, 255), (5, 256), (0, 511), (0, 600)]
    positions = torch.tensor([p for _, p in rows], dtype=torch.int32, device=DEV)
    row_req = torch.tensor([b for b, _ in rows], dtype=torch.int32, device=DEV)
    q = rnd(len(rows), nq, d, dtype=torch.bfloat16, seed=12)
    kind, span = mask
    code, lo_factory = MASKS[kind]
    scale = 1.0 / math.sqrt(d)
    ref = attention_ref(q.cpu(), ks, vs, positions.cpu(), row_req.cpu(), lo_factory(span), scale, nq, nkv)
    out = torch.zeros(len(rows), nq * d, dtype=torch.bfloat16, device=DEV)
    ops.attention_decode(q, kv, table, row_req, positions, out, rows=None, num_rows=len(rows), nq=nq, nkv=nkv, d=d,
                         page_size=ps, mask_kind=code, mask_span=max(span, 1), scale=scale, max_context=1000)
    assert torch.allclose(out.double().cpu(), ref, rtol=2e-2, atol=2e-2)
    # a subset of the rows, named by index; the others stay untouched
    some = torch.tensor([6, 1, 3], dtype=torch.int32, device=DEV)
    out2 = torch.full_like(out, 7.0)
    ops.attention_decode(q, kv, table, row_req, positions, out2, rows=some, num_rows=3, nq=nq, nkv=nkv, d=d,
                         page_size=ps, mask_kind=code, mask_span=max(span, 1), scale=scale, max_context=1000)
    assert torch.equal(out2[some.long()], out[some.long()])
    rest = [i for i in range(len(rows)) if i not in (6, 1, 3)]
    assert bool((out2[rest] == 7.0).all())


def test_attention_decode_many_splits_and_batch_invariance(ops):
    """A row over 70000 keys (274 splits: the merge shares it among more warps) beside short rows; a short
    row's output is the same bits whether the long row is in the launch or not."""
    nq, nkv, d, ps = 4, 1, 64, 64
    lens = [70000, 600, 65536]
    kv, table, ks, vs = paged_setup(lens, nkv, d, ps, torch.bfloat16, seed=77)
    rows = [(0, 69999), (1, 599), (2, 65535), (2, 65279), (1, 0)]        # 274, 3, 256, 255 and 1 splits
    positions = torch.tensor([p for _, p in rows], dtype=torch.int32, device=DEV)
    row_req = torch.tensor([b for b, _ in rows], dtype=torch.int32, device=DEV)
    q = (rnd(len(rows), nq, d, seed=78) * 3.0).to(torch.bfloat16)      # peaked: a few far keys carry the output
    scale = 1.0 / math.sqrt(d)
    ref = attention_ref(q.cpu(), ks, vs, positions.cpu(), row_req.cpu(), lambda p: 0, scale, nq, nkv)
    assert float(ref.abs().max()) > 0.5
    out = torch.zeros(len(rows), nq * d, dtype=torch.bfloat16, device=DEV)
    ops.attention_decode(q, kv, table, row_req, positions, out, rows=None, num_rows=len(rows), nq=nq, nkv=nkv, d=d,
                         page_size=ps, mask_kind=0, mask_span=1, scale=scale, max_context=70000)
    assert torch.allclose(out.double().cpu(), ref, rtol=2e-2, atol=2e-2)
    short = torch.tensor([1, 4], dtype=torch.int32, device=DEV)
    alone = torch.zeros_like(out)
    ops.attention_decode(q, kv, table, row_req, positions, alone, rows=short, num_rows=2, nq=nq, nkv=nkv, d=d,
                         page_size=ps, mask_kind=0, mask_span=1, scale=scale, max_context=600)
    assert torch.equal(alone[short.long()], out[short.long()])
    # told how many keys the rows have together, the launch holds 793 CTAs a kv head instead of 5 x 274: the same bits
    tight = torch.zeros_like(out)
    ops.attention_decode(q, kv, table, row_req, positions, tight, rows=None, num_rows=len(rows), nq=nq, nkv=nkv, d=d,
                         page_size=ps, mask_kind=0, mask_span=1, scale=scale, max_context=70000,
                         max_keys=int((positions.long() + 1).sum()))
    assert torch.equal(tight, out)
    near = torch.tensor([3], dtype=torch.int32, device=DEV)              # 255 splits, launched with narrow blocks
    alone3 = torch.zeros_like(out)
    ops.attention_decode(q, kv, table, row_req, positions, alone3, rows=near, num_rows=1, nq=nq, nkv=nkv, d=d,
                         page_size=ps, mask_kind=0, mask_span=1, scale=scale, max_context=65280)
    assert torch.equal(alone3[3], out[3])


@pytest.mark.parametrize("nq,nkv,d,ps", [(4, 2, 16, 4), (6, 3, 48, 16), (5, 1, 128, 64), (8, 2, 128, 16), (3, 3, 80, 32)])
@pytest.mark.parametrize("mask", [("full", 0), ("chunk", 100), ("chunk", 64), ("window", 50), ("window", 200)])
def test_attention_prefill_tiles(ops, nq, nkv, d, ps, mask):
    """Portions of three requests in one launch: one from an empty cache, one continuing at an odd
    position across a chunk edge, one short."""
    lens = [333, 150, 9]
    kv, table, ks, vs = paged_setup(lens, nkv, d, ps, torch.bfloat16, seed=d + ps)
    portions = [(0, 0, 333), (1, 77, 73), (2, 4, 5)]                     # request, first position, rows
    rows, tiles = [], []
    for b, p0, n in portions:
        for t0 in range(0, n, 64):
            tiles.append([len(rows) + t0, min(64, n - t0), p0 + t0, b])
        rows.extend((b, p0 + i) for i in range(n))
    positions = torch.tensor([p for _, p in rows], dtype=torch.int32)
    row_req = torch.tensor([b for b, _ in rows], dtype=torch.int32)
    q = rnd(len(rows), nq, d, dtype=torch.bfloat16, seed=13)
    kind, span = mask
    code, lo_factory = MASKS[kind]
    scale = 1.0 / math.sqrt(d)
    ref = attention_ref(q.cpu(), ks, vs, positions, row_req, lo_factory(span), scale, nq, nkv)
    out = torch.zeros(len(rows), nq * d, dtype=torch.bfloat16, device=DEV)
    ops.attention_prefill(q, kv, table, torch.tensor(tiles, dtype=torch.int32, device=DEV), out, nq=nq, nkv=nkv, d=d,
                          page_size=ps, mask_kind=code, mask_span=max(span, 1), scale=scale)
    assert torch.allclose(out.double().cpu(), ref, rtol=2e-2, atol=2e-2)
    # the generic kernel agrees too (it is what the float32 path and odd head sizes use)
    gen = ops.paged_attention_generic(q, kv, table, row_req.to(DEV), positions.to(DEV), nq=nq, nkv=nkv, d=d,
                                      page_size=ps, mask_kind=code, mask_span=max(span, 1), scale=scale)
    assert torch.allclose(out.float(), gen.float(), rtol=2e-2, atol=2e-2)


def test_fast_attention_finds_one_far_key_and_respects_edges(ops):
    nq, nkv, d, ps, n = 4, 2, 32, 16, 700
    scale = 1 / math.sqrt(d)
    for far in (0, 1, 15, 16, 63, 64, 255, 256, 257, 511, 512, 698, 699):
        kv, table, ks, vs = paged_setup([n], nkv, d, ps, torch.bfloat16, seed=far)
        q = rnd(64, nq, d, dtype=torch.bfloat16, seed=far + 1)          # rows at positions 636 .. 699
        page, off = int(table[0, far // ps]), far % ps
        for h in range(nkv):
            kv[page, 0, h, off] = (q[63, h * 2].float() * 8.0).to(torch.bfloat16)
        target = [kv[page, 1, h, off].float() for h in range(nkv)]
        positions = torch.arange(n - 64, n, dtype=torch.int32, device=DEV)
        row_req = torch.zeros(64, dtype=torch.int32, device=DEV)
        out_d = torch.zeros(64, nq * d, dtype=torch.bfloat16, device=DEV)
        ops.attention_decode(q, kv, table, row_req, positions, out_d, rows=torch.tensor([63], dtype=torch.int32, device=DEV),
                             num_rows=1, nq=nq, nkv=nkv, d=d, page_size=ps, mask_kind=0, mask_span=1, scale=scale,
                             max_context=n)
        out_p = torch.zeros(64, nq * d, dtype=torch.bfloat16, device=DEV)
        ops.attention_prefill(q, kv, table, torch.tensor([[0, 64, n - 64, 0]], dtype=torch.int32, device=DEV), out_p,
                              nq=nq, nkv=nkv, d=d, page_size=ps, mask_kind=0, mask_span=1, scale=scale)
        for out in (out_d, out_p):
            got = out[63].view(nq, d).float()
            for h in range(nkv):
                assert torch.allclose(got[h * 2], target[h], atol=6e-2), (far, h)
    # edges: the key just outside must not be seen, the one just inside must
    for kind, span, pos, outside, inside in (("chunk", 24, 50, 47, 48), ("chunk", 64, 64, 63, 64), ("window", 9, 60, 51, 52),
                                             ("chunk", 256, 256, 255, 256), ("window", 256, 600, 344, 345)):
        code = {"chunk": 1, "window": 2}[kind]
        for which, key in (("outside", outside), ("inside", inside)):
            kv, table, ks, vs = paged_setup([n], 1, 16, 8, torch.bfloat16, seed=pos)
            q = rnd(1, 2, 16, dtype=torch.bfloat16, seed=3)
            page, off = int(table[0, key // 8]), key % 8
            kv[page, 0, 0, off] = (q[0, 0].float() * 10.0).to(torch.bfloat16)
            kv[page, 1, 0, off] = 50.0
            positions = torch.tensor([pos], dtype=torch.int32, device=DEV)
            zero = torch.zeros(1, dtype=torch.int32, device=DEV)
            out_d = torch.zeros(1, 32, dtype=torch.bfloat16, device=DEV)
            ops.attention_decode(q, kv, table, zero, positions, out_d, rows=None, num_rows=1, nq=2, nkv=1, d=16,
                                 page_size=8, mask_kind=code, mask_span=span, scale=0.25, max_context=pos + 1)
            out_p = torch.zeros(1, 32, dtype=torch.bfloat16, device=DEV)
            ops.attention_prefill(q, kv, table, torch.tensor([[0, 1, pos, 0]], dtype=torch.int32, device=DEV), out_p,
                                  nq=2, nkv=1, d=16, page_size=8, mask_kind=code, mask_span=span, scale=0.25)
            for out in (out_d.float(), out_p.float()):
                if which == "outside":
                    assert float(out[0, :16].abs().max()) < 10.0, (kind, pos, key)
                else:
                    assert float(out[0, :16].min()) > 40.0, (kind, pos, key)


def test_router_rows_do_not_depend_on_the_batch(ops):
    """A token's router logits are the same bits alone, in a small batch (a block per token and expert), in
    a middle one (two tokens share a block) and in a large one (eight do), for widths that are and are not
    multiples of four."""
    for H in (1000, 1001):
        h, wr = rnd(1500, H, seed=21), rnd(16, H, scale=0.05, seed=22)
        e_big, w_big, l_big = ops.router_top1(h, wr, want_logits=True)
        e_mid, w_mid, l_mid = ops.router_top1(h[3:603].contiguous(), wr, want_logits=True)
        e_small, w_small, l_small = ops.router_top1(h[:7].contiguous(), wr, want_logits=True)
        e_one, w_one, l_one = ops.router_top1(h[301:302].contiguous(), wr, want_logits=True)
        assert torch.equal(l_big[:7], l_small) and torch.equal(l_big[301:302], l_one)
        assert torch.equal(l_big[3:603], l_mid) and torch.equal(e_big[3:603], e_mid) and torch.equal(w_big[3:603], w_mid)
        assert torch.equal(e_big[:7], e_small) and torch.equal(w_big[301:302], w_one)


@pytest.mark.parametrize("nq,nkv,d,ps", [(2, 1, 64, 64), (5, 1, 128, 64), (8, 2, 128, 128), (6, 3, 64, 256)])
@pytest.mark.parametrize("mask", [("full", 0), ("chunk", 100), ("chunk", 128), ("window", 50), ("window", 300)])
def test_attention_prefill_tcgen05(ops, nq, nkv, d, ps, mask):
    """The tcgen05 / TMEM kernel: tiles of 128 rows; portions that start at odd positions, cross chunk
    edges and end inside a page."""
    lens = [700, 333, 150, 9]
    kv, table, ks, vs = paged_setup(lens, nkv, d, ps, torch.bfloat16, seed=d + ps + nq)
    portions = [(0, 0, 333), (1, 77, 256), (2, 140, 10), (3, 4, 5), (0, 333, 367)]      # request, first position, rows
    rows, tiles = [], []
    for b, p0, n in portions:
        for t0 in range(0, n, 128):
            tiles.append([len(rows) + t0, min(128, n - t0), p0 + t0, b])
        rows.extend((b, p0 + i) for i in range(n))
    positions = torch.tensor([p for _, p in rows], dtype=torch.int32)
    row_req = torch.tensor([b for b, _ in rows], dtype=torch.int32)
    q = rnd(len(rows), nq, d, dtype=torch.bfloat16, seed=14)
    kind, span = mask
    code, lo_factory = MASKS[kind]
    scale = 1.0 / math.sqrt(d)
    out = torch.zeros(len(rows), nq * d, dtype=torch.bfloat16, device=DEV)
    ops.attention_prefill_tc(q, kv, table, torch.tensor(tiles, dtype=torch.int32, device=DEV), out, nq=nq, nkv=nkv, d=d,
                             page_size=ps, mask_kind=code, mask_span=max(span, 1), scale=scale)
    ops.check_status(DEV)
    ref = attention_ref(q.cpu(), ks, vs, positions, row_req, lo_factory(span), scale, nq, nkv)
    assert torch.allclose(out.double().cpu(), ref, rtol=2e-2, atol=2e-2)


def test_attention_prefill_tcgen05_far_key_and_edges(ops):
    nq, nkv, d, ps, n = 2, 1, 64, 64, 700
    scale = 1 / math.sqrt(d)
    for far in (0, 1, 63, 64, 127, 128, 383, 384, 571, 572, 698, 699):
        kv, table, ks, vs = paged_setup([n], nkv, d, ps, torch.bfloat16, seed=far)
        q = rnd(128, nq, d, dtype=torch.bfloat16, seed=far + 1)           # rows at positions 572 .. 699
        page, off = int(table[0, far // ps]), far % ps
        kv[page, 0, 0, off] = (q[127, 0].float() * 6.0).to(torch.bfloat16)
        target = kv[page, 1, 0, off].float()
        out = torch.zeros(128, nq * d, dtype=torch.bfloat16, device=DEV)
        ops.attention_prefill_tc(q, kv, table, torch.tensor([[0, 128, n - 128, 0]], dtype=torch.int32, device=DEV), out,
                                 nq=nq, nkv=nkv, d=d, page_size=ps, mask_kind=0, mask_span=1, scale=scale)
        ops.check_status(DEV)
        assert torch.allclose(out[127, :d].float(), target, atol=6e-2), far
    for kind, span, pos, outside, inside in (("chunk", 24, 50, 47, 48), ("chunk", 64, 64, 63, 64), ("window", 9, 60, 51, 52),
                                             ("chunk", 256, 256, 255, 256), ("window", 256, 600, 344, 345)):
        code = {"chunk": 1, "window": 2}[kind]
        for which, key in (("outside", outside), ("inside", inside)):
            kv, table, ks, vs = paged_setup([n], 1, 64, 64, torch.bfloat16, seed=pos)
            q = rnd(1, 2, 64, dtype=torch.bfloat16, seed=3)
            page, off = int(table[0, key // 64]), key % 64
            kv[page, 0, 0, off] = (q[0, 0].float() * 4.0).to(torch.bfloat16)
            kv[page, 1, 0, off] = 50.0
            out = torch.zeros(1, 128, dtype=torch.bfloat16, device=DEV)
            ops.attention_prefill_tc(q, kv, table, torch.tensor([[0, 1, pos, 0]], dtype=torch.int32, device=DEV), out,
                                     nq=2, nkv=1, d=64, page_size=64, mask_kind=code, mask_span=span, scale=0.125)
            ops.check_status(DEV)
            if which == "outside":
                assert float(out[0, :64].float().abs().max()) < 10.0, (kind, pos, key)
            else:
                assert float(out[0, :64].float().min()) > 40.0, (kind, pos, key)


# ---------------------------------------------------------------------------------------
# what another architecture's parts would need of the kernels: a bias, a weightless norm, a router that
# weights its experts' outputs; and the path a kernel takes when one of its waits runs out
# ---------------------------------------------------------------------------------------
def test_weightless_norm_and_bias(ops):
    x = rnd(21, 72, seed=1)
    out, _ = ops.add_rmsnorm(x.clone(), None, None, 1e-5, torch.float32)
    ref = x.double() * torch.rsqrt((x.double() ** 2).mean(-1, keepdim=True) + 1e-5)
    assert torch.allclose(out.double(), ref, rtol=2e-6, atol=1e-6)
    y, b = rnd(13, 301, seed=2), rnd(301, seed=3)
    assert torch.equal(ops.add_bias(y.clone(), b), y + b)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gemm_nt_bias_and_row_scale(ops, dtype):
    M, N, K = 45, 70, 52
    a, w, bias, s = rnd(M, K, dtype=dtype, seed=1), rnd(N, K, dtype=dtype, seed=2), rnd(N, seed=3), rnd(M, seed=4)
    out = ops.gemm_nt(a, w, bias=bias, row_scale=s)
    ref = (a.double() @ w.double().T) * s.double()[:, None] + bias.double()
    assert torch.allclose(out.double(), ref, rtol=1e-5, atol=1e-4)
    perm = torch.randperm(M, generator=torch.Generator().manual_seed(5)).to(torch.int32).to(DEV)
    out2 = ops.gemm_nt(a, w, row_scale=s, scale_rows=perm)
    assert torch.allclose(out2.double(), (a.double() @ w.double().T) * s.double()[perm.long()][:, None], rtol=1e-5, atol=1e-4)


@pytest.mark.parametrize("T,E,N,K,row_tile", [(8, 4, 256, 128, 16), (300, 5, 136, 264, 64), (2100, 3, 520, 128, 128),
                                              (700, 3, 520, 128, 0), (3, 2, 384, 1024, 16)])
def test_tc_grouped_gemm_store_weights_its_output_rows(ops, T, E, N, K, row_tile):
    """MODE_STORE with a per-row factor: what a router that weights its experts' outputs needs."""
    expert, order, offsets, a = grouped_case(T, E, K, seed=T + N)
    w = rnd(E, N, K, dtype=torch.bfloat16, scale=0.1, seed=3)
    scale = torch.rand(T, generator=torch.Generator().manual_seed(6)) + 0.5
    sorted_rows = order.to(torch.int32).to(DEV)
    ref = torch.stack([a[t].double() @ w[int(expert[t])].double().cpu().T * float(scale[t]) for t in range(T)])
    base = rnd(T, N, seed=4)
    acc = base.clone()
    ops.tc_grouped_gemm(a[order].contiguous().to(DEV), w, offsets, mode=ops.TC_MODE_STORE, out=acc, out_rows=sorted_rows,
                        accumulate=True, row_tile=row_tile, row_scale=scale.to(DEV), scale_rows=sorted_rows)
    ops.check_status(DEV)
    assert torch.allclose(acc.double().cpu(), base.double().cpu() + ref, rtol=1e-4, atol=1e-3)


def test_a_wait_that_runs_out_is_reported_and_the_kernel_returns(ops):
    """The producer of one launch is told to stop after the first K block and every wait to give up after a few
    thousand polls: the tensor-core warp's wait for the second block runs out, the kernel records the code and
    returns (no fault, no hang), check_status raises it, and the next launch is right again."""
    from sharpinference_b200.kernels.library import KernelError
    expert, order, offsets, a = grouped_case(8, 2, 256, seed=11)
    w = rnd(2, 128, 256, dtype=torch.bfloat16, scale=0.1, seed=3)
    a_sorted = a[order].contiguous().to(DEV)
    ops.check_status(DEV)
    ops.tc_set_wait_test(1 << 12, 1)
    ops.tc_grouped_gemm(a_sorted, w, offsets, mode=ops.TC_MODE_STORE, row_tile=16, k_split=1)
    torch.cuda.synchronize()
    with pytest.raises(KernelError, match="gave up"):
        ops.check_status(DEV)
    ops.check_status(DEV)                                            # the word is back at zero
    out = ops.tc_grouped_gemm(a_sorted, w, offsets, mode=ops.TC_MODE_STORE, row_tile=16, k_split=1)
    ops.check_status(DEV)
    ref = torch.stack([a[t].double() @ w[int(expert[t])].double().cpu().T for t in order.tolist()])
    assert torch.allclose(out.double().cpu(), ref, rtol=1e-4, atol=1e-3)

