"""Each kernel of the pack alone against a plain fp32 torch reference of the
same op, at sizes other than the engine's tiny configurations: widths and
vocabularies that are no power of two, head sizes in steps of 16, odd
numbers of heads and groups, several page sizes, windows."""
import math

import pytest
import torch

import plain_impl

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


@pytest.fixture(scope="module")
def ops():
    from pih_b200.kernels import get_ops
    return get_ops(torch.device(DEV))


def _tol(dtype):
    # fp32: accumulation-order noise; bf16: one rounding of the output (2^-9 relative) plus the same noise
    return dict(rtol=2e-5, atol=2e-6) if dtype == torch.float32 else dict(rtol=8e-3, atol=1e-3)


def _rand(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype).to(DEV)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("vocab,hidden", [(100, 24), (333, 200), (50, 1027)])
def test_embedding(ops, dtype, vocab, hidden):
    table = _rand((vocab, hidden), dtype, 0)
    ids = torch.randint(0, vocab, (37,), dtype=torch.int32, device=DEV)
    out = ops.embedding(table, ids)
    assert torch.equal(out, table[ids.long()])
    ops.check_errors()


def test_embedding_reports_a_bad_token(ops):
    from pih_b200.kernels.ops import KernelError
    table = _rand((10, 8), torch.float32, 0)
    ids = torch.tensor([1, 10, 3], dtype=torch.int32, device=DEV)
    ops.embedding(table, ids)
    with pytest.raises(KernelError, match="vocabulary"):
        ops.check_errors()
    ops.check_errors()          # the word was cleared


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,width,eps", [(5, 24, 1e-6), (33, 200, 1e-5), (7, 1027, 1e-6), (3, 5000, 1e-3)])
def test_rmsnorm_and_fused_add(ops, dtype, rows, width, eps):
    x = _rand((rows, width), dtype, 1, 2.0)
    d = _rand((rows, width), dtype, 2)
    w = (1 + 0.1 * torch.randn(width)).to(dtype).to(DEV)
    # plain norm
    ref = plain_impl.rms_norm(x.cpu().double(), w.cpu().double(), eps)
    out = ops.rmsnorm(x.clone(), w, eps)
    torch.testing.assert_close(out.cpu().double(), ref, **_tol(dtype))
    # fused add: h is updated in place to round(h + d), and that value is normed
    h = x.clone()
    out = ops.rmsnorm(h, w, eps, delta=d)
    s = (x.float() + d.float()).to(dtype)
    assert torch.equal(h, s)
    ref = plain_impl.rms_norm(s.cpu().double(), w.cpu().double(), eps)
    torch.testing.assert_close(out.cpu().double(), ref, **_tol(dtype))
    # gathered rows, h untouched
    h = x.clone()
    pick = torch.tensor([rows - 1, 0, rows // 2], dtype=torch.int32, device=DEV)
    out = ops.rmsnorm(h, w, eps, delta=d, rows=pick)
    assert torch.equal(h, x)
    torch.testing.assert_close(out.cpu().double(), ref[pick.cpu().long()], **_tol(dtype))


def test_rmsnorm_keeps_a_32bit_weight_with_a_bf16_stream(ops):
    x = _rand((4, 96), torch.bfloat16, 1)
    w = (1 + 0.1 * torch.randn(96)).to(DEV)          # float32
    out = ops.rmsnorm(x.clone(), w, 1e-6)
    ref = plain_impl.rms_norm(x.cpu().double(), w.cpu().double(), 1e-6)
    torch.testing.assert_close(out.cpu().double(), ref, **_tol(torch.bfloat16))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,N,K", [(1, 7, 5), (37, 130, 96), (64, 64, 64), (130, 257, 1027), (3, 1000, 33),
                                   (5, 3001, 96), (16, 151, 1024), (9, 2500, 2080)])   # few rows: the fused kernel, fp32 out too
def test_linear(ops, dtype, M, N, K):
    x = _rand((M, K), dtype, 3)
    w = _rand((N, K), dtype, 4, 0.1)
    ref = x.cpu().double() @ w.cpu().double().T
    # a sum of K products in 32-bit: the error grows with K; K <= 1027 here, terms are O(0.1)
    acc = dict(rtol=1e-4, atol=2e-5)
    for fn in (ops.linear, ops.linear_plain):
        out = fn(x, w)
        assert out.dtype == dtype
        torch.testing.assert_close(out.cpu().double(), ref, **(acc if dtype == torch.float32 else _tol(dtype)))
        out32 = fn(x, w, out_dtype=torch.float32)
        assert out32.dtype == torch.float32
        torch.testing.assert_close(out32.cpu().double(), ref, **acc)


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("tile_n", [0, 64, 128, 256])
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (1, 8, 8), (37, 130, 96), (300, 257, 1032), (2048, 1024, 3072),
                                   (129, 1000, 72), (64, 152, 1024), (4000, 2300, 520)])
def test_linear_tcgen05(ops, out_dtype, tile_n, M, N, K):
    """The tcgen05 / TMA product against a float64 reference: tiles that overhang M, N and K, every tile
    width, and enough tiles that a CTA walks over several (both accumulators, ring wrap-around)."""
    x = _rand((M, K), torch.bfloat16, 3)
    w = _rand((N, K), torch.bfloat16, 4, 0.1)
    out = ops.linear_tcgen05(x, w, out_dtype, tile_n=tile_n)
    ops.check_errors()
    assert out is not None and out.dtype == out_dtype and out.shape == (M, N)
    ref = x.cpu().double() @ w.cpu().double().T
    tol = dict(rtol=1e-4, atol=1e-4) if out_dtype == torch.float32 else _tol(torch.bfloat16)
    if out_dtype == torch.bfloat16:
        tol = dict(rtol=8e-3, atol=1e-3 * max(1.0, float(ref.abs().max()) / 4))
    torch.testing.assert_close(out.cpu().double(), ref, **tol)


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("tile_n", [0, 128, 256])
@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (1, 8, 8), (37, 130, 96), (300, 257, 1032), (2048, 1024, 3072),
                                   (129, 1000, 72), (385, 152, 1024), (4000, 4300, 520)])
def test_linear_tcgen05_on_pairs_of_sms(ops, out_dtype, tile_n, M, N, K):
    """The product with two SMs on a 256-row tile (cta_group::2) against a float64 reference: tiles that overhang
    M, N and K — a pair whose second CTA has no rows or no columns at all —, both tile widths, and enough tiles
    that a pair walks over several (both accumulators, ring wrap-around)."""
    x = _rand((M, K), torch.bfloat16, 3)
    w = _rand((N, K), torch.bfloat16, 4, 0.1)
    out = ops.linear_tcgen05(x, w, out_dtype, tile_n=tile_n, pairs=True)
    ops.check_errors()
    assert out is not None and out.dtype == out_dtype and out.shape == (M, N)
    ref = x.cpu().double() @ w.cpu().double().T
    tol = dict(rtol=1e-4, atol=1e-4)
    if out_dtype == torch.bfloat16:
        tol = dict(rtol=8e-3, atol=1e-3 * max(1.0, float(ref.abs().max()) / 4))
    torch.testing.assert_close(out.cpu().double(), ref, **tol)


def test_linear_tcgen05_takes_strided_rows_and_refuses_what_tma_cannot_describe(ops):
    x = _rand((40, 256), torch.bfloat16, 5)
    w = _rand((512, 128), torch.bfloat16, 6, 0.1)
    out = ops.linear_tcgen05(x[:, :128], w[:96])               # row stride 256, first 96 weight rows
    ref = x[:, :128].cpu().double() @ w[:96].cpu().double().T
    torch.testing.assert_close(out.cpu().double(), ref, **_tol(torch.bfloat16))
    assert ops.linear_tcgen05(_rand((4, 20), torch.bfloat16, 7), _rand((8, 20), torch.bfloat16, 8)) is None


@pytest.mark.parametrize("M", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("N,K", [(8, 32), (24, 64), (4096, 1024), (1024, 3072), (1000, 96), (6144, 1024),
                                 (1000, 2080), (40, 2048), (1184, 4096)])
def test_linear_skinny(ops, M, N, K):
    """The few-rows product alone: every row count up to 16, widths that are no multiple of the tile; few
    columns with a long k go to pairs of blocks that split k (an odd number of k blocks among them)."""
    x = _rand((M, K), torch.bfloat16, 3)
    w = _rand((N, K), torch.bfloat16, 4, 0.1)
    out = ops.linear_skinny(x, w)
    assert out is not None and out.shape == (M, N)
    ref = x.cpu().double() @ w.cpu().double().T
    torch.testing.assert_close(out.cpu().double(), ref, rtol=8e-3, atol=1e-3 * max(1.0, float(ref.abs().max()) / 4))
    # a row gives the same bits alone as among others (up to 8 rows and 9 to 16 rows are cut differently: a row
    # among 9 to 16 is compared with itself among 9)
    few = x[M - 1:] if M <= 8 else x[M - 9:]
    assert torch.equal(ops.linear_skinny(few.contiguous(), w)[-1], out[M - 1])


@pytest.mark.parametrize("M", [1, 5, 8, 11, 16, 17])
@pytest.mark.parametrize("N,K", [(151936, 1024), (100003, 2048), (80000, 96)])
def test_the_head_of_a_decode_step(ops, M, N, K):
    """The product with a vocabulary of weight rows and a 32-bit result against float64: up to 8 token rows by the
    kernel that streams the weights straight into MMA operands (a last granule that is not full), more rows by the
    library (faster there); among up to 8 rows a row gives the same bits as alone."""
    x = _rand((M, K), torch.bfloat16, 3)
    w = _rand((N, K), torch.bfloat16, 4, 0.1)
    out = ops.linear(x, w, out_dtype=torch.float32)
    ops.check_errors()
    assert out.dtype == torch.float32 and out.shape == (M, N)
    ref = x.cpu().double() @ w.cpu().double().T
    torch.testing.assert_close(out.cpu().double(), ref, rtol=1e-4, atol=2e-5 * max(1.0, float(ref.abs().max())))
    if M <= 8:
        alone = ops.linear(x[M - 1:].contiguous(), w, out_dtype=torch.float32)
        assert torch.equal(alone[0], out[M - 1])


@pytest.mark.parametrize("M", [1, 8, 13])
@pytest.mark.parametrize("N,K", [(1024, 2048), (1024, 3072), (151, 96), (1000, 1024)])
def test_linear_skinny_adds_the_residual_in_its_epilogue(ops, M, N, K):
    """``round(round(x . w^T) + residual)``: the bits of the separate product followed by the separate add."""
    x = _rand((M, K), torch.bfloat16, 3)
    w = _rand((N, K), torch.bfloat16, 4, 0.1)
    h = _rand((M, N), torch.bfloat16, 5, 2.0)
    fused = ops.linear_add(x, w, h)
    assert fused is not None and fused.shape == (M, N)
    product = ops.linear_skinny(x, w)
    want = (product.float() + h.float()).to(torch.bfloat16)
    assert torch.equal(fused, want)
    ref = plain_impl.residual_add(h.cpu(), plain_impl.linear(x.cpu(), w.cpu(), "bf16"), "bf16")
    torch.testing.assert_close(fused.cpu().double(), ref, rtol=1.6e-2, atol=2e-2)
    ops.check_errors()


@pytest.mark.parametrize("M", [1, 8, 13])
@pytest.mark.parametrize("norm_dtype", [torch.bfloat16, torch.float32])
def test_linear_skinny_fused_add_norm_and_swiglu(ops, M, norm_dtype):
    """h' = h + delta, norm, product, SiLU-mul in one kernel, against the separate roundings of the plain parts."""
    K, inter = 1024, 3072
    h = _rand((M, K), torch.bfloat16, 5, 2.0)
    d = _rand((M, K), torch.bfloat16, 6)
    nw = (1 + 0.1 * torch.randn(K, generator=torch.Generator().manual_seed(9))).to(norm_dtype).to(DEV)
    gate = _rand((inter, K), torch.bfloat16, 7, 0.05)
    up = _rand((inter, K), torch.bfloat16, 8, 0.05)
    w = torch.stack([gate.reshape(-1, 8, K), up.reshape(-1, 8, K)], dim=1).reshape(2 * inter, K).contiguous()
    eps = 1e-6
    # plain: every op rounds once
    hs = plain_impl.residual_add(h.cpu(), d.cpu(), "bf16")
    xn = plain_impl.rms_norm(hs, nw.cpu().double(), eps, "bf16")
    g_ref, u_ref = plain_impl.linear(xn, gate.cpu(), "bf16"), plain_impl.linear(xn, up.cpu(), "bf16")
    act_ref = plain_impl.silu_mul(g_ref, u_ref, "bf16")
    # fused add + norm + product
    h2, qkv = ops.linear_skinny(h, w, delta=d, norm_weight=nw, eps=eps)
    assert torch.equal(h2.cpu().double(), hs) and torch.equal(h, _rand((M, K), torch.bfloat16, 5, 2.0))   # h untouched
    gu_ref = torch.stack([g_ref.reshape(M, -1, 8), u_ref.reshape(M, -1, 8)], dim=2).reshape(M, 2 * inter)
    tol = dict(rtol=1.6e-2, atol=4e-3)          # two roundings upstream of the product may flip
    torch.testing.assert_close(qkv.cpu().double(), gu_ref, **tol)
    # ... and with SiLU-mul in the epilogue
    h3, act = ops.linear_skinny(h, w, delta=d, norm_weight=nw, eps=eps, swiglu=True)
    assert torch.equal(h3, h2) and act.shape == (M, inter)
    # Kernel and reference add the same products in another order, so g and u may each land on the other
    # side of a bf16 rounding boundary (one ulp = 2^-7 of the value's power of two), and so may the result.
    # What one such flip does to silu(g) * u is bounded element by element: near g = -5 the slope of silu is
    # four times silu / g, which a flat relative tolerance does not cover.
    ulp = lambda t: torch.exp2(torch.floor(torch.log2(t.abs().clamp_min(1e-30))) - 7)
    sig = torch.sigmoid(g_ref)
    silu, dsilu = g_ref * sig, sig * (1 + g_ref * (1 - sig))
    bound = ulp(g_ref) * (dsilu * u_ref).abs() + ulp(u_ref) * silu.abs() + ulp(act_ref) + 1e-6
    err = (act.cpu().double() - act_ref).abs()
    assert bool((err <= 1.05 * bound).all()), float((err / bound).max())
    # the unfused path of the same op agrees
    ops.skinny_max_rows = 0
    try:
        h4 = h.clone()
        h4b, act2 = ops.norm_linear(h4, d, nw, eps, w, swiglu_interleave=8)
    finally:
        ops.skinny_max_rows = 16
    assert torch.equal(h4b, h2)
    err2 = (act2.cpu().double() - act.cpu().double()).abs()
    assert bool((err2 <= 2.1 * bound).all()), float((err2 / bound).max())


def test_silu_mul_interleaved(ops):
    for dtype in DTYPES:
        gu = _rand((5, 2 * 48), dtype, 9, 2.0)
        blocks = gu.reshape(5, 6, 2, 8)
        ref = plain_impl.silu_mul(blocks[:, :, 0, :].reshape(5, 48).cpu(), blocks[:, :, 1, :].reshape(5, 48).cpu())
        torch.testing.assert_close(ops.silu_mul(gu, 8).cpu().double(), ref, **_tol(dtype))


def test_linear_fp32_rows_do_not_depend_on_the_batch(ops):
    """The 32-bit product gives a row the same bits alone and among others."""
    x = _rand((77, 300), torch.float32, 5)
    w = _rand((190, 300), torch.float32, 6)
    whole = ops.linear(x, w)
    for lo, hi in [(0, 1), (5, 7), (30, 77)]:
        assert torch.equal(ops.linear(x[lo:hi].contiguous(), w), whole[lo:hi])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,inter", [(3, 24), (17, 224), (5, 1031)])
def test_silu_mul(ops, dtype, rows, inter):
    gu = _rand((rows, 2 * inter), dtype, 7, 2.0)
    ref = plain_impl.silu_mul(gu[:, :inter].cpu(), gu[:, inter:].cpu())
    torch.testing.assert_close(ops.silu_mul(gu).cpu().double(), ref, **_tol(dtype))


def _rope_table(max_pos, rotary, theta):
    cos, sin = plain_impl.rope_angles(range(max_pos), rotary, theta)
    return torch.stack([cos, sin], dim=-1).float().to(DEV).contiguous()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,D,page", [(4, 2, 16, 16), (6, 1, 32, 8), (5, 5, 48, 4), (16, 8, 128, 16),
                                                  (3, 1, 80, 32), (8, 2, 256, 16)])
def test_qk_norm_rope_kv_write(ops, dtype, heads, kv_heads, D, page):
    T, num_pages, eps, theta = 19, 9, 1e-5, 50000.0
    width = (heads + 2 * kv_heads) * D
    qkv = _rand((T, width), dtype, 8)
    qw = (1 + 0.1 * torch.randn(D)).to(dtype).to(DEV)
    kw = (1 + 0.1 * torch.randn(D)).to(dtype).to(DEV)
    positions = torch.randint(0, 300, (T,), dtype=torch.int32, device=DEV)
    slots = torch.randperm(num_pages * page)[:T].to(torch.int32).to(DEV)
    cache = torch.zeros(num_pages, 2, kv_heads, page, D, dtype=dtype, device=DEV)
    table = _rope_table(300, D, theta)
    rounding = "none" if dtype == torch.float32 else "bf16"
    x = qkv.cpu()
    q = x[:, :heads * D].reshape(T, heads, D)
    k = x[:, heads * D:(heads + kv_heads) * D].reshape(T, kv_heads, D)
    v = x[:, (heads + kv_heads) * D:].reshape(T, kv_heads, D)
    cos, sin = plain_impl.rope_angles(positions.cpu().tolist(), D, theta)
    q_ref = plain_impl.rope_apply(plain_impl.rms_norm(q, qw.cpu(), eps, rounding), cos, sin, rounding)
    k_ref = plain_impl.rope_apply(plain_impl.rms_norm(k, kw.cpu(), eps, rounding), cos, sin, rounding)
    ops.qk_norm_rope_kv_write(qkv, heads=heads, kv_heads=kv_heads, head_dim=D, q_norm=qw, k_norm=kw, eps=eps,
                              rope_table=table, rotary_dim=D, positions=positions, slot_mapping=slots,
                              kv_cache=cache, write_kv=True)
    ops.check_errors()
    got_q = qkv[:, :heads * D].cpu().double().reshape(T, heads, D)
    got_k = cache[(slots // page).long(), 0, :, (slots % page).long(), :].cpu().double()
    got_v = cache[(slots // page).long(), 1, :, (slots % page).long(), :].cpu().double()
    for got, ref in ((got_q, q_ref), (got_k, k_ref)):
        if dtype == torch.float32:
            torch.testing.assert_close(got, ref, **_tol(dtype))
        else:
            # two roundings (after the norm, after the rotation): where the 32-bit kernel and the 64-bit
            # reference round the normed value to different neighbours, the rotated value moves by up to one
            # ulp of the normed value (|n| < 8: 2^-5).  That must be rare; everything else is within one rounding.
            err = (got - ref).abs()
            tight = err <= 1e-3 + 8e-3 * ref.abs()
            assert float(tight.double().mean()) > 0.998 and float(err.max()) < 0.04, (float(tight.double().mean()), float(err.max()))
    assert torch.equal(got_v, v.double())
    # nothing else in the cache was touched
    mask = torch.ones(num_pages * page, dtype=torch.bool)
    mask[slots.cpu().long()] = False
    flat = cache.permute(0, 3, 1, 2, 4).reshape(num_pages * page, -1).cpu()
    assert float(flat[mask].abs().max()) == 0.0


def _dense_reference(q, k, v, scale, window):
    return plain_impl.attention(q, k, v, scale, window)


def _paged_setup(dtype, lens, new, heads, kv_heads, D, page, seed, num_pages=None):
    """Requests with ``lens[r]`` tokens in the cache of which the last ``new[r]`` are this step's rows."""
    g = torch.Generator().manual_seed(seed)
    R = len(lens)
    pages_per = [-(-n // page) for n in lens]
    num_pages = num_pages or sum(pages_per) + 3
    perm = torch.randperm(num_pages, generator=g).tolist()
    width = max(pages_per)
    table = torch.full((R, width), -1, dtype=torch.int32)
    cache = torch.zeros(num_pages, 2, kv_heads, page, D, dtype=dtype)
    ks, vs, qs, req_of_row, positions = [], [], [], [], []
    for r in range(R):
        k = (torch.randn(lens[r], kv_heads, D, generator=g)).to(dtype)
        v = (torch.randn(lens[r], kv_heads, D, generator=g)).to(dtype)
        q = (torch.randn(new[r], heads, D, generator=g)).to(dtype)
        ks.append(k), vs.append(v), qs.append(q)
        for i in range(pages_per[r]):
            pg = perm.pop()
            table[r, i] = pg
            n = min(page, lens[r] - i * page)
            cache[pg, 0, :, :n, :] = k[i * page:i * page + n].transpose(0, 1)
            cache[pg, 1, :, :n, :] = v[i * page:i * page + n].transpose(0, 1)
        req_of_row += [r] * new[r]
        positions += list(range(lens[r] - new[r], lens[r]))
    return dict(cache=cache.to(DEV), table=table.to(DEV), ks=ks, vs=vs, qs=qs,
                q=torch.cat(qs).reshape(sum(new), heads * D).contiguous().to(DEV),
                req_of_row=torch.tensor(req_of_row, dtype=torch.int32, device=DEV),
                positions=torch.tensor(positions, dtype=torch.int32, device=DEV))


def _attention_reference(setup, lens, new, scale, window):
    outs = []
    for r in range(len(lens)):
        L, n = lens[r], new[r]
        heads, D = setup["qs"][r].shape[1:]
        qfull = torch.zeros(L, heads, D, dtype=torch.float64)
        qfull[L - n:] = setup["qs"][r].double()
        o = _dense_reference(qfull, setup["ks"][r].double(), setup["vs"][r].double(), scale, window)
        outs.append(o[L - n:].reshape(n, heads * D))
    return torch.cat(outs)


ATTN_CASES = [
    # heads, kv_heads, D, page, lens, new, window
    (4, 2, 16, 16, [5, 40, 17], [5, 1, 17], None),
    (6, 1, 32, 8, [33, 64, 1, 100], [2, 64, 1, 1], None),
    (6, 1, 32, 8, [33, 64, 90, 100], [2, 64, 7, 1], 24),
    (5, 5, 48, 4, [19, 7], [19, 3], 5),
    (16, 8, 128, 16, [300, 129, 2048], [44, 1, 1], None),
    (3, 1, 80, 32, [77, 31], [20, 31], 33),
    (8, 2, 256, 16, [130], [130], None),
    (14, 2, 64, 16, [257, 90], [1, 90], None),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", ATTN_CASES, ids=[f"h{c[0]}kv{c[1]}d{c[2]}p{c[3]}w{c[6]}" for c in ATTN_CASES])
def test_paged_attention_generic(ops, dtype, case):
    heads, kv_heads, D, page, lens, new, window = case
    s = _paged_setup(dtype, lens, new, heads, kv_heads, D, page, seed=9)
    scale = 1.0 / math.sqrt(D)
    out = ops.paged_attention_generic(s["q"], heads=heads, kv_heads=kv_heads, head_dim=D, kv_cache=s["cache"],
                                      block_table=s["table"], request_of_row=s["req_of_row"],
                                      positions=s["positions"], scale=scale, window=window or 0)
    ops.check_errors()
    ref = _attention_reference(s, lens, new, scale, window)
    torch.testing.assert_close(out.cpu().double(), ref, **_tol(dtype))


def _step_of(lens, new):
    from types import SimpleNamespace
    cu = [0]
    for n in new:
        cu.append(cu[-1] + n)
    starts = [l - n for l, n in zip(lens, new)]
    req_of_row = [r for r, n in enumerate(new) for _ in range(n)]
    positions = [starts[r] + i for r, n in enumerate(new) for i in range(n)]
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    return SimpleNamespace(num_requests=len(lens), cu_q=i32(cu), q_start=i32(starts), host_cu_q=cu,
                           host_q_start=starts, request_of_row=i32(req_of_row), positions=i32(positions),
                           attention_plans={}, meta=i32([max(lens), sum(new), len(lens), 0]))


# the tensor-core kernels round the probabilities to bf16 before the PV product (one more 2^-9
# relative rounding per term than the generic kernel) and the output once
MMA_TOL = dict(rtol=1.6e-2, atol=4e-3)
MMA_CASES = [c for c in ATTN_CASES if c[2] != 48] + [
    (16, 8, 128, 16, [2048] * 8, [1] * 8, None),                 # decode batch, several splits each
    (16, 8, 128, 16, [700, 1, 130, 64, 65], [700, 1, 2, 8, 9], None),   # tile + decode-like mixed; G*n = 16 and 18
    (16, 8, 128, 16, [700, 300], [1, 300], 200),
    (32, 2, 64, 8, [90, 40], [1, 40], None),                     # G = 16: one token fills the 16 packed rows
    (40, 2, 32, 16, [90, 33], [1, 2], None),                     # G = 20 > 16: even one token goes to the tile kernel
]


@pytest.fixture(params=["tcgen05+tma", "tcgen05+tma+fetched", "tcgen05+tma+tickets", "mma.sync+cp.async"])
def attention_variant(request, ops):
    """The families of tensor-core attention kernels: tcgen05 tiles with TMA-fed splits that merge as a
    thread-block cluster (small partials sent to the block that finishes them); the same with every partial
    fetched by that block (what larger partials use); with the splits merged through scratch memory and tickets
    (what more than eight splits use); and the mma.sync tile kernel with cp.async splits (which also serve the sizes the
    first does not take)."""
    modern = request.param != "mma.sync+cp.async"
    ops.tcgen05_attention, ops.tma_attention = modern, modern
    ops.set_attention_cluster_merge("fetched" if request.param.endswith("fetched")
                                    else request.param != "tcgen05+tma+tickets")
    yield request.param
    ops.tcgen05_attention, ops.tma_attention = True, True
    ops.set_attention_cluster_merge(True)


MMA_CASES += [
    (16, 8, 128, 16, [2048], [2048], None),                      # a whole 2048-token prompt: 32 row tiles x 16 key tiles
    (16, 8, 128, 16, [1500, 900], [300, 900], 257),              # portions that start deep in the context, window
    (8, 1, 64, 32, [333], [333], None),                          # G = 8, head_dim 64, pages of 32
    (4, 4, 128, 64, [200, 50], [200, 50], None),                 # G = 1, pages of 64
]


@pytest.mark.parametrize("case", MMA_CASES, ids=[f"h{c[0]}kv{c[1]}d{c[2]}p{c[3]}w{c[6]}n{max(c[5])}r{len(c[4])}" for c in MMA_CASES])
def test_paged_attention_tensor_core(ops, attention_variant, case):
    heads, kv_heads, D, page, lens, new, window = case
    s = _paged_setup(torch.bfloat16, lens, new, heads, kv_heads, D, page, seed=13)
    scale = 1.0 / math.sqrt(D)
    step = _step_of(lens, new)
    out = ops.paged_attention_mma(s["q"], heads=heads, kv_heads=kv_heads, head_dim=D, kv_cache=s["cache"],
                                  block_table=s["table"], step=step, scale=scale, window=window or 0)
    ops.check_errors()
    ref = _attention_reference(s, lens, new, scale, window)
    torch.testing.assert_close(out.cpu().double(), ref, **MMA_TOL)
    plain = ops.paged_attention_generic(s["q"], heads=heads, kv_heads=kv_heads, head_dim=D, kv_cache=s["cache"],
                                        block_table=s["table"], request_of_row=step.request_of_row,
                                        positions=step.positions, scale=scale, window=window or 0)
    torch.testing.assert_close(out.float(), plain.float(), **MMA_TOL)


@pytest.mark.parametrize("split", [64, 128, 512])
def test_split_attention_with_a_fixed_cut(ops, split):
    """The keys per split may also be fixed by the host; every cut gives the same attention."""
    heads, kv_heads, D, page, lens, new = 16, 8, 128, 16, [1000, 77, 2048], [1, 1, 1]
    s = _paged_setup(torch.bfloat16, lens, new, heads, kv_heads, D, page, seed=15)
    ops.attention_split = split
    try:
        out = ops.paged_attention_mma(s["q"], heads=heads, kv_heads=kv_heads, head_dim=D, kv_cache=s["cache"],
                                      block_table=s["table"], step=_step_of(lens, new), scale=0.09, window=0)
    finally:
        ops.attention_split = 0
    ops.check_errors()
    torch.testing.assert_close(out.cpu().double(), _attention_reference(s, lens, new, 0.09, None), **MMA_TOL)


def test_tensor_core_attention_reads_q_from_the_fused_projection_buffer(ops):
    """q lives in [rows, (heads + 2 kv_heads) * D] with a row stride larger than heads * D."""
    heads, kv_heads, D, page, lens, new = 6, 2, 64, 16, [50, 200], [50, 1]
    s = _paged_setup(torch.bfloat16, lens, new, heads, kv_heads, D, page, seed=14)
    T = sum(new)
    fused = torch.randn(T, (heads + 2 * kv_heads) * D, device=DEV).to(torch.bfloat16)
    fused[:, :heads * D] = s["q"]
    step = _step_of(lens, new)
    scale = 0.11
    out = ops.paged_attention_mma(fused, heads=heads, kv_heads=kv_heads, head_dim=D, kv_cache=s["cache"],
                                  block_table=s["table"], step=step, scale=scale, window=0)
    torch.testing.assert_close(out.cpu().double(), _attention_reference(s, lens, new, scale, None), **MMA_TOL)


def test_attention_finds_one_far_key_and_respects_the_window_edge(ops):
    """Random keys would hide a dropped key among hundreds: make one far key's
    score dominate, and put it just inside and just outside the window."""
    heads, kv_heads, D, page, L = 4, 2, 32, 16, 700
    for dtype in DTYPES:
        for window, far in [(None, 3), (None, 16 * 20), (64, L - 64), (64, L - 65), (1, L - 1)]:
            s = _paged_setup(dtype, [L], [1], heads, kv_heads, D, page, seed=10)
            q = s["qs"][0][0]                                    # [heads, D]
            # key `far` of kv head 0 points along q head 0, strongly
            k = s["ks"][0]
            k[far, 0] = (q[0].float() / q[0].float().norm() * 40.0).to(dtype)
            pg = int(s["table"][0, far // page])
            s["cache"][pg, 0, 0, far % page] = k[far, 0].to(DEV)
            scale = 1.0 / math.sqrt(D)
            outs = [(ops.paged_attention_generic(s["q"], heads=heads, kv_heads=kv_heads, head_dim=D,
                                                 kv_cache=s["cache"], block_table=s["table"],
                                                 request_of_row=s["req_of_row"], positions=s["positions"],
                                                 scale=scale, window=window or 0), _tol(dtype))]
            if dtype == torch.bfloat16:
                outs.append((ops.paged_attention_mma(s["q"], heads=heads, kv_heads=kv_heads, head_dim=D,
                                                     kv_cache=s["cache"], block_table=s["table"],
                                                     step=_step_of([L], [1]), scale=scale, window=window or 0),
                             MMA_TOL))
            ref = _attention_reference(s, [L], [1], scale, window)
            inside = window is None or far > L - 1 - window
            v_far = s["vs"][0][far, 0].double()
            for out, tol in outs:
                torch.testing.assert_close(out.cpu().double(), ref, **tol)
                close = float((out[0, :D].cpu().double() - v_far).abs().max())
                assert (close < 0.05) == inside, (dtype, window, far, close)


@pytest.mark.parametrize("vocab", [256, 1000, 151936])
def test_argmax_ties_go_to_the_lower_id(ops, vocab):
    logits = _rand((5, vocab), torch.float32, 11)
    logits[1, 7] = logits[1, vocab - 3] = 50.0
    logits[2, vocab - 1] = 60.0
    out = ops.argmax(logits).cpu().tolist()
    ref = [int(torch.argmax(row)) for row in logits.cpu()]
    ref[1] = 7
    assert out == ref


def _sample_rows(ops, logits, rows):
    from pih_b200.sampling import Sampler, SamplingParams
    sampler = Sampler(ops, logits.shape[1], torch.device(DEV))
    params = [SamplingParams(temperature=t, top_p=p, top_k=k, seed=s) for (t, p, k, s, o, sup) in rows]
    return sampler.sample(logits, params, [r[4] for r in rows], [r[5] for r in rows])


@pytest.mark.parametrize("vocab", [384, 5000])
def test_sampler_matches_the_plain_definition(ops, vocab):
    g = torch.Generator().manual_seed(12)
    S = 24
    logits = (torch.randn(S, vocab, generator=g) * 3.0)
    logits[3, 10] = logits[3, 20] = logits[3, 5] = 9.0          # ties at the top
    rows = []
    for i in range(S):
        t = [0.0, 0.8, 1.0, 2.0][i % 4]
        p = 1.0 if t == 0.0 else [1.0, 0.9, 0.5, 0.05][(i // 4) % 4]
        k = None if t == 0.0 else [None, 1, 7, 50, vocab][i % 5]
        sup = [] if i % 3 else [int(torch.argmax(logits[i])), 3]
        rows.append((t, p, k, 1234 + i, i * 3, sup))
    got = _sample_rows(ops, logits.to(DEV), rows)
    ops.check_errors()
    for i, (t, p, k, seed, ordinal, sup) in enumerate(rows):
        ref, _, _ = plain_impl.sample(logits[i].tolist(), temperature=t, top_p=p, top_k=k, seed=seed,
                                      ordinal=ordinal, suppressed=sup)
        assert got[i] == ref, (i, rows[i], got[i], ref)


@pytest.mark.parametrize("vocab", [384, 5000, 151936])
def test_selected_logprob(ops, vocab):
    """The log-probability of the chosen token (the reference's selected_logprob): greedy rows, sampled rows at
    several temperatures, rows with suppressed ids — against the exact value in float64 and, where the
    reference's sequential float32 sum is still accurate, against the plain sampler."""
    from pih_b200.sampling import Sampler, SamplingParams
    g = torch.Generator().manual_seed(21)
    S = 12
    logits = torch.randn(S, vocab, generator=g) * 3.0
    rows = []
    for i in range(S):
        t = [0.0, 0.7, 1.0, 2.0][i % 4]
        sup = [] if i % 3 else [int(torch.argmax(logits[i])), 5]
        rows.append((t, 1.0 if t == 0.0 else 0.9, None, 77 + i, 2 * i, sup))
    sampler = Sampler(ops, vocab, torch.device(DEV))
    params = [SamplingParams(temperature=t, top_p=p, top_k=k, seed=s) for (t, p, k, s, o, sup) in rows]
    ids, lps = sampler.sample_on_device(logits.to(DEV), params, [r[4] for r in rows], [r[5] for r in rows], logprobs=True)
    ids, lps = ids.tolist(), lps.tolist()
    ops.check_errors()
    for i, (t, p, k, seed, ordinal, sup) in enumerate(rows):
        scaled = logits[i].double() / (t if t > 0 else 1.0)
        keep = torch.ones(vocab, dtype=torch.bool)
        keep[sup] = False
        exact = float(scaled[ids[i]] - torch.logsumexp(scaled[keep], dim=0))
        assert abs(lps[i] - exact) <= 2e-5 * max(1.0, abs(exact)), (i, lps[i], exact)
        if vocab <= 5000:
            tok, ref, _ = plain_impl.sample(logits[i].tolist(), temperature=t, top_p=p, top_k=k, seed=seed,
                                            ordinal=ordinal, suppressed=sup)
            assert tok == ids[i] and abs(lps[i] - ref) <= 2e-5 * max(1.0, abs(ref))
    # all rows greedy and nothing suppressed: the argmax path
    greedy = [SamplingParams()] * S
    ids, lps = sampler.sample_on_device(logits.to(DEV), greedy, [0] * S, [[]] * S, logprobs=True)
    want = torch.log_softmax(logits.double(), dim=-1).max(dim=-1).values
    torch.testing.assert_close(lps.cpu().double(), want, rtol=2e-5, atol=2e-5)
    assert ids.tolist() == torch.argmax(logits, dim=-1).tolist()


@pytest.mark.parametrize("vocab,count", [(384, 20), (5000, 7), (151936, 20), (151936, 1), (400001, 3)])
def test_top_logprobs(ops, vocab, count):
    """The most probable ids with their log-probabilities (the reference's top_logprobs): greedy and scaled rows,
    rows whose best ids are suppressed, a plateau of equal logits (ties go to the lower id) that spans slices of the
    vocabulary — against the plain ordering and the exact log-probabilities in float64."""
    from pih_b200.sampling import Sampler, SamplingParams
    g = torch.Generator().manual_seed(23)
    S = 6
    logits = torch.randn(S, vocab, generator=g) * 3.0
    logits[1, torch.randperm(vocab, generator=g)[:40]] = 9.5           # a plateau above everything else
    logits[2, vocab - 1] = 20.0                                          # the last id of the last slice
    rows = []
    for i in range(S):
        t = [0.0, 0.7, 1.0, 2.0][i % 4]
        sup = [] if i % 3 else sorted(set(torch.topk(logits[i], 3).indices.tolist() + [5]))
        rows.append((t, sup))
    sampler = Sampler(ops, vocab, torch.device(DEV))
    params = [SamplingParams(temperature=t, seed=i, logprobs=True, top_logprobs=count) for i, (t, _) in enumerate(rows)]
    ids, lps, (top_ids, top_lps) = sampler.sample_on_device(logits.to(DEV), params, [0] * S, [sup for _, sup in rows],
                                                            logprobs=True, top_logprobs=count)
    ops.check_errors()
    top_ids, top_lps = top_ids.tolist(), top_lps.tolist()
    for i, (t, sup) in enumerate(rows):
        want = plain_impl.top_logprobs(logits[i].numpy(), count, temperature=t, suppressed=sup)
        assert top_ids[i] == [a for a, _ in want], (i, top_ids[i], want)
        for got, (_, lp) in zip(top_lps[i], want):
            assert abs(got - lp) <= 2e-5 * max(1.0, abs(lp)), (i, got, lp)
    # all rows greedy and nothing suppressed: the argmax path; the first of the list is the chosen token
    greedy = [SamplingParams(logprobs=True, top_logprobs=count)] * S
    ids, lps, (top_ids, top_lps) = sampler.sample_on_device(logits.to(DEV), greedy, [0] * S, [[]] * S, logprobs=True,
                                                            top_logprobs=count)
    assert top_ids[:, 0].tolist() == ids.tolist()
    torch.testing.assert_close(top_lps[:, 0], lps, rtol=1e-6, atol=1e-6)


def test_sampler_at_the_full_vocabulary(ops):
    """The vocabulary that serving samples from (151 936): the radix selection's two-level counts and the
    fixed-point mass over 150 000 terms.  Temperature alone, top-k 50, top-p 0.9, both, a suppressed arg-max,
    greedy with a suppressed arg-max, a plateau of equal logits.

    The kernel adds masses exactly (2^-44 fixed point); the definition adds them one after the other in
    float32 (plugins/model-qwen3/qwen3_sampler.cpp:140-170), which over 150 000 terms loses up to a few
    thousandths of the total — every term below half an ulp of the running sum is dropped.  So the kernel is
    held to the definition evaluated without that loss (float64: its choice is the first place where the
    cumulative share exceeds u, to 2e-6), and its distance from the plain float32 sampler's choice may be no
    more than the mass that float32 summation can lose.  Where few terms are summed (top-k) the two agree."""
    import numpy as np
    vocab = 151936
    g = torch.Generator().manual_seed(19)
    rows = [(0.8, 1.0, None, 7, 0, []), (0.7, 1.0, 50, 8, 3, []), (1.0, 0.9, None, 9, 100, []),
            (1.3, 0.5, 50, 10, 2**33 + 5, []), (0.8, 1.0, None, 11, 1, "argmax"), (0.0, 1.0, None, 0, 4, "argmax"),
            (2.0, 0.95, 1000, 2**40 + 3, 77, []), (0.6, 0.05, None, 13, 9, [5, 6])]
    logits = torch.randn(len(rows), vocab, generator=g) * 2.5
    logits[2, 1000:1040] = 9.0                                   # a plateau of equal logits at the top
    rows = [(t, p, k, s, o, [int(torch.argmax(logits[i])), 17] if sup == "argmax" else sup)
            for i, (t, p, k, s, o, sup) in enumerate(rows)]
    got = _sample_rows(ops, logits.to(DEV), rows)
    ops.check_errors()
    for i, (t, p, k, seed, ordinal, sup) in enumerate(rows):
        ref, _, word = plain_impl.sample(logits[i].tolist(), temperature=t, top_p=p, top_k=k, seed=seed,
                                         ordinal=ordinal, suppressed=sup)
        assert got[i] not in sup
        if t == 0.0 or (k is not None and k <= 50):
            assert got[i] == ref, (i, rows[i], got[i], ref)
            continue
        scaled = (logits[i].numpy() / np.float32(t)).astype(np.float32)
        order = np.lexsort((np.arange(vocab), -scaled.astype(np.float64)))
        order = order[~np.isin(order, sup)]
        if k is not None:
            order = order[:k]
        w = np.exp((scaled[order] - scaled[order[0]]).astype(np.float64))
        share = np.cumsum(w) / w.sum()
        kept = min(len(order), int(np.searchsorted(share, p, side="left")) + 1)
        cum = np.concatenate([[0.0], np.cumsum(w[:kept]) / w[:kept].sum()])
        at = {int(tok): j for j, tok in enumerate(order)}
        u = (word + 0.5) / 2.0 ** 32
        j = at[got[i]]
        assert j < kept and cum[j] - 2e-6 <= u < cum[j + 1] + 2e-6, (i, rows[i], got[i], j, kept, u)
        jr = min(at[ref], kept - 1)
        assert abs(cum[j + 1] - cum[jr + 1]) < 1e-2, (i, rows[i], got[i], ref)


def test_sampler_draws_follow_the_distribution(ops):
    """Many ordinals of one request: frequencies follow softmax(logits / T)."""
    vocab, n = 12, 4000
    row = torch.tensor([2.0, 1.0, 0.5, 0.0, -1.0, 3.0, 1.5, -2.0, 0.2, 0.1, 2.5, -0.5])
    logits = row.repeat(n, 1).to(DEV)
    got = _sample_rows(ops, logits, [(0.7, 1.0, None, 99, o, []) for o in range(n)])
    freq = torch.bincount(torch.tensor(got), minlength=vocab).double() / n
    prob = torch.softmax(row.double() / 0.7, dim=0)
    assert float((freq - prob).abs().max()) < 0.03
    # the same (seed, ordinal) gives the same token whatever else is in the batch
    again = _sample_rows(ops, logits[:7], [(0.7, 1.0, None, 99, o, []) for o in (5, 900, 17, 3, 2500, 0, 41)])
    assert again == [got[o] for o in (5, 900, 17, 3, 2500, 0, 41)]


FUSED_QK_CASES = [
    # heads, kv_heads, D, page, lens, new, window, norms, rope, write_kv
    (16, 8, 128, 16, [2048] * 8, [1] * 8, None, True, True, True),          # the decode step of the benchmark
    (16, 8, 128, 16, [1, 64, 65, 130, 2047, 513], [1, 1, 1, 2, 8, 3], None, True, True, True),   # tile edges, small portions
    (16, 8, 128, 16, [700, 300, 64], [1, 4, 2], 200, True, True, True),     # window
    (8, 2, 64, 8, [90, 40, 33], [1, 2, 1], None, True, True, True),         # head_dim 64, G = 4, pages of 8
    (4, 4, 256, 64, [200, 50], [1, 3], None, True, True, True),             # head_dim 256, G = 1, pages of 64
    (16, 8, 128, 32, [300, 129], [1, 1], None, False, True, True),          # no q/k norm
    (16, 8, 128, 16, [300, 129], [2, 1], None, True, False, True),          # no rotation
    (16, 8, 128, 16, [300, 129], [1, 1], None, True, True, False),          # another entry's cache: nothing appended
]


@pytest.mark.parametrize("splits", [0, 64])
@pytest.mark.parametrize("case", FUSED_QK_CASES, ids=[f"h{c[0]}kv{c[1]}d{c[2]}p{c[3]}w{c[6]}n{max(c[5])}{'' if c[7] else '-nonorm'}{'' if c[8] else '-norope'}{'' if c[9] else '-nowrite'}" for c in FUSED_QK_CASES])
def test_qk_attention_fused_matches_the_two_kernels(ops, case, splits):
    """The decode attention that norms and rotates q and k and appends to the cache itself gives the bits of
    the q/k kernel followed by the attention kernel — output and cache — with the splits merged as a cluster
    (automatic cut) and through tickets (64-key splits: more than eight of them)."""
    heads, kv_heads, D, page, lens, new, window, norms, rope, write_kv = case
    s = _paged_setup(torch.bfloat16, lens, new, heads, kv_heads, D, page, seed=31)
    T = sum(new)
    g = torch.Generator().manual_seed(32)
    kv_new = torch.randn(T, 2 * kv_heads * D, generator=g).to(torch.bfloat16).to(DEV)
    qkv = torch.cat([s["q"], kv_new], dim=1).contiguous()
    qw = (1 + 0.2 * torch.randn(D, generator=g)).to(torch.bfloat16).to(DEV) if norms else None
    kw = (1 + 0.2 * torch.randn(D, generator=g)).to(torch.bfloat16).to(DEV) if norms else None
    table = _rope_table(2100, D, 10000.0) if rope else None
    step = _step_of(lens, new)
    slots = []
    for r, (L, n) in enumerate(zip(lens, new)):
        for pos in range(L - n, L):
            slots.append(int(s["table"][r, pos // page]) * page + pos % page)
    slots = torch.tensor(slots, dtype=torch.int32, device=DEV)
    kw_args = dict(heads=heads, kv_heads=kv_heads, head_dim=D, q_norm=qw, k_norm=kw, eps=1e-6, rope_table=table,
                   rotary_dim=D if rope else 0)
    ops.attention_split = splits
    try:
        # the two kernels
        qkv_a, cache_a = qkv.clone(), s["cache"].clone()
        ops.qk_norm_rope_kv_write(qkv_a, positions=s["positions"], slot_mapping=slots, kv_cache=cache_a,
                                  write_kv=write_kv, **kw_args)
        out_a = ops.paged_attention_mma(qkv_a, heads=heads, kv_heads=kv_heads, head_dim=D, kv_cache=cache_a,
                                        block_table=s["table"], step=step, scale=1.0 / math.sqrt(D), window=window or 0)
        # one kernel
        qkv_b, cache_b = qkv.clone(), s["cache"].clone()
        step_b = _step_of(lens, new)
        out_b = ops.qk_attention_fused(qkv_b, kv_cache=cache_b, block_table=s["table"], step=step_b,
                                       scale=1.0 / math.sqrt(D), window=window or 0, write_kv=write_kv, **kw_args)
    finally:
        ops.attention_split = 0
    ops.check_errors()
    assert out_b is not None
    assert torch.equal(qkv_b, qkv)                                   # the raw rows are left as they were
    assert torch.equal(cache_b, cache_a)
    assert torch.equal(out_b, out_a)
    if not write_kv:
        assert torch.equal(cache_b, s["cache"])


def test_qk_attention_fused_declines_what_it_does_not_take(ops):
    heads, kv_heads, D, page = 16, 8, 128, 16
    lens, new = [300, 40], [1, 40]                                   # a prompt portion in the step
    s = _paged_setup(torch.bfloat16, lens, new, heads, kv_heads, D, page, seed=33)
    qkv = torch.cat([s["q"], torch.zeros(sum(new), 2 * kv_heads * D, dtype=torch.bfloat16, device=DEV)], dim=1).contiguous()
    kw_args = dict(heads=heads, kv_heads=kv_heads, head_dim=D, q_norm=None, k_norm=None, eps=1e-6, rope_table=None,
                   rotary_dim=0, kv_cache=s["cache"], block_table=s["table"], scale=0.1, window=0, write_kv=True)
    assert ops.qk_attention_fused(qkv, step=_step_of(lens, new), **kw_args) is None
    lens, new = [300, 40], [1, 1]
    table = _rope_table(400, D, 10000.0)
    s = _paged_setup(torch.bfloat16, lens, new, heads, kv_heads, D, page, seed=34)
    qkv = torch.cat([s["q"], torch.zeros(2, 2 * kv_heads * D, dtype=torch.bfloat16, device=DEV)], dim=1).contiguous()
    kw_args.update(kv_cache=s["cache"], block_table=s["table"], rope_table=table, rotary_dim=D // 2)   # partial rotation
    assert ops.qk_attention_fused(qkv, step=_step_of(lens, new), **kw_args) is None
    ops.check_errors()


@pytest.mark.parametrize("M,I,K", [(300, 264, 200), (2048, 3072, 1024), (130, 8, 64), (129, 1000, 1032), (513, 136, 96)])
def test_linear_tcgen05_swiglu(ops, M, I, K):
    """The tcgen05 product with SiLU-mul in its epilogue against the plain parts: gate and up rounded to bf16, then
    silu(g) * u rounded — each element within what one rounding flip per stage can do (see the few-rows test)."""
    x = _rand((M, K), torch.bfloat16, 51)
    gate = _rand((I, K), torch.bfloat16, 52, 0.05)
    up = _rand((I, K), torch.bfloat16, 53, 0.05)
    w = torch.stack([gate.reshape(-1, 8, K), up.reshape(-1, 8, K)], dim=1).reshape(2 * I, K).contiguous()
    act = ops.linear_tcgen05_swiglu(x, w)
    ops.check_errors()
    assert act is not None and act.shape == (M, I)
    g_ref = plain_impl.linear(x.cpu(), gate.cpu(), "bf16")
    u_ref = plain_impl.linear(x.cpu(), up.cpu(), "bf16")
    act_ref = plain_impl.silu_mul(g_ref, u_ref, "bf16")
    ulp = lambda t: torch.exp2(torch.floor(torch.log2(t.abs().clamp_min(1e-30))) - 7)
    sig = torch.sigmoid(g_ref)
    silu, dsilu = g_ref * sig, sig * (1 + g_ref * (1 - sig))
    # ... and, where g or u is a small difference of large products, the 32-bit accumulation's own noise
    # (about K * 2^-24 of the products' size) weighs more than a rounding step of the tiny value
    noise = 1e-5
    bound = (ulp(g_ref) + noise) * (dsilu * u_ref).abs() + (ulp(u_ref) + noise) * silu.abs() + ulp(act_ref) + 1e-6
    err = (act.cpu().double() - act_ref).abs()
    assert bool((err <= 1.05 * bound).all()), float((err / bound).max())
    # and the separate kernels of the pack
    act2 = ops.silu_mul(ops.linear(x, w), 8)
    err2 = (act2.cpu().double() - act.cpu().double()).abs()
    assert bool((err2 <= 2.1 * bound).all()), float((err2 / bound).max())
