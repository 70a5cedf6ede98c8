"""Each CUDA kernel alone against a plain float64/float32 restatement of the same operation, at
sizes other than the tiny models' (odd widths, tails, head sizes in steps of 16, many groups)."""
import math

import pytest
import torch

from kernel_inputs import attention_case
from plain import llama_moe_plain as P

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def _lib():
    from transformer_b200.csrc import lib
    return lib


def _tol(dtype, scale=1.0):
    return (2e-5 if dtype == torch.float32 else 2.0 ** -7) * scale


def _rand(shape, dtype, seed, std=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * std).to(dtype).cuda()


# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
def test_embed(dtype):
    lib = _lib()
    V, d = 301, 72
    table = _rand((V, d), dtype, 0)
    tok = torch.tensor([5, 300, 0, 5, 17], dtype=torch.int32, device="cuda")
    x = torch.empty((5, d), dtype=torch.float32, device="cuda")
    lib.call("tb_embed_" + lib.suffix(dtype), tok.data_ptr(), table.data_ptr(), x.data_ptr(), 5, d)
    assert torch.equal(x, table[tok.long()].float())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d", [72, 4100])
def test_add_rmsnorm(dtype, d):
    lib = _lib()
    n, eps = 7, 3e-6
    x = _rand((n, d), torch.float32, 1, 2.0)
    delta = _rand((n, d), dtype, 2)
    w = _rand((d,), torch.float32, 3)
    y = torch.empty((n, d), dtype=dtype, device="cuda")
    x_in = x.clone()
    lib.call("tb_add_rmsnorm_" + lib.suffix(dtype), x.data_ptr(), delta.data_ptr(), 0, 0, 0, 0, 0, w.data_ptr(), eps,
             y.data_ptr(), n, d, w.data_ptr(), 4 * d)          # and some weight to fetch meanwhile: changes nothing
    v = x_in.double() + delta.double()
    assert torch.allclose(x.double(), v, atol=1e-6), "the stream is updated in place with a float sum"
    ref = P.rms_norm(v.cpu(), w.double().cpu(), eps)
    assert float((y.double().cpu() - ref).abs().max()) <= _tol(dtype, float(ref.abs().max()))
    # gathered rows, no delta, no write-back
    rows = torch.tensor([6, 0, 6], dtype=torch.int32, device="cuda")
    y2 = torch.empty((3, d), dtype=dtype, device="cuda")
    before = x.clone()
    lib.call("tb_add_rmsnorm_" + lib.suffix(dtype), x.data_ptr(), 0, 0, 0, 0, 0, rows.data_ptr(), w.data_ptr(), eps,
             y2.data_ptr(), 3, d, 0, 0)
    assert torch.equal(x, before)
    ref2 = P.rms_norm(before[rows.long()].double().cpu(), w.double().cpu(), eps)
    assert float((y2.double().cpu() - ref2).abs().max()) <= _tol(dtype, float(ref2.abs().max()))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d,E,k", [(72, 6, 3), (4096, 16, 4), (136, 33, 1), (8192, 5, 5)])
def test_add_rmsnorm_that_also_routes(dtype, d, E, k):
    """The norm that also routes: the same stream and rows as the norm alone, and the experts and weights that the
    router kernel finds in those rows; what it does not take is refused with nothing done."""
    lib = _lib()
    n, eps = 9, 1e-5
    x = _rand((n, d), torch.float32, 4, 2.0)
    delta = _rand((n, d), dtype, 5)
    w = _rand((d,), torch.float32, 6)
    wr = _rand((E, d), dtype, 7, 0.3)
    x2 = x.clone()
    y, y2 = (torch.empty((n, d), dtype=dtype, device="cuda") for _ in range(2))
    idx, idx2 = (torch.empty((n, k), dtype=torch.int32, device="cuda") for _ in range(2))
    sc, sc2 = (torch.empty((n, k), dtype=torch.float32, device="cuda") for _ in range(2))
    took = lib.try_call("tb_add_rmsnorm_router_" + lib.suffix(dtype), x.data_ptr(), delta.data_ptr(), 0, 0, 0, 0, 0,
                        w.data_ptr(), eps, y.data_ptr(), wr.data_ptr(), idx.data_ptr(), sc.data_ptr(), n, d, E, k)
    assert took
    lib.call("tb_add_rmsnorm_" + lib.suffix(dtype), x2.data_ptr(), delta.data_ptr(), 0, 0, 0, 0, 0, w.data_ptr(), eps,
             y2.data_ptr(), n, d, 0, 0)
    assert torch.equal(x, x2) and torch.equal(y, y2)
    lg = torch.empty((n, E), dtype=torch.float32, device="cuda")
    lib.call("tb_router_" + lib.suffix(dtype), y2.data_ptr(), wr.data_ptr(), idx2.data_ptr(), sc2.data_ptr(),
             lg.data_ptr(), 0, 0, 0, 0, n, d, E, k)
    assert torch.equal(idx, idx2), "the same sums in the same order: the same choice"
    assert float((sc - sc2).abs().max()) < 1e-6
    rows = torch.tensor([2, 2, 7], dtype=torch.int32, device="cuda")      # gathered rows, as the final norm has them
    y3 = torch.empty((3, d), dtype=dtype, device="cuda")
    i3 = torch.empty((3, k), dtype=torch.int32, device="cuda")
    s3 = torch.empty((3, k), dtype=torch.float32, device="cuda")
    assert lib.try_call("tb_add_rmsnorm_router_" + lib.suffix(dtype), x.data_ptr(), 0, 0, 0, 0, 0, rows.data_ptr(),
                        w.data_ptr(), eps, y3.data_ptr(), wr.data_ptr(), i3.data_ptr(), s3.data_ptr(), 3, d, E, k)
    assert torch.equal(i3, idx[rows.long()]) and torch.equal(y3, y[rows.long()])
    assert not lib.try_call("tb_add_rmsnorm_router_" + lib.suffix(dtype), x.data_ptr(), delta.data_ptr(), 0, 0, 0, 0, 0,
                            w.data_ptr(), eps, y.data_ptr(), wr.data_ptr(), idx.data_ptr(), sc.data_ptr(), n, d - 4,
                            E, k), "a width that is no multiple of 8 is refused"
    many = torch.zeros((300, d), dtype=torch.float32, device="cuda")
    assert not lib.try_call("tb_add_rmsnorm_router_" + lib.suffix(dtype), many.data_ptr(), 0, 0, 0, 0, 0, 0, w.data_ptr(),
                            eps, torch.empty((300, d), dtype=dtype, device="cuda").data_ptr(), wr.data_ptr(),
                            torch.empty((300, k), dtype=torch.int32, device="cuda").data_ptr(),
                            torch.empty((300, k), dtype=torch.float32, device="cuda").data_ptr(), 300, d, E, k), \
        "more rows than it takes: refused (the router's own kernels serve prompts)"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("pairing", ["adjacent", "half"])
def test_rope_and_cache_write(dtype, pairing):
    lib = _lib()
    nh, nkvh, dh, theta, nctx = 5, 1, 48, 12345.0, 300
    pos = [0, 1, 63, 64, 200, 299]
    seqs = [0, 1, 1, 1, 0, 1]
    nt = len(pos)
    qkv = _rand((nt, (nh + 2 * nkvh) * dh), dtype, 4)
    orig = qkv.clone()
    i = torch.arange(dh // 2, dtype=torch.float64)
    ang = torch.arange(nctx, dtype=torch.float64)[:, None] * theta ** (-2.0 * i / dh)[None]
    cos, sin = torch.cos(ang).float().cuda(), torch.sin(ang).float().cuda()
    n_pages, max_pages = 12, 5
    table = torch.tensor([[3, 7, 1, 9, 11], [2, 8, 0, 4, 10]], dtype=torch.int32, device="cuda")
    kc = torch.zeros((n_pages, nkvh, 64, dh), dtype=dtype, device="cuda")
    vc = torch.zeros_like(kc)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    seq_t, pos_t = i32(seqs), i32(pos)      # kept alive: a temporary's memory would be handed out again
    lib.call("tb_rope_cache_" + lib.suffix(dtype), qkv.data_ptr(), seq_t.data_ptr(), pos_t.data_ptr(),
             table.data_ptr(), max_pages, cos.data_ptr(), sin.data_ptr(), kc.data_ptr(), vc.data_ptr(), nt, nh,
             nkvh, dh, 1 if pairing == "half" else 0)
    o = orig.double().cpu().reshape(nt, nh + 2 * nkvh, dh)
    q_ref = P.rope(o[:, :nh], pos, theta, pairing)
    k_ref = P.rope(o[:, nh:nh + nkvh], pos, theta, pairing)
    got = qkv.double().cpu().reshape(nt, nh + 2 * nkvh, dh)
    tol = _tol(dtype, 4.0)
    assert float((got[:, :nh] - q_ref).abs().max()) <= tol
    for a in range(nt):
        page = int(table[seqs[a], pos[a] // 64])
        assert float((kc[page, :, pos[a] % 64].double().cpu() - k_ref[a]).abs().max()) <= tol
        assert torch.equal(vc[page, :, pos[a] % 64].cpu(), orig.cpu().reshape(nt, -1, dh)[a, nh + nkvh:])
    assert int((kc.abs().sum(dim=(1, 3)) > 0).sum()) == nt, "nothing else in the cache was touched"


# ---------------------------------------------------------------------------------------------
def _run_attention(lib, c, dtype, splits, decode, ring=False, done=None):
    nt, nh, dh = c["nt"], c["nh"], c["dh"]
    out = torch.zeros(nt, nh * dh, dtype=dtype, device="cuda")
    partial = torch.empty(max(1, nt * nh * splits * (dh + 2)), dtype=torch.float32, device="cuda")
    scale = 1.0 / math.sqrt(dh)
    if decode:
        seq = torch.repeat_interleave(c["tile_seq"], c["tile_nq"])
        if ring:       # the kernel with a ring of cache pages: TMA, products on the tensor cores
            ok = lib.try_call("tb_attention_decode_mma_bf16", c["q"].data_ptr(), out.data_ptr(), c["kc"].data_ptr(),
                              c["vc"].data_ptr(), seq.data_ptr(), c["tok_pos"].data_ptr(), c["table"].data_ptr(),
                              partial.data_ptr(), 0 if done is None else done.data_ptr(), nt, c["max_pages"], nh * dh,
                              nh, c["nkvh"], dh, splits, c["kc"].shape[0], scale)
            assert lib.gemm_tc_status() == 0
            return out.double().cpu().reshape(nt, nh, dh) if ok else None
        ok = lib.try_call("tb_attention_decode_" + lib.suffix(dtype), c["q"].data_ptr(), out.data_ptr(),
                          c["kc"].data_ptr(), c["vc"].data_ptr(), seq.data_ptr(), c["tok_pos"].data_ptr(),
                          c["table"].data_ptr(), partial.data_ptr(), nt, c["max_pages"], nh * dh, nh, c["nkvh"], dh,
                          splits, scale)
        if not ok:
            return None
    else:
        lib.call("tb_attention_" + lib.suffix(dtype), c["q"].data_ptr(), out.data_ptr(), c["kc"].data_ptr(),
                 c["vc"].data_ptr(), c["tile_seq"].data_ptr(), c["tile_t0"].data_ptr(), c["tile_nq"].data_ptr(),
                 c["tok_pos"].data_ptr(), c["table"].data_ptr(), partial.data_ptr(), c["tiles"], nt, c["max_pages"],
                 nh * dh, nh, c["nkvh"], dh, splits, scale)
    return out.double().cpu().reshape(nt, nh, dh)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkvh,dh", [(4, 2, 16), (3, 1, 48), (6, 6, 80), (40, 2, 32), (2, 1, 256), (8, 8, 128)])
def test_attention_general(dtype, nh, nkvh, dh):
    lib = _lib()
    tq = lib.attention_tile_tokens(nh, nkvh)
    # prompts from zero, a continued prompt, single tokens: all in one ragged batch
    c = attention_case([37, 1, 9, 1, 70], [0, 130, 64, 0, 31], nh, nkvh, dh, dtype, tq, seed=nh + dh)
    for splits in (1, 3):
        got = _run_attention(lib, c, dtype, splits, decode=False)
        assert float((got - c["ref"]).abs().max()) <= _tol(dtype, 4.0), f"splits {splits}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkvh,dh", [(4, 2, 16), (3, 1, 32), (8, 8, 128), (12, 2, 64), (20, 2, 128), (2, 1, 256)])
def test_attention_decode(dtype, nh, nkvh, dh):
    lib = _lib()
    c = attention_case([1, 1, 1, 1, 1], [0, 63, 64, 700, 129], nh, nkvh, dh, dtype, 1, seed=3 * nh + dh)
    for splits in (1, 2, 7):
        got = _run_attention(lib, c, dtype, splits, decode=True)
        if got is None:
            assert dtype == torch.float32 and dh == 256, "only a float head of 256 is refused here"
            return
        assert float((got - c["ref"]).abs().max()) <= _tol(dtype, 4.0), f"splits {splits}"


@pytest.mark.parametrize("decode", [False, True])
def test_attention_finds_one_far_key(decode):
    """Among hundreds of keys one, far back and on an early page, is made to dominate: the output
    must be its value.  Shows a wrong page, a dropped key slice, a wrong mask."""
    lib = _lib()
    nh, nkvh, dh = 4, 2, 64
    for far in (0, 5, 64, 391):
        c = attention_case([1], [900], nh, nkvh, dh, torch.float32, 1, seed=far, scale_key=(0, far, 40.0))
        # the query that points at that key: q = k_far (already scaled), so its score towers
        kfar_page = int(c["table"][0, far // 64])
        kfar = c["kc"][kfar_page, :, far % 64]                    # [nkvh, dh]
        c["q"] = kfar.repeat_interleave(nh // nkvh, dim=0).reshape(1, nh * dh).contiguous() * 0.05
        vfar = c["vc"][kfar_page, :, far % 64].double().cpu()
        for splits in (1, 4):
            got = _run_attention(lib, c, torch.float32, splits, decode)
            for h in range(nh):
                assert float((got[0, h] - vfar[h // 2]).abs().max()) < 1e-3, f"far key {far}, splits {splits}"


# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,N,K", [(1, 16, 8), (5, 50, 24), (70, 129, 100), (3, 688, 4096), (130, 64, 688)])
def test_gemm_simt_dense(dtype, M, N, K):
    from transformer_b200.parts.linear import gemm_simt
    a, w = _rand((M, K), dtype, 5), _rand((N, K), dtype, 6, 0.1)
    ref = a.double() @ w.double().T
    for out_dtype, kind in ((dtype, 0), (torch.float32, 1)):
        out = torch.empty((M, N), dtype=out_dtype, device="cuda")
        gemm_simt(a, w, out, out_kind=kind)
        assert float((out.double() - ref).abs().max()) <= _tol(out_dtype, float(ref.abs().max()))


def _grouped_case(dtype, E, k, nt, d, di, seed):
    g = torch.Generator().manual_seed(seed)
    x = _rand((nt, d), dtype, seed + 1)
    wgu = _rand((E, 2 * di, d), dtype, seed + 2, 0.1)
    wd = _rand((E, d, di), dtype, seed + 3, 0.1)
    idx = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(nt)]).to(torch.int32).cuda()
    return x, wgu, wd, idx


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("E,k,nt,d,di", [(4, 2, 9, 64, 40), (16, 4, 8, 256, 86), (6, 3, 200, 96, 80), (3, 3, 1, 72, 16),
                                          (16, 4, 64, 128, 88), (5, 2, 13, 2048, 48)])
def test_dispatch_grouped_products_and_combine(dtype, E, k, nt, d, di):
    """token -> expert dispatch, the grouped gate/up product with swiglu, the grouped down product
    and the weighted combine, against a per-token loop."""
    lib = _lib()
    from transformer_b200.parts.linear import grouped_matmul, gemm_simt
    x, wgu, wd, idx = _grouped_case(dtype, E, k, nt, d, di, seed=E + nt)
    w = torch.softmax(_rand((nt, k), torch.float32, 9), dim=1).contiguous()
    M = nt * k
    off = torch.empty(E + 1, dtype=torch.int32, device="cuda")
    st = torch.empty(M, dtype=torch.int32, device="cuda")
    pr = torch.empty(M, dtype=torch.int32, device="cuda")
    lib.call("tb_moe_dispatch", idx.data_ptr(), off.data_ptr(), st.data_ptr(), pr.data_ptr(), M, k, E)
    offc, stc, prc = off.cpu(), st.cpu(), pr.cpu()
    assert offc[0] == 0 and offc[-1] == M and sorted(prc.tolist()) == list(range(M))
    for p in range(M):
        e = int(idx.view(-1)[p])
        assert offc[e] <= prc[p] < offc[e + 1] and stc[prc[p]] == p // k
    ref = torch.zeros(nt, d, dtype=torch.float64)
    for t in range(nt):
        for j in range(k):
            e = int(idx[t, j])
            ref[t] += float(w[t, j]) * P.expert_ffn(x[t].double().cpu(), wgu[e].double().cpu(), wd[e].double().cpu())
    uses = ("auto", "simt") + (("unsorted",) if dtype == torch.bfloat16 and M <= 256 and d % 8 == 0 and di % 8 == 0 else ())
    for use in uses:
        h = torch.empty((M, di), dtype=dtype, device="cuda")
        y = torch.empty((M, d), dtype=dtype, device="cuda")
        rows = pr
        if use == "unsorted":
            # no lists: row p is pair p, and every block picks its expert's pairs out of the router's answer
            from transformer_b200.parts.linear import gemm_skinny
            pairs = idx.view(-1)
            assert gemm_skinny(x, wgu, h, groups=E, out_kind=2, max_group_rows=nt, row_group=pairs, x_div=k)
            assert gemm_skinny(h, wd, y, groups=E, max_group_rows=nt, row_group=pairs)
            rows = torch.arange(M, dtype=torch.int32, device="cuda")
        elif use == "auto":
            grouped_matmul(x, wgu, h, a_rows=st, group_offsets=off, groups=E, swiglu=True)
            grouped_matmul(h, wd, y, group_offsets=off, groups=E)
        else:
            gemm_simt(x, wgu, h, a_rows=st, group_offsets=off, groups=E, out_kind=2)
            gemm_simt(h, wd, y, group_offsets=off, groups=E, out_kind=0)
        out = torch.empty((nt, d), dtype=dtype, device="cuda")
        lib.call("tb_moe_combine_" + lib.suffix(dtype), y.data_ptr(), rows.data_ptr(), w.data_ptr(), out.data_ptr(),
                 nt, d, k)
        assert float((out.double().cpu() - ref).abs().max()) <= 2 * _tol(dtype, float(ref.abs().max())), use


def test_an_expert_that_nearly_every_token_picks():
    """The decode product sizes a pass by the usual group (one and a half times the mean), so a group far larger
    than that takes several passes over its weights: every token picks expert 3 and one other expert."""
    from transformer_b200.parts.linear import gemm_skinny, grouped_matmul
    lib = _lib()
    E, k, nt, d, di = 8, 2, 40, 128, 48
    x, wgu, wd, _ = _grouped_case(torch.bfloat16, E, k, nt, d, di, seed=77)
    g = torch.Generator().manual_seed(5)
    other = torch.randint(0, E - 1, (nt,), generator=g)
    other = other + (other >= 3).long()                          # any expert but 3
    idx = torch.stack([torch.full((nt,), 3), other], dim=1).to(torch.int32).cuda()
    idx[::2] = idx[::2].flip(1)                                  # expert 3 is not always the first choice
    M = nt * k
    assert int((idx == 3).sum()) == nt and (3 * M // E + 1) // 2 < nt, "one group is larger than a pass"
    ref = torch.zeros(M, d, dtype=torch.float64)
    for p in range(M):
        e = int(idx.view(-1)[p])
        ref[p] = P.expert_ffn(x[p // k].double().cpu(), wgu[e].double().cpu(), wd[e].double().cpu())
    tol = 2 * _tol(torch.bfloat16, float(ref.abs().max()))
    h = torch.empty((M, di), dtype=torch.bfloat16, device="cuda")
    y = torch.empty((M, d), dtype=torch.bfloat16, device="cuda")
    pairs = idx.view(-1)
    assert gemm_skinny(x, wgu, h, groups=E, out_kind=2, max_group_rows=nt, row_group=pairs, x_div=k)
    assert gemm_skinny(h, wd, y, groups=E, max_group_rows=nt, row_group=pairs)
    assert float((y.double().cpu() - ref).abs().max()) <= tol, "rows unsorted"
    off = torch.empty(E + 1, dtype=torch.int32, device="cuda")
    st = torch.empty(M, dtype=torch.int32, device="cuda")
    pr = torch.empty(M, dtype=torch.int32, device="cuda")
    lib.call("tb_moe_dispatch", idx.data_ptr(), off.data_ptr(), st.data_ptr(), pr.data_ptr(), M, k, E)
    h.zero_(), y.zero_()
    grouped_matmul(x, wgu, h, a_rows=st, group_offsets=off, groups=E, swiglu=True, max_group_rows=nt)
    grouped_matmul(h, wd, y, group_offsets=off, groups=E, max_group_rows=nt)
    assert float((y[pr.long()].double().cpu() - ref).abs().max()) <= tol, "rows sorted by expert"


@pytest.mark.parametrize("M,N,K", [(1, 16, 8), (8, 50, 24), (9, 129, 104), (33, 688, 4096), (64, 4096, 688), (3, 1000, 72),
                                   (17, 48, 1000)])
def test_gemm_skinny_dense(M, N, K):
    from transformer_b200.parts.linear import gemm_skinny
    a, w = _rand((M, K), torch.bfloat16, 7), _rand((N, K), torch.bfloat16, 8, 0.1)
    ref = a.double() @ w.double().T
    for out_dtype, kind in ((torch.bfloat16, 0), (torch.float32, 1)):
        out = torch.empty((M, N), dtype=out_dtype, device="cuda")
        assert gemm_skinny(a, w, out, out_kind=kind)
        assert float((out.double() - ref).abs().max()) <= _tol(out_dtype, float(ref.abs().max()))
    # a width that is no multiple of 8 is refused, not computed wrongly
    a2, w2 = _rand((M, 20), torch.bfloat16, 7), _rand((N, 20), torch.bfloat16, 8)
    assert not gemm_skinny(a2[:, :12].contiguous(), w2[:, :12].contiguous(),
                           torch.empty((M, N), dtype=torch.bfloat16, device="cuda"))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("E,k,d,nt", [(4, 2, 64, 5), (16, 4, 4096, 3), (6, 3, 100, 40), (70, 70, 24, 2), (33, 5, 72, 1100)])
def test_router(dtype, E, k, d, nt):
    lib = _lib()
    x, wr = _rand((nt, d), dtype, 10), _rand((E, d), dtype, 11, 0.3)
    idx = torch.empty((nt, k), dtype=torch.int32, device="cuda")
    w = torch.empty((nt, k), dtype=torch.float32, device="cuda")
    lg = torch.empty((nt, E), dtype=torch.float32, device="cuda")
    lib.call("tb_router_" + lib.suffix(dtype), x.data_ptr(), wr.data_ptr(), idx.data_ptr(), w.data_ptr(),
             lg.data_ptr(), 0, 0, 0, 0, nt, d, E, k)
    # the same kernel with the dispatch lists built by its last block, twice (the counter is left at zero)
    offs = torch.empty(E + 1, dtype=torch.int32, device="cuda")
    tok = torch.empty(nt * k, dtype=torch.int32, device="cuda")
    row = torch.empty(nt * k, dtype=torch.int32, device="cuda")
    done = torch.zeros(1, dtype=torch.int32, device="cuda")
    idx2, w2 = torch.empty_like(idx), torch.empty_like(w)
    for _ in range(2):
        offs.fill_(-1), tok.fill_(-1), row.fill_(-1)
        lib.call("tb_router_" + lib.suffix(dtype), x.data_ptr(), wr.data_ptr(), idx2.data_ptr(), w2.data_ptr(), 0,
                 offs.data_ptr(), tok.data_ptr(), row.data_ptr(), done.data_ptr(), nt, d, E, k)
        assert torch.equal(idx2, idx) and torch.equal(w2, w) and int(done) == 0
        flat = idx.flatten().cpu()
        counts = torch.bincount(flat, minlength=E)
        assert offs.cpu().tolist() == [0] + torch.cumsum(counts, 0).tolist()
        r = row.cpu().long()
        assert sorted(r.tolist()) == list(range(nt * k)), "every pair has a row of its own"
        assert torch.equal(tok.cpu()[r], torch.arange(nt * k, dtype=torch.int32) // k), "a row reads its pair's token"
        e_of_row = torch.bucketize(r, offs.cpu().long()[1:], right=True)
        assert torch.equal(e_of_row, flat.long()), "a pair's row lies in its expert's range"
    ref_lg = x.double() @ wr.double().T
    assert float((lg.double() - ref_lg).abs().max()) <= 2e-5 * max(1.0, float(ref_lg.abs().max())), \
        "router logits are float whatever the storage type"
    for t in range(0, nt, max(1, nt // 50)):
        experts, weights = P.route(lg[t].double().cpu(), k)     # from the kernel's own logits: exact rule
        assert idx[t].tolist() == experts
        assert float((w[t].double().cpu() - weights).abs().max()) < 1e-5


@pytest.mark.parametrize("E,k,d,nt", [(16, 4, 4096, 2048), (8, 2, 96, 17), (6, 3, 64, 300), (24, 5, 1024, 1000),
                                      (60, 7, 320, 333), (64, 64, 32, 16)])
def test_router_for_many_tokens(E, k, d, nt):
    """The router that takes 16 tokens' logits as one tensor-core tile: widths from one 32-column chunk (fewer
    chunks than warps) to 4,096, expert counts that are no multiple of 8, a last block of 1, 5, 12 and 16 tokens;
    logits against float64, the choice against the plain rule from the kernel's own logits, against the per-token
    kernel, and the dispatch lists that its last block builds, twice."""
    lib = _lib()
    dtype = torch.bfloat16
    x, wr = _rand((nt, d), dtype, 13), _rand((E, d), dtype, 14, 0.3)
    idx = torch.empty((nt, k), dtype=torch.int32, device="cuda")
    w = torch.empty((nt, k), dtype=torch.float32, device="cuda")
    lg = torch.empty((nt, E), dtype=torch.float32, device="cuda")
    lib.call("tb_router_rows_bf16", x.data_ptr(), wr.data_ptr(), idx.data_ptr(), w.data_ptr(), lg.data_ptr(), 0, 0, 0, 0,
             nt, d, E, k)
    ref_lg = x.double() @ wr.double().T
    assert float((lg.double() - ref_lg).abs().max()) <= 2e-5 * max(1.0, float(ref_lg.abs().max())), \
        "router logits are float whatever the storage type"
    for t in list(range(0, nt, max(1, nt // 50))) + [nt - 1]:
        experts, weights = P.route(lg[t].double().cpu(), k)     # from the kernel's own logits: exact rule
        assert idx[t].tolist() == experts, t
        assert float((w[t].double().cpu() - weights).abs().max()) < 1e-5
    # the per-token kernel sums in another order: the same experts wherever its two candidates are a clear gap apart
    idx1, w1, lg1 = torch.empty_like(idx), torch.empty_like(w), torch.empty_like(lg)
    lib.call("tb_router_bf16", x.data_ptr(), wr.data_ptr(), idx1.data_ptr(), w1.data_ptr(), lg1.data_ptr(), 0, 0, 0, 0,
             nt, d, E, k)
    assert float((lg - lg1).abs().max()) <= 2e-5 * max(1.0, float(ref_lg.abs().max()))
    top = torch.sort(lg, dim=1, descending=True).values
    clear = ((top[:, :-1] - top[:, 1:])[:, :k].min(dim=1).values > 1e-4) if k < E else \
        ((top[:, :-1] - top[:, 1:]).min(dim=1).values > 1e-4)
    assert int(clear.sum()) > nt // 2
    assert torch.equal(idx[clear], idx1[clear])
    offs = torch.empty(E + 1, dtype=torch.int32, device="cuda")
    tok = torch.empty(nt * k, dtype=torch.int32, device="cuda")
    row = torch.empty(nt * k, dtype=torch.int32, device="cuda")
    done = torch.zeros(1, dtype=torch.int32, device="cuda")
    idx2, w2 = torch.empty_like(idx), torch.empty_like(w)
    for _ in range(2):
        offs.fill_(-1), tok.fill_(-1), row.fill_(-1)
        lib.call("tb_router_rows_bf16", x.data_ptr(), wr.data_ptr(), idx2.data_ptr(), w2.data_ptr(), 0,
                 offs.data_ptr(), tok.data_ptr(), row.data_ptr(), done.data_ptr(), nt, d, E, k)
        assert torch.equal(idx2, idx) and torch.equal(w2, w) and int(done) == 0
        flat = idx.flatten().cpu()
        counts = torch.bincount(flat, minlength=E)
        assert offs.cpu().tolist() == [0] + torch.cumsum(counts, 0).tolist()
        r = row.cpu().long()
        assert sorted(r.tolist()) == list(range(nt * k)), "every pair has a row of its own"
        assert torch.equal(tok.cpu()[r], torch.arange(nt * k, dtype=torch.int32) // k), "a row reads its pair's token"
        e_of_row = torch.bucketize(r, offs.cpu().long()[1:], right=True)
        assert torch.equal(e_of_row, flat.long()), "a pair's row lies in its expert's range"
    assert not lib.try_call("tb_router_rows_bf16", x.data_ptr(), wr.data_ptr(), idx.data_ptr(), w.data_ptr(), 0, 0, 0, 0, 0,
                            nt, 40, E, k), "a width that is no multiple of 32 is refused"


def test_router_ties_go_to_the_lower_expert():
    lib = _lib()
    E, k, d = 8, 3, 16
    x = torch.ones((1, d), dtype=torch.float32, device="cuda")
    wr = torch.zeros((E, d), dtype=torch.float32, device="cuda")
    wr[[1, 4, 6, 7]] = 0.5                                  # four equal best logits
    idx = torch.empty((1, k), dtype=torch.int32, device="cuda")
    w = torch.empty((1, k), dtype=torch.float32, device="cuda")
    lib.call("tb_router_f32", x.data_ptr(), wr.data_ptr(), idx.data_ptr(), w.data_ptr(), 0, 0, 0, 0, 0, 1, d, E, k)
    assert idx[0].tolist() == [1, 4, 6] and torch.allclose(w, torch.full_like(w, 1 / 3))


# ---------------------------------------------------------------------------------------------
def _sample(lib, logits, u, t, k, p):
    rows = logits.shape[0]
    idx = torch.empty(rows, dtype=torch.int32, device="cuda")
    val = torch.empty(rows, dtype=torch.float32, device="cuda")
    uu = torch.tensor(u, dtype=torch.float32, device="cuda")
    lib.call("tb_sample", logits.data_ptr(), logits.stride(0), uu.data_ptr(), rows, logits.shape[1], float(t), int(k),
             float(p), idx.data_ptr(), val.data_ptr())
    return idx.cpu().tolist(), val.cpu()


@pytest.mark.parametrize("V", [5, 384, 32000, 50257])
def test_sampling_argmax_and_ties(V):
    lib = _lib()
    lg = _rand((3, V), torch.float32, 12)
    lg[1, [V // 2, V - 1]] = 50.0      # two equal maxima: the lower id wins
    lg[2, 0] = 60.0
    ids, vals = _sample(lib, lg, [0.5] * 3, 0.0, 0, 1.0)
    assert ids == [int(torch.argmax(lg[0])), V // 2, 0]
    assert torch.equal(vals, lg.cpu()[torch.arange(3), torch.tensor(ids)])
    assert _sample(lib, lg, [0.9] * 3, 0.7, 1, 1.0)[0] == ids, "top_k = 1 is the argmax"


@pytest.mark.parametrize("V,t,k,p", [(384, 0.8, 0, 1.0), (1000, 1.0, 40, 1.0), (1000, 1.3, 0, 0.9), (32000, 0.7, 50, 0.8),
                                     (50, 1.0, 7, 0.5), (50, 2.0, 49, 0.999)])
def test_sampling_draws_from_the_stated_distribution(V, t, k, p):
    """For many uniform numbers the kernel's token must be the one whose interval of the cumulative
    distribution (kept tokens in ascending id) holds u; a hair's breadth at an edge is allowed."""
    lib = _lib()
    rows = 64
    lg = (_rand((1, V), torch.float32, 13) * 3).repeat(rows, 1).contiguous()
    lg[0, 3] = lg[0, 11]          # equal logits inside the row
    lg = lg[0:1].repeat(rows, 1).contiguous()
    us = [(i + 0.37) / rows for i in range(rows)]
    ids, _ = _sample(lib, lg, us, t, k, p)
    kept, probs = P.sample_distribution(lg[0].cpu(), t, k, p)
    cdf = [0.0]
    for q in probs:
        cdf.append(cdf[-1] + q)
    for u, tok in zip(us, ids):
        assert tok in kept, f"token {tok} is outside the kept set"
        j = kept.index(tok)
        assert cdf[j] - 1e-4 <= u <= cdf[j + 1] + 1e-4, f"u = {u}: token {tok} covers [{cdf[j]}, {cdf[j + 1]}]"


# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 256, 256), (300, 688, 4096), (1000, 1376, 136), (77, 40, 688),
                                   (1024, 256, 64), (1100, 300, 520), (2500, 1376, 1000), (4096, 688, 136)])
def test_gemm_tc_dense(M, N, K):
    """The tcgen05 product against float64, bfloat16 and float outputs, with tails in M, N and K; from 1,024 rows
    on, two blocks share a tile (cta_group::2)."""
    lib = _lib()
    from transformer_b200.parts.linear import gemm_tc
    a, w = _rand((M, K), torch.bfloat16, 20), _rand((N, K), torch.bfloat16, 21, 0.1)
    ref = a.double() @ w.double().T
    for out_dtype, kind in ((torch.bfloat16, 0), (torch.float32, 1)):
        out = torch.full((M, N), 7.0, dtype=out_dtype, device="cuda")
        assert gemm_tc(a, w, out, out_kind=kind)
        assert lib.gemm_tc_status() == 0, "a wait inside the kernel gave up"
        assert float((out.double() - ref).abs().max()) <= _tol(out_dtype, float(ref.abs().max()))


@pytest.mark.parametrize("E,k,nt,d,di", [(4, 2, 300, 128, 96), (16, 4, 700, 256, 688), (3, 1, 130, 64, 200),
                                         (2, 2, 1300, 128, 176), (3, 2, 1700, 64, 80),       # these two: pairs of blocks
                                         (16, 4, 64, 256, 688), (5, 2, 20, 64, 440)])        # few rows: narrower tiles
def test_gemm_tc_grouped_swiglu_and_down(E, k, nt, d, di):
    """Experts through the prompt path: gather, grouped gate/up with swiglu, grouped down product."""
    lib = _lib()
    from transformer_b200.parts.linear import grouped_matmul
    import transformer_b200.parts.linear as L
    x, wgu, wd, idx = _grouped_case(torch.bfloat16, E, k, nt, d, di, seed=31 + E)
    M = nt * k
    off = torch.empty(E + 1, dtype=torch.int32, device="cuda")
    st = torch.empty(M, dtype=torch.int32, device="cuda")
    pr = torch.empty(M, dtype=torch.int32, device="cuda")
    lib.call("tb_moe_dispatch", idx.data_ptr(), off.data_ptr(), st.data_ptr(), pr.data_ptr(), M, k, E)
    bufs = {}
    scratch = lambda name, shape, dt: bufs.setdefault(name, torch.empty(shape, dtype=dt, device="cuda"))
    old = L.SKINNY_MAX_PAIRS
    L.SKINNY_MAX_PAIRS = 0          # force the prompt kernel whatever the size
    try:
        h = torch.empty((M, di), dtype=torch.bfloat16, device="cuda")
        y = torch.empty((M, d), dtype=torch.bfloat16, device="cuda")
        grouped_matmul(x, wgu, h, a_rows=st, group_offsets=off, groups=E, swiglu=True, scratch=scratch)
        grouped_matmul(h, wd, y, group_offsets=off, groups=E)
    finally:
        L.SKINNY_MAX_PAIRS = old
    assert "grouped.sorted_rows" in bufs, "the tensor-core path was taken"
    assert lib.gemm_tc_status() == 0
    prc = pr.cpu()
    xs, wg, wdd = x.double().cpu(), wgu.double().cpu(), wd.double().cpu()
    worst = 0.0
    for t in range(0, nt, max(1, nt // 40)):
        for j in range(k):
            e = int(idx[t, j])
            gu = wg[e] @ xs[t]
            href = P.silu(gu[:di]) * gu[di:]
            r = int(prc[t * k + j])
            assert float((h[r].double().cpu() - href).abs().max()) <= _tol(torch.bfloat16, float(href.abs().max()) + 1e-3)
            yref = wdd[e] @ h[r].double().cpu()
            worst = max(worst, float((y[r].double().cpu() - yref).abs().max()) / (float(yref.abs().max()) + 1e-6))
    assert worst <= 2.0 ** -7


@pytest.mark.parametrize("nh,nkvh,dh", [(4, 2, 64), (8, 8, 128), (6, 1, 128), (4, 2, 16), (3, 1, 48), (6, 3, 80), (4, 1, 96),
                                        (2, 2, 112), (2, 1, 144), (4, 2, 160), (2, 1, 192), (3, 3, 208), (2, 1, 240),
                                        (4, 2, 256)])
def test_attention_prompt_kernel(nh, nkvh, dh):
    """The tensor-core prompt kernel on a ragged batch: prompts from zero (shorter and longer than a
    tile, not multiples of 64), a continued prompt whose cache already holds 130 tokens, a single token; at head sizes
    from 16 to 256 (rows of shared memory padded to a multiple of 64 values)."""
    lib = _lib()
    dtype = torch.bfloat16
    tq = lib.attention_prefill_tile_tokens()
    c = attention_case([150, 1, 64, 37, 200], [0, 90, 0, 130, 64], nh, nkvh, dh, dtype, tq, seed=nh + dh)
    nt = c["nt"]
    out = torch.zeros(nt, nh * dh, dtype=dtype, device="cuda")
    assert lib.try_call("tb_attention_prefill_bf16", c["q"].data_ptr(), out.data_ptr(), c["kc"].data_ptr(),
                        c["vc"].data_ptr(), c["tile_seq"].data_ptr(), c["tile_t0"].data_ptr(), c["tile_nq"].data_ptr(),
                        c["tok_pos"].data_ptr(), c["table"].data_ptr(), c["tiles"], c["max_pages"], nh * dh, nh,
                        c["nkvh"], dh, 1.0 / math.sqrt(dh))
    got = out.double().cpu().reshape(nt, nh, dh)
    # P is rounded to bfloat16 before P.V: allow for that on top of the storage rounding
    assert float((got - c["ref"]).abs().max()) <= _tol(dtype, 4.0)
    # a head size it does not take is refused, not computed wrongly
    assert not lib.try_call("tb_attention_prefill_bf16", c["q"].data_ptr(), out.data_ptr(), c["kc"].data_ptr(),
                            c["vc"].data_ptr(), c["tile_seq"].data_ptr(), c["tile_t0"].data_ptr(),
                            c["tile_nq"].data_ptr(), c["tok_pos"].data_ptr(), c["table"].data_ptr(), c["tiles"],
                            c["max_pages"], nh * 40, nh, c["nkvh"], 40, 1.0)


@pytest.mark.parametrize("nh,nkvh,dh", [(4, 2, 64), (8, 8, 128), (6, 1, 128)])
def test_attention_tcgen05_kernel(nh, nkvh, dh):
    """The tcgen05 prompt kernel (S and O in tensor memory) on a ragged batch: prompts from zero, shorter and
    longer than its 128-token tile, a continued prompt over 130 cached tokens, a single token."""
    lib = _lib()
    dtype = torch.bfloat16
    tq = lib.attention_tc_tile_tokens()
    c = attention_case([150, 1, 64, 37, 300], [0, 90, 0, 130, 64], nh, nkvh, dh, dtype, tq, seed=nh + dh)
    nt = c["nt"]
    out = torch.zeros(nt, nh * dh, dtype=dtype, device="cuda")
    assert lib.try_call("tb_attention_tc_bf16", c["q"].data_ptr(), out.data_ptr(), c["kc"].data_ptr(),
                        c["vc"].data_ptr(), c["tile_seq"].data_ptr(), c["tile_t0"].data_ptr(), c["tile_nq"].data_ptr(),
                        c["tok_pos"].data_ptr(), c["table"].data_ptr(), c["tiles"], nt, c["max_pages"], nh * dh, nh,
                        c["nkvh"], dh, c["kc"].shape[0], 1.0 / math.sqrt(dh))
    assert lib.gemm_tc_status() == 0, "a wait inside the kernel gave up"
    got = out.double().cpu().reshape(nt, nh, dh)
    assert float((got - c["ref"]).abs().max()) <= _tol(dtype, 4.0)


@pytest.mark.parametrize("nh,nkvh,dh", [(4, 4, 64), (8, 8, 128), (12, 2, 64), (20, 2, 128), (3, 1, 128), (32, 8, 128),
                                        (16, 1, 64), (40, 2, 128), (51, 3, 64), (6, 2, 192), (3, 3, 256), (8, 2, 256)])
def test_attention_decode_on_tensor_cores(nh, nkvh, dh):
    """The decode kernel whose products run as mma.sync with a group's query heads as rows: groups of 1, 3, 4, 6, 10,
    exactly 16, 17 and 20 heads (more than 16 take two blocks); contexts of one token, exactly one page, a page and a
    bit, many pages; key slices that leave some slices empty; both ways of merging the slices."""
    lib = _lib()
    c = attention_case([1, 1, 1, 1, 1, 1], [0, 63, 64, 700, 129, 15], nh, nkvh, dh, torch.bfloat16, 1, seed=7 * nh + dh)
    for splits in (1, 2, 7):
        done = torch.zeros(6 * nh, dtype=torch.int32, device="cuda")
        for counters in (None, done, done):
            got = _run_attention(lib, c, torch.bfloat16, splits, decode=True, ring=True, done=counters)
            assert got is not None
            assert float((got - c["ref"]).abs().max()) <= _tol(torch.bfloat16, 4.0), f"splits {splits}"
            assert int(done.abs().sum()) == 0
    if (nh, nkvh, dh) == (12, 2, 64):
        pos = [(37 * i * i + 11 * i) % 900 for i in range(70)]
        big = attention_case([1] * 70, pos, 24, 4, 64, torch.bfloat16, 1, seed=78)
        done = torch.zeros(70 * 24, dtype=torch.int32, device="cuda")
        for splits in (1, 5):
            got = _run_attention(lib, big, torch.bfloat16, splits, decode=True, ring=True, done=done)
            assert float((got - big["ref"]).abs().max()) <= _tol(torch.bfloat16, 4.0), f"70 sequences, splits {splits}"
            assert int(done.abs().sum()) == 0 and lib.gemm_tc_status() == 0
    c48 = attention_case([1], [10], 2, 1, 48, torch.bfloat16, 1, seed=1)
    assert _run_attention(lib, c48, torch.bfloat16, 1, decode=True, ring=True) is None, "a head of 48 is refused"


@pytest.mark.parametrize("pairing", ["adjacent", "half"])
@pytest.mark.parametrize("nh,nkvh,dh", [(4, 4, 64), (8, 2, 128), (12, 2, 64), (40, 2, 128), (3, 1, 128), (6, 2, 192),
                                        (4, 1, 256)])
def test_decode_attention_that_also_rotates_and_writes_the_cache(nh, nkvh, dh, pairing):
    """The fused form against the two kernels it stands for (rotary kernel, then the attention over the finished
    cache), from the same unrotated q-k-v rows: the same output, the same cache rows written, q-k-v left alone; with
    the new rows poisoned in the cache beforehand, so that a kernel that read them from there would show; and against
    float64 attention over the cache that the rotary kernel left.  Then for a layer that reads another layer's cache
    (nothing to write: only the queries are rotated)."""
    lib = _lib()
    dtype = torch.bfloat16
    pos = [0, 63, 64, 700, 129, 15]
    c = attention_case([1] * len(pos), pos, nh, nkvh, dh, dtype, 1, seed=11 * nh + dh)
    nt, width = c["nt"], (nh + 2 * nkvh) * dh
    qkv = _rand((nt, width), dtype, 21)
    theta = 10000.0
    i = torch.arange(dh // 2, dtype=torch.float64)
    ang = torch.arange(1024, dtype=torch.float64)[:, None] * theta ** (-2.0 * i / dh)[None]
    cos, sin = torch.cos(ang).float().cuda(), torch.sin(ang).float().cuda()
    half = 1 if pairing == "half" else 0
    seq = torch.repeat_interleave(c["tile_seq"], c["tile_nq"])
    scale = 1.0 / math.sqrt(dh)
    # the two kernels
    qkv_a, kc_a, vc_a = qkv.clone(), c["kc"].clone(), c["vc"].clone()
    lib.call("tb_rope_cache_bf16", qkv_a.data_ptr(), seq.data_ptr(), c["tok_pos"].data_ptr(), c["table"].data_ptr(),
             c["max_pages"], cos.data_ptr(), sin.data_ptr(), kc_a.data_ptr(), vc_a.data_ptr(), nt, nh, nkvh, dh, half)
    # float64 attention over that cache
    ref = torch.zeros(nt, nh, dh, dtype=torch.float64)
    table = c["table"].cpu()
    q_rot = qkv_a[:, :nh * dh].double().cpu().reshape(nt, nh, dh)
    for t in range(nt):
        n = pos[t] + 1
        pages = table[t, :(n + 63) // 64].long()
        k = kc_a[pages.cuda()].double().cpu().permute(1, 0, 2, 3).reshape(nkvh, -1, dh)[:, :n]
        v = vc_a[pages.cuda()].double().cpu().permute(1, 0, 2, 3).reshape(nkvh, -1, dh)[:, :n]
        for h in range(nh):
            g = h // (nh // nkvh)
            ref[t, h] = torch.softmax(k[g] @ q_rot[t, h] * scale, 0) @ v[g]
    poison_k, poison_v = c["kc"].clone(), c["vc"].clone()
    for t in range(nt):
        page = int(table[t, pos[t] // 64])
        poison_k[page, :, pos[t] % 64] = 300.0
        poison_v[page, :, pos[t] % 64] = -300.0
    for splits in (1, 2, 7):
        partial = torch.empty(nt * nh * splits * (dh + 2), dtype=torch.float32, device="cuda")
        done = torch.zeros(nt * nh, dtype=torch.int32, device="cuda")
        out_a = torch.zeros(nt, nh * dh, dtype=dtype, device="cuda")
        lib.call("tb_attention_decode_mma_bf16", qkv_a.data_ptr(), out_a.data_ptr(), kc_a.data_ptr(), vc_a.data_ptr(),
                 seq.data_ptr(), c["tok_pos"].data_ptr(), c["table"].data_ptr(), partial.data_ptr(), done.data_ptr(), nt,
                 c["max_pages"], width, nh, nkvh, dh, splits, kc_a.shape[0], scale)
        for write in (1, 0):
            qkv_b = qkv.clone()
            kc_b, vc_b = (poison_k.clone(), poison_v.clone()) if write else (kc_a.clone(), vc_a.clone())
            out_b = torch.zeros_like(out_a)
            lib.call("tb_attention_decode_rope_bf16", qkv_b.data_ptr(), out_b.data_ptr(), kc_b.data_ptr(), vc_b.data_ptr(),
                     seq.data_ptr(), c["tok_pos"].data_ptr(), c["table"].data_ptr(), partial.data_ptr(), done.data_ptr(),
                     cos.data_ptr(), sin.data_ptr(), nt, c["max_pages"], width, nh, nkvh, dh, splits, kc_b.shape[0], half,
                     write, scale)
            assert lib.gemm_tc_status() == 0 and int(done.abs().sum()) == 0
            assert torch.equal(qkv_b, qkv), "the q-k-v rows are read, not rotated in place"
            assert torch.equal(vc_b, vc_a), "the value rows written are the rotary kernel's"
            # the rotated key: the same arithmetic in another kernel, at most the last bit of a bfloat16 apart
            dk = (kc_b.float() - kc_a.float()).abs()
            assert float((dk / kc_a.float().abs().clamp_min(1e-3)).max()) <= 2.0 ** -7, "key rows written"
            got = out_b.double().cpu().reshape(nt, nh, dh)
            assert float((got - ref).abs().max()) <= _tol(dtype, 4.0), f"splits {splits}, write {write}"
            assert float((out_b.float() - out_a.float()).abs().max()) <= _tol(dtype, 1.0), "against the two kernels"


def test_decode_on_tensor_cores_finds_one_far_key():
    """Among 1,500 keys one (position 3, in the first page of the first slice, held by the first warp) is scaled so
    that it takes nearly all the weight of every head; then one at the context's very end (the newest key, the last
    row a warp reads before the mask).  A page, a warp's share of a page or a slice that was lost shows at once."""
    lib = _lib()
    for where in (3, 1499, 1087):
        c = attention_case([1, 1], [1499, 1499], 12, 2, 128, torch.bfloat16, 1, seed=40 + where, scale_key=(0, where, 6.0))
        for splits in (1, 4, 11):
            done = torch.zeros(2 * 12, dtype=torch.int32, device="cuda")
            got = _run_attention(lib, c, torch.bfloat16, splits, decode=True, ring=True, done=done)
            assert float((got - c["ref"]).abs().max()) <= _tol(torch.bfloat16, 4.0), f"key {where}, splits {splits}"


# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
def test_random_fill_is_the_rule_bit_for_bit(dtype):
    """The fill kernel against the tests' own restatement of the rule (plain/counter_weights.py), at sizes with
    tails, at an odd offset into the stream, into a tensor that does not start on a 16-byte boundary."""
    from plain import counter_weights as C
    from transformer_b200.weights import counter_random as R
    lib = _lib()
    for seed, name, n, first, std in ((0, "token_embd.weight", 1, 0, 0.02), (3, "blk.1.attn_qkv.weight", 8 * 257 + 5, 0, 0.02),
                                      (2 ** 33 + 1, "output.weight", 100003, 77, 1.0), (9, "x", 4096, 2 ** 33 + 3, 0.5)):
        buf = torch.full((n + 3,), 7.0, dtype=dtype, device="cuda")
        out = buf[1:1 + n]                                   # misaligned for 16-byte stores: the scalar path
        lib.call("tb_random_fill_" + lib.suffix(dtype), out.data_ptr(), n, R.stream_base(seed, name), first,
                 float(R.scale_for(std)))
        want = C.values(seed, name, (n,), std, dtype=dtype, first=first)
        assert torch.equal(out.float().cpu(), want), (seed, name, n)
        assert float(buf[0]) == 7.0 and float(buf[n + 1]) == 7.0, "wrote outside its range"
        whole = torch.empty(n, dtype=dtype, device="cuda")
        lib.random_fill(whole, R.stream_base(seed, name), float(R.scale_for(std)), first)
        assert torch.equal(whole.float().cpu(), want)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_weights_drawn_on_the_device_are_the_folders(dtype, tmp_path):
    import transformer_b200 as tb
    from tiny import CONFIGS
    cfg, seed = CONFIGS["B"]
    on_device = tb.random_model(cfg, seed=seed, dtype=dtype, std=0.1, max_tokens=64)
    from_file = tb.load(tb.write_random_model(str(tmp_path / "m"), cfg, seed=seed, dtype=dtype, std=0.1), dtype=dtype,
                        max_tokens=64)
    assert torch.equal(on_device.embedding, from_file.embedding) and torch.equal(on_device.head, from_file.head)
    assert on_device.head.data_ptr() == on_device.embedding.data_ptr(), "a tied head shares the table's storage"
    for a, b in zip(on_device.layers, from_file.layers):
        for name, part in a.parts().items():
            for wname, w in part.weights.items():
                assert torch.equal(w, b.parts()[name].weights[wname]), (name, wname)


# ---------------------------------------------------------------------------------------------
def test_attention_over_a_long_context():
    """Twelve thousand cached tokens (188 scrambled pages), bfloat16, heads of 128: the tcgen05 and the mma.sync prompt
    kernels continue a prompt by 300 tokens, the page-ring and the register-staged decode kernels take one token with
    the keys cut into 1, 8 and 32 slices.  One early key (position 7) is scaled up so that a lost first page or slice
    would show in every row."""
    lib = _lib()
    nh, nkvh, dh, dtype = 4, 2, 128, torch.bfloat16
    scale = 1.0 / math.sqrt(dh)
    # prompts: a long continuation, and a short sequence beside it
    tq = lib.attention_tc_tile_tokens()
    c = attention_case([300, 70], [11700, 0], nh, nkvh, dh, dtype, tq, seed=91, scale_key=(0, 7, 3.0))
    nt = c["nt"]
    out = torch.zeros(nt, nh * dh, dtype=dtype, device="cuda")
    assert lib.try_call("tb_attention_tc_bf16", c["q"].data_ptr(), out.data_ptr(), c["kc"].data_ptr(), c["vc"].data_ptr(),
                        c["tile_seq"].data_ptr(), c["tile_t0"].data_ptr(), c["tile_nq"].data_ptr(), c["tok_pos"].data_ptr(),
                        c["table"].data_ptr(), c["tiles"], nt, c["max_pages"], nh * dh, nh, nkvh, dh, c["kc"].shape[0],
                        scale)
    assert lib.gemm_tc_status() == 0
    assert float((out.double().cpu().reshape(nt, nh, dh) - c["ref"]).abs().max()) <= _tol(dtype, 4.0), "tcgen05 prompt kernel"
    tq2 = lib.attention_prefill_tile_tokens()
    c2 = attention_case([300, 70], [11700, 0], nh, nkvh, dh, dtype, tq2, seed=91, scale_key=(0, 7, 3.0))
    out.zero_()
    assert lib.try_call("tb_attention_prefill_bf16", c2["q"].data_ptr(), out.data_ptr(), c2["kc"].data_ptr(),
                        c2["vc"].data_ptr(), c2["tile_seq"].data_ptr(), c2["tile_t0"].data_ptr(), c2["tile_nq"].data_ptr(),
                        c2["tok_pos"].data_ptr(), c2["table"].data_ptr(), c2["tiles"], c2["max_pages"], nh * dh, nh,
                        nkvh, dh, scale)
    assert float((out.double().cpu().reshape(nt, nh, dh) - c2["ref"]).abs().max()) <= _tol(dtype, 4.0), "mma.sync prompt kernel"
    # decoding: three sequences of 12,001, 8,192 and 4,096 tokens
    d = attention_case([1, 1, 1], [12000, 8191, 4095], nh, nkvh, dh, dtype, 1, seed=92, scale_key=(0, 7, 3.0))
    for splits in (1, 8, 32):
        done = torch.zeros(3 * nh, dtype=torch.int32, device="cuda")
        for ring, counters in ((True, done), (True, None), (False, None)):
            got = _run_attention(lib, d, dtype, splits, decode=True, ring=ring, done=counters)
            assert got is not None
            assert float((got - d["ref"]).abs().max()) <= _tol(dtype, 4.0), f"decode, splits {splits}, ring {ring}"
        assert int(done.abs().sum()) == 0
