"""Each kernel alone against a plain PyTorch float32/float64 statement of the same op, at
sizes other than the engine's tiny models: odd widths, head sizes 16..256, groups, windows,
rings, chunked keys."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return 2e-5 if dtype == torch.float32 else 2e-2


def close(got, want, dtype, scale=None):
    got, want = got.double().cpu(), want.double().cpu()
    s = float(want.abs().max()) if scale is None else scale
    err = float((got - want).abs().max()) / max(s, 1e-30)
    assert err < tol(dtype), err


def status():
    return torch.zeros(1, dtype=torch.int32, device="cuda")


def test_embed_and_bad_token_flag():
    from minfer_b200.kernels import api as K
    for dt in DTYPES:
        table = torch.randn(131, 72).to(dt).cuda()
        ids = torch.tensor([0, 130, 5, 5, 77], dtype=torch.int32, device="cuda")
        out = torch.empty(5, 72, device="cuda")
        st = status()
        K.embed(table, ids, out, st)
        assert torch.equal(out, table.float()[ids.long()]) and int(st) == 0
        K.embed(table, ids, out, st, scale=2.5)
        assert torch.equal(out, table.float()[ids.long()] * 2.5) and int(st) == 0
    bad = torch.tensor([3, 131], dtype=torch.int32, device="cuda")
    out = torch.full((2, 72), 9.0, device="cuda")
    K.embed(table, bad, out, st)
    assert int(st) & 1 and float(out[1].abs().sum()) == 0.0


@pytest.mark.parametrize("width", [64, 200, 3584, 5000])
def test_rmsnorm(width):
    from minfer_b200.kernels import api as K
    x = (torch.randn(7, width) * 3).cuda()
    w = (1 + 0.1 * torch.randn(width)).cuda()
    want = x.double() / torch.sqrt((x.double() ** 2).mean(-1, keepdim=True) + 1e-5) * w.double()
    for dt in DTYPES:
        out = torch.empty(7, width, dtype=dt, device="cuda")
        K.rmsnorm(x, w, 1e-5, out)
        close(out, want, dt)
    rows = torch.tensor([6, 0, 3], dtype=torch.int32, device="cuda")
    out = torch.empty(3, width, device="cuda")
    K.rmsnorm(x, w, 1e-5, out, rows)
    close(out, want[[6, 0, 3]], torch.float32)


@pytest.mark.parametrize("m,n,k", [(1, 1, 16), (5, 130, 72), (64, 64, 64), (65, 67, 200),
                                   (130, 389, 328), (3, 1000, 1031)])
def test_gemm_simt_all_precisions(m, n, k):
    from minfer_b200.kernels import api as K
    g = torch.Generator().manual_seed(m * 1000 + n)
    a32, w32 = torch.randn(m, k, generator=g), torch.randn(n, k, generator=g)
    bias = torch.randn(n, generator=g).cuda()
    for ta in DTYPES:
        for tw in DTYPES:
            a, w = a32.to(ta).cuda(), w32.to(tw).cuda()
            want = a.double() @ w.double().t() + bias.double()
            for tc in DTYPES:
                out = torch.empty(m, n, dtype=tc, device="cuda")
                K.gemm_simt(a, w, bias, out)
                close(out, want, tc if tc == torch.bfloat16 else torch.float32)
            acc = torch.randn(m, n, generator=g).cuda()
            before = acc.clone()
            K.gemm_simt(a, w, None, acc, accumulate=True)
            close(acc, before.double() + a.double() @ w.double().t(), torch.float32)


def test_gemm_rows_do_not_depend_on_the_batch():
    """A row's result is bit-identical whether it is multiplied alone or among others."""
    from minfer_b200.kernels import api as K
    a = torch.randn(70, 200).cuda()
    w = torch.randn(90, 200).cuda()
    whole = torch.empty(70, 90, device="cuda")
    K.gemm_simt(a, w, None, whole)
    for r in (0, 33, 69):
        one = torch.empty(1, 90, device="cuda")
        K.gemm_simt(a[r:r + 1].contiguous(), w, None, one)
        assert torch.equal(one[0], whole[r])


def rope_reference(x, pos, inv_freq, rotary_dim, style):
    """x [T, H, hd] float64."""
    out = x.clone()
    ang = pos.double()[:, None] * inv_freq.double()[None, :]
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    h = rotary_dim // 2
    if style == 0:
        a, b = x[..., :h], x[..., h:rotary_dim]
        out[..., :h], out[..., h:rotary_dim] = a * cos - b * sin, a * sin + b * cos
    else:
        a, b = x[..., 0:rotary_dim:2], x[..., 1:rotary_dim:2]
        out[..., 0:rotary_dim:2], out[..., 1:rotary_dim:2] = a * cos - b * sin, a * sin + b * cos
    return out


@pytest.mark.parametrize("hd,rotary_dim,style", [(16, 16, 0), (48, 48, 0), (64, 32, 0),
                                                 (128, 128, 1), (32, 16, 1), (256, 256, 0)])
def test_rope_kvstore_pages_and_rotation(hd, rotary_dim, style):
    from minfer_b200.kernels import api as K
    nh, nk = 3, 2
    # two sequences: row 0 holds positions 100..104 (5 tokens), row 1 position 63 and 64
    positions = torch.tensor([100, 101, 102, 103, 104, 63, 64], dtype=torch.int32)
    rows = torch.tensor([0, 0, 0, 0, 0, 1, 1], dtype=torch.int32)
    T = 7
    qkv = torch.randn(T, (nh + 2 * nk) * hd)
    inv_freq = 1.0 / (10000.0 ** (torch.arange(rotary_dim // 2).double() * 2 / rotary_dim))
    n_pages = 6
    table = torch.tensor([[4, 2, -1], [5, 0, -1]], dtype=torch.int32)   # logical page -> physical
    for dt in DTYPES:
        kc = torch.zeros(n_pages, nk, 64, hd, dtype=dt, device="cuda")
        vc = torch.zeros_like(kc)
        q = torch.empty(T, nh, hd, dtype=dt, device="cuda")
        ks = torch.empty(T, nk, hd, dtype=dt, device="cuda")
        vs = torch.empty_like(ks)
        st = status()
        K.rope_kvstore(qkv.cuda(), positions.cuda(), rows.cuda(),
                       torch.tensor([105, 65], dtype=torch.int32, device="cuda"), inv_freq.cuda(),
                       q, ks, vs, kc, vc, table.cuda(), 3, 0, nh, nk, hd, rotary_dim, style, st)
        x = qkv.double().reshape(T, nh + 2 * nk, hd)
        want_q = rope_reference(x[:, :nh], positions, inv_freq, rotary_dim, style)
        want_k = rope_reference(x[:, nh:nh + nk], positions, inv_freq, rotary_dim, style)
        want_v = x[:, nh + nk:]
        close(q, want_q, dt); close(ks, want_k, dt); close(vs, want_v, dt)
        assert int(st) == 0
        for t in range(T):
            p, b = int(positions[t]), int(rows[t])
            page = int(table[b, p // 64])
            assert torch.equal(kc[page, :, p % 64, :], ks[t]) and torch.equal(vc[page, :, p % 64, :], vs[t])
        written = {(int(table[int(rows[t]), int(positions[t]) // 64]), int(positions[t]) % 64)
                   for t in range(T)}
        mask = torch.ones(n_pages, 64, dtype=torch.bool)
        for pg, off in written:
            mask[pg, off] = False
        untouched = kc.float().cpu().permute(0, 2, 1, 3)[mask]          # [page, offset] pairs
        assert float(untouched.abs().sum()) == 0.0                       # nothing else was touched


def test_rope_kvstore_ring_keeps_only_the_tail_and_flags_missing_pages():
    from minfer_b200.kernels import api as K
    nh, nk, hd, T = 1, 1, 16, 150
    qkv = torch.randn(T, 3 * hd).cuda()
    positions = torch.arange(T, dtype=torch.int32, device="cuda")
    rows = torch.zeros(T, dtype=torch.int32, device="cuda")
    kc = torch.zeros(2, nk, 64, hd, device="cuda"); vc = torch.zeros_like(kc)
    q = torch.empty(T, nh, hd, device="cuda")
    ks = torch.empty(T, nk, hd, device="cuda"); vs = torch.empty_like(ks)
    st = status()
    table = torch.tensor([[1, 0]], dtype=torch.int32, device="cuda")
    K.rope_kvstore(qkv, positions, rows, torch.tensor([T], dtype=torch.int32, device="cuda"), None,
                   q, ks, vs, kc, vc, table, 2, 128, nh, nk, hd, 0, 0, st)
    assert int(st) == 0
    for p in range(T - 128, T):                     # the last 128 positions, at p % 128
        page = int(table[0, (p % 128) // 64])
        assert torch.equal(vc[page, 0, p % 64], vs[p, 0])
    assert torch.equal(ks, qkv[:, hd:2 * hd].reshape(T, 1, hd))       # no rotation asked for
    bad = torch.tensor([[1, -1]], dtype=torch.int32, device="cuda")
    K.rope_kvstore(qkv, positions, rows, torch.tensor([T], dtype=torch.int32, device="cuda"), None,
                   q, ks, vs, kc, vc, bad, 2, 128, nh, nk, hd, 0, 0, st)
    assert int(st) & 2


def attention_reference(q, k, v, scale, window):
    """q [T, nh, hd], k/v [T, nk, hd] of one sequence, float64."""
    T, nh, hd = q.shape
    g = nh // k.shape[1]
    out = torch.zeros_like(q)
    idx = torch.arange(T)
    mask = idx[None, :] <= idx[:, None]
    if window > 0:
        mask &= (idx[:, None] - idx[None, :]) < window
    for h in range(nh):
        s = (q[:, h] @ k[:, h // g].t()) * scale
        s = s.masked_fill(~mask, -math.inf)
        out[:, h] = torch.softmax(s, dim=-1) @ v[:, h // g]
    return out


@pytest.mark.parametrize("hd,nh,nk,window", [(16, 4, 1, 0), (32, 6, 2, 16), (48, 3, 3, 70),
                                             (64, 14, 2, 0), (128, 7, 1, 33), (256, 2, 2, 0),
                                             (80, 5, 5, 0), (112, 9, 3, 50), (128, 34, 2, 0)])
def test_attention_packed_unequal_sequences(hd, nh, nk, window):
    from minfer_b200.kernels import api as K
    lens = [37, 1, 100, 65]
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    T = cu[-1]
    g = torch.Generator().manual_seed(hd + nh)
    q32, k32, v32 = (torch.randn(T, h, hd, generator=g) for h in (nh, nk, nk))
    row_seq = torch.cat([torch.full((n,), b, dtype=torch.int32) for b, n in enumerate(lens)])
    row_pos = torch.cat([torch.arange(n, dtype=torch.int32) for n in lens])
    scale = 1.0 / math.sqrt(hd)
    for dt in DTYPES:
        q, k, v = q32.to(dt).cuda(), k32.to(dt).cuda(), v32.to(dt).cuda()
        out = torch.empty(T, nh * hd, dtype=dt, device="cuda")
        K.attention_packed(q, k, v, row_seq.cuda(), row_pos.cuda(),
                           torch.tensor(cu, dtype=torch.int32, device="cuda"), out, nh, nk, hd,
                           window, scale)
        for b, n in enumerate(lens):
            sl = slice(cu[b], cu[b + 1])
            want = attention_reference(q[sl].double().cpu(), k[sl].double().cpu(),
                                       v[sl].double().cpu(), scale, window)
            close(out[sl].reshape(n, nh, hd), want, dt, scale=float(v32.abs().max()))


def test_attention_finds_a_far_key_among_hundreds():
    """One key far back gets a score that stands out; the output must be its value."""
    from minfer_b200.kernels import api as K
    T, hd = 700, 64
    q = torch.randn(T, 1, hd) * 0.1
    k = torch.randn(T, 1, hd) * 0.1
    v = torch.randn(T, 1, hd)
    k[13, 0] = 0.0; k[13, 0, 5] = 40.0
    q[T - 1, 0] = 0.0; q[T - 1, 0, 5] = 40.0            # score 1600 * scale at key 13
    out = torch.empty(T, hd, device="cuda")
    K.attention_packed(q.cuda(), k.cuda(), v.cuda(), torch.zeros(T, dtype=torch.int32, device="cuda"),
                       torch.arange(T, dtype=torch.int32, device="cuda"),
                       torch.tensor([0, T], dtype=torch.int32, device="cuda"), out, 1, 1, hd, 0, 0.125)
    assert torch.allclose(out[T - 1].cpu(), v[13, 0], atol=1e-5)
    # with a window that ends before key 13 it must NOT be seen
    K.attention_packed(q.cuda(), k.cuda(), v.cuda(), torch.zeros(T, dtype=torch.int32, device="cuda"),
                       torch.arange(T, dtype=torch.int32, device="cuda"),
                       torch.tensor([0, T], dtype=torch.int32, device="cuda"), out, 1, 1, hd,
                       T - 1 - 13, 0.125)
    assert not torch.allclose(out[T - 1].cpu(), v[13, 0], atol=1e-2)
    K.attention_packed(q.cuda(), k.cuda(), v.cuda(), torch.zeros(T, dtype=torch.int32, device="cuda"),
                       torch.arange(T, dtype=torch.int32, device="cuda"),
                       torch.tensor([0, T], dtype=torch.int32, device="cuda"), out, 1, 1, hd,
                       T - 13, 0.125)                   # the window's edge: key 13 is the oldest seen
    assert torch.allclose(out[T - 1].cpu(), v[13, 0], atol=1e-5)


@pytest.mark.parametrize("hd,nh,nk,window,ring", [(16, 4, 1, 0, 0), (32, 6, 2, 16, 64),
                                                  (48, 3, 3, 70, 128), (128, 28, 4, 0, 0),
                                                  (64, 2, 1, 100, 0), (96, 6, 3, 0, 0),
                                                  (128, 34, 2, 0, 0), (240, 3, 1, 0, 0)])
def test_attention_paged_matches_packed_history(hd, nh, nk, window, ring):
    """Queries at the ends of sequences of unequal lengths over a scattered paged cache."""
    from minfer_b200.kernels import api as K
    lens = [600, 1, 64, 65, 300]
    B = len(lens)
    n_pages = 40
    g = torch.Generator().manual_seed(7)
    perm = torch.randperm(n_pages, generator=g).tolist()
    scale = 1.0 / math.sqrt(hd)
    for dt in DTYPES:
        kc = torch.randn(n_pages, nk, 64, hd, generator=g).to(dt).cuda()   # stale values everywhere
        vc = torch.randn(n_pages, nk, 64, hd, generator=g).to(dt).cuda()
        width = 10
        table = torch.full((B, width), -1, dtype=torch.int32)
        hist_k, hist_v = [], []
        for b, n in enumerate(lens):
            kk = torch.randn(n, nk, hd, generator=g).to(dt)
            vv = torch.randn(n, nk, hd, generator=g).to(dt)
            hist_k.append(kk); hist_v.append(vv)
            lo = max(0, n - ring) if ring else 0
            for p in range(lo, n):
                pe = p % ring if ring else p
                lp = pe // 64
                if table[b, lp] < 0:
                    table[b, lp] = perm.pop()
                kc[table[b, lp], :, p % 64] = kk[p].cuda()
                vc[table[b, lp], :, p % 64] = vv[p].cuda()
        q32 = torch.randn(B, nh, hd, generator=g)
        q = q32.to(dt).cuda()
        row_seq = torch.arange(B, dtype=torch.int32, device="cuda")
        row_pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device="cuda")
        for chunk, n_chunks in ((256, 3), (64, 10), (1024, 1)):
            out = torch.empty(B, nh * hd, dtype=dt, device="cuda")
            partial = torch.empty(B * nh * n_chunks * (hd + 2), device="cuda")
            K.attention_paged(q, kc, vc, row_seq, row_pos, table.cuda(), width, ring, out, partial,
                              nh, nk, hd, window, chunk, n_chunks, scale)
            for b, n in enumerate(lens):
                qq = torch.zeros(n, nh, hd, dtype=torch.float64)
                qq[n - 1] = q[b].double().cpu()
                want = attention_reference(qq, hist_k[b].double(), hist_v[b].double(), scale, window)
                close(out[b].reshape(nh, hd), want[n - 1], dt, scale=3.0)


def test_swiglu_gather_cast():
    from minfer_b200.kernels import api as K
    gu = torch.randn(5, 2 * 328).cuda()
    want = torch.nn.functional.silu(gu[:, :328].double()) * gu[:, 328:].double()
    for dt in DTYPES:
        out = torch.empty(5, 328, dtype=dt, device="cuda")
        K.swiglu(gu, out)
        close(out, want, dt)
    out = torch.empty(5, 328, dtype=torch.bfloat16, device="cuda")
    K.swiglu(gu.bfloat16(), out)
    close(out, torch.nn.functional.silu(gu.bfloat16()[:, :328].double()) * gu.bfloat16()[:, 328:].double(),
          torch.bfloat16)
    il = torch.stack([gu[:, :328], gu[:, 328:]], dim=2).reshape(5, 656).contiguous()
    out = torch.empty(5, 328, device="cuda")
    K.swiglu(il, out, interleaved=True)
    close(out, want, torch.float32)
    x = torch.randn(9, 100).cuda()
    rows = torch.tensor([8, 8, 0, 3], dtype=torch.int32, device="cuda")
    picked = torch.empty(4, 100, device="cuda")
    K.gather_rows(x, rows, picked)
    assert torch.equal(picked, x[rows.long()])
    b = torch.empty(9, 100, dtype=torch.bfloat16, device="cuda")
    K.cast(x, b)
    assert torch.equal(b, x.bfloat16())
    back = torch.empty(9, 100, device="cuda")
    K.cast(b, back)
    assert torch.equal(back, b.float())


def test_unsupported_sizes_are_refused_not_miscomputed():
    from minfer_b200.kernels import api as K
    q = torch.zeros(1, 1, 24, device="cuda")
    with pytest.raises(K.KernelError, match="does not take"):
        K.attention_packed(q, q, q, torch.zeros(1, dtype=torch.int32, device="cuda"),
                           torch.zeros(1, dtype=torch.int32, device="cuda"),
                           torch.tensor([0, 1], dtype=torch.int32, device="cuda"),
                           torch.zeros(1, 24, device="cuda"), 1, 1, 24, 0, 1.0)
    with pytest.raises(K.KernelError, match="CUDA device"):
        K.rmsnorm(torch.zeros(1, 8), torch.zeros(8), 1e-6, torch.zeros(1, 8))
    from minfer_b200.parts.attention import Attention
    with pytest.raises(ValueError, match="multiples of 16"):
        Attention(hidden_size=40, n_heads=2, n_kv_heads=1, head_dim=20, scale=1.0)


@pytest.mark.parametrize("m,n,k", [(1, 128, 64), (8, 256, 128), (5, 130, 72), (16, 389, 328),
                                   (33, 640, 200), (64, 512, 1024), (100, 384, 512),
                                   (300, 640, 3584), (8, 3584, 3584), (700, 1000, 264),
                                   (2048, 3584, 128), (2048, 4608, 64), (16576, 256, 64),
                                   (14208, 256, 72), (64, 896, 896), (8, 1152, 896),
                                   (40, 896, 4864)])
def test_gemm_tensor_core_against_float64(m, n, k):
    """The tcgen05 kernels at every token tile (16..128 for one CTA; 160, 192, 208, 224 and 256
    for the CTA pair: the last four sizes each pick another one), with and without K splits,
    ragged edges in all three dimensions, every epilogue.  The last three are small weights,
    which are cut along K until a CTA has two k-blocks (7 splits; 16 with a short last one)."""
    from minfer_b200.kernels import api as K
    g = torch.Generator().manual_seed(m + n + k)
    x = (torch.randn(m, k, generator=g) * 0.5).bfloat16().cuda()
    w = (torch.randn(n, k, generator=g) * 0.5).bfloat16().cuda()
    bias = torch.randn(n, generator=g).cuda()
    st = status()
    want = x.double() @ w.double().t()
    out = torch.zeros(m, n, device="cuda")
    K.gemm_tc(x, w, bias, out, K.EPI_STORE, st)
    close(out, want + bias.double(), torch.float32)
    outb = torch.zeros(m, n, dtype=torch.bfloat16, device="cuda")
    K.gemm_tc(x, w, None, outb, K.EPI_STORE, st)
    close(outb, want, torch.bfloat16)
    acc = torch.randn(m, n, generator=g).cuda()
    before = acc.clone()
    K.gemm_tc(x, w, None, acc, K.EPI_ACCUM, st)
    close(acc, before.double() + want, torch.float32)
    if n % 2 == 0:
        act = torch.zeros(m, n // 2, dtype=torch.bfloat16, device="cuda")
        K.gemm_tc(x, w, None, act, K.EPI_SWIGLU, st)
        close(act, torch.nn.functional.silu(want[:, 0::2]) * want[:, 1::2], torch.bfloat16)
    assert int(st) == 0
    # run twice: the same bits (splits are added in a fixed order)
    again = torch.zeros(m, n, device="cuda")
    K.gemm_tc(x, w, bias, again, K.EPI_STORE, st)
    assert torch.equal(again, out)


@pytest.mark.parametrize("m,n,k", [(300, 640, 328), (2048, 512, 200), (777, 1000, 520),
                                   (256, 256, 64), (1300, 768, 1024), (3000, 300, 136)])
def test_gemm_pair_kernel_two_token_tiles_at_once(m, n, k):
    """The CTA-pair kernel with two token tiles a pair (forced on: the cost model picks it only
    for long K): one token tile alone, a second one with a few tokens, an odd number of token
    tiles, ragged edges, every epilogue.  Against float64, and bit for bit against the form
    with one token tile a pair."""
    from minfer_b200.kernels import api as K
    g = torch.Generator().manual_seed(m * 3 + n + k)
    x = (torch.randn(m, k, generator=g) * 0.5).bfloat16().cuda()
    w = (torch.randn(n, k, generator=g) * 0.5).bfloat16().cuda()
    bias = torch.randn(n, generator=g).cuda()
    start = torch.randn(m, n, generator=g).cuda()
    st = status()
    want = x.double() @ w.double().t()
    results = {}
    try:
        for mode in (2, 0):
            K.gemm_pair_dual_mode(mode)
            assert K.gemm_pair_plan(m, n, k)[1] == (mode == 2)
            out = torch.zeros(m, n, device="cuda")
            K.gemm_tc(x, w, bias, out, K.EPI_STORE, st)
            acc = start.clone()
            K.gemm_tc(x, w, None, acc, K.EPI_ACCUM, st)
            accb = start.clone()
            K.gemm_tc(x, w, bias, accb, K.EPI_ACCUM, st)
            act = torch.zeros(m, n // 2, dtype=torch.bfloat16, device="cuda")
            K.gemm_tc(x, w, None, act, K.EPI_SWIGLU, st)
            results[mode] = (out, acc, accb, act)
    finally:
        K.gemm_pair_dual_mode(1)
    out, acc, accb, act = results[2]
    close(out, want + bias.double(), torch.float32)
    close(acc, start.double() + want, torch.float32)
    close(accb, start.double() + want + bias.double(), torch.float32)
    close(act, torch.nn.functional.silu(want[:, 0::2]) * want[:, 1::2], torch.bfloat16)
    for a, b in zip(results[2], results[0]):
        assert torch.equal(a, b)
    assert int(st) == 0


@pytest.mark.parametrize("m,n,k", [(3000, 600, 136), (5000, 300, 72)])
def test_gemm_pair_kernel_walks_the_tiles_in_groups(m, n, k):
    """The CTA-pair kernel takes the token tiles in groups (within a group the weight tiles
    change slowest), so that prompts of many thousand tokens do not fetch every token row once
    per weight tile.  Every group width, a last group that is narrower, one and two token
    tiles a pair: the same bits as the ungrouped order, and right against float64."""
    from minfer_b200.kernels import api as K
    g = torch.Generator().manual_seed(m + n + k)
    x = (torch.randn(m, k, generator=g) * 0.5).bfloat16().cuda()
    w = (torch.randn(n, k, generator=g) * 0.5).bfloat16().cuda()
    start = torch.randn(m, n, generator=g).cuda()
    st = status()
    want = start.double() + x.double() @ w.double().t()
    try:
        for dual in (0, 2):
            K.gemm_pair_dual_mode(dual)
            K.gemm_pair_group_m(1 << 20)                   # one group: all token tiles side by side
            base = start.clone()
            K.gemm_tc(x, w, None, base, K.EPI_ACCUM, st)
            close(base, want, torch.float32)
            for group in (0, 1, 3, 5, 7):
                K.gemm_pair_group_m(group)
                acc = start.clone()
                K.gemm_tc(x, w, None, acc, K.EPI_ACCUM, st)
                assert torch.equal(acc, base), (dual, group)
    finally:
        K.gemm_pair_dual_mode(1)
        K.gemm_pair_group_m(0)
    assert int(st) == 0


def test_gemm_pair_plan_takes_two_token_tiles_for_a_long_k():
    """The cost model's choices at the sizes it was measured on: the down projection of a
    2,048-token prompt (K 18,944, 14 weight tiles) takes two token tiles a pair, the gate|up
    projection (16 rounds of tiles, whose epilogues hide behind the next tile) does not, and
    neither does a product with fewer tiles than pairs."""
    from minfer_b200.kernels import api as K
    K.gemm_pair_dual_mode(1)
    assert K.gemm_pair_plan(2048, 3584, 18944) == (208, True)
    assert K.gemm_pair_plan(4096, 3584, 18944) == (208, True)
    assert K.gemm_pair_plan(2048, 37888, 3584) == (256, False)
    assert K.gemm_pair_plan(2048, 4608, 3584) == (256, False)
    assert K.gemm_pair_plan(512, 3584, 18944)[1] is False
    assert K.gemm_pair_plan(8192, 5120, 5120) == (256, False)
    assert K.gemm_pair_plan(2048, 3584, 3584) == (208, True)
    assert K.gemm_pair_plan(8192, 5120, 13824)[1] is False


def test_gemm_tensor_core_refuses_unaligned_rows():
    from minfer_b200.kernels import api as K
    x = torch.zeros(4, 20, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(8, 20, dtype=torch.bfloat16, device="cuda")
    assert not K.gemm_tc_supported(x, w)
    with pytest.raises(K.KernelError, match="aligned"):
        K.gemm_tc(x, w, None, torch.zeros(4, 8, device="cuda"), K.EPI_STORE, status())
    # the projection falls back to the FP32-pipe kernel for such widths
    from minfer_b200.parts.linear import Linear
    xr = torch.randn(4, 20).bfloat16().cuda()
    wr = torch.randn(8, 20).bfloat16().cuda()
    got = Linear(wr).forward(xr, torch.float32)
    close(got, xr.double() @ wr.double().t(), torch.float32)


@pytest.mark.parametrize("hd,nh,nk,window,ring", [(128, 28, 4, 0, 0), (64, 14, 2, 0, 0),
                                                  (128, 16, 1, 0, 0), (64, 3, 3, 100, 128),
                                                  (128, 8, 2, 300, 0), (64, 12, 4, 40, 64)])
def test_attention_decode_tensor_core_kernel(hd, nh, nk, window, ring):
    """The mma decode kernel (bfloat16, head size 64/128) against float64 attention over the
    same cache, with sequences ending inside a page, at a page edge and at a chunk edge,
    and a far key that must be found; also against the generic kernel."""
    from minfer_b200.kernels import api as K
    lens = [600, 1, 64, 65, 256, 257, 1000]
    B = len(lens)
    n_pages = 60
    g = torch.Generator().manual_seed(hd + nh)
    perm = torch.randperm(n_pages, generator=g).tolist()
    scale = 1.0 / math.sqrt(hd)
    dt = torch.bfloat16
    kc = torch.randn(n_pages, nk, 64, hd, generator=g).to(dt).cuda()       # stale values everywhere
    vc = torch.randn(n_pages, nk, 64, hd, generator=g).to(dt).cuda()
    width = 16
    table = torch.full((B, width), -1, dtype=torch.int32)
    hist_k, hist_v = [], []
    q32 = torch.randn(B, nh, hd, generator=g)
    for b, n in enumerate(lens):
        kk = torch.randn(n, nk, hd, generator=g)
        vv = torch.randn(n, nk, hd, generator=g)
        if n == 1000 and window == 0:           # a far key that dominates head 0
            kk[17, 0] = 0.0; kk[17, 0, 3] = 30.0
            q32[b, 0] = 0.0; q32[b, 0, 3] = 30.0
        kk, vv = kk.to(dt), vv.to(dt)
        hist_k.append(kk); hist_v.append(vv)
        lo = max(0, n - ring) if ring else 0
        for p in range(lo, n):
            pe = p % ring if ring else p
            lp = pe // 64
            if table[b, lp] < 0:
                table[b, lp] = perm.pop()
            kc[table[b, lp], :, p % 64] = kk[p].cuda()
            vc[table[b, lp], :, p % 64] = vv[p].cuda()
    q = q32.to(dt).cuda()
    row_seq = torch.arange(B, dtype=torch.int32, device="cuda")
    row_pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device="cuda")
    n_chunks = 4
    outs = {}
    for force in (False, True):
        out = torch.empty(B, nh * hd, dtype=dt, device="cuda")
        partial = torch.full((B * nh * n_chunks * (hd + 2),), float("nan"), device="cuda")
        K.attention_paged(q, kc, vc, row_seq, row_pos, table.cuda(), width, ring, out, partial,
                          nh, nk, hd, window, 256, n_chunks, scale, force_generic=force)
        outs[force] = out
    # chunks of several 256-key blocks: a CTA walks them with a running softmax, its warps
    # loading their own keys (no status word) or fed by the TMA ring (with one)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for chunk, chunks, st in ((512, 2, None), (1024, 1, None), (768, 2, None),
                              (512, 2, status), (1024, 1, status), (768, 2, status)):
        out = torch.full((B, nh * hd), float("nan"), dtype=dt, device="cuda")
        partial = torch.full((B * nh * chunks * (hd + 2),), float("nan"), device="cuda")
        K.attention_paged(q, kc, vc, row_seq, row_pos, table.cuda(), width, ring, out, partial,
                          nh, nk, hd, window, chunk, chunks, scale, status=st,
                          old_keys_final=st is not None and chunk != 768)
        assert int(status.item()) == 0
        close(out, outs[False].double(), dt, scale=3.0)
        for b, n in enumerate(lens):
            qq = torch.zeros(n, nh, hd, dtype=torch.float64)
            qq[n - 1] = q[b].double().cpu()
            want = attention_reference(qq, hist_k[b].double(), hist_v[b].double(), scale, window)
            close(out[b].reshape(nh, hd), want[n - 1], dt, scale=3.0)
    close(outs[False], outs[True].double(), dt, scale=3.0)
    if window == 0:
        assert torch.allclose(outs[False][6, :hd].float().cpu(), hist_v[6][17, 0].float(), atol=2e-2)


@pytest.mark.parametrize("hd,nh,nk,window", [(128, 14, 2, 0), (64, 16, 1, 0), (128, 6, 2, 3000)])
def test_attention_decode_ring_long_chunks(hd, nh, nk, window):
    """The TMA-ring decode kernel on chunks of thousands of keys (the ring wraps many times and
    the producer fetches page ids more than once), pages scattered over the cache, sequences
    ending at a page edge, inside a page and in the first page of a chunk; a far key in an
    early page must be found.  Against float64 attention."""
    from minfer_b200.kernels import api as K
    lens = [5000, 2049, 4096, 70, 2561]
    B, width = len(lens), 80
    n_pages = sum((n + 63) // 64 for n in lens) + 7
    g = torch.Generator().manual_seed(hd + nh + window)
    perm = torch.randperm(n_pages, generator=g).tolist()
    scale = 1.0 / math.sqrt(hd)
    dt = torch.bfloat16
    kc = torch.randn(n_pages, nk, 64, hd, generator=g).to(dt).cuda()
    vc = torch.randn(n_pages, nk, 64, hd, generator=g).to(dt).cuda()
    table = torch.full((B, width), -1, dtype=torch.int32)
    hist_k, hist_v = [], []
    q32 = torch.randn(B, nh, hd, generator=g)
    for b, n in enumerate(lens):
        kk = torch.randn(n, nk, hd, generator=g)
        vv = torch.randn(n, nk, hd, generator=g)
        if n == 5000 and window == 0:           # position 2077 dominates head 1 of the first sequence
            kk[2077, 0] = 0.0; kk[2077, 0, 5] = 30.0
            q32[b, 1] = 0.0; q32[b, 1, 5] = 30.0
        kk, vv = kk.to(dt), vv.to(dt)
        hist_k.append(kk); hist_v.append(vv)
        pages = [perm.pop() for _ in range((n + 63) // 64)]
        table[b, :len(pages)] = torch.tensor(pages, dtype=torch.int32)
        for i, pg in enumerate(pages):
            m = min(64, n - 64 * i)
            kc[pg, :, :m] = kk[64 * i:64 * i + m].transpose(0, 1).cuda()
            vc[pg, :, :m] = vv[64 * i:64 * i + m].transpose(0, 1).cuda()
    q = q32.to(dt).cuda()
    row_seq = torch.arange(B, dtype=torch.int32, device="cuda")
    row_pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    want = []
    for b, n in enumerate(lens):
        qq = torch.zeros(n, nh, hd, dtype=torch.float64)
        qq[n - 1] = q[b].double().cpu()
        want.append(attention_reference(qq, hist_k[b].double(), hist_v[b].double(), scale, window)[n - 1])
    for chunk, chunks, final in ((5120, 1, True), (4096, 2, False), (2560, 2, True), (512, 10, True),
                                 (256, 20, True), (256, 20, False)):
        out = torch.full((B, nh * hd), float("nan"), dtype=dt, device="cuda")
        partial = torch.full((B * nh * chunks * (hd + 2),), float("nan"), device="cuda")
        K.attention_paged(q, kc, vc, row_seq, row_pos, table.cuda(), width, 0, out, partial,
                          nh, nk, hd, window, chunk, chunks, scale, status=status,
                          old_keys_final=final)
        assert int(status.item()) == 0
        for b in range(B):
            close(out[b].reshape(nh, hd), want[b], dt, scale=3.0)
        if window == 0:
            assert torch.allclose(out[0, hd:2 * hd].float().cpu(), hist_v[0][2077, 0].float(), atol=2e-2)


@pytest.mark.parametrize("hd", [64, 128])
def test_attention_decode_many_rows(hd):
    """Many rows at once: the decode kernel's variant for grids of several rounds of CTAs
    (three CTAs per SM) against the generic kernel over the same random cache."""
    from minfer_b200.kernels import api as K
    B, nh, nk, n_chunks, width = 200, 8, 4, 3, 12
    g = torch.Generator().manual_seed(hd)
    dt = torch.bfloat16
    n_pages = B * width
    kc = torch.randn(n_pages, nk, 64, hd, generator=g).to(dt).cuda()
    vc = torch.randn(n_pages, nk, 64, hd, generator=g).to(dt).cuda()
    table = torch.randperm(n_pages, generator=g).to(torch.int32).reshape(B, width).cuda()
    lens = torch.randint(1, 64 * width + 1, (B,), generator=g)
    lens[:4] = torch.tensor([1, 256, 257, 64 * width])
    q = torch.randn(B, nh, hd, generator=g).to(dt).cuda()
    row_seq = torch.arange(B, dtype=torch.int32, device="cuda")
    row_pos = (lens - 1).to(torch.int32).cuda()
    outs = []
    for force in (False, True):
        out = torch.full((B, nh * hd), float("nan"), dtype=dt, device="cuda")
        partial = torch.full((B * nh * n_chunks * (hd + 2),), float("nan"), device="cuda")
        K.attention_paged(q, kc, vc, row_seq, row_pos, table, width, 0, out, partial, nh, nk, hd, 0,
                          256, n_chunks, 1.0 / math.sqrt(hd), force_generic=force)
        outs.append(out)
    assert not torch.isnan(outs[0].float()).any()
    close(outs[0], outs[1].double(), dt, scale=3.0)


@pytest.mark.parametrize("hd,nh,nk,window", [(128, 7, 1, 0), (64, 14, 2, 0), (128, 4, 4, 33),
                                             (64, 6, 2, 200), (128, 2, 1, 64), (64, 3, 1, 1)])
def test_attention_prefill_tensor_core_kernel(hd, nh, nk, window):
    """Whole prompts of unequal lengths (one token, tile edges, several tiles) on the mma
    kernel against float64 attention and against the generic kernel."""
    from minfer_b200.kernels import api as K
    lens = [37, 1, 64, 65, 128, 300, 129]
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    T = cu[-1]
    g = torch.Generator().manual_seed(hd * 3 + nh)
    dt = torch.bfloat16
    q = torch.randn(T, nh, hd, generator=g).to(dt).cuda()
    k = torch.randn(T, nk, hd, generator=g).to(dt).cuda()
    v = torch.randn(T, nk, hd, generator=g).to(dt).cuda()
    if window == 0:       # a far key that dominates: the last query of the 300-token sequence
        b0 = cu[5]
        k[b0 + 3, 0] = 0.0; k[b0 + 3, 0, 7] = 30.0
        q[b0 + 299, 0] = 0.0; q[b0 + 299, 0, 7] = 30.0
    scale = 1.0 / math.sqrt(hd)
    cu_t = torch.tensor(cu, dtype=torch.int32, device="cuda")
    out = torch.full((T, nh * hd), float("nan"), dtype=dt, device="cuda")
    K.attention_prefill(q, k, v, cu_t, out, len(lens), max(lens), nh, nk, hd, window, scale)
    row_seq = torch.cat([torch.full((n,), b, dtype=torch.int32) for b, n in enumerate(lens)]).cuda()
    row_pos = torch.cat([torch.arange(n, dtype=torch.int32) for n in lens]).cuda()
    gen = torch.empty_like(out)
    K.attention_packed(q, k, v, row_seq, row_pos, cu_t, gen, nh, nk, hd, window, scale)
    for b, n in enumerate(lens):
        sl = slice(cu[b], cu[b + 1])
        want = attention_reference(q[sl].double().cpu(), k[sl].double().cpu(), v[sl].double().cpu(),
                                   scale, window)
        close(out[sl].reshape(n, nh, hd), want, dt, scale=3.0)
    close(out, gen.double(), dt, scale=3.0)
    if window == 0:
        assert torch.allclose(out[cu[5] + 299, :hd].float().cpu(), v[cu[5] + 3, 0].float().cpu(), atol=2e-2)


@pytest.mark.parametrize("hd,nh,nk,window", [(128, 7, 1, 0), (64, 14, 2, 0), (128, 4, 4, 33),
                                             (64, 6, 2, 200), (128, 2, 1, 64), (64, 3, 1, 1),
                                             (128, 3, 1, 129), (64, 2, 2, 300)])
def test_attention_prefill_tcgen05_kernel(hd, nh, nk, window):
    """Whole prompts of unequal lengths on the tcgen05 kernel (two query tiles of 128 per CTA,
    key tiles of 128): one token, the edges of a query tile and of a pair of tiles, a second
    query tile with one row, many key tiles; against float64 attention and the generic kernel.
    Without a window one far key is made to dominate a late query."""
    from minfer_b200.kernels import api as K
    lens = [37, 1, 128, 129, 256, 257, 700, 383, 1000]
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    T = cu[-1]
    g = torch.Generator().manual_seed(hd * 5 + nh)
    dt = torch.bfloat16
    q = torch.randn(T, nh, hd, generator=g).to(dt).cuda()
    k = torch.randn(T, nk, hd, generator=g).to(dt).cuda()
    v = torch.randn(T, nk, hd, generator=g).to(dt).cuda()
    if window == 0:       # key 3 of the 1000-token sequence dominates its query 999
        b0 = cu[8]
        k[b0 + 3, 0] = 0.0; k[b0 + 3, 0, 7] = 30.0
        q[b0 + 999, 0] = 0.0; q[b0 + 999, 0, 7] = 30.0
    scale = 1.0 / math.sqrt(hd)
    cu_t = torch.tensor(cu, dtype=torch.int32, device="cuda")
    out = torch.full((T, nh * hd), float("nan"), dtype=dt, device="cuda")
    st = status()
    K.attention_prefill_tc(q, k, v, cu_t, out, len(lens), max(lens), nh, nk, hd, window, scale, st)
    assert int(st.item()) == 0
    row_seq = torch.cat([torch.full((n,), b, dtype=torch.int32) for b, n in enumerate(lens)]).cuda()
    row_pos = torch.cat([torch.arange(n, dtype=torch.int32) for n in lens]).cuda()
    gen = torch.empty_like(out)
    K.attention_packed(q, k, v, row_seq, row_pos, cu_t, gen, nh, nk, hd, window, scale)
    for b, n in enumerate(lens):
        sl = slice(cu[b], cu[b + 1])
        want = attention_reference(q[sl].double().cpu(), k[sl].double().cpu(), v[sl].double().cpu(),
                                   scale, window)
        close(out[sl].reshape(n, nh, hd), want, dt, scale=3.0)
    close(out, gen.double(), dt, scale=3.0)
    if window == 0:
        assert torch.allclose(out[cu[8] + 999, :hd].float().cpu(), v[cu[8] + 3, 0].float().cpu(), atol=2e-2)


def test_attention_prefill_tcgen05_refuses_other_head_sizes():
    from minfer_b200.kernels import api as K
    q = torch.zeros(4, 2, 96, dtype=torch.bfloat16, device="cuda")
    cu = torch.tensor([0, 4], dtype=torch.int32, device="cuda")
    with pytest.raises(K.KernelError):
        K.attention_prefill_tc(q, q, q, cu, torch.empty(4, 192, dtype=torch.bfloat16, device="cuda"),
                               1, 4, 2, 2, 96, 0, 0.1, status())


def test_deferred_split_sums_feed_the_next_kernel():
    """A small projection leaves its K splits; add_rmsnorm and rope_kvstore add them (and the
    bias) themselves: the same numbers as reducing first."""
    from minfer_b200.kernels import api as K
    g = torch.Generator().manual_seed(5)
    m, n, k = 8, 3584, 3584
    x = (torch.randn(m, k, generator=g) * 0.3).bfloat16().cuda()
    w = (torch.randn(n, k, generator=g) * 0.05).bfloat16().cuda()
    bias = torch.randn(n, generator=g).cuda()
    st = status()
    partial = K.gemm_tc_partial_sums(x, w, st)
    assert partial is not None and partial.shape[0] > 1 and partial.shape[1:] == (m, n)
    full = x.double() @ w.double().t()
    close(partial.sum(0), full, torch.float32)
    # reduce, accumulate
    h = torch.randn(m, n, generator=g).cuda()
    h0 = h.clone()
    K.splitk_reduce(partial, bias, h, accumulate=True)
    close(h, h0.double() + full + bias.double(), torch.float32)
    # add + norm in one kernel
    wn = (1 + 0.1 * torch.randn(n, generator=g)).cuda()
    for dt in DTYPES:
        h2 = h0.clone()
        y = torch.empty(m, n, dtype=dt, device="cuda")
        K.add_rmsnorm(h2, partial, partial.shape[0], bias, wn, 1e-6, y)
        assert torch.equal(h2, h)                      # the same sums in the same order
        hd_ = h.double()
        want = hd_ / torch.sqrt((hd_ ** 2).mean(-1, keepdim=True) + 1e-6) * wn.double()
        close(y, want, dt)
    # no partial sums: plain residual + norm
    h3 = h0.clone()
    y = torch.empty(m, n, device="cuda")
    K.add_rmsnorm(h3, None, 0, None, wn, 1e-6, y)
    assert torch.equal(h3, h0)
    # a product that is not split leaves nothing
    assert K.gemm_tc_partial_sums(torch.zeros(2048, 64, dtype=torch.bfloat16, device="cuda"),
                                  torch.zeros(256, 64, dtype=torch.bfloat16, device="cuda"), st) is None
    # rotary kernel adding the splits: equals the kernel run on the reduced projection
    nh, nk, hd = 20, 4, 128
    assert (nh + 2 * nk) * hd == n
    red = torch.empty(m, n, device="cuda")
    K.splitk_reduce(partial, bias, red, accumulate=False)
    pos = torch.arange(100, 100 + m, dtype=torch.int32, device="cuda")
    rows = torch.zeros(m, dtype=torch.int32, device="cuda")
    end = torch.tensor([100 + m], dtype=torch.int32, device="cuda")
    inv_freq = (1.0 / (1e6 ** (torch.arange(hd // 2).double() * 2 / hd))).cuda()
    outs = []
    for src, npart, b in ((red, 0, None), (partial, partial.shape[0], bias)):
        q = torch.empty(m, nh, hd, dtype=torch.bfloat16, device="cuda")
        ks = torch.empty(m, nk, hd, dtype=torch.bfloat16, device="cuda")
        vs = torch.empty_like(ks)
        K.rope_kvstore(src, pos, rows, end, inv_freq, q, ks, vs, None, None, None, 0, 0, nh, nk, hd,
                       hd, 0, st, n_partials=npart, bias=b)
        outs.append((q, ks, vs))
    for a, b in zip(outs[0], outs[1]):
        assert torch.equal(a, b)
    assert int(st) == 0


def _norm_ref(h, g, eps):
    h = h.double()
    return h / torch.sqrt((h * h).mean(-1, keepdim=True) + eps) * g.double()


@pytest.mark.parametrize("m", [1, 8, 17, 64, 300, 700])
@pytest.mark.parametrize("n,k", [(3584, 3584), (896, 4864), (200, 1024), (64, 128), (384, 264)])
def test_product_that_completes_the_residual_and_prepares_the_next_norm(m, n, k):
    """EPI_ACCUM with the next norm folded in (few tokens: K split over a cluster of CTAs that add
    their tiles through distributed shared memory; many tokens: refused, the norm stays a
    kernel): the residual, x' = bfloat16(h * g) and the sums of squares against float64; then a
    product that reads x' with the row scale against norm-then-product in float64."""
    from minfer_b200.kernels import api as K
    g0 = torch.Generator().manual_seed(m + n + k)
    x = (torch.randn(m, k, generator=g0) * 0.5).bfloat16().cuda()
    w = (torch.randn(n, k, generator=g0) * 0.05).bfloat16().cuda()
    h0 = torch.randn(m, n, generator=g0).cuda()
    gw = (1 + 0.1 * torch.randn(n, generator=g0)).cuda()
    bias = (torch.randn(n, generator=g0) * 0.1).cuda()
    parts = K.gemm_tc_prep_parts(m, n, k)
    if parts == 0:
        # nothing folds the norm in at these sizes: the call says so instead of computing
        with pytest.raises(K.KernelError):
            K.gemm_tc_fused(x, w, None, h0.clone(), K.EPI_ACCUM, status(),
                            prep_x=torch.empty(m, n, dtype=torch.bfloat16, device="cuda"),
                            prep_weight=gw, prep_ssq=torch.empty(1, m, device="cuda"))
        return
    h = h0.clone()
    xp = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    # guards behind the sums of squares: nothing may be written past the parts that exist
    ssq_all = torch.full((parts + 2, m), float("nan"), device="cuda")
    ssq = ssq_all[:parts]
    st = status()
    K.gemm_tc_fused(x, w, bias, h, K.EPI_ACCUM, st, prep_x=xp, prep_weight=gw, prep_ssq=ssq)
    assert int(st.item()) == 0
    assert torch.isnan(ssq_all[parts:]).all() and not torch.isnan(ssq).any()
    want_h = h0.double() + x.double() @ w.double().t() + bias.double()
    close(h, want_h, torch.float32)                     # exact bfloat16 products, float32 sums
    close(xp, h.double() * gw.double(), torch.bfloat16)
    close(ssq.sum(0), (h.double() ** 2).sum(-1), torch.float32, scale=float((h.double() ** 2).sum(-1).max()) * 10)
    # the consumer: a second product reads x' and applies 1/rms in its epilogue
    n2 = 256
    w2 = (torch.randn(n2, n, generator=g0) * 0.05).bfloat16().cuda()
    b2 = torch.randn(n2, generator=g0).cuda()
    eps = 1e-5
    want = _norm_ref(h, gw, eps) @ w2.double().t() + b2.double()
    rs = K.RowScale(ssq, n, eps)
    out = torch.empty(m, n2, device="cuda")
    K.gemm_tc_fused(xp, w2, b2, out, K.EPI_STORE, st, row_scale=rs)
    close(out, want, torch.bfloat16)
    part = K.gemm_tc_fused(xp, w2, None, None, K.EPI_STORE, st, row_scale=rs, defer=True)
    if part is not None:                               # split along K: the splits carry the scale
        close(part.sum(0) + b2, want, torch.bfloat16)
    # and SwiGLU over interleaved gate/up rows
    act = torch.empty(m, n2 // 2, dtype=torch.bfloat16, device="cuda")
    K.gemm_tc_fused(xp, w2, None, act, K.EPI_SWIGLU, st, row_scale=rs)
    y = _norm_ref(h, gw, eps) @ w2.double().t()
    close(act, torch.nn.functional.silu(y[:, 0::2]) * y[:, 1::2], torch.bfloat16)
    assert int(st.item()) == 0
