"""The bfloat16 tensor-core attention kernels at the places where an off-by-one would hide
behind random keys: the window's edge, a page's edge, a chunk's edge, a ring's wrap, and
the line between the keys a step brings and the keys the cache held before.

Random keys cannot show one key too many or too few (it moves the output by about
1/window).  Here every query of head 0 points along one dimension with weight 30 and a few
*marked* keys point the same way, so a marked key's score stands out by e^70: a query's
output is the value of the marked key it sees, and the float64 reference gives something
else entirely as soon as the kernel sees one key more or fewer than it should.
"""
import math

import pytest
import torch

from test_kernels_gpu import attention_reference, close, status

pytestmark = pytest.mark.gpu
DT = torch.bfloat16
DIM, BIG = 5, 30.0


def _history(n, nk, hd, marked, g):
    """Keys and values of one sequence of ``n`` positions; ``marked`` positions dominate head 0's
    key/value head along DIM."""
    k = torch.randn(n, nk, hd, generator=g)
    v = torch.randn(n, nk, hd, generator=g)
    for j in marked:
        if 0 <= j < n:
            k[j, 0] = 0.0
            k[j, 0, DIM] = BIG
    return k.to(DT), v.to(DT)


def _queries(n, nh, hd, g):
    q = torch.randn(n, nh, hd, generator=g)
    q[:, 0] = 0.0
    q[:, 0, DIM] = BIG
    return q.to(DT)


class PagedCache:
    """Pages scattered over storage that holds stale values everywhere."""

    def __init__(self, n_pages, nk, hd, width, n_seqs, ring, g):
        self.k = torch.randn(n_pages, nk, 64, hd, generator=g).to(DT).cuda()
        self.v = torch.randn(n_pages, nk, 64, hd, generator=g).to(DT).cuda()
        self.table = torch.full((n_seqs, width), -1, dtype=torch.int32)
        self.free = torch.randperm(n_pages, generator=g).tolist()
        self.ring, self.width = ring, width

    def write(self, b, k, v, lo=0):
        """Positions lo.. of sequence b (a ring keeps what its wrap leaves)."""
        n = k.shape[0]
        first = max(lo, n - self.ring) if self.ring else lo
        for p in range(first, n):
            pe = p % self.ring if self.ring else p
            if self.table[b, pe // 64] < 0:
                self.table[b, pe // 64] = self.free.pop()
            self.k[self.table[b, pe // 64], :, p % 64] = k[p].cuda()
            self.v[self.table[b, pe // 64], :, p % 64] = v[p].cuda()


def _marks(window, n):
    """Marked keys further apart than the window, at odd offsets: each query sees at most
    one, and the edges fall inside pages, on page edges and on tile edges over the run."""
    step = window + 37 if window else 10 ** 9
    return [j for j in range(11, n, step)] if window else [17]


@pytest.mark.parametrize("hd,nh,nk,window", [(64, 6, 2, 33), (128, 4, 1, 64), (64, 2, 2, 100),
                                             (128, 7, 1, 129), (64, 3, 1, 256), (128, 8, 2, 0)])
@pytest.mark.parametrize("kernel", ["mma", "tcgen05"])
def test_whole_prompt_kernels_at_the_window_edge(kernel, hd, nh, nk, window):
    from minfer_b200.kernels import api as K
    lens = [700, 129, 64, 385]
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    g = torch.Generator().manual_seed(hd + nh + window)
    ks, vs, qs = [], [], []
    for n in lens:
        k, v = _history(n, nk, hd, _marks(window, n), g)
        ks.append(k); vs.append(v); qs.append(_queries(n, nh, hd, g))
    q, k, v = torch.cat(qs).cuda(), torch.cat(ks).cuda(), torch.cat(vs).cuda()
    scale = 1.0 / math.sqrt(hd)
    cu_t = torch.tensor(cu, dtype=torch.int32, device="cuda")
    out = torch.full((cu[-1], nh * hd), float("nan"), dtype=DT, device="cuda")
    if kernel == "mma":
        K.attention_prefill(q, k, v, cu_t, out, len(lens), max(lens), nh, nk, hd, window, scale)
    else:
        st = status()
        K.attention_prefill_tc(q, k, v, cu_t, out, len(lens), max(lens), nh, nk, hd, window, scale, st)
        assert int(st.item()) == 0
    for b, n in enumerate(lens):
        want = attention_reference(qs[b].double(), ks[b].double(), vs[b].double(), scale, window)
        got = out[cu[b]:cu[b + 1]].reshape(n, nh, hd)
        close(got, want, DT, scale=3.0)
        for j in _marks(window, n):
            last = min(n, j + window) - 1 if window else n - 1      # the last query that sees key j
            assert torch.allclose(got[last, 0].float().cpu(), vs[b][j, 0].float(), atol=2e-2), (b, j)
            if window and last + 1 < n:                             # the next one must not
                assert not torch.allclose(got[last + 1, 0].float().cpu(), vs[b][j, 0].float(), atol=0.3)


@pytest.mark.parametrize("hd,nh,nk,window,ring", [(64, 6, 2, 33, 64), (128, 4, 1, 64, 128),
                                                  (64, 2, 2, 100, 0), (128, 7, 1, 129, 256),
                                                  (64, 3, 1, 256, 320), (128, 16, 1, 300, 0)])
@pytest.mark.parametrize("with_status", [False, True])
def test_decode_kernels_at_the_window_edge(with_status, hd, nh, nk, window, ring):
    """One query at the end of each sequence over the paged cache.  The marked key sits at
    pos - window (just outside) or pos - window + 1 (the oldest key seen), with that edge
    inside a page, on a page edge and on a chunk edge; both decode kernels (warps that load
    their own keys; the TMA ring) with chunks of one and of several blocks."""
    from minfer_b200.kernels import api as K
    # pos - window + 1 = 300 (inside a page), 320 (page edge), 512 (chunk edge), 256, 0
    edges = [300, 320, 512, 256, 0]
    cases = []
    for e in edges:
        cases.append((e + window, e, True))             # (length, marked key, seen)
        cases.append((e + window + 1, e, False))
    B = len(cases)
    g = torch.Generator().manual_seed(hd + nh + window + ring)
    width = 16
    cache = PagedCache(B * width + 4, nk, hd, width, B, ring, g)
    hist = []
    for b, (n, j, _) in enumerate(cases):
        k, v = _history(n, nk, hd, [j], g)
        cache.write(b, k, v)
        hist.append((k, v))
    q = _queries(B, nh, hd, g).cuda()
    row_seq = torch.arange(B, dtype=torch.int32, device="cuda")
    row_pos = torch.tensor([n - 1 for n, _, _ in cases], dtype=torch.int32, device="cuda")
    scale = 1.0 / math.sqrt(hd)
    st = status() if with_status else None
    max_end = max(n for n, _, _ in cases)
    for chunk in (256, 512, 1024):
        n_chunks = -(-max_end // chunk)
        out = torch.full((B, nh * hd), float("nan"), dtype=DT, device="cuda")
        partial = torch.full((B * nh * n_chunks * (hd + 2),), float("nan"), device="cuda")
        K.attention_paged(q, cache.k, cache.v, row_seq, row_pos, cache.table.cuda(), width, ring,
                          out, partial, nh, nk, hd, window, chunk, n_chunks, scale, status=st,
                          old_keys_final=with_status)
        if st is not None:
            assert int(st.item()) == 0
        for b, (n, j, seen) in enumerate(cases):
            qq = torch.zeros(n, nh, hd, dtype=torch.float64)
            qq[n - 1] = q[b].double().cpu()
            want = attention_reference(qq, hist[b][0].double(), hist[b][1].double(), scale, window)
            got = out[b].reshape(nh, hd)
            close(got, want[n - 1], DT, scale=3.0)
            is_value = torch.allclose(got[0].float().cpu(), hist[b][1][j, 0].float(), atol=2e-2)
            assert is_value == seen, (chunk, b, n, j)


@pytest.mark.parametrize("hd,nh,nk,window,ring", [(64, 6, 2, 0, 0), (128, 4, 1, 0, 0),
                                                  (64, 2, 2, 33, 384), (128, 7, 1, 129, 448),
                                                  (64, 3, 1, 100, 0), (128, 28, 4, 300, 640)])
def test_portions_over_the_paged_cache_tcgen05(hd, nh, nk, window, ring):
    """The step's rows go on from what the cache holds: sequences that held 0, 1, 63, 64, 200
    and 700 positions bring 1 to 300 tokens each; the cache holds old and new keys; marked keys
    lie in the old part, in the new part and at the window's edge of queries on both sides of
    the line between them.  Against float64 attention of the whole sequences and against the
    generic kernel."""
    from minfer_b200.kernels import api as K
    olds = [0, 1, 63, 64, 200, 700, 130, 511]
    news = [300, 129, 2, 256, 57, 257, 1, 128]
    B = len(olds)
    g = torch.Generator().manual_seed(hd + nh + window)
    width = 16
    if ring:
        assert all(n <= ring - window + 1 for n in news)
    cache = PagedCache(B * width + 4, nk, hd, width, B, ring, g)
    hist, qs = [], []
    for b in range(B):
        n = olds[b] + news[b]
        if window:
            marks = _marks(window, n)
        else:       # one marked key: in what the cache held before (even rows) or in the step's own
            marks = [3] if b % 2 == 0 or news[b] < 2 else [olds[b] + 1]
        k, v = _history(n, nk, hd, marks, g)
        cache.write(b, k[:olds[b]], v[:olds[b]])        # what earlier steps left (a ring: its last part)
        cache.write(b, k, v, lo=olds[b])                # the step's own positions
        hist.append((k, v, marks))
        qs.append(_queries(news[b], nh, hd, g))
    cu = [0]
    for n in news:
        cu.append(cu[-1] + n)
    q = torch.cat(qs).cuda()
    scale = 1.0 / math.sqrt(hd)
    cu_t = torch.tensor(cu, dtype=torch.int32, device="cuda")
    seq_end = torch.tensor([o + n for o, n in zip(olds, news)], dtype=torch.int32, device="cuda")
    out = torch.full((cu[-1], nh * hd), float("nan"), dtype=DT, device="cuda")
    st = status()
    K.attention_prefill_tc_paged(q, cache.k, cache.v, cu_t, seq_end, cache.table.cuda(), width, ring,
                                 out, B, max(news), nh, nk, hd, window, scale, st)
    assert int(st.item()) == 0
    row_seq = torch.cat([torch.full((n,), b, dtype=torch.int32) for b, n in enumerate(news)]).cuda()
    row_pos = torch.cat([torch.arange(o, o + n, dtype=torch.int32) for o, n in zip(olds, news)]).cuda()
    gen = torch.empty_like(out)
    K.attention_paged(q, cache.k, cache.v, row_seq, row_pos, cache.table.cuda(), width, ring, gen, None,
                      nh, nk, hd, window, 0, 1, scale, force_generic=True)
    close(out, gen.double(), DT, scale=3.0)
    for b in range(B):
        k, v, marks = hist[b]
        n = olds[b] + news[b]
        qq = torch.zeros(n, nh, hd, dtype=torch.float64)
        qq[olds[b]:] = qs[b].double()
        want = attention_reference(qq, k.double(), v.double(), scale, window)[olds[b]:]
        got = out[cu[b]:cu[b + 1]].reshape(news[b], nh, hd)
        close(got, want, DT, scale=3.0)
        for j in marks:
            last = min(n, j + window) - 1 if window else n - 1
            if last >= olds[b] and j < n:
                assert torch.allclose(got[last - olds[b], 0].float().cpu(), v[j, 0].float(), atol=2e-2), (b, j)
                if window and last + 1 < n:
                    assert not torch.allclose(got[last + 1 - olds[b], 0].float().cpu(), v[j, 0].float(), atol=0.3)
