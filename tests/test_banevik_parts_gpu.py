"""The mechanisms Banevik brought, each alone against the plain formulas: the token-pair embedding with its
kept token, the router, the grouped products (experts and heads), the latent mixer in prompts and in
decoding, and the sink and the shared key/value rows in every attention kernel, with keys made to stand out
at the places where a fault would hide: a window's edge, a page's border, far back, the first token."""
import math

import pytest
import torch

import brolm_b200 as bb
from brolm_b200 import kernels
from brolm_b200.cache import Cache
from brolm_b200.parts import LatentAttention, RotaryEmbedding, RoutedExperts
from tests.plain import banevik_plain as plain
from tests.test_parts_gpu import make_ctx

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
TOL = {torch.float32: 2e-5, torch.bfloat16: 4e-2}


def rel(got, ref):
    ref = ref.double().cpu()
    return float((got.double().cpu() - ref).abs().max()) / max(1e-30, float(ref.abs().max()))


def i32(v):
    return torch.tensor(v, dtype=torch.int32, device=DEV)


# ---------------------------------------------------------------------------------------------------------
def test_pair_embedding_with_the_kept_token():
    V, D, buckets, mp, mc = 40, 24, 11, 7, 3
    g = torch.Generator().manual_seed(0)
    w = {"embed": torch.randn(V, D, generator=g), "bigram": torch.randn(buckets + 1, D, generator=g)}
    config = {"embedding": {"bigram": {"buckets": buckets, "mul_prev": mp, "mul_cur": mc}}}
    seqs = [torch.randint(0, V, (n,), generator=g).tolist() for n in (9, 1, 5)]
    last = torch.full((5,), 12345, dtype=torch.int32, device=DEV)        # stale numbers of earlier tenants
    slots = [3, 0, 2]

    def run(chunks, starts):
        n = [len(c) for c in chunks]
        cu = [0]
        for k in n:
            cu.append(cu[-1] + k)
        out = torch.empty((cu[-1], D), dtype=torch.float32, device=DEV)
        kernels.embed_pairs(i32([t for c in chunks for t in c]), i32([a + j for a, k in zip(starts, n) for j in range(k)]),
                            i32([b for b, k in enumerate(n) for _ in range(k)]), i32(cu), i32(slots[:len(chunks)]), last,
                            w["embed"].to(DEV), w["bigram"].to(DEV), 1.0, mp, mc, buckets, out)
        return out.cpu()

    refs = [plain.embed(config, w, s) for s in seqs]
    got = run([s[:max(1, len(s) - 2)] for s in seqs], [0, 0, 0])
    at = 0
    for s, r in zip(seqs, refs):
        k = max(1, len(s) - 2)
        assert rel(got[at:at + k], r[:k]) < 1e-6
        at += k
    # the two long ones go on token by token: the token before comes from what the step before kept
    for step in (2, 1):
        live = [0, 2]
        order = [slots[0], slots[2]]
        chunks = [[seqs[i][len(seqs[i]) - step]] for i in live]
        n = len(chunks)
        out = torch.empty((n, D), dtype=torch.float32, device=DEV)
        kernels.embed_pairs(i32([c[0] for c in chunks]), i32([len(seqs[i]) - step for i in live]), i32([0, 1]), i32([0, 1, 2]),
                            i32(order), last, w["embed"].to(DEV), w["bigram"].to(DEV), 1.0, mp, mc, buckets, out)
        for r, i in enumerate(live):
            assert rel(out[r], refs[i][len(seqs[i]) - step]) < 1e-6
    assert last.tolist()[3] == seqs[0][-1] and last.tolist()[2] == seqs[2][-1] and last.tolist()[0] == seqs[1][-1]
    # a padding row (position -1) takes the token's row alone and keeps nothing
    out = torch.empty((1, D), dtype=torch.float32, device=DEV)
    kernels.embed_pairs(i32([4]), i32([-1]), i32([0]), i32([0, 1]), i32([4]), last, w["embed"].to(DEV), w["bigram"].to(DEV),
                        1.0, mp, mc, buckets, out)
    assert rel(out[0], w["embed"][4]) < 1e-6 and last.tolist()[4] == 12345


# ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("E,top,D", [(5, 2, 40), (7, 7, 64), (33, 4, 24), (3, 1, 100)])
def test_router(dtype, E, top, D):
    g = torch.Generator().manual_seed(E)
    x = torch.randn(70, D, generator=g).to(dtype)
    wr = torch.randn(E, D, generator=g).to(dtype)
    ids = torch.empty((70, top), dtype=torch.int32, device=DEV)
    wts = torch.empty((70, top), dtype=torch.float32, device=DEV)
    kernels.route_topk(x.to(DEV), wr.to(DEV), top, ids, wts)
    z = x.double() @ wr.double().T
    ref = torch.topk(z, top, dim=1)
    assert torch.equal(ids.cpu().long(), ref.indices)                  # (the operands are the same numbers: no close calls)
    assert rel(wts, torch.sigmoid(ref.values)) < 1e-5
    # the choice alone, from scores in memory (rows further apart than E)
    held = torch.zeros((70, E + 3), dtype=torch.float32, device=DEV)
    held[:, :E] = z.float().to(DEV)
    ids2, wts2 = torch.empty_like(ids), torch.empty_like(wts)
    kernels.route_pick(held[:, :E], top, ids2, wts2)
    assert torch.equal(ids2.cpu().long(), ref.indices) and rel(wts2, torch.sigmoid(ref.values)) < 1e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,E,top,D,F", [(1, 4, 2, 32, 16), (7, 6, 1, 40, 24), (70, 3, 3, 48, 40), (300, 5, 2, 36, 20),
                                         (3, 9, 1, 64, 72), (300, 4, 2, 64, 136), (5, 8, 2, 64, 72), (40, 2, 1, 128, 64),
                                         (100, 4, 2, 64, 136), (700, 4, 2, 72, 264), (520, 2, 1, 320, 128)])
def test_routed_experts_part(dtype, T, E, top, D, F):
    """Experts with many rows (several tiles), with one row, with none; sizes that are no multiples of 8 (the plain
    kernel), aligned sizes with many rows per expert (the tcgen05 kernel, also with sizes that are no multiples of
    its tiles), with fewer (the pipelined kernel) and with a few (the streaming kernel)."""
    part = RoutedExperts(D, F, E, top)
    g = torch.Generator().manual_seed(T)
    ws = {n: (torch.randn(s.shape, generator=g) * (1.0 if n == "router" else 0.25)).to(dtype)
          for n, s in part.param_specs().items()}
    part.bind({n: t.to(DEV) for n, t in ws.items()})
    x = torch.randn(T, D, generator=g).to(dtype)

    class Ctx:
        pass
    ctx = Ctx()
    ctx.dtype = dtype
    y = part.forward(x.to(DEV), ctx)
    assert y.shape == (top, T, D) and y.dtype == torch.float32
    m = {"router": {"experts": E, "top": top}}
    w = {f"p.{n}": t for n, t in ws.items()}
    margins = []
    ref = plain.experts(m, w, "p.", x.double(), margins)
    got = y.sum(dim=0).double().cpu()
    # a token whose choice is a close call for rounded products is left out (none in float32)
    keep = [t for t in range(T) if margins[t] > (1e-5 if dtype == torch.float32 else 0.02)]
    assert len(keep) >= T * 0.7
    assert rel(got[keep], ref[keep]) <= TOL[dtype]


@pytest.mark.parametrize("counts", [[0, 1, 128, 129, 300, 0, 70], [256, 0, 0, 127], [5, 600], [257, 15, 16, 17, 255]])
@pytest.mark.parametrize("N,K", [(256, 64), (40, 200), (520, 72)])
def test_grouped_products_on_tcgen05_with_uneven_experts(counts, N, K):
    """The two products over hand-made expert loads: experts without rows, with one, with a full tile and one more,
    with several tiles; outputs narrower and wider than a tile, a depth that is no multiple of a stage."""
    E, top = len(counts), 2
    g = torch.Generator().manual_seed(sum(counts) + N)
    expert_of = torch.cat([torch.full((c,), e, dtype=torch.int32) for e, c in enumerate(counts)])
    pairs = expert_of.numel() + (expert_of.numel() & 1)
    ids = torch.full((pairs,), E - 1, dtype=torch.int32)
    ids[torch.randperm(pairs, generator=g)[:expert_of.numel()]] = expert_of
    tokens = pairs // top
    ids = ids.view(tokens, top).to(DEV)
    perm = torch.empty(pairs, dtype=torch.int32, device=DEV)
    offsets = torch.empty(E + 1, dtype=torch.int32, device=DEV)
    tiles = torch.empty((2, kernels.group_tiles(pairs, E, kernels.GROUP_ROWS_TC)), dtype=torch.int32, device=DEV)
    kernels.group_pairs(ids, E, perm, offsets, tiles, kernels.GROUP_ROWS_TC)
    x = torch.randn(tokens, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(E, N, K, generator=g) * 0.2).to(torch.bfloat16)
    gates = torch.rand(tokens, top, generator=g) + 0.25
    xs = torch.empty((pairs, K), dtype=torch.bfloat16, device=DEV)
    kernels.gather_rows(x.to(DEV), perm, top, xs)
    order = perm.cpu().long()
    assert torch.equal(xs.cpu(), x[order // top])
    assert torch.equal(ids.view(-1).cpu()[order], torch.sort(ids.view(-1).cpu()).values)
    u = torch.empty((pairs, N), dtype=torch.bfloat16, device=DEV)
    kernels.experts_linear_tc(xs, w.to(DEV), u, perm, offsets, tiles, top, tokens, scale=gates.to(DEV), activation="relu2")
    y = torch.empty((top, tokens, N), dtype=torch.float32, device=DEV)
    kernels.experts_linear_tc(xs, w.to(DEV), y, perm, offsets, tiles, top, tokens, down=True)
    assert kernels.grouped_tc_status() == 0
    flat_ids = ids.view(-1).cpu().long()
    sums = torch.einsum("pk,pnk->pn", x.double()[torch.arange(pairs) // top], w.double()[flat_ids])      # by pair
    ref_u = torch.relu(sums * gates.view(-1, 1).double()) ** 2
    assert rel(u.cpu()[torch.argsort(order)], ref_u) < 8e-3
    ref_y = sums.view(tokens, top, N).transpose(0, 1)
    assert rel(y, ref_y) < 1e-5 + 1e-6 * K


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,H,N,K,a_head,o_head", [(1, 3, 16, 8, 24, 16), (70, 5, 40, 24, 24, 48), (130, 2, 9, 13, 20, 11),
                                                   (65, 18, 12, 6, 10, 16)])
def test_product_per_head(dtype, T, H, N, K, a_head, o_head):
    g = torch.Generator().manual_seed(H)
    a = torch.randn(T, H * a_head + 3, generator=g).to(dtype)
    w = torch.randn(H, N, K, generator=g).to(dtype)
    for out_dtype in {dtype, torch.float32}:
        out = torch.full((T, H * o_head), 7.0, dtype=out_dtype, device=DEV)
        kernels.heads_linear(a.to(DEV), a_head, w.to(DEV), out, o_head)
        ref = torch.full((T, H, o_head), 7.0, dtype=torch.float64)
        ref[:, :, :N] = torch.einsum("thk,hnk->thn", a[:, :H * a_head].view(T, H, a_head)[:, :, :K].double(), w.double())
        assert rel(out, ref.view(T, -1)) <= (1e-5 if out_dtype == torch.float32 and dtype == torch.float32 else 1e-2)


# ---------------------------------------------------------------------------------------------------------
def plain_rows_attention(q, rows, scale, window, sink, first_pos):
    """q [T, H, D] at positions first_pos .., rows [n, D] the cached rows of positions 0 .. n-1 (key and value at
    once): out [T, H, D]."""
    T, H, D = q.shape
    out = torch.zeros(T, H, D, dtype=torch.float64)
    for t in range(T):
        p = first_pos + t
        lo = 0 if not window else max(0, p - window + 1)
        for h in range(H):
            s = (rows[lo:p + 1] @ q[t, h]) * scale
            e = torch.exp(s - s.max())
            den = e.sum() + (math.exp(float(sink[h]) - float(s.max())) if sink is not None else 0.0)
            out[t, h] = (e / den) @ rows[lo:p + 1]
    return out


def standout(n, D, H, window, g):
    """Rows and queries such that, for the last query, the keys just inside and just outside its window (or, without
    a window, the first key) would each take nearly all the weight if they were seen."""
    rows = torch.randn(n, D, generator=g) * 0.3
    q = torch.randn(n, H, D, generator=g) * 0.3
    mark = torch.zeros(D)
    mark[5] = 1.0
    q[-1] += 6.0 * mark
    edge = n - window if window else 0                  # the last key the last query still sees
    rows[edge] += 5.0 * mark
    if window and edge > 0:
        rows[edge - 1] += 9.0 * mark                    # would win if the window were one wider
    return q, rows


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,window", [(200, 0), (200, 64), (200, 65), (130, 9), (64, 64), (65, 64), (300, 136), (40, 1)])
@pytest.mark.parametrize("H", [3, 8, 18])
def test_attention_over_shared_rows_with_a_sink(dtype, n, window, H):
    """Prompts (packed rows) and decoding (paged rows, scattered pages), exact kernel and tensor-core kernels."""
    D, scale = 48, 0.5
    g = torch.Generator().manual_seed(n + window + H)
    q, rows = standout(n, D, H, window, g)
    q, rows = q.to(dtype), rows.to(dtype)
    sink = torch.randn(H, generator=g) + 1.0
    ref = plain_rows_attention(q.double(), rows.double(), scale, window, sink.double(), 0)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    qd, rd, sd = q.reshape(n, H * D).to(DEV), rows.to(DEV), sink.to(DEV)
    cu, kvl = i32([0, n]), i32([n])
    common = dict(n_kv=1, group=H, head_dim=D, scale=scale, cap=0.0, window=window, batch=1, sink=sd)
    out = torch.empty_like(qd)
    kernels.attention_simt(qd, out, cu, kvl, k=rd, v=rd, max_q_len=n, **common)
    assert rel(out, ref.view(n, -1)) <= tol, "exact kernel, prompt"
    if dtype == torch.bfloat16:
        out = torch.empty_like(qd)
        kernels.attention_prefill_mma(qd, out, cu, rd, rd, max_q_len=n, **common)
        assert rel(out, ref.view(n, -1)) <= tol, "tensor cores, prompt"
    # the last query alone, over pages in a scattered order (a ring when there is a window)
    ring = (window + 63) // 64 * 64 if window else 1 << 30
    n_pages = ring // 64 if window else (n + 63) // 64
    order = torch.randperm(n_pages + 3, generator=g)[:n_pages].tolist()
    pages = torch.full((n_pages + 3, 1, 64, D), float("nan")).to(dtype)          # never written: NaN
    first_kept = max(0, n - ring) if window else 0
    for p in range(first_kept, n):
        r = p % ring
        pages[order[r // 64], 0, r % 64] = rows[p]
    table = i32([order])
    q1 = qd[n - 1:n].contiguous()
    kw = dict(common, batch=1)
    out1 = torch.empty_like(q1)
    kernels.attention_simt(q1, out1, i32([0, 1]), kvl, k_pages=pages.to(DEV), v_pages=pages.to(DEV), page_table=table,
                           ring=ring, page_size=64, max_q_len=1, **kw)
    assert rel(out1, ref[n - 1].view(1, -1)) <= tol, "exact kernel, decoding"
    if dtype == torch.bfloat16 and H <= 16:
        pd = pages.to(DEV)
        for splits in (1, 2, 3, 5):
            out1 = torch.empty_like(q1)
            kernels.attention_decode_mma(q1, out1, i32([0, 1]), kvl, pd, pd, table, ring=ring, page_size=64,
                                         n_splits=splits, **{k: v for k, v in kw.items()})
            assert rel(out1, ref[n - 1].view(1, -1)) <= tol, f"tensor cores, decoding, {splits} splits"


# ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,dn,dr,dv,R,rd,window", [(3, 8, 16, 24, 24, 8, 9), (18, 6, 4, 10, 12, 4, 64), (2, 16, 8, 8, 40, 8, 70),
                                                     (5, 8, 8, 16, 16, 8, None), (1, 24, 8, 32, 56, 0, 5)])
def test_latent_mixer_prompt_then_decode(dtype, H, dn, dr, dv, R, rd, window):
    hidden, eps, base, scale = 40, 1e-5, 300.0, 0.3
    rope = RotaryEmbedding(dr, base, rd) if rd else None
    att = LatentAttention(hidden, H, dn, dr, dv, R, scale, eps, window, True, rope)
    g = torch.Generator().manual_seed(H)
    ws = {n: (torch.randn(s.shape, generator=g) * (0.3 if n != "sink" else 1.0)).to(dtype)
          for n, s in att.param_specs().items()}
    att.bind({n: t.to(DEV) for n, t in ws.items()})
    cache = Cache([att.cache_spec()], 1024, dtype, DEV)
    att.prepare(1024, DEV)
    lengths = [150, 3, 66]
    extra = 70                                              # decoded tokens: past the ring of every window here
    xs = [torch.randn(n + extra, hidden, generator=g).to(dtype) for n in lengths]
    m = dict(heads=H, dim=dn, rot_dim=dr, vdim=dv, kv_rank=R, scale=scale, rot=dict(base=base, dims=rd))
    if window:
        m["mask"] = dict(size=window)
    w = {"p." + n.replace("dkv_norm", "dkv.norm"): t for n, t in ws.items()}
    refs = [plain.latent_attention(m, w, "p.", x.double(), eps) for x in xs]
    tol = TOL[dtype]
    ctx = make_ctx(cache, "prefill", [0, 0, 0], lengths, dtype)
    y = att.forward(torch.cat([x[:n] for x, n in zip(xs, lengths)]).to(DEV), ctx, cache.entries[0])
    y = y.sum(dim=0) if y.dim() == 3 else y
    at = 0
    for r, n in zip(refs, lengths):
        assert rel(y[at:at + n], r[:n]) <= tol
        at += n
    for j in range(extra):
        ctx = make_ctx(cache, "decode", [n + j for n in lengths], [1, 1, 1], dtype)
        y = att.forward(torch.stack([x[n + j] for x, n in zip(xs, lengths)]).to(DEV), ctx, cache.entries[0])
        y = y.sum(dim=0) if y.dim() == 3 else y
        for b, (r, n) in enumerate(zip(refs, lengths)):
            assert rel(y[b], r[n + j]) <= tol, (j, b)
