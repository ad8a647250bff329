"""Neburax's mechanisms one by one on the GPU, each against its function of the plain implementation, with
made-up inputs where random ones would hide a fault: one key that carries the weight just inside and just outside
a chunk, at a page border and hundreds of places back; states that remember for thousands of tokens; a router
whose correction changes the choice but not the weights; experts with identity choices; sizes that the shipped
kernels treat differently (states per thread, taps, blocks)."""
import math

import pytest
import torch

from brolm_b200 import kernels
from brolm_b200.cache import Cache
from brolm_b200.parts import Attention, DenseFeedForward, GatedFeedForward, GatedRecurrence, RoutedExperts, SideBySide, StateSpace
from tests.plain import neburax_plain as plain
from tests.test_parts_gpu import make_ctx

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = {torch.float32: 2e-5, torch.bfloat16: 3e-2}


def rel(got, ref):
    ref = ref.double()
    return float((got.double().cpu() - ref).abs().max()) / max(float(ref.abs().max()), 1e-6)


def i32(v):
    return torch.tensor(v, dtype=torch.int32, device=DEV)


def weights(part, g, dtype, std=0.3, scales=None):
    ws = {}
    for n, s in part.param_specs().items():
        ws[n] = (torch.randn(s.shape, generator=g) * (scales or {}).get(n, std)).to(dtype)
    return ws


def run_part(part, cache, xs, lengths, extra, dtype, refs, tol, what):
    """A prompt of ``lengths[b]`` tokens per sequence in one step, then ``extra`` tokens one by one."""
    ctx = make_ctx(cache, "prefill", [0] * len(lengths), lengths, dtype)
    y = part.forward(torch.cat([x[:n] for x, n in zip(xs, lengths)]).to(DEV), ctx, cache.entries[0])
    y = y.sum(dim=0) if y.dim() == 3 else y
    at = 0
    for b, (r, n) in enumerate(zip(refs, lengths)):
        assert rel(y[at:at + n], r[:n]) <= tol, f"{what}: prompt of sequence {b}"
        at += n
    for j in range(extra):
        ctx = make_ctx(cache, "decode", [n + j for n in lengths], [1] * len(lengths), dtype)
        y = part.forward(torch.stack([x[n + j] for x, n in zip(xs, lengths)]).to(DEV), ctx, cache.entries[0])
        y = y.sum(dim=0) if y.dim() == 3 else y
        for b, (r, n) in enumerate(zip(refs, lengths)):
            assert rel(y[b], r[n + j]) <= tol * max(1.0, float(r.abs().max() / r[n + j].abs().max().clamp_min(1e-9)) ** 0), \
                f"{what}: decoded token {j} of sequence {b}"


# ---------------------------------------------------------------------------------------------------------
def chunk_ref(q, k, v, H, G, d, dv, scale, chunk):
    T = q.shape[0]
    q, k, v = q.double().view(T, H, d), k.double().view(T, G, d), v.double().view(T, G, dv)
    seen = plain.chunk_mask(T, chunk)
    outs = []
    for h in range(H):
        s = (q[:, h] @ k[:, h // (H // G)].T) * scale
        outs.append(torch.softmax(s.masked_fill(~seen, float("-inf")), dim=-1) @ v[:, h // (H // G)])
    return torch.cat(outs, dim=-1)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,dv,chunk,n", [(4, 2, 8, 16, 9, 40), (3, 3, 24, 24, 64, 200), (6, 1, 12, 6, 70, 200), (5, 5, 10, 14, 33, 100),
                                             (2, 1, 16, 32, 1, 20), (4, 2, 64, 128, 512, 700), (8, 2, 32, 8, 128, 300)])
def test_chunked_attention_kernel_with_one_key_that_carries_the_weight(dtype, H, G, d, dv, chunk, n):
    """The key at a chunk's first place carries the weight for the chunk's last query (hundreds of places back when
    the chunk is long); the key one place earlier, just outside, is made ten times as loud and must not be heard.
    Packed keys (a prompt) and paged keys (decoding) with scattered pages, chunk edges on and off page borders."""
    g = torch.Generator().manual_seed(n + chunk)
    scale = 0.25
    q = torch.randn(n, H * d, generator=g) * 0.3
    k = torch.randn(n, G * d, generator=g) * 0.3
    v = torch.randn(n, G * dv, generator=g)
    last_start = (n - 1) // chunk * chunk                       # first place of the last chunk
    probe = min(n - 1, last_start + chunk - 1)                  # its last query present
    q[probe] = 0.0
    q[probe].view(H, d)[:, 0] = 6.0
    k[last_start].view(G, d)[:, 0] = 6.0
    if last_start > 0:
        k[last_start - 1].view(G, d)[:, 0] = 60.0               # just outside: louder, and unseen
    q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
    ref = chunk_ref(q, k, v, H, G, d, dv, scale, chunk)
    if chunk > 1 and probe > last_start:
        want = torch.cat([v.double().view(n, G, dv)[last_start, h // (H // G)] for h in range(H)])
        assert rel(ref[probe], want) < 0.05                     # the made-up key does carry the weight in the oracle
    common = dict(n_kv=G, group=H // G, head_dim=d, scale=scale, cap=0.0, window=0, batch=1, v_dim=dv, chunk=chunk)
    out = torch.empty(n, H * dv, dtype=dtype, device=DEV)
    kernels.attention_simt(q.to(DEV), out, i32([0, n]), i32([n]), k=k.to(DEV), v=v.to(DEV), max_q_len=n, **common)
    assert rel(out, ref) <= TOL[dtype], "packed"
    # paged: the ring a chunk needs, pages scattered, only the last chunk's places filled (the rest holds NaN)
    ring = (chunk + 63) // 64 * 64
    n_pages = ring // 64
    table = torch.randperm(n_pages + 3, generator=g)[:n_pages].to(torch.int32)
    kp = torch.full((n_pages + 3, G, 64, d), float("nan"), dtype=dtype)
    vp = torch.full((n_pages + 3, G, 64, dv), float("nan"), dtype=dtype)
    for pos in range(max(0, n - ring), n):
        r = pos % ring
        kp[table[r // 64], :, r % 64] = k[pos].view(G, d)
        vp[table[r // 64], :, r % 64] = v[pos].view(G, dv)
    for pos in (n - 1, probe):
        if pos < n - 1:
            continue
        one = torch.empty(1, H * dv, dtype=dtype, device=DEV)
        kernels.attention_simt(q[pos:pos + 1].to(DEV), one, i32([0, 1]), i32([pos + 1]), k_pages=kp.to(DEV),
                               v_pages=vp.to(DEV), page_table=table.view(1, -1).to(DEV), ring=ring, page_size=64,
                               max_q_len=1, **common)
        assert rel(one, ref[pos:pos + 1]) <= TOL[dtype], "paged"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,dv,chunk", [(4, 2, 8, 16, 9), (3, 3, 24, 24, 64), (6, 1, 12, 6, 70), (5, 5, 10, 14, 33), (2, 1, 16, 32, 1),
                                            # key and value rows of one size, a multiple of 16: in bfloat16 the tensor-core kernels
                                            (4, 2, 32, 32, 9), (2, 1, 64, 64, 70), (2, 2, 128, 128, 100), (4, 1, 16, 16, 1),
                                            (2, 1, 48, 48, 33), (8, 2, 64, 64, 64), (2, 1, 32, 32, 1000)])
def test_attention_part_with_whole_row_norm_prompt_then_decode(dtype, H, G, d, dv, chunk):
    hidden, eps, scale = 40, 1e-5, 0.3
    att = Attention(hidden, H, G, d, scale, v_dim=dv, qk_norm="whole", eps=eps, chunk=chunk)
    g = torch.Generator().manual_seed(H * 100 + chunk)
    ws = weights(att, g, dtype, scales={"q_norm": 1.0, "k_norm": 1.0})
    att.bind({n: t.to(DEV) for n, t in ws.items()})
    cache = Cache([att.cache_spec()], 1024, dtype, DEV)
    lengths, extra = [150, 3, 66], 80
    xs = [torch.randn(n + extra, hidden, generator=g).to(dtype) for n in lengths]
    m = dict(heads=H, kv_heads=G, dim=d, vdim=dv, scale=scale, mask=dict(size=chunk))
    w = {"p." + n.replace("_norm", ".norm"): t.double() for n, t in ws.items()}
    refs = [plain.chunked_attention(x.double(), w, "p.", m, eps) for x in xs]
    run_part(att, cache, xs, lengths, extra, dtype, refs, TOL[dtype], "chunked attention")


# ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("C,K", [(5, 1), (40, 2), (300, 4), (33, 7)])
def test_causal_convolution_prompt_then_tokens(C, K):
    g = torch.Generator().manual_seed(C)
    lengths, extra = [1, 2, K + 3, 70], 2 * K + 1           # 76 tokens and more in the prompt step: a thread takes a run of tokens
    taps, bias, in_bias = torch.randn(C, K, generator=g), torch.randn(C, generator=g), torch.randn(C, generator=g)
    xs = [torch.randn(n + extra, C, generator=g) for n in lengths]
    refs = [plain.silu(plain.causal_conv(x.double() + in_bias.double(), taps.double(), bias.double())) for x in xs]
    state = torch.zeros(len(lengths) + 1, 7 + (K - 1) * C, device=DEV)
    slots, B = i32(list(range(len(lengths)))), len(lengths)
    consts = (in_bias.to(DEV), taps.to(DEV), bias.to(DEV), "silu")

    def step(rows, before, n_new):
        x = torch.cat(rows).to(DEV)
        cu = [0]
        for n in n_new:
            cu.append(cu[-1] + n)
        seq = (i32(cu), i32([a + b for a, b in zip(before, n_new)]), slots, state)
        out = torch.empty(x.shape, dtype=torch.float32, device=DEV)
        kernels.causal_conv(x, *consts, i32([b for b, n in enumerate(n_new) for _ in range(n)]),
                            i32([p for a, n in zip(before, n_new) for p in range(a, a + n)]), *seq, 7, out)
        kernels.conv_tail(x, consts[0], K, *seq, 7, B)
        return out

    out = step([x[:n] for x, n in zip(xs, lengths)], [0] * B, lengths)
    at = 0
    for r, n in zip(refs, lengths):
        assert rel(out[at:at + n], r[:n]) <= 2e-6
        at += n
    for j in range(extra):
        out = step([x[n + j:n + j + 1] for x, n in zip(xs, lengths)], [n + j for n in lengths], [1] * B)
        for b, (r, n) in enumerate(zip(refs, lengths)):
            assert rel(out[b], r[n + j]) <= 2e-6, (j, b)
    assert float(state[:, :7].abs().max()) == 0.0 and float(state[B].abs().max()) == 0.0      # only the tails, only its rows


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,blocks,taps", [(32, 2, 4), (40, 1, 1), (24, 3, 2), (256, 4, 3), (48, 48, 5)])
def test_gated_recurrence_prompt_then_decode(dtype, width, blocks, taps):
    hidden = 40
    part = GatedRecurrence(hidden, width, blocks, taps, decay_scale=8.0)
    g = torch.Generator().manual_seed(width + taps)
    ws = weights(part, g, dtype, scales={"lam": 1.5, "ra_bias": 1.0, "ri_bias": 1.0})
    part.bind({n: t.to(DEV) for n, t in ws.items()})
    cache = Cache([part.cache_spec()], 1024, dtype, DEV)
    lengths, extra = [150, 3, 66], 40
    xs = [torch.randn(n + extra, hidden, generator=g).to(dtype) for n in lengths]
    m = dict(width=width, blocks=blocks, conv=taps)
    w = {"p." + n.replace("_bias", ".b"): t.double() for n, t in ws.items()}
    refs = [plain.gated_recurrence(x.double(), w, "p.", m) for x in xs]
    run_part(part, cache, xs, lengths, extra, dtype, refs, TOL[dtype], "gated recurrence")


def test_gated_scan_remembers_for_thousands_of_tokens():
    """Decays within 1e-4 of one: the first token's input is still most of the state 3,000 tokens later, in a prompt
    and token by token alike."""
    W, T = 64, 3000
    g = torch.Generator().manual_seed(9)
    pre = torch.zeros(T, 2 * W)
    pre[:, :W] = -3.0 + 0.1 * torch.randn(T, W, generator=g)          # r small: slow decay
    pre[:, W:] = 4.0
    u = torch.randn(T, W, generator=g) * 1e-3
    u[0] = 50.0
    lam = torch.full((W,), -8.0)
    y_raw = torch.randn(T, W, generator=g)
    r, i = torch.sigmoid(pre[:, :W].double()), torch.sigmoid(pre[:, W:].double())
    log_a = -8.0 * r * plain.softplus(lam.double())
    a = torch.exp(log_a)
    S, ref = torch.zeros(W, dtype=torch.float64), []
    for t in range(T):
        S = a[t] * S + torch.sqrt(1 - a[t] ** 2) * i[t] * u[t].double()
        ref.append(S * plain.gelu_tanh(y_raw[t].double()))
    ref = torch.stack(ref)
    zeros = torch.zeros(W, device=DEV)
    for cut in (T, 1, 2000):
        state = torch.zeros(2, W, device=DEV)
        out = torch.empty(T, W, device=DEV)
        args = lambda lo, hi: (pre[lo:hi].to(DEV), u[lo:hi].to(DEV), y_raw[lo:hi].to(DEV), None, zeros, zeros, lam.to(DEV), 8.0, W)
        kernels.gated_scan(*args(0, cut), i32(list(range(cut))), i32([0, cut]), i32([cut]), i32([0]), state, out[:cut], 1, cut)
        for t in range(cut, T):
            kernels.gated_scan(*args(t, t + 1), i32([t]), i32([0, 1]), i32([t + 1]), i32([0]), state, out[t:t + 1], 1, 1)
            if cut == 2000 and t > 2040:
                out[t + 1:] = ref[t + 1:].float().to(DEV)
                break
        assert rel(out, ref) <= 2e-5, cut
    assert float(ref[-1].abs().max()) > 0.1 * float(ref[1].abs().max())


def test_two_halves_keep_sixteen_bits_and_two_part_gate_sums_add_up():
    g = torch.Generator().manual_seed(3)
    u = torch.randn(37, 50, generator=g) * torch.logspace(-6, 3, 50)
    out = torch.empty(74, 50, dtype=torch.bfloat16, device=DEV)
    kernels.split_halves(u.to(DEV), out)
    back = out[:37].double().cpu() + out[37:].double().cpu()
    assert float(((back - u.double()).abs() / u.double().abs().clamp_min(1e-30)).max()) <= 2.0 ** -16
    assert torch.equal(out[:37].cpu(), u.to(torch.bfloat16))
    # the recurrence from sums given in two parts is the recurrence from their sum
    W, T = 32, 100
    pre, u2, y_raw = torch.randn(T, 2 * W, generator=g), torch.randn(T, W, generator=g), torch.randn(T, W, generator=g)
    part = torch.randn(T, 2 * W, generator=g)
    vecs = [torch.randn(W, generator=g).to(DEV) for _ in range(4)]
    outs = []
    for a, b in ((pre, None), (pre - part, part)):
        state = torch.zeros(2, W, device=DEV)
        o = torch.empty(T, W, device=DEV)
        kernels.gated_scan(a.to(DEV), u2.to(DEV), y_raw.to(DEV), *vecs, 8.0, 8, i32(list(range(T))), i32([0, T]), i32([T]), i32([0]),
                           state, o, 1, T, pre_lo=b.to(DEV) if b is not None else None)
        outs.append(o)
    assert rel(outs[1], outs[0].cpu()) <= 1e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,P,N,groups,norm_groups,taps", [(4, 8, 16, 2, 1, 2), (2, 24, 12, 1, 3, 5), (5, 8, 40, 5, 5, 3),
                                                                (1, 32, 64, 1, 2, 4), (2, 16, 100, 2, 4, 4), (2, 8, 128, 1, 1, 1),
                                                                (3, 40, 256, 3, 1, 2), (8, 64, 2, 4, 8, 4)])
def test_state_space_prompt_then_decode(dtype, heads, P, N, groups, norm_groups, taps):
    hidden, eps = 40, 1e-5
    part = StateSpace(hidden, heads, P, N, groups, norm_groups, taps, eps)
    g = torch.Generator().manual_seed(heads * 1000 + N)
    ws = weights(part, g, dtype, std=0.2, scales={"A_log": 1.0, "D": 1.0, "dt_bias": 1.0, "norm": 1.0})
    part.bind({n: t.to(DEV) for n, t in ws.items()})
    cache = Cache([part.cache_spec()], 1024, dtype, DEV)
    lengths, extra = [150, 3, 17], 20
    xs = [torch.randn(n + extra, hidden, generator=g).to(dtype) for n in lengths]
    m = dict(heads=heads, vdim=P, state=N, groups=groups, norm_groups=norm_groups, conv=taps)
    w = {"p." + n.replace("_bias", ".b").replace("dt.b", "dt_bias"): t.double() for n, t in ws.items()}
    refs = [plain.state_space(x.double(), w, "p.", m, eps) for x in xs]
    run_part(part, cache, xs, lengths, extra, dtype, refs, TOL[dtype] * (2 if dtype == torch.bfloat16 else 1), "state space")


def test_state_space_scan_remembers_for_thousands_of_tokens():
    heads, P, N, T = 2, 8, 16, 3000
    g = torch.Generator().manual_seed(5)
    xbc = torch.randn(T, heads * P + 2 * N, generator=g) * 1e-3
    xbc[0, :heads * P] = 30.0
    xbc[0, heads * P:heads * P + N] = 1.0                                  # B of the first token
    xbc[-1, heads * P + N:] = 1.0                                          # C of the last one asks for it
    dt_raw = torch.full((T, heads), -7.0) + 0.1 * torch.randn(T, heads, generator=g)
    a_log, d, dtb = torch.tensor([-2.0, -1.0]), torch.tensor([0.5, -0.5]), torch.zeros(heads)
    dt = plain.softplus(dt_raw.double())
    ref = torch.zeros(T, heads, P, dtype=torch.float64)
    for h in range(heads):
        S = torch.zeros(N, P, dtype=torch.float64)
        for t in range(T):
            x = xbc[t, h * P:(h + 1) * P].double()
            S = torch.exp(-torch.exp(a_log[h].double()) * dt[t, h]) * S + dt[t, h] * torch.outer(xbc[t, heads * P:heads * P + N].double(), x)
            ref[t, h] = S.T @ xbc[t, heads * P + N:].double() + d[h] * x
    ref = ref.view(T, heads * P)
    assert float(ref[-1].abs().max()) > 0.2                                # the first token is what the last one hears
    for cut in (T, 1):
        state = torch.zeros(2, heads * P * N, device=DEV)
        y = torch.empty(T, heads * P, device=DEV)
        consts = (dtb.to(DEV), a_log.to(DEV), d.to(DEV), heads, 1, P, N)
        kernels.ssm_scan(xbc[:cut].to(DEV), dt_raw[:cut].to(DEV), *consts, i32([0, cut]), i32([cut]), i32([0]), state, y[:cut], 1, cut)
        for t in range(cut, T):
            kernels.ssm_scan(xbc[t:t + 1].to(DEV), dt_raw[t:t + 1].to(DEV), *consts, i32([0, 1]), i32([t + 1]), i32([0]), state,
                             y[t:t + 1], 1, 1)
        assert rel(y, ref) <= 2e-5, cut


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_two_mixers_side_by_side(dtype):
    hidden, eps = 48, 1e-5
    left = Attention(hidden, 4, 2, 8, 0.3, v_dim=16, qk_norm="whole", eps=eps, chunk=70)
    right = GatedRecurrence(hidden, 32, 2, 4)
    both = SideBySide(left, right, 0.7, 1.3)
    g = torch.Generator().manual_seed(21)
    wl, wr = weights(left, g, dtype, scales={"q_norm": 1.0, "k_norm": 1.0}), weights(right, g, dtype, scales={"lam": 1.0})
    left.bind({n: t.to(DEV) for n, t in wl.items()})
    right.bind({n: t.to(DEV) for n, t in wr.items()})
    cache = Cache([both.cache_spec()], 1024, dtype, DEV)
    lengths, extra = [100, 5], 50
    xs = [torch.randn(n + extra, hidden, generator=g).to(dtype) for n in lengths]
    w = {"p.left." + n.replace("_norm", ".norm"): t.double() for n, t in wl.items()}
    w.update({"p.right." + n.replace("_bias", ".b"): t.double() for n, t in wr.items()})
    m = dict(left=dict(heads=4, kv_heads=2, dim=8, vdim=16, scale=0.3, mask=dict(size=70)),
             right=dict(width=32, blocks=2, conv=4), left_scale=0.7, right_scale=1.3)
    refs = [plain.parallel_mixer(x.double(), w, "p.", m, eps) for x in xs]
    run_part(both, cache, xs, lengths, extra, dtype, refs, TOL[dtype], "two mixers side by side")


# ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_dense_feed_forward_with_biases(dtype):
    part = DenseFeedForward(40, 56, "relu2", True)
    g = torch.Generator().manual_seed(2)
    ws = weights(part, g, dtype)
    part.bind({n: t.to(DEV) for n, t in ws.items()})
    w = {"p." + n.replace("_bias", ".b"): t.double() for n, t in ws.items()}
    for T in (1, 5, 40, 300):
        x = torch.randn(T, 40, generator=g).to(dtype)
        ctx = type("Ctx", (), {"dtype": dtype})()
        assert rel(part.forward(x.to(DEV), ctx), plain.dense_ff(x.double(), w, "p.")) <= TOL[dtype]


@pytest.mark.parametrize("tokens", [1, 7, 300])
@pytest.mark.parametrize("E,ident,top", [(5, 2, 2), (4, 0, 1), (0, 2, 2), (3, 1, 4), (16, 3, 6)])
def test_softmax_router_with_a_correction_that_moves_the_choice_only(E, ident, top, tokens):
    g = torch.Generator().manual_seed(E * 10 + top)
    n, W = E + ident, 40
    x, wr = torch.randn(tokens, W, generator=g), torch.randn(n, W, generator=g) * 0.3
    corr = torch.randn(n, generator=g) * 0.5
    s = torch.softmax(x.double() @ wr.double().T, dim=-1)
    want_ids = torch.topk(s + corr.double(), top, dim=-1).indices
    want_w = torch.gather(s, 1, want_ids)
    want_w = want_w / (want_w.sum(-1, keepdim=True) + 1e-20)
    ids = torch.empty(tokens, top, dtype=torch.int32, device=DEV)
    wts = torch.empty(tokens, top, dtype=torch.float32, device=DEV)
    kernels.route_topk(x.to(DEV), wr.to(DEV), top, ids, wts, "softmax", corr.to(DEV))
    assert torch.equal(ids.cpu().long(), want_ids) and rel(wts, want_w) <= 1e-5
    z = (x @ wr.T).to(DEV)
    kernels.route_pick(z, top, ids, wts, "softmax", corr.to(DEV))
    assert torch.equal(ids.cpu().long(), want_ids) and rel(wts, want_w) <= 1e-5
    if top < n:
        plain_ids = torch.topk(s, top, dim=-1).indices
        assert not torch.equal(plain_ids, want_ids) or tokens == 1            # the correction does move choices


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("E,ident,top,shared", [(5, 2, 2, 16), (4, 0, 1, 0), (0, 2, 2, 24), (3, 1, 4, 8)])
@pytest.mark.parametrize("tokens", [1, 9, 700])
def test_routed_experts_with_identity_and_shared_experts(dtype, E, ident, top, shared, tokens):
    """Whatever the run chose (a rounded run may choose otherwise than float64 would where scores are close), its
    result must be the plain weighted sum for that choice; in float32 the choice itself is the oracle's."""
    W, ff = 40, 24
    sh = GatedFeedForward(W, shared, "silu") if shared else None
    part = RoutedExperts(W, ff, E, top, activation="silu", scale_input=False, router="softmax", correction=True, gated=True,
                         identity=ident, shared=sh)
    g = torch.Generator().manual_seed(E + tokens)
    ws = weights(part, g, dtype, scales={"correction": 0.3})
    part.bind({n: t.to(DEV) for n, t in ws.items()})
    w = {"p." + n: t.double() for n, t in ws.items()}
    if sh is not None:
        wsh = weights(sh, g, dtype)
        sh.bind({n: t.to(DEV) for n, t in wsh.items()})
        w.update({"p.shared." + n: t.double() for n, t in wsh.items()})
    x = torch.randn(tokens, W, generator=g).to(dtype)
    ctx = type("Ctx", (), {"dtype": dtype})()
    got = part.forward(x.to(DEV), ctx)
    assert got.shape == (tokens, W) and got.dtype == torch.float32
    mlp = dict(kind="moe", expert=dict(ff=ff), router=dict(experts=E, top=top, identity=ident), shared=dict(ff=shared) if shared else None)
    choices = []
    ref = plain.mixture_ff(x.double(), w, "p.", mlp, choices)
    if dtype == torch.float32 or top == E + ident:
        assert rel(got, ref) <= TOL[dtype]
    else:
        err = ((got.double().cpu() - ref).abs().amax(dim=1) / ref.abs().max()).sort().values
        assert float(err[len(err) // 2]) <= TOL[dtype]
