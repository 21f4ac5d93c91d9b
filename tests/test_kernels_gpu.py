"""Each kernel alone against a plain 32-bit torch statement of the same operation,
at sizes other than the engine's (odd widths, head sizes in steps of 16, page
edges, windows)."""
import math
import random

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
# error relative to the largest |expected| value
TOL = {"float32": 3e-6, "bfloat16": 1.2e-2}


def ops():
    from ferrox_b200.kernels import ops as o

    return o


def rel(got, want):
    return float((got.float() - want.float()).abs().max() / want.float().abs().max().clamp_min(1e-30))


def rnd(*shape, dtype=torch.float32, scale=1.0, seed=None):
    g = torch.Generator().manual_seed(seed if seed is not None else sum(shape) + len(shape))
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


# ------------------------------------------------------------------ matrix products
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("M,N,K", [(1, 7, 5), (3, 130, 77), (70, 65, 64), (129, 33, 250), (64, 64, 16)])
def test_gemm_generic(dtype, M, N, K):
    o, dt = ops(), DT[dtype]
    a, w, bias = rnd(M, K, dtype=dt), rnd(N, K, dtype=dt), rnd(N, dtype=torch.float32)
    want = a.float() @ w.float().T + bias
    out = torch.empty(M, N, dtype=dt, device=DEV)
    o.gemm(a, w, out, bias=bias)
    assert rel(out, want) < TOL[dtype]
    acc = rnd(M, N, dtype=torch.float32, seed=5)
    base = acc.clone()
    o.gemm(a, w, acc, accumulate=True)  # 32-bit output, added to what is there
    assert rel(acc, base + a.float() @ w.float().T) < (3e-6 if dtype == "float32" else 1e-5)


def test_gemm_mixed_precision_weights_stay_32_bit():
    o = ops()
    a, w = rnd(5, 96, dtype=torch.bfloat16), rnd(40, 96, dtype=torch.float32)
    out = torch.empty(5, 40, dtype=torch.float32, device=DEV)
    o.gemm(a, w, out)
    assert rel(out, a.float() @ w.T) < 3e-6  # no rounding of the 32-bit weights


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_gemm_grouped_with_gather(dtype):
    o, dt = ops(), DT[dtype]
    G, N, K, T = 5, 37, 48, 23
    x, w = rnd(T, K, dtype=dt), rnd(G, N, K, dtype=dt)
    counts = [0, 9, 1, 0, 13]
    offsets = torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int32, device=DEV)
    rows = torch.randint(0, T, (sum(counts),), generator=torch.Generator().manual_seed(1)).to(torch.int32).to(DEV)
    out = torch.zeros(sum(counts), N, dtype=dt, device=DEV)
    o.gemm(x, w, out, a_rows=rows, group_offsets=offsets)
    r = 0
    for g, c in enumerate(counts):
        for _ in range(c):
            want = x[rows[r]].float() @ w[g].float().T
            assert rel(out[r], want) < TOL[dtype]
            r += 1


@pytest.mark.parametrize("T", [1, 3, 8, 9, 17, 40, 64])
@pytest.mark.parametrize("N,K", [(16, 32), (60, 64), (1, 96), (200, 2048), (33, 160), (9493, 64)])
def test_gemm_skinny(T, N, K):
    o = ops()
    x, w, bias = rnd(T, K, dtype=torch.bfloat16), rnd(N, K, dtype=torch.bfloat16, scale=0.1), rnd(N)
    want = x.float() @ w.float().T + bias
    out = torch.empty(T, N, dtype=torch.bfloat16, device=DEV)
    o.gemm_skinny(x, w, out, bias=bias)
    assert rel(out, want) < TOL["bfloat16"]
    acc = rnd(T, N, seed=3)
    base = acc.clone()
    o.gemm_skinny(x, w, acc, accumulate=True)
    assert rel(acc, base + x.float() @ w.float().T) < 2e-5
    # gated: silu(gate) * up in the epilogue
    if N > 1:
        wg = rnd(2 * N, K, dtype=torch.bfloat16, scale=0.1, seed=9)
        gate, up = x.float() @ wg[:N].float().T, x.float() @ wg[N:].float().T
        got = torch.empty(T, N, dtype=torch.float32, device=DEV)
        o.gemm_skinny(x, wg, got, gated=True)
        assert rel(got, gate / (1 + torch.exp(-gate)) * up) < 2e-5


@pytest.mark.parametrize("T", [1, 5, 8, 13, 32])
@pytest.mark.parametrize("N,K", [(6144, 2048), (1000, 384), (2048, 2048), (61, 128), (7, 1408), (3001, 1024)])
def test_gemm_slab_holds_its_rows_of_the_matrix_in_shared_memory(T, N, K):
    """The product for a few tokens that asks for the whole matrix before it waits for the kernel before it:
    against the 32-bit product, with a bias, added to a 32-bit result, rows of x wider than K, after a kernel
    that is still running when it starts (the same stream: its wait is what orders them)."""
    o = ops()
    xw = rnd(T, K + 24, dtype=torch.bfloat16)
    x = xw[:, :K]
    w, bias = rnd(N, K, dtype=torch.bfloat16, scale=0.1), rnd(N)
    assert o.slab_ok(x, w)
    want = x.float() @ w.float().T
    out = torch.empty(T, N, dtype=torch.bfloat16, device=DEV)
    o.gemm_slab(x, w, out, bias=bias)
    assert rel(out, want + bias) < TOL["bfloat16"]
    acc = rnd(T, N, seed=3)
    base = acc.clone()
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    o.gemm_slab(x, w, acc, accumulate=True, status=status)
    assert rel(acc, base + want) < 2e-5 and int(status) == 0
    # x written by the kernel just before it on the stream
    x2 = torch.empty_like(xw)
    out2 = torch.empty(T, N, dtype=torch.float32, device=DEV)
    o.residual_add(acc, out)                      # some kernel of the library: the product's wait is for it
    x2.copy_(xw)
    o.gemm_slab(x2[:, :K], w, out2)
    assert rel(out2, want) < 2e-5
    # each token's result does not depend on the others
    if T > 1:
        one = torch.empty(1, N, dtype=torch.float32, device=DEV)
        o.gemm_slab(x[T - 1:T], w, one)
        assert torch.equal(one[0], out2[T - 1])


def test_gemm_slab_refuses_what_does_not_fit():
    o = ops()
    big = torch.empty(40000, 2048, dtype=torch.bfloat16, device=DEV)      # 164 MB: no SM's share fits
    x = rnd(4, 2048, dtype=torch.bfloat16)
    assert not o.slab_ok(x, big)
    assert not o.slab_ok(rnd(4, 96, dtype=torch.bfloat16), rnd(64, 96, dtype=torch.bfloat16))      # K no multiple of 128
    assert not o.slab_ok(rnd(40, 128, dtype=torch.bfloat16), rnd(64, 128, dtype=torch.bfloat16))   # too many tokens
    assert not o.slab_ok(rnd(4, 128), rnd(64, 128))                                                  # 32-bit
    with pytest.raises(o.KernelError):
        o.gemm_slab(x, big, torch.empty(4, 40000, dtype=torch.float32, device=DEV))


@pytest.mark.parametrize("T,K_top", [(1, 2), (8, 4), (33, 3)])
def test_gemm_skinny_grouped_against_routing(T, K_top):
    o = ops()
    E, I, H = 7, 64, 96
    x = rnd(T, H, dtype=torch.bfloat16)
    w_gu, w_down = rnd(E, 2 * I, H, dtype=torch.bfloat16, scale=0.1), rnd(E, H, I, dtype=torch.bfloat16, scale=0.1)
    g = torch.Generator().manual_seed(T)
    ids = torch.stack([torch.randperm(E, generator=g)[:K_top] for _ in range(T)]).to(torch.int32).to(DEV)
    scratch = torch.zeros(2 * E, dtype=torch.int32, device=DEV)
    offsets = torch.empty(E + 1, dtype=torch.int32, device=DEV)
    src = torch.empty(T * K_top, dtype=torch.int32, device=DEV)
    inv = torch.empty(T * K_top, dtype=torch.int32, device=DEV)
    active = torch.empty(min(E, T * K_top), dtype=torch.int32, device=DEV)
    o.moe_align(ids, E, scratch, offsets, src, inv, active)
    # bookkeeping: a permutation, rows grouped by expert, active = experts with rows
    counts = torch.bincount(ids.flatten().long(), minlength=E)
    assert offsets.tolist() == [0] + counts.cumsum(0).tolist()
    assert sorted(inv.tolist()) == list(range(T * K_top))
    for i in range(T * K_top):
        r = int(inv[i])
        e = int(ids.flatten()[i])
        assert int(offsets[e]) <= r < int(offsets[e + 1]) and int(src[r]) == i // K_top
    act_list = [e for e in active.tolist() if e >= 0]
    assert act_list == [e for e in range(E) if counts[e] > 0] and all(e == -1 for e in active.tolist()[len(act_list):])
    act = torch.empty(T * K_top, I, dtype=torch.bfloat16, device=DEV)
    o.gemm_skinny(x, w_gu, act, gated=True, x_rows=src, group_offsets=offsets, active_groups=active, tokens_hint=T)
    y = torch.empty(T * K_top, H, dtype=torch.float32, device=DEV)
    o.gemm_skinny(act, w_down, y, group_offsets=offsets, active_groups=active, tokens_hint=T)
    for i in range(T * K_top):
        t, e, r = i // K_top, int(ids.flatten()[i]), int(inv[i])
        gu = x[t].float() @ w_gu[e].float().T
        a = (gu[:I] / (1 + torch.exp(-gu[:I])) * gu[I:])
        assert rel(act[r], a) < TOL["bfloat16"]
        assert rel(y[r], act[r].float() @ w_down[e].float().T) < 2e-5


def test_skinny_refuses_what_it_cannot_do():
    o = ops()
    x, w = rnd(2, 40, dtype=torch.bfloat16), rnd(16, 40, dtype=torch.bfloat16)
    assert not o.skinny_ok(x, w)
    with pytest.raises(o.KernelError, match="size"):
        o.gemm_skinny(x, w, torch.empty(2, 16, dtype=torch.bfloat16, device=DEV))
    with pytest.raises(o.KernelError, match="CUDA tensors"):
        o.gemm(x.cpu(), w, torch.empty(2, 16, dtype=torch.bfloat16, device=DEV))


# ------------------------------------------------------------------ element-wise
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H", [16, 80, 333, 2048])
def test_rmsnorm_embed_silu(dtype, H):
    o, dt = ops(), DT[dtype]
    x, w = rnd(9, H, scale=3.0), rnd(H, dtype=dt) + 1
    eps = 1e-5
    want = x * (1.0 / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)) * w.float()
    out = torch.empty(9, H, dtype=dt, device=DEV)
    o.rmsnorm(x, w, eps, out)
    assert rel(out, want) < (1e-6 if dtype == "float32" else 5e-3)
    rows = torch.tensor([7, 0, 7, 3], dtype=torch.int32, device=DEV)
    picked = torch.empty(4, H, dtype=dt, device=DEV)
    o.rmsnorm(x, w, eps, picked, rows=rows)
    assert torch.equal(picked, out[rows.long()])
    table = rnd(50, H, dtype=dt)
    ids = torch.tensor([3, 49, 0, 3], dtype=torch.int32, device=DEV)
    h = torch.empty(4, H, dtype=torch.float32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    o.embed(table, ids, h, status)
    assert torch.equal(h, table[ids.long()].float()) and int(status) == 0
    o.embed(table, torch.tensor([50], dtype=torch.int32, device=DEV), h[:1], status)
    assert int(status) == 1  # a token id outside the table is reported, not read
    gu = rnd(5, 2 * H, dtype=dt)
    act = torch.empty(5, H, dtype=dt, device=DEV)
    o.silu_mul(gu, act)
    g, u = gu[:, :H].float(), gu[:, H:].float()
    assert rel(act, g / (1 + torch.exp(-g)) * u) < (1e-6 if dtype == "float32" else 5e-3)


def test_router_topk_and_ties():
    o = ops()
    logits = torch.arange(1.0, 9.0, device=DEV).reshape(1, 8)
    ids = torch.empty(1, 3, dtype=torch.int32, device=DEV)
    w = torch.empty(1, 3, dtype=torch.float32, device=DEV)
    o.router_topk(logits, 3, False, ids, w)
    assert ids.tolist() == [[7, 6, 5]]
    # the reference's golden for these logits (crates/ferrox-moe/src/lib.rs:864-893), its tolerance
    assert torch.allclose(w.cpu(), torch.tensor([[0.6323223, 0.2326232, 0.0855683]]), atol=1e-4)
    o.router_topk(logits, 3, True, ids, w)
    assert abs(float(w.sum()) - 1) < 1e-6
    tie = torch.tensor([[0.5, 2.0, 2.0, 0.1, 2.0]], device=DEV)
    ids2 = torch.empty(1, 2, dtype=torch.int32, device=DEV)
    o.router_topk(tie, 2, False, ids2, torch.empty(1, 2, device=DEV))
    assert ids2.tolist() == [[1, 2]]  # equal probabilities: the lowest index first
    g = torch.Generator().manual_seed(0)
    big = torch.randn(300, 61, generator=g).to(DEV)
    ids3 = torch.empty(300, 5, dtype=torch.int32, device=DEV)
    w3 = torch.empty(300, 5, device=DEV)
    o.router_topk(big, 5, False, ids3, w3)
    p = torch.softmax(big, -1)
    tv, ti = torch.topk(p, 5, dim=-1)
    assert torch.equal(ids3.long(), ti) and rel(w3, tv) < 1e-6


def test_moe_combine_in_rank_order():
    o = ops()
    T, K, H = 6, 3, 40
    y, shared = rnd(T * K, H), rnd(T, H)
    inv = torch.randperm(T * K, generator=torch.Generator().manual_seed(0)).to(torch.int32).to(DEV)
    w = torch.rand(T, K, generator=torch.Generator().manual_seed(1)).to(DEV)
    gate = rnd(T, 1)
    h = rnd(T, H, seed=2)
    want = h.clone()
    for t in range(T):
        acc = torch.zeros(H, device=DEV)
        for k in range(K):
            acc = acc + w[t, k] * y[inv[t * K + k]]
        want[t] += acc + torch.sigmoid(gate[t]) * shared[t]
    o.moe_combine(h, y, inv, w, shared, gate)
    assert rel(h, want) < 1e-6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H", [40, 2048, 3584, 8192, 1000])
@pytest.mark.parametrize("with_shared", [True, False])
def test_moe_combine_with_the_norm_that_follows(dtype, H, with_shared):
    """The combine that also applies the next RMSNorm: the same residual rows, bit for bit, as the combine alone, and
    the normed rows of the norm kernel on them (sums of squares in another order: a rounding apart)."""
    o, dt = ops(), DT[dtype]
    T, K = 5, 4
    y, shared = rnd(T * K, H, dtype=dt), (rnd(T, H, dtype=dt) if with_shared else None)
    inv = torch.randperm(T * K, generator=torch.Generator().manual_seed(0)).to(torch.int32).to(DEV)
    w = torch.rand(T, K, generator=torch.Generator().manual_seed(1)).to(DEV)
    logits = rnd(T, 7)
    gate = logits[:, 6:] if with_shared else None      # a strided column, as the router's product leaves it
    nw = (1 + 0.1 * rnd(H, seed=5)).to(dt)
    h0 = rnd(T, H, seed=2)
    h_a, h_b = h0.clone(), h0.clone()
    o.moe_combine(h_a, y, inv, w, shared, gate)
    x_a = o.rmsnorm(h_a, nw, 1e-5, torch.empty(T, H, dtype=dt, device=DEV))
    assert o.combine_norm_ok(h_b, y) == (H % (4 if dtype == "float32" else 8) == 0 and H // (4 if dtype == "float32" else 8) <= 1024)
    if not o.combine_norm_ok(h_b, y):
        return
    x_b = o.moe_combine(h_b, y, inv, w, shared, gate, norm=(nw, 1e-5, torch.empty(T, H, dtype=dt, device=DEV)))
    assert torch.equal(h_a, h_b)
    assert rel(x_b.float(), x_a.float()) < (1e-6 if dtype == "float32" else 8e-3)
    want = h_a / torch.sqrt((h_a * h_a).mean(dim=1, keepdim=True) + 1e-5) * nw.float()
    assert rel(x_b.float(), want) < (1e-6 if dtype == "float32" else 8e-3)


# ------------------------------------------------------------------ rotary + cache write + attention
def build_cache(dtype, seqs, nkv, d, page_size, n_pages, seed=0):
    """Random K/V for requests of the given lengths, scattered into shuffled pages."""
    rng = random.Random(seed)
    free = list(range(n_pages))
    rng.shuffle(free)
    width = max(-(-L // page_size) for L in seqs) + 1
    table = torch.full((len(seqs) + 2, width), -1, dtype=torch.int32)
    kp = torch.zeros(n_pages, nkv, page_size, d)
    vp = torch.zeros(n_pages, nkv, page_size, d)
    ks, vs = [], []
    for s, L in enumerate(seqs):
        k = torch.randn(L, nkv, d, generator=torch.Generator().manual_seed(seed * 100 + s)).to(dtype).float()
        v = torch.randn(L, nkv, d, generator=torch.Generator().manual_seed(seed * 100 + 50 + s)).to(dtype).float()
        ks.append(k)
        vs.append(v)
        for j in range(-(-L // page_size)):
            pg = free.pop()
            table[s + 1, j] = pg  # slot = s + 1: slots and entries are different things
            n = min(page_size, L - j * page_size)
            kp[pg, :, :n] = k[j * page_size:j * page_size + n].transpose(0, 1)
            vp[pg, :, :n] = v[j * page_size:j * page_size + n].transpose(0, 1)
    return kp.to(dtype).to(DEV), vp.to(dtype).to(DEV), table.to(DEV), ks, vs


def plain_attention(q, k, v, pos, window, scale):
    """One query (heads, d) at position pos over keys k[:pos+1] (nkv heads)."""
    nh, nkv = q.shape[0], k.shape[1]
    lo = max(0, pos - window + 1) if window else 0
    out = torch.zeros_like(q)
    for h in range(nh):
        kv = h // (nh // nkv)
        s = (k[lo:pos + 1, kv] @ q[h]) * scale
        out[h] = torch.softmax(s, 0) @ v[lo:pos + 1, kv]
    return out


ATT_CASES = [
    # nh, nkv, d, page, window, lengths
    (4, 2, 16, 4, 0, [1, 5, 33]),
    (2, 1, 64, 16, 16, [70, 16, 17]),
    (6, 3, 48, 8, 7, [40, 9]),
    (16, 16, 128, 64, 0, [300, 64, 65]),
    (28, 4, 128, 64, 100, [130]),
    (3, 3, 256, 16, 0, [50]),
    (12, 1, 32, 16, 0, [90]),
    # head sizes in steps of 64 on pages of a multiple of 64: in bfloat16 the decode kernel that streams pages by TMA
    (8, 2, 64, 64, 0, [200, 129, 1]),
    (6, 2, 192, 128, 150, [318, 70]),
    (40, 2, 64, 128, 0, [150, 260]),
    (4, 4, 256, 64, 33, [140, 64]),
    (16, 16, 128, 64, 70, [319]),
]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", ATT_CASES)
@pytest.mark.parametrize("kernel", ["generic", "decode"])
def test_attention_over_pages(dtype, case, kernel):
    o, dt = ops(), DT[dtype]
    nh, nkv, d, ps, window, lens = case
    kp, vp, table, ks, vs = build_cache(dt, lens, nkv, d, ps, n_pages=sum(-(-L // ps) for L in lens) + 3)
    # queries: for each request its last position, one in the middle and position 0
    toks = []
    for s, L in enumerate(lens):
        for pos in sorted({L - 1, L // 2, 0}):
            toks.append((s, pos))
    T = len(toks)
    q = rnd(T, nh * d + 8, dtype=dt)[:, : nh * d + 8]  # rows wider than the heads: a strided view
    positions = torch.tensor([p for _, p in toks], dtype=torch.int32, device=DEV)
    token_seq = torch.tensor([s for s, _ in toks], dtype=torch.int32, device=DEV)
    seq_slot = torch.tensor([s + 1 for s in range(len(lens))], dtype=torch.int32, device=DEV)
    out = torch.empty(T, nh * d, dtype=dt, device=DEV)
    scale = 1 / math.sqrt(d)
    if kernel == "generic":
        o.paged_attention(q, kp, vp, table, ps, positions, token_seq, seq_slot, out, nh, nkv, d, window, scale)
    else:
        for split_len, n_splits in ((64, 5), (128, 3), (4096, 1), (0, 1), (0, 3), (0, 7)):
            pa = torch.empty(T, nh, n_splits, d, device=DEV)
            pm = torch.empty(T, nh, n_splits, 2, device=DEV)
            out.zero_()
            o.decode_attention(q, kp, vp, table, ps, positions, token_seq, seq_slot, out, nh, nkv, d, window, scale,
                               split_len, n_splits, pa, pm)
            _check_attention(out, q, ks, vs, toks, nh, d, window, scale, dtype)
            # the key ranges merged by the kernel's last blocks instead of the merge kernel: the same bits, twice
            # in a row with the same counters, which it leaves zeroed
            counters = torch.zeros(T * nkv * -(-(nh // nkv) // 16), dtype=torch.int32, device=DEV)
            for _ in range(2):
                fused = torch.zeros_like(out)
                o.decode_attention(q, kp, vp, table, ps, positions, token_seq, seq_slot, fused, nh, nkv, d, window,
                                   scale, split_len, n_splits, torch.empty_like(pa), torch.empty_like(pm),
                                   counters=counters)
                assert torch.equal(fused, out)
                assert int(counters.abs().sum()) == 0
        return
    _check_attention(out, q, ks, vs, toks, nh, d, window, scale, dtype)


def _check_attention(out, q, ks, vs, toks, nh, d, window, scale, dtype):
    for i, (s, pos) in enumerate(toks):
        want = plain_attention(q[i, : nh * d].float().cpu().reshape(nh, d), ks[s], vs[s], pos, window, scale)
        got = out[i].float().cpu().reshape(nh, d)
        assert rel(got, want) < (2e-6 if dtype == "float32" else 1e-2), (s, pos)


@pytest.mark.parametrize("kernel", ["generic", "decode"])
def test_attention_finds_one_far_key_and_respects_the_window_edge(kernel):
    """One key among hundreds is made to stand out; the output must be its value when
    it is visible and must not contain it one position past the window."""
    o = ops()
    nh = nkv = 2
    d, ps, L = 32, 16, 400
    kp, vp, table, ks, vs = build_cache(torch.float32, [L], nkv, d, ps, n_pages=30, seed=4)
    far = 37
    q = torch.zeros(1, nh * d)
    spike = torch.randn(d, generator=torch.Generator().manual_seed(1))
    spike = spike / spike.norm() * 12
    q[0, :d], q[0, d:] = spike, spike
    page, off = int(table[1, far // ps]), far % ps
    kp[page, :, off, :] = (spike * 8).to(DEV)  # score far above every other key
    ks[0][far, :, :] = spike * 8
    q = q.to(DEV)
    args = dict(n_heads=nh, n_kv_heads=nkv, head_dim=d, scale=1 / math.sqrt(d))
    positions = torch.tensor([L - 1], dtype=torch.int32, device=DEV)
    z = torch.zeros(1, dtype=torch.int32, device=DEV)
    slot = torch.ones(1, dtype=torch.int32, device=DEV)

    def run(window):
        out = torch.empty(1, nh * d, device=DEV)
        if kernel == "generic":
            o.paged_attention(q, kp, vp, table, ps, positions, z, slot, out, window=window, **args)
        else:
            pa, pm = torch.empty(1, nh, 7, d, device=DEV), torch.empty(1, nh, 7, 2, device=DEV)
            o.decode_attention(q, kp, vp, table, ps, positions, z, slot, out, window=window, split_len=64, n_splits=7,
                               part_acc=pa, part_ml=pm, **args)
        return out.cpu().reshape(nh, d)

    full = run(0)
    assert rel(full[0], vs[0][far, 0]) < 1e-4  # all the weight on the far key
    inside = run(L - far)  # window reaches back exactly to the far key
    assert rel(inside[0], vs[0][far, 0]) < 1e-4
    outside = run(L - far - 1)  # one less: the far key is out
    want = plain_attention(q[0].cpu().reshape(nh, d), ks[0], vs[0], L - 1, L - far - 1, args["scale"])
    assert rel(outside, want) < 1e-5 and rel(outside[0], vs[0][far, 0]) > 0.1


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nh,nkv,d,rot", [(4, 2, 16, 16), (3, 1, 48, 48), (2, 2, 128, 64)])
def test_rope_and_cache_write(dtype, nh, nkv, d, rot):
    o, dt = ops(), DT[dtype]
    ps, T = 4, 7
    theta = 10000.0
    width = nh * d + 2 * nkv * d
    qkv = rnd(T, width, dtype=dt)
    before = qkv.clone()
    positions = torch.tensor([0, 1, 2, 3, 9, 10, 150], dtype=torch.int32, device=DEV)
    token_seq = torch.tensor([0, 0, 0, 0, 1, 1, 2], dtype=torch.int32, device=DEV)
    seq_slot = torch.tensor([2, 0, 1], dtype=torch.int32, device=DEV)
    table = torch.full((3, 40), -1, dtype=torch.int32)
    table[2, 0], table[0, 2], table[1, 37] = 5, 1, 3
    table = table.to(DEV)
    kp = torch.zeros(6, nkv, ps, d, dtype=dt, device=DEV)
    vp = torch.zeros_like(kp)
    inv_freq = (1.0 / torch.pow(torch.tensor(theta), torch.arange(0, rot // 2).float() * 2 / rot)).to(DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    o.rope_kv_write(qkv, positions, token_seq, seq_slot, inv_freq, rot, kp, vp, table, ps, nh, nkv, d, True, status)
    assert int(status) == 0
    x = before.float().cpu()
    ang = positions.cpu().float()[:, None] * inv_freq.cpu()[None, :]
    cos, sin = torch.cos(ang), torch.sin(ang)
    tol = 2e-6 if dtype == "float32" else 8e-3
    for t in range(T):
        for hh in range(nh + nkv):
            a, b = x[t, hh * d: hh * d + rot // 2], x[t, hh * d + rot // 2: hh * d + rot]
            want = torch.cat([a * cos[t] - b * sin[t], a * sin[t] + b * cos[t], x[t, hh * d + rot:(hh + 1) * d]])
            assert rel(qkv[t, hh * d:(hh + 1) * d].cpu(), want) < tol
        assert torch.equal(qkv[t, (nh + nkv) * d:], before[t, (nh + nkv) * d:])  # v untouched
    # where the rows landed: page table[slot][pos // ps], offset pos % ps
    where = {0: (5, 0), 1: (5, 1), 2: (5, 2), 3: (5, 3), 4: (1, 1), 5: (1, 2), 6: (3, 2)}
    for t, (pg, off) in where.items():
        assert torch.equal(kp[pg, :, off, :].reshape(-1), qkv[t, nh * d:(nh + nkv) * d])
        assert torch.equal(vp[pg, :, off, :].reshape(-1), qkv[t, (nh + nkv) * d:])
    assert int((kp != 0).any(dim=-1).sum()) == T * nkv  # nothing else was written
    # a position without a page is reported, not written
    o.rope_kv_write(qkv[:1], torch.tensor([20], dtype=torch.int32, device=DEV), token_seq[:1], seq_slot, inv_freq, rot,
                    kp, vp, table, ps, nh, nkv, d, True, status)
    assert int(status) == 2


@pytest.mark.parametrize("T,E,K", [(1, 4, 2), (8, 60, 4), (33, 61, 5), (256, 8, 3)])
def test_route_small_equals_the_two_step_routing(T, E, K):
    o = ops()
    logits = rnd(T, E, scale=2.0, seed=T)
    i32 = dict(dtype=torch.int32, device=DEV)
    ids_a, w_a = torch.empty(T, K, **i32), torch.empty(T, K, device=DEV)
    o.router_topk(logits, K, True, ids_a, w_a)
    ids_b, w_b = torch.empty(T, K, **i32), torch.empty(T, K, device=DEV)
    offsets, src, inv = torch.empty(E + 1, **i32), torch.empty(T * K, **i32), torch.empty(T * K, **i32)
    active = torch.empty(min(E, T * K), **i32)
    o.route_small(logits, K, True, ids_b, w_b, offsets, src, inv, active)
    assert torch.equal(ids_a, ids_b) and torch.equal(w_a, w_b)
    counts = torch.bincount(ids_b.flatten().long(), minlength=E)
    assert offsets.tolist() == [0] + counts.cumsum(0).tolist()
    assert sorted(inv.tolist()) == list(range(T * K))
    flat = ids_b.flatten().tolist()
    for i, r in enumerate(inv.tolist()):
        assert int(offsets[flat[i]]) <= r < int(offsets[flat[i] + 1]) and int(src[r]) == i // K
    act = [e for e in active.tolist() if e >= 0]
    assert act == [e for e in range(E) if counts[e] > 0]


@pytest.mark.parametrize("T,E,K", [(1, 4, 2), (70, 60, 4), (2048, 61, 5), (700, 1000, 8), (300, 8, 3)])
def test_route_in_two_kernels_equals_the_separate_steps(T, E, K):
    o = ops()
    logits = rnd(T, E + 1, scale=2.0, seed=T)      # one more column than experts, as with the shared expert's gate
    i32 = dict(dtype=torch.int32, device=DEV)
    ids_a, w_a = torch.empty(T, K, **i32), torch.empty(T, K, device=DEV)
    o.router_topk(logits, K, True, ids_a, w_a, n_experts=E)
    ids_b, w_b = torch.empty(T, K, **i32), torch.empty(T, K, device=DEV)
    offsets, src, inv = torch.empty(E + 1, **i32), torch.empty(T * K, **i32), torch.empty(T * K, **i32)
    active = torch.empty(min(E, T * K), **i32)
    scratch = torch.full((2 * E,), 7, **i32)       # the call clears it itself
    for _ in range(2):
        o.route(logits, K, True, ids_b, w_b, scratch, offsets, src, inv, active, n_experts=E)
        assert torch.equal(ids_a, ids_b) and torch.equal(w_a, w_b)
        counts = torch.bincount(ids_b.flatten().long(), minlength=E)
        assert offsets.tolist() == [0] + counts.cumsum(0).tolist()
        inv_l, src_l, off_l, flat = inv.tolist(), src.tolist(), offsets.tolist(), ids_b.flatten().tolist()
        assert sorted(inv_l) == list(range(T * K))
        assert all(off_l[flat[i]] <= r < off_l[flat[i] + 1] and src_l[r] == i // K for i, r in enumerate(inv_l))
        act = [e for e in active.tolist() if e >= 0]
        assert act == [e for e in range(E) if counts[e] > 0][: active.numel()]


def test_rope_table_matches_inline_angles():
    o = ops()
    nh, nkv, d, ps = 2, 1, 32, 8
    T = 5
    positions = torch.tensor([0, 3, 77, 1000, 4095], dtype=torch.int32, device=DEV)
    inv_freq = (1.0 / torch.pow(torch.tensor(1e6), torch.arange(0, d // 2).float() * 2 / d)).to(DEV)
    table = torch.empty(T, d // 2, 2, device=DEV)
    o.rope_table(positions, inv_freq, table)
    ang = positions.float()[:, None] * inv_freq[None, :]
    assert rel(table[..., 0], torch.cos(ang)) < 1e-6 and rel(table[..., 1], torch.sin(ang)) < 1e-6
    qkv = rnd(T, (nh + 2 * nkv) * d)
    a, b = qkv.clone(), qkv.clone()
    z = torch.zeros(T, dtype=torch.int32, device=DEV)
    slot = torch.zeros(1, dtype=torch.int32, device=DEV)
    bt = torch.arange(0, 520, dtype=torch.int32, device=DEV).reshape(1, -1)
    kp = torch.zeros(520, nkv, ps, d, device=DEV)
    vp = torch.zeros_like(kp)
    o.rope_kv_write(a, positions, z, slot, inv_freq, d, kp, vp, bt, ps, nh, nkv, d)
    o.rope_kv_write(b, positions, z, slot, inv_freq, d, kp, vp, bt, ps, nh, nkv, d, cos_sin=table)
    assert torch.equal(a, b)  # the table holds exactly the angles the kernel would compute


# ------------------------------------------------------------------ tcgen05 products
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 384, 512), (65, 60, 72), (300, 200, 2048), (129, 130, 200),
                                   (2048, 256, 1408), (2048, 6144, 2048), (1000, 1000, 520), (4096, 640, 72)])
def test_gemm_tc_dense(M, N, K):
    o = ops()
    x, w, bias = rnd(M, K, dtype=torch.bfloat16), rnd(N, K, dtype=torch.bfloat16, scale=0.1), rnd(N)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    want = x.float() @ w.float().T
    out = torch.full((M, N), 7.0, dtype=torch.bfloat16, device=DEV)
    o.gemm_tc(x, w, out, bias=bias, status=status)
    assert int(status) == 0
    assert rel(out, want + bias) < TOL["bfloat16"]
    acc = rnd(M, N, seed=3)
    base = acc.clone()
    o.gemm_tc(x, w, acc, accumulate=True, status=status)
    assert int(status) == 0 and rel(acc, base + want) < 2e-5
    # a strided view of wider rows, as the attention output is inside the fused q|k|v rows
    wide = rnd(M, K + 64, dtype=torch.bfloat16, seed=11)
    out32 = torch.empty(M, N, dtype=torch.float32, device=DEV)
    o.gemm_tc(wide[:, :K], w, out32, status=status)
    assert rel(out32, wide[:, :K].float() @ w.float().T) < 2e-5


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (300, 520, 136), (2048, 2048, 2048), (70, 100, 96), (1000, 6144, 264)])
def test_gemm_tc2_pairs_of_sms(M, N, K):
    """The dense product on pairs of SMs (cta_group::2): plain with bias, accumulating, into a strided view."""
    o = ops()
    x, w = rnd(M, K, dtype=torch.bfloat16), rnd(N, K, dtype=torch.bfloat16, scale=0.2)
    bias = rnd(N, seed=5)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    want = x.float() @ w.float().T
    out = torch.full((M, N), 7.0, dtype=torch.bfloat16, device=DEV)
    o.gemm_tc2(x, w, out, bias=bias, status=status)
    assert int(status) == 0
    assert rel(out, want + bias) < TOL["bfloat16"]
    acc = rnd(M, N, seed=3)
    base = acc.clone()
    o.gemm_tc2(x, w, acc, accumulate=True, status=status)
    assert int(status) == 0 and rel(acc, base + want) < 2e-5
    wide = torch.full((M, N + 5), 7.0, device=DEV)
    o.gemm_tc2(x, w, wide[:, :N], status=status)
    assert rel(wide[:, :N], want) < 2e-5 and float(wide[:, N:].min()) == 7.0


@pytest.mark.parametrize("M,I,K", [(256, 128, 64), (200, 1408, 256), (70, 100, 96), (2048, 5632, 2048)])
def test_gemm_tc2_gated(M, I, K):
    o = ops()
    x, w = rnd(M, K, dtype=torch.bfloat16), rnd(2 * I, K, dtype=torch.bfloat16, scale=0.2)
    gate, up = x.float() @ w[:I].float().T, x.float() @ w[I:].float().T
    out = torch.empty(M, I, dtype=torch.float32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    o.gemm_tc2(x, w, out, gated=True, status=status)
    assert int(status) == 0 and rel(out, gate / (1 + torch.exp(-gate)) * up) < 3e-5


@pytest.mark.parametrize("M,I,K", [(128, 64, 64), (200, 1408, 256), (70, 100, 96), (2048, 5632, 2048), (700, 300, 136)])
def test_gemm_tc_gated(M, I, K):
    o = ops()
    x, w = rnd(M, K, dtype=torch.bfloat16), rnd(2 * I, K, dtype=torch.bfloat16, scale=0.2)
    gate, up = x.float() @ w[:I].float().T, x.float() @ w[I:].float().T
    out = torch.empty(M, I, dtype=torch.float32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    o.gemm_tc(x, w, out, gated=True, status=status)
    assert int(status) == 0 and rel(out, gate / (1 + torch.exp(-gate)) * up) < 3e-5


@pytest.mark.parametrize("counts", [[0, 130, 1, 0, 128, 255], [3, 0, 0, 0, 0, 700], [64, 64, 64, 64, 64, 64],
                                    [137, 0, 512, 9] * 15, [136] * 60, [129, 8, 260, 256, 257, 1, 384, 385, 127, 128],
                                    [1000, 0, 0, 513]])
def test_gemm_tc_grouped(counts):
    o = ops()
    G = len(counts)
    I, H = (96, 128) if G < 10 else (320, 520)   # the large case takes 128 x 256 tiles and several tiles per CTA
    R = sum(counts)
    x = rnd(R, H, dtype=torch.bfloat16)
    w_gu, w_down = rnd(G, 2 * I, H, dtype=torch.bfloat16, scale=0.1), rnd(G, H, I, dtype=torch.bfloat16, scale=0.1)
    offsets = torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    act = torch.full((R, I), 9.0, dtype=torch.bfloat16, device=DEV)
    o.gemm_tc(x, w_gu, act, gated=True, group_offsets=offsets, status=status)
    y = torch.empty(R, H, dtype=torch.float32, device=DEV)
    o.gemm_tc(act, w_down, y, group_offsets=offsets, status=status)
    assert int(status) == 0
    r = 0
    for g, c in enumerate(counts):
        if c == 0:
            continue
        gu = x[r:r + c].float() @ w_gu[g].float().T
        want = gu[:, :I] / (1 + torch.exp(-gu[:, :I])) * gu[:, I:]
        assert rel(act[r:r + c], want) < TOL["bfloat16"], g
        assert rel(y[r:r + c], act[r:r + c].float() @ w_down[g].float().T) < 2e-5, g
        r += c


@pytest.mark.parametrize("M,N,K,tnb", [(40, 300, 136, 0), (17, 128, 64, 32), (64, 2048, 5632, 0), (130, 520, 264, 0),
                                       (300, 200, 96, 64), (5, 61, 2048, 0)])
def test_gemm_tc_swap(M, N, K, tnb):
    """Features in the lanes, tokens in the columns: plain, with bias, accumulating, into a strided view."""
    o = ops()
    x, w = rnd(M, K, dtype=torch.bfloat16), rnd(N, K, dtype=torch.bfloat16, scale=0.2)
    bias = rnd(N, seed=5)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    want = x.float() @ w.float().T
    out = torch.full((M, N), 7.0, dtype=torch.bfloat16, device=DEV)
    o.gemm_tc_swap(x, w, out, bias=bias, tokens_per_tile=tnb, status=status)
    assert int(status) == 0
    assert rel(out, want + bias) < TOL["bfloat16"]
    acc = rnd(M, N, seed=3)
    base = acc.clone()
    o.gemm_tc_swap(x, w, acc, accumulate=True, tokens_per_tile=tnb, status=status)
    assert int(status) == 0 and rel(acc, base + want) < 2e-5
    wide = torch.full((M, N + 5), 7.0, device=DEV)
    o.gemm_tc_swap(x, w, wide[:, :N], tokens_per_tile=tnb, status=status)
    assert rel(wide[:, :N], want) < 2e-5 and float(wide[:, N:].min()) == 7.0


@pytest.mark.parametrize("M,N,K,splits", [(64, 2048, 5632, 8), (40, 300, 136, 3), (17, 128, 64, 1), (5, 61, 2048, 4)])
def test_gemm_tc_swap_runs_of_k(M, N, K, splits):
    """K cut into runs taken by separate CTAs, partial sums added in run order: bias, accumulation, a strided view;
    the same bits every time."""
    o = ops()
    x, w = rnd(M, K, dtype=torch.bfloat16), rnd(N, K, dtype=torch.bfloat16, scale=0.2)
    bias = rnd(N, seed=5)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    want = x.float() @ w.float().T
    out = torch.full((M, N), 7.0, dtype=torch.bfloat16, device=DEV)
    o.gemm_tc_swap(x, w, out, bias=bias, k_splits=splits, status=status)
    assert int(status) == 0 and rel(out, want + bias) < TOL["bfloat16"]
    acc = rnd(M, N, seed=3)
    base = acc.clone()
    o.gemm_tc_swap(x, w, acc, accumulate=True, k_splits=splits, status=status)
    assert int(status) == 0 and rel(acc, base + want) < 2e-5
    wide = torch.full((M, N + 5), 7.0, device=DEV)
    o.gemm_tc_swap(x, w, wide[:, :N], k_splits=splits, status=status)
    first = wide.clone()
    assert rel(wide[:, :N], want) < 2e-5 and float(wide[:, N:].min()) == 7.0
    for _ in range(3):
        o.gemm_tc_swap(x, w, wide[:, :N], k_splits=splits, status=status)
        assert torch.equal(wide, first)
    if splits > 1:
        with pytest.raises(o.KernelError):   # more runs than there are k-blocks
            o.gemm_tc_swap(x, w, out, k_splits=K // 64 + 2, status=status)


@pytest.mark.parametrize("M,I,K", [(48, 100, 96), (64, 5632, 2048), (33, 1408, 256), (200, 300, 136)])
def test_gemm_tc_swap_gated(M, I, K):
    o = ops()
    x, w = rnd(M, K, dtype=torch.bfloat16), rnd(2 * I, K, dtype=torch.bfloat16, scale=0.2)
    gate, up = x.float() @ w[:I].float().T, x.float() @ w[I:].float().T
    out = torch.empty(M, I, dtype=torch.float32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    o.gemm_tc_swap(x, w, out, gated=True, status=status)
    assert int(status) == 0 and rel(out, gate / (1 + torch.exp(-gate)) * up) < 3e-5


@pytest.mark.parametrize("counts", [[0, 130, 1, 0, 128, 255], [3, 0, 0, 0, 0, 700], [16, 17, 15, 64, 129, 1],
                                    [137, 0, 512, 9] * 15])
def test_gemm_tc_swap_grouped(counts):
    o = ops()
    G = len(counts)
    I, H = (96, 128) if G < 10 else (320, 520)
    R = sum(counts)
    x = rnd(R, H, dtype=torch.bfloat16)
    w_gu, w_down = rnd(G, 2 * I, H, dtype=torch.bfloat16, scale=0.1), rnd(G, H, I, dtype=torch.bfloat16, scale=0.1)
    offsets = torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    act = torch.full((R, I), 9.0, dtype=torch.bfloat16, device=DEV)
    o.gemm_tc_swap(x, w_gu, act, gated=True, group_offsets=offsets, status=status)
    y = torch.empty(R, H, dtype=torch.float32, device=DEV)
    o.gemm_tc_swap(act, w_down, y, group_offsets=offsets, status=status)
    assert int(status) == 0
    r = 0
    for g, c in enumerate(counts):
        if c == 0:
            continue
        gu = x[r:r + c].float() @ w_gu[g].float().T
        want = gu[:, :I] / (1 + torch.exp(-gu[:, :I])) * gu[:, I:]
        assert rel(act[r:r + c], want) < TOL["bfloat16"], g
        assert rel(y[r:r + c], act[r:r + c].float() @ w_down[g].float().T) < 2e-5, g
        r += c


def test_gather_rows():
    o = ops()
    x = rnd(9, 72, dtype=torch.bfloat16)
    rows = torch.tensor([8, 0, 0, 3, 5], dtype=torch.int32, device=DEV)
    out = torch.empty(5, 72, dtype=torch.bfloat16, device=DEV)
    o.gather_rows(x, rows, out)
    assert torch.equal(out, x[rows.long()])
    xf = rnd(9, 7)
    outf = torch.empty(5, 7, device=DEV)
    o.gather_rows(xf, rows, outf)
    assert torch.equal(outf, xf[rows.long()])


@pytest.mark.parametrize("case", ATT_CASES + [(4, 4, 80, 16, 33, [200, 70]), (2, 2, 16, 4, 0, [129])])
def test_prefill_attention_tiles(case):
    """Prompt portions (whole prompts and continuations after a cached prefix) through
    the tiled tensor-core kernel, against the plain per-query statement."""
    o = ops()
    nh, nkv, d, ps, window, lens = case
    dt = torch.bfloat16
    kp, vp, table, ks, vs = build_cache(dt, lens, nkv, d, ps, n_pages=sum(-(-L // ps) for L in lens) + 3, seed=2)
    starts = [0 if i % 2 == 0 else min(L - 1, max(1, L // 3)) for i, L in enumerate(lens)]
    toks, tiles, flat = [], [], 0
    for s, (L, st) in enumerate(zip(lens, starts)):
        n = L - st
        for i in range(0, n, 64):
            tiles.append((flat + i, min(64, n - i), s, st + i))
        toks += [(s, p) for p in range(st, L)]
        flat += n
    T = len(toks)
    q = rnd(T, nh * d + 2 * nkv * d, dtype=dt, seed=T)
    tiles_t = torch.tensor(tiles, dtype=torch.int32, device=DEV)
    seq_slot = torch.tensor([s + 1 for s in range(len(lens))], dtype=torch.int32, device=DEV)
    out = torch.zeros(T, nh * d, dtype=dt, device=DEV)
    scale = 1 / math.sqrt(d)
    o.prefill_attention(q, kp, vp, table, ps, tiles_t, seq_slot, out, nh, nkv, d, window, scale)
    assert torch.isfinite(out.float()).all()
    step = max(1, T // 40)  # a spread of tokens, plus tile edges
    check = sorted(set(list(range(0, T, step)) + [t for t in (0, 1, 63, 64, 65, 127, 128, T - 1) if t < T]))
    for i in check:
        s, pos = toks[i]
        want = plain_attention(q[i, : nh * d].float().cpu().reshape(nh, d), ks[s], vs[s], pos, window, scale)
        assert rel(out[i].float().cpu().reshape(nh, d), want) < 1.5e-2, (i, s, pos)


TC_ATT_CASES = [
    # nh, nkv, d, page, window, lengths
    (16, 16, 128, 64, 0, [300, 64, 65]),
    (28, 4, 128, 64, 100, [130, 517]),
    (6, 2, 64, 128, 0, [700, 129]),
    (3, 1, 64, 64, 300, [900]),
    (2, 2, 128, 192, 129, [400, 2, 128]),
    (4, 2, 128, 64, 0, [2300, 300]),
    (2, 1, 128, 64, 0, [6000]),
    (2, 2, 64, 64, 2048, [4300]),
]


@pytest.mark.parametrize("run_blocks", [-1, 0, 1, 3])
@pytest.mark.parametrize("case", TC_ATT_CASES)
def test_prefill_attention_tcgen05(case, run_blocks):
    """Prompt portions through the tcgen05 kernel (tiles of 256 queries, blocks of 128 keys), whole prompts and
    continuations after a cached prefix, against the plain per-query statement; with the planner's own cut of
    long tiles into runs of key blocks, and with runs of one and of three blocks (every tile with more is then added
    up from partial results by the second kernel).  One far key of the longest request is made to stand out for its
    last query, so that a block that is skipped or masked wrongly shows."""
    o = ops()
    nh, nkv, d, ps, window, lens = case
    dt = torch.bfloat16
    kp, vp, table, ks, vs = build_cache(dt, lens, nkv, d, ps, n_pages=sum(-(-L // ps) for L in lens) + 3, seed=5)
    # stale finite values in the unused places of every page, as pages that are used again hold
    starts = [0 if i % 2 == 0 else min(L - 1, max(1, L // 3)) for i, L in enumerate(lens)]
    toks = []
    for s, (L, st) in enumerate(zip(lens, starts)):
        toks += [(s, p) for p in range(st, L)]
    T = len(toks)
    items, merges, parts = o.prefill_tc_plan([(L - st, st) for L, st in zip(lens, starts)], window, nh, run_blocks=run_blocks)
    if run_blocks == 1:
        assert parts >= max(lens) // 128 and len(merges) >= 1
    if window:
        # pages that the window has left behind are given back before a later portion runs: no page there
        for s, st in enumerate(starts):
            for j in range(max(0, st - window + 1) // ps):
                table[s + 1, j] = -1
    q = rnd(T, nh * d + 2 * nkv * d, dtype=dt, seed=T)
    # the last query of request 0 looks hard at one far key that is still inside its window
    L0 = lens[0]
    far = max(0, L0 - 1 - (window - 2 if window else L0))
    last0 = L0 - starts[0] - 1
    q[last0, :d] = (ks[0][far, 0] * 4).to(dt).to(DEV)
    seq_slot = torch.tensor([s + 1 for s in range(len(lens))], dtype=torch.int32, device=DEV)
    out = torch.zeros(T, nh * d, dtype=dt, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    scale = 1 / math.sqrt(d)
    assert o.prefill_tc_ok(q, out, kp, ps, d)
    part_o = torch.full((max(parts, 1), nh, 256, d), float("nan"), device=DEV)      # what a run does not write is not read
    part_ml = torch.full((max(parts, 1), nh, 256, 2), float("nan"), device=DEV)
    o.prefill_attention_tc(q, kp, vp, table, ps, torch.from_numpy(items).to(DEV), seq_slot, out, nh, nkv, d, window, scale,
                           status=status, merges=torch.from_numpy(merges).to(DEV) if parts else None, part_o=part_o,
                           part_ml=part_ml)
    assert int(status) == 0
    assert torch.isfinite(out.float()).all()
    step = max(1, T // 40)  # a spread of tokens, plus tile edges
    check = sorted(set(list(range(0, T, step)) + [t for t in (0, 1, 63, 64, 127, 128, 129, 255, 256, last0, T - 1) if t < T]))
    for i in check:
        s, pos = toks[i]
        want = plain_attention(q[i, : nh * d].float().cpu().reshape(nh, d), ks[s], vs[s], pos, window, scale)
        assert rel(out[i].float().cpu().reshape(nh, d), want) < 1.5e-2, (i, s, pos)
    # the far key carries (nearly) all the weight of that query's first head
    got = out[last0, :d].float().cpu()
    assert rel(got, vs[0][far, 0]) < 5e-2


def test_prefill_attention_tcgen05_refuses_other_sizes():
    o = ops()
    q = rnd(4, 3 * 48, dtype=torch.bfloat16)
    kp = torch.zeros(2, 1, 64, 48, dtype=torch.bfloat16, device=DEV)
    out = torch.zeros(4, 48, dtype=torch.bfloat16, device=DEV)
    assert not o.prefill_tc_ok(q, out, kp, 64, 48)
    tiles = torch.tensor([[0, 4, 0, 0, 0, 1, -1, 0]], dtype=torch.int32, device=DEV)
    table = torch.zeros(1, 2, dtype=torch.int32, device=DEV)
    slots = torch.zeros(1, dtype=torch.int32, device=DEV)
    with pytest.raises(o.KernelError):
        o.prefill_attention_tc(q, kp, kp, table, 64, tiles, slots, out, 1, 1, 48, 0, 1.0)


def test_gemm_skinny_transposed_store_and_linear_picks_it_for_narrow_outputs():
    o = ops()
    T, N, K = 300, 61, 256
    x, w = rnd(T, K, dtype=torch.bfloat16), rnd(N, K, dtype=torch.bfloat16, scale=0.1)
    want = x.float() @ w.float().T
    out = torch.full((T, N), 7.0, device=DEV)
    o.gemm_skinny(w, x, out, transposed_out=True)   # roles swapped: w is the few "tokens", x the streamed matrix
    assert rel(out, want) < 2e-5
    wide = torch.full((T, N + 3), 7.0, device=DEV)   # a view with a row pitch of its own
    o.linear(x, w, wide[:, :N])
    assert rel(wide[:, :N], want) < 2e-5 and float(wide[:, N:].min()) == 7.0


# ------------------------------------------------------------------ random weights
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape,mean,std", [((7,), 0.0, 0.02), ((33, 129), 1.0, 0.02), ((5, 64, 48), 0.0, 1.0),
                                            ((1408, 2048), 0.0, 0.02)])
def test_random_weights_are_the_same_bits_on_the_device_and_on_the_cpu(dtype, shape, mean, std):
    """The device draw against the host's statement of the same rule, bit for bit (odd lengths end inside a pair;
    the last shape is one expert matrix at the real width, its checksum compared as well)."""
    from ferrox_b200.weights import random_init as ri

    key = ri.tensor_key(11, f"t{shape}")
    dev = ri.normal(key, shape, DT[dtype], mean, std, device=DEV).cpu()
    cpu = ri.normal(key, shape, DT[dtype], mean, std, device="cpu")
    assert dev.dtype == cpu.dtype == DT[dtype] and dev.shape == cpu.shape == shape
    ibits = torch.int32 if dtype == "float32" else torch.int16
    assert torch.equal(dev.view(ibits), cpu.view(ibits))
    assert int(dev.view(ibits).to(torch.int64).sum()) == int(cpu.view(ibits).to(torch.int64).sum())


def test_a_model_drawn_on_the_device_is_the_model_of_the_folder(tmp_path):
    """Engine.from_random(on_device=True) and a folder written on the CPU for the same configuration and seed hold
    the same weights: their logits are equal bit for bit."""
    from ferrox_b200 import Engine, StepEntry, write_random_model
    from tiny_configs import TINY_B

    folder = write_random_model(str(tmp_path / "m"), TINY_B, seed=5, norm_init="around_one")
    toks = [(i * 37 + 11) % TINY_B["vocab_size"] for i in range(41)]
    outs = []
    for make in (lambda: Engine.from_folder(folder, dtype="float32", page_size=16, n_pages=8, max_slots=2),
                 lambda: Engine.from_random(TINY_B, seed=5, norm_init="around_one", dtype="float32", on_device=True,
                                            page_size=16, n_pages=8, max_slots=2)):
        eng = make()
        slot = eng.open_request()
        outs.append(eng.step([StepEntry(slot, toks, want=list(range(len(toks))))]).cpu())
    assert torch.equal(outs[0], outs[1])


# ------------------------------------------------------------------ the rotary kernel's other pairing rule
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nh,nkv,d,rot", [(4, 2, 16, 16), (3, 1, 48, 20), (2, 2, 128, 128)])
def test_rope_adjacent_pairs_with_a_frequency_table(dtype, nh, nkv, d, rot):
    """Pairs (2i, 2i+1) rotated by pos * inv_freq[i] for an arbitrary table (the reference's interleaved form with
    per-band factors, crates/ferrox-core/src/attention.rs:340-352, 319-337); the rest of the head passes through;
    the keys reach their pages as rotated."""
    o, dt = ops(), DT[dtype]
    ps, T = 8, 5
    width = nh * d + 2 * nkv * d
    qkv = rnd(T, width, dtype=dt)
    before = qkv.clone()
    positions = torch.tensor([0, 1, 2, 40, 41], dtype=torch.int32, device=DEV)
    token_seq = torch.tensor([0, 0, 0, 1, 1], dtype=torch.int32, device=DEV)
    seq_slot = torch.tensor([1, 0], dtype=torch.int32, device=DEV)
    table = torch.full((2, 8), -1, dtype=torch.int32)
    table[1, 0], table[0, 5] = 2, 0
    table = table.to(DEV)
    kp = torch.zeros(3, nkv, ps, d, dtype=dt, device=DEV)
    vp = torch.zeros_like(kp)
    inv_freq = (torch.rand(rot // 2, generator=torch.Generator().manual_seed(rot)) + 0.01).to(DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    o.rope_kv_write(qkv, positions, token_seq, seq_slot, inv_freq, rot, kp, vp, table, ps, nh, nkv, d, True, status,
                    pairing=o.PAIR_ADJACENT)
    assert int(status) == 0
    x = before.float().cpu()
    ang = positions.cpu().float()[:, None] * inv_freq.cpu()[None, :]
    cos, sin = torch.cos(ang), torch.sin(ang)
    tol = 2e-6 if dtype == "float32" else 8e-3
    for t in range(T):
        for hh in range(nh + nkv):
            head = x[t, hh * d:(hh + 1) * d]
            want = head.clone()
            a, b = head[0:rot:2], head[1:rot:2]
            want[0:rot:2] = a * cos[t] - b * sin[t]
            want[1:rot:2] = a * sin[t] + b * cos[t]
            assert rel(qkv[t, hh * d:(hh + 1) * d].cpu(), want) < tol
    for t, (pg, off) in {0: (2, 0), 2: (2, 2), 3: (0, 0), 4: (0, 1)}.items():
        assert torch.equal(kp[pg, :, off, :].reshape(-1), qkv[t, nh * d:(nh + nkv) * d])
        assert torch.equal(vp[pg, :, off, :].reshape(-1), before[t, (nh + nkv) * d:])


# ------------------------------------------------------------------ decode attention right after a long write
@pytest.mark.parametrize("page_size,d", [(64, 128), (16, 48)])
def test_decode_attention_waits_for_a_write_of_many_positions(page_size, d):
    """The public entry makes no assumption about the kernel before it: 100 positions of one request are written by
    the rotary kernel and read by the decode attention launched right behind it (more than any early fetch could
    skip), many times over, against the plain attention."""
    o = ops()
    nh, nkv, n_new, L0 = 4, 2, 100, 90
    dt = torch.bfloat16
    scale = 1 / math.sqrt(d)
    n_pages = -(-(L0 + n_new) // page_size) + 1
    table = torch.full((1, n_pages + 2), -1, dtype=torch.int32)
    table[0, :n_pages] = torch.randperm(n_pages, generator=torch.Generator().manual_seed(3)).int()
    table = table.to(DEV)
    seq_slot = torch.zeros(1, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for trial in range(5):
        kp = torch.zeros(n_pages, nkv, page_size, d, dtype=dt, device=DEV)
        vp = torch.zeros_like(kp)
        # the old positions, then the new ones in the very launch before the attention
        rows = rnd(L0 + n_new, (nh + 2 * nkv) * d, dtype=dt, seed=trial)
        want_rows = rows.clone()
        pos_all = torch.arange(L0 + n_new, dtype=torch.int32, device=DEV)
        seq_all = torch.zeros(L0 + n_new, dtype=torch.int32, device=DEV)
        o.rope_kv_write(rows[:L0], pos_all[:L0], seq_all[:L0], seq_slot, None, 0, kp, vp, table, page_size, nh, nkv, d,
                        True, status)
        torch.cuda.synchronize()
        out = torch.zeros(n_new, nh * d, dtype=dt, device=DEV)
        n_splits = 3
        pa = torch.empty(n_new, nh, n_splits, d, device=DEV)
        pm = torch.empty(n_new, nh, n_splits, 2, device=DEV)
        o.rope_kv_write(rows[L0:], pos_all[L0:], seq_all[L0:], seq_slot, None, 0, kp, vp, table, page_size, nh, nkv, d,
                        True, status)
        o.decode_attention(rows[L0:], kp, vp, table, page_size, pos_all[L0:], seq_all[L0:], seq_slot, out, nh, nkv, d,
                           0, scale, 0, n_splits, pa, pm)
        torch.cuda.synchronize()
        assert int(status) == 0
        x = want_rows.float().cpu()
        k = x[:, nh * d:(nh + nkv) * d].reshape(-1, nkv, d)
        v = x[:, (nh + nkv) * d:].reshape(-1, nkv, d)
        for i in (0, 1, 37, n_new - 1):
            want = plain_attention(x[L0 + i, :nh * d].reshape(nh, d), k, v, L0 + i, 0, scale)
            assert rel(out[i].float().cpu().reshape(nh, d), want) < 1e-2, (trial, i)


# ------------------------------------------------------------------ decode attention that rotates and stores itself
@pytest.mark.parametrize("nh,nkv,d,ps,window,lens", [
    (16, 16, 128, 64, 0, [300, 64, 65, 1]),
    (28, 4, 128, 64, 100, [130, 517]),
    (40, 2, 64, 128, 0, [150, 260, 129]),       # 20 query heads a kv head: two blocks of heads share a key's tile
    (6, 2, 192, 128, 150, [318, 70]),
    (4, 4, 256, 64, 33, [140, 64]),
])
@pytest.mark.parametrize("rotate", [True, False])
def test_decode_attention_does_the_rotary_kernels_work_itself(nh, nkv, d, ps, window, lens, rotate):
    """One new token a request: the decode attention given the fused rows as projected (store_new) against the
    rotary kernel followed by the decode attention: the same pages bit for bit, the same output within rounding;
    with one and with several key ranges, merged by the kernel and by the merge kernel; and against plain."""
    o, dt = ops(), torch.bfloat16
    assert o.decode_tma_blocks_per_sm(dt, d, ps) > 0
    kp0, vp0, table, ks, vs = build_cache(dt, lens, nkv, d, ps, n_pages=sum(-(-L // ps) for L in lens) + 3, seed=9)
    B = len(lens)
    positions = torch.tensor([L - 1 for L in lens], dtype=torch.int32, device=DEV)     # the new token is each request's last
    token_seq = torch.arange(B, dtype=torch.int32, device=DEV)
    seq_slot = torch.tensor([s + 1 for s in range(B)], dtype=torch.int32, device=DEV)
    qkv0 = rnd(B, (nh + 2 * nkv) * d + 8, dtype=dt, seed=d)[:, :(nh + 2 * nkv) * d]
    inv_freq = (1.0 / torch.pow(torch.tensor(1e4), torch.arange(0, d // 2).float() * 2 / d)).to(DEV) if rotate else None
    cos_sin = None
    if rotate:
        cos_sin = torch.empty(B, d // 2, 2, device=DEV)
        o.rope_table(positions, inv_freq, cos_sin)
    scale = 1 / math.sqrt(d)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    # the two-kernel way
    qkv_a, kp_a, vp_a = qkv0.clone(), kp0.clone(), vp0.clone()
    o.rope_kv_write(qkv_a, positions, token_seq, seq_slot, inv_freq, d if rotate else 0, kp_a, vp_a, table, ps, nh, nkv, d,
                    True, status, cos_sin=cos_sin)
    for n_splits, with_counters in ((1, False), (3, False), (2, True), (5, True)):
        pa, pm = torch.empty(B, nh, n_splits, d, device=DEV), torch.empty(B, nh, n_splits, 2, device=DEV)
        counters = torch.zeros(B * nkv * -(-(nh // nkv) // 16), dtype=torch.int32, device=DEV) if with_counters else None
        want = torch.zeros(B, nh * d, dtype=dt, device=DEV)
        o.decode_attention(qkv_a, kp_a, vp_a, table, ps, positions, token_seq, seq_slot, want, nh, nkv, d, window, scale,
                           0, n_splits, pa, pm, status=status, counters=counters)
        qkv_b, kp_b, vp_b = qkv0.clone(), kp0.clone(), vp0.clone()
        got = torch.zeros_like(want)
        o.decode_attention(qkv_b, kp_b, vp_b, table, ps, positions, token_seq, seq_slot, got, nh, nkv, d, window, scale,
                           0, n_splits, torch.empty_like(pa), torch.empty_like(pm), status=status, counters=counters,
                           store_new=True, write_pages=True, cos_sin=cos_sin, fresh_positions=1)
        assert int(status) == 0
        assert torch.equal(kp_b, kp_a) and torch.equal(vp_b, vp_a), n_splits       # the pages hold the same bits
        assert torch.equal(qkv_b, qkv0)                                            # the rows stay as projected
        assert rel(got, want) < 4e-3, n_splits
        # a layer that reads another layer's cache: nothing is stored, the token's own key still counts
        kp_c, vp_c = kp0.clone(), vp0.clone()
        got_c = torch.zeros_like(want)
        o.decode_attention(qkv0.clone(), kp_c, vp_c, table, ps, positions, token_seq, seq_slot, got_c, nh, nkv, d, window,
                           scale, 0, n_splits, torch.empty_like(pa), torch.empty_like(pm), status=status, counters=counters,
                           store_new=True, write_pages=False, cos_sin=cos_sin)
        assert torch.equal(kp_c, kp0) and torch.equal(got_c, got)
    # and against the plain statement, with the new key and value in their places
    x = qkv_a.float().cpu()
    for s, L in enumerate(lens):
        ks[s][L - 1] = x[s, nh * d:(nh + nkv) * d].reshape(nkv, d)
        vs[s][L - 1] = x[s, (nh + nkv) * d:].reshape(nkv, d)
        ref = plain_attention(x[s, :nh * d].reshape(nh, d), ks[s], vs[s], L - 1, window, scale)
        assert rel(got[s].float().cpu().reshape(nh, d), ref) < 1e-2, s
    # what the kernel cannot do itself is refused, not approximated
    with pytest.raises(o.KernelError):
        o.decode_attention(qkv0.float(), kp0.float(), vp0.float(), table, ps, positions, token_seq, seq_slot,
                           torch.zeros(B, nh * d, device=DEV), nh, nkv, d, window, scale, 0, 1, pa, pm, store_new=True)


# ------------------------------------------------------------------ router product, routing and gather in one launch
@pytest.mark.parametrize("T,E,K,H,extra", [(1, 60, 4, 2048, 1), (8, 60, 4, 2048, 1), (3, 5, 1, 80, 0), (7, 64, 8, 3584, 0),
                                           (2, 131, 6, 520, 1), (5, 8, 3, 128, 1)])
def test_route_fused_is_product_routing_and_gather(T, E, K, H, extra):
    """One cluster does what three kernels do: logits = x . w^T (E router rows and `extra` further rows, 32-bit sums),
    the routing over the first E, and the rows in expert order.  The logits against a 32-bit product, everything else
    equal to route_small run on those very logits, the gathered rows equal to the rows they copy."""
    o = ops()
    x = rnd(T + 1, H + 8, dtype=torch.bfloat16, seed=T)[1:, :H]        # a strided view
    w = rnd(E + extra, H, dtype=torch.bfloat16, scale=0.3, seed=E)
    assert o.route_fused_ok(x, w, E)
    i32 = dict(dtype=torch.int32, device=DEV)
    R = E + extra
    for renorm in (False, True):
        for gather in (True, False):
            logits = torch.full((T, R), float("nan"), device=DEV)
            ids_a, w_a = torch.empty(T, K, **i32), torch.empty(T, K, device=DEV)
            offsets, src, inv = torch.empty(E + 1, **i32), torch.empty(T * K, **i32), torch.empty(T * K, **i32)
            active = torch.empty(min(E, T * K), **i32)
            xp = torch.full((T * K, H), float("nan"), dtype=torch.bfloat16, device=DEV) if gather else None
            o.route_fused(x, w, logits, K, renorm, ids_a, w_a, offsets, src, inv, active, n_experts=E, xp_out=xp)
            assert rel(logits, x.float() @ w.float().T) < 3e-6
            ids_b, w_b = torch.empty(T, K, **i32), torch.empty(T, K, device=DEV)
            off_b, src_b, inv_b = torch.empty(E + 1, **i32), torch.empty(T * K, **i32), torch.empty(T * K, **i32)
            act_b = torch.empty(min(E, T * K), **i32)
            o.route_small(logits, K, renorm, ids_b, w_b, off_b, src_b, inv_b, act_b, n_experts=E)
            assert torch.equal(ids_a, ids_b) and torch.equal(w_a, w_b) and torch.equal(offsets, off_b)
            assert torch.equal(active, act_b)
            flat = ids_a.flatten().tolist()
            assert sorted(inv.tolist()) == list(range(T * K))
            for i, r in enumerate(inv.tolist()):
                assert int(offsets[flat[i]]) <= r < int(offsets[flat[i] + 1]) and int(src[r]) == i // K
            if gather:
                assert torch.equal(xp, x[src.long()])
    # what it does not take is said beforehand
    assert not o.route_fused_ok(rnd(9, H, dtype=torch.bfloat16), w, E) and not o.route_fused_ok(x.float(), w, E)
