"""Each CUDA kernel alone against a plain PyTorch float32/float64 restatement of its
formula, at sizes other than the engine's tiny models (widths that are no power of two,
odd head sizes, many groups)."""
import json
import math

import numpy as np
import pytest
import torch

import helpers
import plain_qwen2moe as P
from test_plain import oracle_inputs

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


@pytest.fixture(scope="module")
def K():
    from cajeta_llm_b200.csrc import kernels
    return kernels


def rnd(*shape, seed=0, scale=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


def tol(dtype):
    return dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed_gather(K, dtype):
    table = rnd(301, 72, seed=1, dtype=dtype)
    ids = torch.tensor([0, 300, 17, 17, 5], dtype=torch.int32, device=DEV)
    out = torch.empty(5, 72, device=DEV)
    K.embed_gather(out, table, ids)
    assert torch.equal(out, table[ids.long()].float())
    K.embed_gather(out, table, ids, 1.75)                      # an embedding scale (0 = none)
    assert torch.equal(out, table[ids.long()].float() * 1.75)


# four elements a load: 72, 1000, 2048, 3584 (two loads a thread), 5000 (four); one at a time: 1002, 10000
@pytest.mark.parametrize("H", [72, 1000, 1002, 2048, 3584, 5000, 10000])
def test_rmsnorm(K, H):
    x = rnd(7, H, seed=2, scale=3.0)
    w = rnd(H, seed=3)
    want = P.rmsnorm(x.double().cpu(), w.double().cpu(), 1e-5)
    out = torch.empty(7, H, device=DEV)
    K.rmsnorm(x, w, 1e-5, out)
    assert torch.allclose(out.cpu().double(), want, atol=1e-5, rtol=1e-5)
    out_b = torch.empty(3, H, device=DEV, dtype=torch.bfloat16)
    out_f = torch.empty(3, H, device=DEV)
    rows = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEV)
    K.rmsnorm(x, w, 1e-5, out_b, out_f, rows)
    assert torch.allclose(out_f.cpu().double(), want[[6, 0, 3]], atol=1e-5, rtol=1e-5)
    assert torch.equal(out_b, out_f.to(torch.bfloat16))            # one rounding, from the float32 value


def test_rmsnorm_adds_pending_partial_sums_first(K):
    H = 200
    x = rnd(5, H, seed=2, scale=2.0)
    parts = rnd(3, 5, H, seed=8)
    w = rnd(H, seed=3)
    total = x.double() + parts.double().sum(0)
    out = torch.empty(5, H, device=DEV, dtype=torch.bfloat16)
    out32 = torch.empty(5, H, device=DEV)
    K.rmsnorm(x, w, 1e-6, out, out32, None, parts)
    assert torch.allclose(x.double(), total, atol=1e-6)                      # the residual stream keeps the sum
    assert torch.allclose(out32.double().cpu(), P.rmsnorm(total.cpu(), w.double().cpu(), 1e-6), atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("H", [200, 202, 3584])
def test_rmsnorm_partial_sums_and_three_term_form(K, H):
    """Partial sums are added first whatever the row's width; the three bfloat16 terms add up to
    the float32 result to 2^-24 of its size (hi is the ordinary bfloat16 result)."""
    x = rnd(6, H, seed=4, scale=2.0)
    parts = rnd(2, 6, H, seed=9)
    w = rnd(H, seed=5)
    total = x.double() + parts.double().sum(0)
    out = torch.empty(6, H, device=DEV, dtype=torch.bfloat16)
    split = torch.empty(6, 3 * H, device=DEV, dtype=torch.bfloat16)
    K.rmsnorm(x, w, 1e-6, out, None, None, parts, split)
    want = P.rmsnorm(total.cpu(), w.double().cpu(), 1e-6)
    assert torch.allclose(x.double(), total, atol=1e-6)
    assert torch.equal(split[:, :H], out)
    three = split.double().view(6, 3, H).sum(1).cpu()
    assert torch.allclose(three, want, atol=1e-5, rtol=1e-5)
    exact = torch.empty(6, H, device=DEV)
    K.rmsnorm(x, w, 1e-6, out, exact, None, None, None)
    assert float((three - exact.double().cpu()).abs().max()) <= 2.0 ** -22 * float(exact.abs().max())


@pytest.mark.parametrize("H", [2048, 1540, 3584, 384])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_of_a_row_does_not_depend_on_the_rows_beside_it(K, H, out_dtype):
    """Hundreds of rows in one call (wide rows then take the kernel with a quarter of the threads) against
    the plain norm, and bit for bit against the same rows normed a few at a time - with pending partial
    sums, the float32 copy and the three-term form."""
    rows, few = 333, 9
    x0 = rnd(rows, H, seed=41, scale=3.0)
    w = rnd(H, seed=42)
    parts = rnd(3, rows, H, seed=43)
    want = P.rmsnorm((x0.double() + parts.double().sum(0)).cpu(), w.double().cpu(), 1e-6)
    x = x0.clone()
    out, out32 = torch.empty(rows, H, device=DEV, dtype=out_dtype), torch.empty(rows, H, device=DEV)
    split = torch.empty(rows, 3 * H, device=DEV, dtype=torch.bfloat16)
    K.rmsnorm(x, w, 1e-6, out, out32, None, parts, split)
    assert torch.allclose(out32.double().cpu(), want, atol=1e-5, rtol=1e-5)
    for lo in (0, 100, rows - few):
        xs = x0[lo:lo + few].clone()
        o, o32 = torch.empty(few, H, device=DEV, dtype=out_dtype), torch.empty(few, H, device=DEV)
        sp = torch.empty(few, 3 * H, device=DEV, dtype=torch.bfloat16)
        K.rmsnorm(xs, w, 1e-6, o, o32, None, parts[:, lo:lo + few].contiguous(), sp)
        assert torch.equal(xs, x[lo:lo + few]) and torch.equal(o, out[lo:lo + few])
        assert torch.equal(o32, out32[lo:lo + few]) and torch.equal(sp, split[lo:lo + few])
    plain = torch.empty(rows, H, device=DEV, dtype=out_dtype)             # and without any of the extras
    K.rmsnorm(x0, w, 1e-6, plain)
    one = torch.empty(1, H, device=DEV, dtype=out_dtype)
    K.rmsnorm(x0[200:201].contiguous(), w, 1e-6, one)
    assert torch.equal(one[0], plain[200])


@pytest.mark.parametrize("dtype,H", [(torch.bfloat16, 2048), (torch.bfloat16, 72), (torch.float32, 100), (torch.bfloat16, 67)])
@pytest.mark.parametrize("rows", [5, 300, 700])
def test_gather_rows(K, dtype, H, rows):
    """Few rows: a block a row; many rows of a multiple of 16 bytes: a warp a row."""
    x = rnd(41, H, seed=11, dtype=dtype)
    g = torch.Generator().manual_seed(rows)
    index = torch.randint(0, 41, (rows,), generator=g, dtype=torch.int32).to(DEV)
    out = torch.empty(rows, H, device=DEV, dtype=dtype)
    K.gather_rows(x, index, out)
    assert torch.equal(out, x[index.long()])


@pytest.mark.parametrize("M,N,K_", [(1, 5, 7), (3, 70, 100), (65, 129, 33), (130, 64, 257)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gemm_plain_bias_accumulate(K, M, N, K_, dtype):
    a = rnd(M, K_, seed=4, dtype=dtype)
    w = rnd(N, K_, seed=5, dtype=dtype)
    b = rnd(N, seed=6)
    want = a.double() @ w.double().t()
    out = torch.empty(M, N, device=DEV)
    K.gemm(a, w, out)
    assert torch.allclose(out.double(), want, atol=1e-4, rtol=1e-5)
    K.gemm(a, w, out, bias=b)
    assert torch.allclose(out.double(), want + b.double(), atol=1e-4, rtol=1e-5)
    base = rnd(M, N, seed=7)
    acc = base.clone()
    K.gemm(a, w, acc, accumulate=True)
    assert torch.allclose(acc.double(), want + base.double(), atol=1e-4, rtol=1e-5)
    if dtype == torch.bfloat16:
        out_b = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
        K.gemm(a, w, out_b)
        assert torch.equal(out_b, out_from(want, a, w, K).to(torch.bfloat16))


def out_from(want, a, w, K):
    out = torch.empty(want.shape, device=DEV)
    K.gemm(a, w, out)
    return out


def test_gemm_rows_do_not_depend_on_the_batch(K):
    a = rnd(90, 77, seed=8)
    w = rnd(50, 77, seed=9)
    full = torch.empty(90, 50, device=DEV)
    K.gemm(a, w, full)
    for lo, hi in ((0, 1), (13, 14), (60, 90)):
        part = torch.empty(hi - lo, 50, device=DEV)
        K.gemm(a[lo:hi].contiguous(), w, part)
        assert torch.equal(part, full[lo:hi])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gemm_swiglu_and_grouped(K, dtype):
    T, H, I, E, k = 37, 52, 44, 5, 2
    x = rnd(T, H, seed=10, dtype=dtype)
    wg, wu = rnd(E, I, H, seed=11, scale=0.3, dtype=dtype), rnd(E, I, H, seed=12, scale=0.3, dtype=dtype)
    wd = rnd(E, H, I, seed=13, scale=0.3, dtype=dtype)
    # dense SwiGLU with expert 0's matrices
    act = torch.empty(T, I, device=DEV, dtype=dtype)
    K.gemm(x, wg[0], act, w_up=wu[0])
    want = P.silu(x.double() @ wg[0].double().t()) * (x.double() @ wu[0].double().t())
    assert torch.allclose(act.double(), want, **tol(dtype))
    # grouped: random picks, counting sort, per-expert products
    g = torch.Generator().manual_seed(14)
    sel = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(torch.int32).to(DEV)
    sel[:, 0] = torch.where(sel[:, 0] == 3, sel[:, 1], sel[:, 0])       # expert 3 may end up empty
    offsets = torch.empty(E + 1, dtype=torch.int32, device=DEV)
    slot_token = torch.empty(T * k, dtype=torch.int32, device=DEV)
    slot_of_pick = torch.empty(T * k, dtype=torch.int32, device=DEV)
    K.moe_group(sel, k, E, offsets, slot_token, slot_of_pick)
    off = offsets.cpu().tolist()
    flat = sel.flatten().cpu().tolist()
    assert off[0] == 0 and off[-1] == T * k and all(off[e + 1] - off[e] == flat.count(e) for e in range(E))
    st, sp = slot_token.cpu().tolist(), slot_of_pick.cpu().tolist()
    for i, e in enumerate(flat):
        assert off[e] <= sp[i] < off[e + 1] and st[sp[i]] == i // k
    for e in range(E):      # stable: within an expert the picks keep their order
        mine = [sp[i] for i, x_ in enumerate(flat) if x_ == e]
        assert mine == sorted(mine)
    act = torch.empty(T * k, I, device=DEV, dtype=dtype)
    K.gemm(x, wg, act, w_up=wu, group_offsets=offsets, a_row_index=slot_token)
    y = torch.empty(T * k, H, device=DEV)
    K.gemm(act, wd, y, group_offsets=offsets)
    for i, e in enumerate(flat):
        row = x[i // k].double()
        a_want = P.silu(wg[e].double() @ row) * (wu[e].double() @ row)
        assert torch.allclose(act[sp[i]].double(), a_want, **tol(dtype)), (i, e)
        y_want = wd[e].double() @ act[sp[i]].double()
        assert torch.allclose(y[sp[i]].double(), y_want, atol=1e-4, rtol=1e-4), (i, e)
    # combine in selection order with a gated shared row
    w = rnd(T, k, seed=15).abs()
    shared, gate = rnd(T, H, seed=16), rnd(T, seed=17).abs()
    hs = rnd(T, H, seed=18)
    want = hs.double().clone()
    for t in range(T):
        acc = sum(w[t, j].double() * y[sp[t * k + j]].double() for j in range(k)) + gate[t].double() * shared[t].double()
        want[t] += acc
    K.moe_combine(hs, y, slot_of_pick, w, k, shared, gate)
    assert torch.allclose(hs.double(), want, atol=1e-5, rtol=1e-5)
    # groups that hold every token follow the routed ones; the shared rows come in chunks
    C = 3
    offsets2 = torch.empty(E + C + 1, dtype=torch.int32, device=DEV)
    slot_token2 = torch.empty(T * k + C * T, dtype=torch.int32, device=DEV)
    K.moe_group(sel, k, E, offsets2, slot_token2, slot_of_pick, extra_groups=C)
    assert offsets2.cpu().tolist() == off + [T * k + (c + 1) * T for c in range(C)]
    assert slot_token2[:T * k].cpu().tolist() == st and slot_token2[T * k:].cpu().tolist() == list(range(T)) * C
    chunks = rnd(C, T, H, seed=19)
    hs2 = rnd(T, H, seed=18)
    K.moe_combine(hs2, y, slot_of_pick, w, k, chunks, gate)
    want2 = want - gate.double()[:, None] * shared.double() + gate.double()[:, None] * chunks.double().sum(0)
    assert torch.allclose(hs2.double(), want2, atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("k", [1, 2, 3, 4, 6, 8])
@pytest.mark.parametrize("H,C", [(136, 0), (136, 1), (200, 5), (75, 3)])
def test_combine_of_few_rows_and_of_many_gives_the_same_bits(K, k, H, C):
    """Few rows take a form whose loads are written out per pick, many rows a loop: both hold to the
    weighted sum in selection order plus the gated chunks of a shared expert in chunk order, and a row
    has the same bits in either (the first rows of the large call are the small call's rows)."""
    few, many = 7, 300
    slots = many * k
    g = torch.Generator().manual_seed(100 * k + H)
    y = rnd(slots, H, seed=31)
    slot_of_pick = torch.randperm(slots, generator=g).to(torch.int32).to(DEV)
    w = rnd(many, k, seed=32).abs()
    shared = rnd(C, many, H, seed=33) if C else None
    gate = rnd(many, seed=34).abs() if C else None
    hs0 = rnd(many, H, seed=35)
    want = hs0.double().clone()
    picks = slot_of_pick.view(many, k).long()
    for j in range(k):
        want += w[:, j].double()[:, None] * y[picks[:, j]].double()
    if C:
        want += gate.double()[:, None] * shared.double().sum(0)
    big = hs0.clone()
    K.moe_combine(big, y, slot_of_pick, w, k, shared, gate)
    assert torch.allclose(big.double(), want, atol=1e-5, rtol=1e-5)
    small = hs0[:few].clone()
    K.moe_combine(small, y, slot_of_pick[:few * k].contiguous(), w[:few].contiguous(), k,
                  shared[:, :few].contiguous() if C else None, gate[:few].contiguous() if C else None)
    assert torch.equal(small, big[:few])


@pytest.mark.parametrize("T,k,E,extra", [(9, 2, 5, 0), (511, 4, 60, 0), (513, 4, 60, 2), (3000, 3, 7, 1)])
def test_grouping_is_a_stable_sort_by_expert(K, T, k, E, extra):
    """Few picks (8 warps a block) and thousands (32 warps): offsets count each expert's picks, the
    slots of an expert keep pick order, every pick finds its slot; groups of every token follow."""
    g = torch.Generator().manual_seed(T)
    sel = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(torch.int32)
    n = T * k
    offsets = torch.empty(E + extra + 1, dtype=torch.int32, device=DEV)
    slot_token = torch.empty(n + extra * T, dtype=torch.int32, device=DEV)
    slot_of_pick = torch.empty(n, dtype=torch.int32, device=DEV)
    K.moe_group(sel.to(DEV), k, E, offsets, slot_token, slot_of_pick, extra_groups=extra)
    flat = sel.flatten()
    order = torch.sort(flat, stable=True).indices                      # slot -> pick
    counts = torch.bincount(flat, minlength=E)
    want_off = torch.cat([torch.zeros(1, dtype=torch.long), counts.cumsum(0)]).tolist() + [n + (c + 1) * T for c in range(extra)]
    assert offsets.cpu().tolist() == want_off
    assert slot_token[:n].cpu().tolist() == (order // k).tolist()
    want_slot = torch.empty(n, dtype=torch.long)
    want_slot[order] = torch.arange(n)
    assert slot_of_pick.cpu().tolist() == want_slot.tolist()
    assert slot_token[n:].cpu().tolist() == list(range(T)) * extra


def test_router_kernel_meets_the_reference_constants(K):
    o, router, probe, gate = oracle_inputs()
    x = torch.stack([probe, -probe]).to(DEV)
    sel = torch.empty(2, 2, dtype=torch.int32, device=DEV)
    w = torch.empty(2, 2, device=DEV)
    sig = torch.empty(2, device=DEV)
    K.router_topk(x, router.to(DEV), gate.to(DEV), 2, False, sel, w, sig)
    assert sel.cpu().tolist() == [o["probe"]["sel"], o["probe_negated"]["sel"]]
    assert np.allclose(w.cpu().numpy(), [o["probe"]["w_raw"], o["probe_negated"]["w_raw"]], atol=o["tolerance"])
    assert abs(float(sig[0]) - o["shared_gate_sigmoid"]) < o["tolerance"]
    K.router_topk(x, router.to(DEV), None, 2, True, sel, w, None)
    assert np.allclose(w[0].cpu().numpy(), o["probe"]["w_norm"], atol=o["tolerance"])


@pytest.mark.parametrize("E,k,H", [(7, 3, 100), (60, 4, 2048), (130, 8, 333)])
def test_router_kernel_against_plain(K, E, k, H):
    T = 19
    x = rnd(T, H, seed=20)
    wr = rnd(E, H, seed=21, scale=0.1)
    x[3] = 0.0                                  # all logits equal: ties go to the lowest indices
    for norm in (False, True):
        sel = torch.empty(T, k, dtype=torch.int32, device=DEV)
        w = torch.empty(T, k, device=DEV)
        K.router_topk(x, wr, None, k, norm, sel, w, None)
        for t in range(T):
            s_want, w_want = P.route(P.linear(x[t].double().cpu(), wr.double().cpu()), k, norm)
            assert sel[t].cpu().tolist() == s_want, t
            assert torch.allclose(w[t].cpu().double(), w_want, atol=1e-6, rtol=1e-5)
        assert sel[3].cpu().tolist() == list(range(k))


def paged_setup(lengths, n_kv, hd, page, dtype, seed, scramble=True, live_from=None):
    """K/V of several requests laid into scrambled pages; returns planes, table, dense copies.

    ``live_from[r]``: request r has given back every page that lies wholly below that position
    (what a windowed group does once the window has passed a page): the table entry is -1 and
    the page itself, like every page no table names, holds NaN - another request may own it by
    now, and nothing of it may reach a result.  The planes are views behind a guard page of NaN,
    so that a kernel that did follow a -1 entry would show in the result instead of reading
    outside the allocation."""
    g = torch.Generator().manual_seed(seed)
    pages_per = [-(-L // page) for L in lengths]
    total = sum(pages_per) + 3
    perm = torch.randperm(total, generator=g).tolist() if scramble else list(range(total))
    width = max(pages_per) + 2
    table = torch.full((len(lengths), width), -1, dtype=torch.int32)
    fill = float("nan") if live_from is not None else 0.0
    kp = torch.full((total + 1, n_kv, page, hd), fill)
    vp = torch.full((total + 1, n_kv, page, hd), fill)
    ks, vs = [], []
    nxt = 0
    for r, L in enumerate(lengths):
        k = torch.randn(L, n_kv, hd, generator=g)
        v = torch.randn(L, n_kv, hd, generator=g)
        ks.append(k), vs.append(v)
        for j in range(pages_per[r]):
            pg = perm[nxt]
            nxt += 1
            if live_from is not None and (j + 1) * page <= live_from[r]:
                continue                                   # given back: -1 in the table, NaN in the page
            table[r, j] = pg
            n = min(page, L - j * page)
            kp[1 + pg, :, :n] = k[j * page: j * page + n].transpose(0, 1)
            vp[1 + pg, :, :n] = v[j * page: j * page + n].transpose(0, 1)
            if live_from is not None:
                kp[1 + pg, :, n:] = 1000.0                 # what an earlier owner left behind the request's end
                vp[1 + pg, :, n:] = 1000.0
    return kp.to(dtype).to(DEV)[1:], vp.to(dtype).to(DEV)[1:], table.to(DEV), ks, vs


def window_start(p, window):
    return p + 1 - window if window > 0 and p + 1 > window else 0


@pytest.mark.parametrize("heads,n_kv,hd,page,window", [(4, 2, 16, 16, 0), (4, 1, 24, 16, 8), (6, 3, 40, 4, 0),
                                                         (16, 16, 128, 16, 0), (14, 2, 128, 16, 33), (2, 1, 256, 8, 0)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_paged_attention(K, heads, n_kv, hd, page, window, dtype):
    lengths = [70, 1, 33, 16]
    kp, vp, table, ks, vs = paged_setup(lengths, n_kv, hd, page, dtype, seed=30)
    # rows: every position of request 2 (a whole prompt), the last of the others (decode rows), mixed order
    rows = [(0, 69), (1, 0)] + [(2, p) for p in range(33)] + [(3, 15), (0, 31), (0, 32)]
    g = torch.Generator().manual_seed(31)
    q = torch.randn(len(rows), heads, hd, generator=g).to(dtype).to(DEV)
    out = torch.empty_like(q)
    pos = torch.tensor([p for _, p in rows], dtype=torch.int32, device=DEV)
    req = torch.tensor([r for r, _ in rows], dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(hd)
    K.paged_attention(q, out, kp, vp, pos, req, table, page, heads, n_kv, hd, window, scale)
    for i, (r, p) in enumerate(rows):
        kd = ks[r].to(dtype).double()
        vd = vs[r].to(dtype).double()
        qq = torch.zeros(p + 1, heads, hd, dtype=torch.float64)
        qq[p] = q[i].double().cpu()
        want = P.attention(qq, kd[:p + 1], vd[:p + 1], window, scale)[p]
        assert torch.allclose(out[i].double().cpu(), want, **tol(dtype)), (i, r, p)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_finds_one_far_key_among_hundreds_and_the_edge_of_the_window(K, dtype):
    heads, n_kv, hd, page = 4, 2, 32, 16
    L = 600
    kp, vp, table, ks, vs = paged_setup([L], n_kv, hd, page, dtype, seed=40)
    g = torch.Generator().manual_seed(41)
    q = torch.randn(1, heads, hd, generator=g)
    far = 37                                               # a key in the third page, far behind
    # scale one key so that its score stands out: it is the query direction, blown up
    pg, slot = int(table[0, far // page]), far % page
    for h in range(n_kv):
        kp[pg, h, slot] = (q[0, h * 2] * 40.0).to(dtype).to(DEV)
    qd = q.to(dtype).to(DEV)
    out = torch.empty_like(qd)
    pos = torch.tensor([L - 1], dtype=torch.int32, device=DEV)
    req = torch.zeros(1, dtype=torch.int32, device=DEV)
    K.paged_attention(qd, out, kp, vp, pos, req, table, page, heads, n_kv, hd, 0, 1.0 / math.sqrt(hd))
    for h in (0, 2):                                       # the heads whose query the key was built from
        assert torch.allclose(out[0, h].float().cpu(), vp[pg, h // 2, slot].float().cpu(), atol=2e-2)
    # window: with w = L - far the far key is the first inside, with one less it is outside
    for w, inside in ((L - far, True), (L - far - 1, False)):
        K.paged_attention(qd, out, kp, vp, pos, req, table, page, heads, n_kv, hd, w, 1.0 / math.sqrt(hd))
        close = torch.allclose(out[0, 0].float().cpu(), vp[pg, 0, slot].float().cpu(), atol=2e-2)
        assert close == inside, (w, inside)


# units of four dims: (16, 16), (24, 24), (64, 32), (128, 128); of two: (20, 12); one at a time: (18, 6)
@pytest.mark.parametrize("hd,rot", [(16, 16), (24, 24), (64, 32), (128, 128), (20, 12), (18, 6)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rope_and_cache_write(K, hd, rot, dtype):
    heads, n_kv, page, T = 3, 2, 4, 11
    qd, kvd = heads * hd, n_kv * hd
    qkv = rnd(T, qd + 2 * kvd, seed=50)
    positions = [5, 6, 7, 8, 0, 1, 2, 3, 4, 400, 17]
    req = [0, 0, 0, 0, 1, 1, 1, 1, 1, 2, 3]
    table = torch.full((4, 101), -1, dtype=torch.int32)
    table[0, 1], table[0, 2], table[1, 0], table[1, 1], table[2, 100], table[3, 4] = 9, 2, 5, 0, 7, 3
    table = table.to(DEV)
    kp = torch.zeros(10, n_kv, page, hd, dtype=dtype, device=DEV)
    vp = torch.zeros_like(kp)
    inv = P.inv_freq(rot, 10000.0, torch.float32).to(DEV)
    q_out = torch.empty(T, heads, hd, dtype=dtype, device=DEV)
    K.rope_kv_write(qkv, 0, qd, qd + kvd, q_out, kp, vp, torch.tensor(positions, dtype=torch.int32, device=DEV),
                    torch.tensor(req, dtype=torch.int32, device=DEV), table, page, heads, n_kv, hd, rot, inv, True)
    pos_t = torch.tensor(positions)
    x = qkv.cpu().double()

    def want_rope(t, n):
        t = t.reshape(T, n, hd)
        return torch.cat([P.rope(t[..., :rot], pos_t, inv.cpu().double()), t[..., rot:]], dim=-1)

    wq, wk = want_rope(x[:, :qd], heads), want_rope(x[:, qd:qd + kvd], n_kv)
    wv = x[:, qd + kvd:].reshape(T, n_kv, hd)
    t_ = dict(atol=2e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=1e-2)
    assert torch.allclose(q_out.double().cpu(), wq, **t_)
    tab = table.cpu()
    for i, (r, p) in enumerate(zip(req, positions)):
        pg = int(tab[r, p // page])
        assert torch.allclose(kp[pg, :, p % page].double().cpu(), wk[i], **t_), i
        assert torch.allclose(vp[pg, :, p % page].double().cpu(), wv[i], **t_), i
    assert int((kp != 0).any(dim=-1).sum()) == T * n_kv        # nothing else was written


def test_argmax_takes_the_first_of_equals(K):
    V = 151_936
    logits = rnd(3, V, seed=60)
    logits[0, 777] = logits[0, 150_000] = 9.0
    logits[1, V - 1] = 11.0
    logits[2] = 0.25
    out = torch.empty(3, dtype=torch.int32, device=DEV)
    K.argmax(logits, out)
    assert out.cpu().tolist() == [777, V - 1, 0]


@pytest.mark.parametrize("V", [257, 5003])
def test_sampler_distribution_and_draws_follow_the_plain_sampler(K, V):
    cases = [dict(t=0.8, k=0, p=0.0, pen=1.0), dict(t=1.3, k=40, p=0.0, pen=1.0), dict(t=0.7, k=0, p=0.9, pen=1.0),
             dict(t=1.0, k=50, p=0.8, pen=1.3), dict(t=0.0, k=0, p=0.0, pen=1.0), dict(t=0.0, k=5, p=0.5, pen=2.0),
             dict(t=1.0, k=3, p=0.0, pen=1.0)]
    n = len(cases)
    logits = rnd(n, V, seed=61, scale=2.0)
    logits[6] = 0.5                                        # all equal: top-3 keeps ids 0, 1, 2
    hist = [[], [], [], [3, 9, 3, 100], [], [int(logits[5].argmax()), 7], []]
    us = [0.0, 0.37, 0.93, 0.5, 0.2, 0.6, 0.66]
    flat = [t for h in hist for t in h]
    off = np.cumsum([0] + [len(h) for h in hist]).astype(np.int32)
    scratch = torch.empty(n * V, device=DEV)
    out = torch.empty(n, dtype=torch.int32, device=DEV)

    def up(a, dt):
        return torch.tensor(a, dtype=dt, device=DEV)

    K.sample(logits, up([c["t"] for c in cases], torch.float32), up(us, torch.float32), scratch, out,
             top_k=up([c["k"] for c in cases], torch.int32), top_p=up([c["p"] for c in cases], torch.float32),
             repeat_penalty=up([c["pen"] for c in cases], torch.float32), history=up(flat, torch.int32),
             history_offsets=torch.from_numpy(off).to(DEV))
    e = scratch.view(n, V).cpu()
    got = out.cpu().tolist()
    for i, c in enumerate(cases):
        want = P.prepared_distribution(logits[i].cpu(), c["t"], c["k"], c["p"], c["pen"], hist[i])
        dist = e[i] / e[i].sum()
        assert ((dist > 0) == (want > 0)).all(), i
        assert torch.allclose(dist, want, atol=1e-6, rtol=1e-4), i
        assert got[i] == P.draw(want, us[i]), (i, got[i])
    assert (e[6] > 0).nonzero().flatten().tolist() == [0, 1, 2]
    # many draws of one row land where the plain sampler puts them
    m = 64
    row = logits[1:2].expand(m, V).contiguous()
    us = [(i + 0.5) / m for i in range(m)]
    out = torch.empty(m, dtype=torch.int32, device=DEV)
    scratch = torch.empty(m * V, device=DEV)
    K.sample(row, up([1.1] * m, torch.float32), up(us, torch.float32), scratch, out)
    want = P.prepared_distribution(logits[1].cpu(), 1.1, 0, 0.0, 1.0, [])
    agree = sum(int(g == P.draw(want, u)) for g, u in zip(out.cpu().tolist(), us))
    assert agree >= m - 1               # a draw within rounding of a boundary may fall either way


@pytest.mark.parametrize("heads,n_kv,hd,page,window", [(16, 16, 128, 16, 0), (14, 2, 128, 16, 0), (6, 3, 64, 8, 0),
                                                         (8, 4, 64, 16, 200), (4, 1, 128, 16, 130), (24, 2, 64, 16, 0),
                                                         (4, 2, 128, 16, 40), (6, 3, 64, 16, 150)])
@pytest.mark.parametrize("chunk", [64, 128, 0])
def test_decode_attention_split_kv(K, heads, n_kv, hd, page, window, chunk):
    """Rows of very different lengths (1 key, exactly one chunk, several chunks and a
    remainder) against the plain attention, on the FMA pipe (chunks of 64 or 128) and on the
    tensor cores (chunk 0); run twice to see the arrival counters reset.  With a window the
    pages behind it have been given back (-1 in the table, NaN where they were)."""
    lengths = [1, 128, 129, 700, 300, 17, 64, 65]
    dtype = torch.bfloat16
    live_from = [window_start(L - 1, window) for L in lengths] if window > 0 else None
    kp, vp, table, ks, vs = paged_setup(lengths, n_kv, hd, page, dtype, seed=70, live_from=live_from)
    rows = [(r, L - 1) for r, L in enumerate(lengths)]
    g = torch.Generator().manual_seed(71)
    q = torch.randn(len(rows), heads, hd, generator=g).to(dtype).to(DEV)
    pos = torch.tensor([p for _, p in rows], dtype=torch.int32, device=DEV)
    req = torch.tensor([r for r, _ in rows], dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(hd)
    scratch = K.DecodeScratch()
    outs = []
    for _ in range(2):
        out = torch.full_like(q, 7.0)
        K.decode_attention(q, out, kp, vp, pos, req, table, page, heads, n_kv, hd, window, scale, max(lengths), scratch,
                           chunk=chunk)
        outs.append(out)
    assert torch.equal(outs[0], outs[1])
    assert int(scratch.counters.abs().sum()) == 0
    for i, (r, p) in enumerate(rows):
        qq = torch.zeros(p + 1, heads, hd, dtype=torch.float64)
        qq[p] = q[i].double().cpu()
        want = P.attention(qq, ks[r].to(dtype).double()[:p + 1], vs[r].to(dtype).double()[:p + 1], window, scale)[p]
        assert torch.allclose(outs[0][i].double().cpu(), want, atol=2e-2, rtol=2e-2), (i, r, p)
    if chunk == 0:
        # the chunks merged by a kernel of its own (what steps with many rows do): the same bits
        out2 = torch.full_like(q, 7.0)
        K.decode_attention(q, out2, kp, vp, pos, req, table, page, heads, n_kv, hd, window, scale, max(lengths), scratch,
                           merge_later=True)
        assert torch.equal(out2, outs[0]) and int(scratch.counters.abs().sum()) == 0
    # the same row alone gives the same bits: the chunking depends on the row only
    out1 = torch.empty_like(q[3:4])
    K.decode_attention(q[3:4].contiguous(), out1, kp, vp, pos[3:4].contiguous(), req[3:4].contiguous(), table, page, heads,
                       n_kv, hd, window, scale, lengths[3], K.DecodeScratch(), chunk=chunk)
    assert torch.equal(out1[0], outs[0][3])


def test_decode_merge_kernel_with_nothing_to_merge(K):
    """Many short rows under a large context bound (what a captured decode step of a long
    bucket sees early on): the launch has several chunks a row, the separate merge kernel is
    launched, and no row has anything to merge.  The merge kernel must still order itself
    behind the attention kernel, or the kernel after it could read the output too early; the
    result must equal the in-kernel merge's, also when another kernel follows at once."""
    heads, n_kv, hd, page = 16, 16, 128, 16
    lengths = [1 + (7 * i) % 127 for i in range(64)]             # 64 rows x 16 heads = 1024 pairs, all below 128 keys
    dtype = torch.bfloat16
    kp, vp, table, ks, vs = paged_setup(lengths, n_kv, hd, page, dtype, seed=75)
    g = torch.Generator().manual_seed(76)
    q = torch.randn(len(lengths), heads, hd, generator=g).to(dtype).to(DEV)
    pos = torch.tensor([L - 1 for L in lengths], dtype=torch.int32, device=DEV)
    req = torch.arange(len(lengths), dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(hd)
    scratch = K.DecodeScratch()
    ref = torch.full_like(q, 7.0)
    K.decode_attention(q, ref, kp, vp, pos, req, table, page, heads, n_kv, hd, 0, scale, 1024, scratch, merge_later=False)
    for _ in range(5):
        out = torch.full_like(q, 7.0)
        copy = torch.empty_like(out)
        K.decode_attention(q, out, kp, vp, pos, req, table, page, heads, n_kv, hd, 0, scale, 1024, scratch, merge_later=True)
        K.gather_rows(out.view(len(lengths), -1), req, copy.view(len(lengths), -1))     # a kernel of this library right behind
        assert torch.equal(out, ref) and torch.equal(copy, ref)


@pytest.mark.parametrize("block_rows", [64, 128])
@pytest.mark.parametrize("heads,n_kv,hd,page,window", [(4, 4, 128, 16, 0), (6, 2, 64, 16, 0), (8, 1, 128, 8, 70), (4, 2, 64, 16, 17),
                                                         (6, 3, 64, 16, 150), (4, 2, 128, 16, 40)])
def test_prefill_attention_tiles(K, heads, n_kv, hd, page, window, block_rows):
    """Requests with and without earlier tokens, portions that end inside a tile, a single
    token riding along; every row against the plain attention."""
    dtype = torch.bfloat16
    totals = [200, 64, 131, 40, 300]
    new = [200, 1, 67, 40, 130]                       # rows this step brings; the rest is already cached
    # with a window, what lies behind the window of a request's first new row has been given back
    live_from = [window_start(t - n, window) for t, n in zip(totals, new)] if window > 0 else None
    kp, vp, table, ks, vs = paged_setup(totals, n_kv, hd, page, dtype, seed=90, live_from=live_from)
    starts = [0]
    for n in new:
        starts.append(starts[-1] + n)
    prior = [t - n for t, n in zip(totals, new)]
    g = torch.Generator().manual_seed(91)
    q = torch.randn(starts[-1], heads, hd, generator=g).to(dtype).to(DEV)
    out = torch.full_like(q, 5.0)
    scale = 1.0 / math.sqrt(hd)
    K.prefill_attention(q, out, kp, vp, torch.tensor(starts, dtype=torch.int32, device=DEV),
                        torch.tensor(prior, dtype=torch.int32, device=DEV), table, page, heads, n_kv, hd, window, scale,
                        block_rows=block_rows)
    for r, (T, n) in enumerate(zip(totals, new)):
        qq = torch.zeros(T, heads, hd, dtype=torch.float64)
        qq[T - n:] = q[starts[r]:starts[r + 1]].double().cpu()
        want = P.attention(qq, ks[r].to(dtype).double(), vs[r].to(dtype).double(), window, scale)[T - n:]
        got = out[starts[r]:starts[r + 1]].double().cpu()
        assert torch.allclose(got, want, atol=2e-2, rtol=2e-2), (r, float((got - want).abs().max()))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_random_fill_on_the_device_equals_the_host_generator(K, dtype):
    """A tensor drawn by the kernel holds the same bits as the same tensor drawn by the numpy
    generator (more elements than one pass of the grid covers, a count that is no multiple of
    anything), and a few of them are held to the restatement with Python integers."""
    import plain_random as PR
    from cajeta_llm_b200.parts.plan import ParamSpec
    from cajeta_llm_b200.weights.sources import RandomWeights
    name, seed = "model.layers.0.self_attn.q_proj.weight", 31
    spec = ParamSpec((1531, 1013), std=0.02)
    on_host = RandomWeights(seed, dtype, device="cpu").get(name, spec)
    on_device = RandomWeights(seed, dtype, device=DEV).get(name, spec)
    assert on_device.is_cuda and on_device.dtype == dtype
    assert torch.equal(on_device.cpu(), on_host)
    flat = on_device.flatten().cpu().float()
    for i in (0, 1, 1012, 1013, 1_550_902):
        want = PR.value(seed, name, i, 0.02)
        assert float(flat[i]) == (PR.to_bfloat16(want) if dtype == torch.bfloat16 else want), i
