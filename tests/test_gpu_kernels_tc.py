"""The tensor-core (tcgen05 / TMA) products against a float64 product of the same bfloat16
operands, in both orientations, every epilogue, grouped and split along K, at sizes that
leave partial tiles in every dimension."""
import pytest
import torch

import plain_qwen2moe as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def K():
    from cajeta_llm_b200.csrc import kernels
    yield kernels
    assert kernels.gemm_tc_error() == 0          # no bounded wait ran out during these tests


def rnd(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(torch.bfloat16).to(DEV)


def close(got, want, atol=2e-3, rtol=2e-3):
    d = (got.double() - want.double()).abs()
    bound = atol + rtol * want.double().abs()
    assert bool((d <= bound).all()), f"max diff {float(d.max()):.4e} at {int(d.argmax())}, want max {float(want.abs().max()):.3f}"


@pytest.mark.parametrize("swap,n_mma,T,N,Kd", [(False, 128, 300, 384, 512), (False, 256, 129, 520, 264), (False, 128, 128, 128, 64),
                                                (True, 16, 5, 300, 512), (True, 32, 40, 128, 200), (True, 64, 64, 1000, 2048),
                                                (True, 128, 130, 260, 128), (True, 16, 1, 2048, 2048)])
def test_store_accumulate_bias(K, swap, n_mma, T, N, Kd):
    x, w = rnd(T, Kd, seed=1), rnd(N, Kd, seed=2, scale=0.1)
    bias = torch.randn(N, generator=torch.Generator().manual_seed(3)).to(DEV)
    want = x.double() @ w.double().t()
    out = torch.full((T, N), 7.0, device=DEV)
    K.gemm_tc(x, w, out, K.EPI_STORE_F32, swap, n_mma)
    close(out, want)
    K.gemm_tc(x, w, out, K.EPI_STORE_F32, swap, n_mma, bias=bias)
    close(out, want + bias.double())
    base = torch.randn(T, N, generator=torch.Generator().manual_seed(4)).to(DEV)
    acc = base.clone()
    K.gemm_tc(x, w, acc, K.EPI_ACC_F32, swap, n_mma)
    close(acc, want + base.double())
    ob = torch.empty(T, N, device=DEV, dtype=torch.bfloat16)
    K.gemm_tc(x, w, ob, K.EPI_STORE_BF16, swap, n_mma)
    close(ob, want, atol=2e-2, rtol=1e-2)


@pytest.mark.parametrize("swap,n_mma,T", [(False, 128, 200), (True, 16, 9), (True, 64, 50)])
def test_swiglu(K, swap, n_mma, T):
    N, Kd = 328, 256
    x, wg, wu = rnd(T, Kd, seed=5), rnd(N, Kd, seed=6, scale=0.1), rnd(N, Kd, seed=7, scale=0.1)
    want = P.silu(x.double() @ wg.double().t()) * (x.double() @ wu.double().t())
    out = torch.empty(T, N, device=DEV, dtype=torch.bfloat16)
    K.gemm_tc(x, wg, out, K.EPI_SWIGLU_BF16, swap, n_mma, w_up=wu)
    close(out, want, atol=2e-2, rtol=1e-2)


@pytest.mark.parametrize("swap,n_mma", [(False, 128), (True, 16), (True, 32), (True, 96), (True, 128), (True, 160), (True, 192), (True, 256)])
def test_grouped(K, swap, n_mma):
    E, N, Kd = 6, 200, 192
    counts = [0, 3, 1, 20, 0, 7] if (swap and n_mma <= 32) else [0, 37, 1, 300, 0, 520]
    T = sum(counts)
    offsets = torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int32, device=DEV)
    x = rnd(T, Kd, seed=8)
    wg, wu = rnd(E, N, Kd, seed=9, scale=0.1), rnd(E, N, Kd, seed=10, scale=0.1)
    out = torch.full((T, N), -3.0, device=DEV)
    K.gemm_tc(x, wg, out, K.EPI_STORE_F32, swap, n_mma, group_offsets=offsets)
    act = torch.empty(T, N, device=DEV, dtype=torch.bfloat16)
    K.gemm_tc(x, wg, act, K.EPI_SWIGLU_BF16, swap, n_mma, w_up=wu, group_offsets=offsets)
    lo = 0
    for e, c in enumerate(counts):
        xe = x[lo:lo + c].double()
        close(out[lo:lo + c], xe @ wg[e].double().t())
        close(act[lo:lo + c], P.silu(xe @ wg[e].double().t()) * (xe @ wu[e].double().t()), atol=2e-2, rtol=1e-2)
        lo += c


@pytest.mark.parametrize("live", [20, 27, 40])
def test_grouped_products_of_many_live_groups_choose_their_tile_height(K, live):
    """A decode step's grouped product with more tiles than the machine has SMs picks, inside the kernel,
    tiles of 112 or 96 weight rows when that evens out the rounds (20 live groups of 1,408 features: 112;
    27: 96; 40: 128 stays); 1,408 is a multiple of neither, so the last tile of a group is a partial one
    beside another group's rows.  Against the float64 products, plain and SwiGLU."""
    E, N, Kd = 40, 1408, 256
    g = torch.Generator().manual_seed(live)
    chosen = sorted(torch.randperm(E, generator=g)[:live].tolist())
    counts = [0] * E
    for i, e in enumerate(chosen):
        counts[e] = 1 + i % 3
    T = sum(counts)
    offsets = torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int32, device=DEV)
    x = rnd(T, Kd, seed=27)
    wg, wu = rnd(E, N, Kd, seed=28, scale=0.1), rnd(E, N, Kd, seed=29, scale=0.1)
    out = torch.full((T, N), -3.0, device=DEV)
    K.gemm_tc(x, wg, out, K.EPI_STORE_F32, True, 16, group_offsets=offsets)
    act = torch.empty(T, N, device=DEV, dtype=torch.bfloat16)
    K.gemm_tc(x, wg, act, K.EPI_SWIGLU_BF16, True, 16, w_up=wu, group_offsets=offsets, offsets_settled=True)
    lo = 0
    for e, c in enumerate(counts):
        xe = x[lo:lo + c].double()
        close(out[lo:lo + c], xe @ wg[e].double().t())
        close(act[lo:lo + c], P.silu(xe @ wg[e].double().t()) * (xe @ wu[e].double().t()), atol=2e-2, rtol=1e-2)
        lo += c


@pytest.mark.parametrize("splits", [2, 4, 7])
def test_split_k_partials_sum_to_the_product(K, splits):
    T, N, Kd = 8, 384, 1408
    x, w = rnd(T, Kd, seed=11), rnd(N, Kd, seed=12, scale=0.1)
    bias = torch.randn(N, generator=torch.Generator().manual_seed(13)).to(DEV)
    parts = torch.full((splits, T, N), 9.0, device=DEV)
    K.gemm_tc(x, w, parts, K.EPI_STORE_F32, True, 16, bias=bias, k_splits=splits)
    close(parts.sum(0), x.double() @ w.double().t() + bias.double())


def test_refusals(K):
    x, w = rnd(4, 100, seed=14), rnd(8, 100, seed=15)
    out = torch.empty(4, 8, device=DEV)
    with pytest.raises(K.KernelError, match="alignment"):
        K.gemm_tc(x, w, out, K.EPI_STORE_F32, True, 16)               # K = 100 is not a multiple of 8
    x, w = rnd(4, 64, seed=14), rnd(8, 64, seed=15)
    with pytest.raises(K.KernelError, match="size"):
        K.gemm_tc(x, w, out, K.EPI_STORE_F32, True, 24)


@pytest.mark.parametrize("block_rows", [0, 128, 256])
@pytest.mark.parametrize("heads,n_kv,window", [(4, 4, 0), (6, 2, 0), (8, 1, 150), (4, 2, 40), (2, 2, 128)])
def test_prefill_attention_tcgen05(K, heads, n_kv, window, block_rows):
    """Both attention products on tcgen05: requests with and without earlier tokens, portions
    that end inside a tile, a single token riding along, several key tiles (so the running
    maximum moves and the output is rescaled), a window that starts inside a tile; every
    row against the plain attention, with 256 query rows a block, with 128, and with the choice
    left to the launch.  One far key is made to stand out for the last rows."""
    from test_gpu_kernels import paged_setup, window_start
    import math
    dtype, hd, page = torch.bfloat16, 128, 16
    totals = [700, 64, 131, 300, 513]
    new = [700, 1, 67, 130, 257]                      # rows this step brings; the rest is already cached
    # with a window, the pages behind the window of a request's first new row have been given
    # back: -1 in the table, NaN where they were
    live_from = [window_start(t - n, window) for t, n in zip(totals, new)] if window > 0 else None
    kp, vp, table, ks, vs = paged_setup(totals, n_kv, hd, page, dtype, seed=190, live_from=live_from)
    # stale data in a page's unused tail must not reach the result
    tail = totals[2] % page
    kp[table[2, totals[2] // page].item(), :, tail:] = 3.0
    vp[table[2, totals[2] // page].item(), :, tail:] = 100.0
    starts = [0]
    for n in new:
        starts.append(starts[-1] + n)
    prior = [t - n for t, n in zip(totals, new)]
    g = torch.Generator().manual_seed(191)
    q = torch.randn(starts[-1], heads, hd, generator=g)
    # the last 40 rows of request 0 look hard at key 5 (far behind, in the first tile)
    kdir = ks[0][5].to(dtype).float()                  # [n_kv, hd]
    for h in range(heads):
        q[starts[1] - 40:starts[1], h] = 6.0 * kdir[h // (heads // n_kv)] / kdir[h // (heads // n_kv)].norm() * math.sqrt(hd) / 4
    q = q.to(dtype).to(DEV)
    out = torch.full_like(q, 5.0)
    scale = 1.0 / math.sqrt(hd)
    for _ in range(2):
        K.prefill_attention_tc(q, out, kp, vp, torch.tensor(starts, dtype=torch.int32, device=DEV),
                               torch.tensor(prior, dtype=torch.int32, device=DEV), table, page, heads, n_kv, hd, window, scale,
                               block_rows=block_rows)
    torch.cuda.synchronize()
    assert K.prefill_attention_tc_error() == 0
    for r, (T, n) in enumerate(zip(totals, new)):
        qq = torch.zeros(T, heads, hd, dtype=torch.float64)
        qq[T - n:] = q[starts[r]:starts[r + 1]].double().cpu()
        want = P.attention(qq, ks[r].to(dtype).double(), vs[r].to(dtype).double(), window, scale)[T - n:]
        got = out[starts[r]:starts[r + 1]].double().cpu()
        assert torch.allclose(got, want, atol=2e-2, rtol=2e-2), (r, float((got - want).abs().max()))


def test_prefill_attention_tcgen05_late_standout_key(K):
    """A key that stands out far above the rest appears late, in the second 64 keys of a key
    tile: rows after it must move their reference maximum there (the pass over those scores is
    repeated and the output so far rescaled while the product over the tile's first keys may
    still run).  The portion starts at a position that is no multiple of a tile, and the
    kernel gives the same bits twice."""
    from test_gpu_kernels import paged_setup
    import math
    dtype, hd, page, heads, n_kv = torch.bfloat16, 128, 16, 4, 2
    total, new, late = 1100, 900, 1000                  # 1000 % 128 = 104: the tile's second half
    kp, vp, table, ks, vs = paged_setup([total], n_kv, hd, page, dtype, seed=210)
    g = torch.Generator().manual_seed(211)
    q = torch.randn(new, heads, hd, generator=g)
    kdir = ks[0][late].to(dtype).float()
    for h in range(heads):
        d = kdir[h // (heads // n_kv)]
        q[late - (total - new):, h] += 40.0 * d / d.norm() * math.sqrt(hd) / d.norm()      # score about +40 at that key
    q = q.to(dtype).to(DEV)
    scale = 1.0 / math.sqrt(hd)
    starts = torch.tensor([0, new], dtype=torch.int32, device=DEV)
    prior = torch.tensor([total - new], dtype=torch.int32, device=DEV)
    outs = []
    for _ in range(2):
        out = torch.full_like(q, 5.0)
        K.prefill_attention_tc(q, out, kp, vp, starts, prior, table, page, heads, n_kv, hd, 0, scale)
        outs.append(out)
    torch.cuda.synchronize()
    assert K.prefill_attention_tc_error() == 0
    assert torch.equal(outs[0], outs[1])
    qq = torch.zeros(total, heads, hd, dtype=torch.float64)
    qq[total - new:] = q.double().cpu()
    want = P.attention(qq, ks[0].to(dtype).double(), vs[0].to(dtype).double(), 0, scale)[total - new:]
    got = outs[0].double().cpu()
    assert torch.allclose(got, want, atol=2e-2, rtol=2e-2), float((got - want).abs().max())
    # the rows after the late key do look at it almost alone
    v_late = vs[0][late].to(dtype).double()
    assert (want[late - (total - new) + 1][0] - v_late[0]).abs().max() < 0.05


def test_prefill_attention_tcgen05_refuses(K):
    q = torch.zeros(4, 2, 64, dtype=torch.bfloat16, device=DEV)
    kp = torch.zeros(2, 2, 16, 64, dtype=torch.bfloat16, device=DEV)
    z = torch.zeros(2, dtype=torch.int32, device=DEV)
    with pytest.raises(K.KernelError):
        K.prefill_attention_tc(q, q.clone(), kp, kp, z, z[:1], z.view(1, 2), 16, 2, 2, 64, 0, 1.0)


@pytest.mark.parametrize("n_tok", [128, 256])
def test_pair_product_dense(K, n_tok):
    """The two-SM product (tcgen05 cta_group::2): every epilogue, partial tiles in every
    dimension (300 tokens, 384 features = one and a half pairs of 128 rows, K = 520)."""
    T, N, Kd = 300, 384, 520
    x, w, wu = rnd(T, Kd, seed=1), rnd(N, Kd, seed=2, scale=0.1), rnd(N, Kd, seed=7, scale=0.1)
    bias = torch.randn(N, generator=torch.Generator().manual_seed(3)).to(DEV)
    want = x.double() @ w.double().t()
    out = torch.full((T, N), 7.0, device=DEV)
    K.gemm_tc2(x, w, out, K.EPI_STORE_F32, n_tok, bias=bias)
    close(out, want + bias.double())
    base = torch.randn(T, N, generator=torch.Generator().manual_seed(4)).to(DEV)
    acc = base.clone()
    K.gemm_tc2(x, w, acc, K.EPI_ACC_F32, n_tok)
    close(acc, want + base.double())
    ob = torch.empty(T, N, device=DEV, dtype=torch.bfloat16)
    K.gemm_tc2(x, w, ob, K.EPI_STORE_BF16, n_tok)
    close(ob, want, atol=2e-2, rtol=1e-2)
    os_ = torch.empty(T, N, device=DEV, dtype=torch.bfloat16)
    K.gemm_tc2(x, w, os_, K.EPI_SWIGLU_BF16, n_tok, w_up=wu)
    close(os_, P.silu(want) * (x.double() @ wu.double().t()), atol=2e-2, rtol=1e-2)
    torch.cuda.synchronize()
    assert K.wait_errors() == {}


@pytest.mark.parametrize("n_tok", [128, 256])
def test_pair_product_grouped(K, n_tok):
    """Ragged groups (empty, 1 row, exactly a tile, a tile and one) through the two-SM product."""
    G, N, Kd = 7, 320, 264
    counts = [0, 5, 130, 300, 1, 257, 64]
    offs = [0]
    for c in counts:
        offs.append(offs[-1] + c)
    Tt = offs[-1]
    x, w, wu = rnd(Tt, Kd, seed=11), rnd(G, N, Kd, seed=12, scale=0.1), rnd(G, N, Kd, seed=13, scale=0.1)
    go = torch.tensor(offs, dtype=torch.int32, device=DEV)
    want = torch.zeros(Tt, N, dtype=torch.float64, device=DEV)
    wantu = torch.zeros_like(want)
    for g in range(G):
        want[offs[g]:offs[g + 1]] = x[offs[g]:offs[g + 1]].double() @ w[g].double().t()
        wantu[offs[g]:offs[g + 1]] = x[offs[g]:offs[g + 1]].double() @ wu[g].double().t()
    out = torch.full((Tt, N), 7.0, device=DEV)
    K.gemm_tc2(x, w, out, K.EPI_STORE_F32, n_tok, group_offsets=go)
    close(out, want)
    os_ = torch.full((Tt, N), 3.0, device=DEV, dtype=torch.bfloat16)
    K.gemm_tc2(x, w, os_, K.EPI_SWIGLU_BF16, n_tok, w_up=wu, group_offsets=go)
    close(os_, P.silu(want) * wantu, atol=2e-2, rtol=1e-2)
    torch.cuda.synchronize()
    assert K.wait_errors() == {}


def test_pair_product_refuses(K):
    x, w = rnd(64, 128, seed=1), rnd(200, 128, seed=2)
    out = torch.empty(64, 200, device=DEV, dtype=torch.bfloat16)
    with pytest.raises(K.KernelError):
        K.gemm_tc2(x, w, torch.empty(64, 200, device=DEV), K.EPI_STORE_F32, 64)          # token tiles of 128 or 256
    with pytest.raises(K.KernelError):
        K.gemm_tc2(x, w, out, K.EPI_STORE_F32, 128)                                     # float32 epilogue, bf16 out


@pytest.mark.parametrize("rows", [1, 8, 64, 200])
def test_language_model_head_at_the_real_vocabulary(K, rows):
    """The head's product at 151,936 features x 2,048 (1,187 feature tiles; an output row of
    151,936 floats) through the engine's own dispatch, every logit against a float64 product
    of the same bfloat16 operands.  A slip in the tile table or in the output index at this
    width would show as a wrong or an unwritten stretch of the row."""
    from cajeta_llm_b200.parts.base import Runtime
    from cajeta_llm_b200.parts.linear import project
    V, H = 151_936, 2048
    from cajeta_llm_b200.parts.plan import ParamSpec
    from cajeta_llm_b200.weights.sources import RandomWeights
    w = RandomWeights(5, torch.bfloat16, device=DEV).get("lm_head.weight", ParamSpec((V, H), std=0.02))
    x = rnd(rows, H, seed=500 + rows)
    out = torch.full((rows, V), float("nan"), device=DEV)
    project(Runtime("bfloat16", device=DEV), x, w, out)
    xd = x.double()
    worst = 0.0
    for lo in range(0, V, 16384):
        want = xd @ w[lo:lo + 16384].double().t()
        got = out[:, lo:lo + 16384].double()
        assert bool(torch.isfinite(got).all()), f"unwritten logits in columns {lo}.."
        d = (got - want).abs()
        assert bool((d <= 2e-3 + 2e-3 * want.abs()).all()), (lo, float(d.max()))
        worst = max(worst, float(d.max()))
    print(f"\nhead {rows} rows: worst |diff| {worst:.3e}")


