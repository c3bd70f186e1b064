"""Each part alone (norm, position encoding, attention mixer, dense and sparse
feed-forward, block) against the plain functions, at sizes other than the tiny models',
built through the part registry exactly as a model builds them."""
import math
from types import SimpleNamespace

import pytest
import torch

import helpers
import plain_qwen2moe as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def runtime(dtype):
    from cajeta_llm_b200.parts.base import Runtime
    return Runtime(dtype, device=DEV)


def make(category, spec, prefix, dtype, seed, **extra):
    import cajeta_llm_b200  # noqa: F401
    from cajeta_llm_b200.parts.base import make_part
    part = make_part(category, spec, prefix, runtime(dtype), **extra)
    weights = helpers.random_weights_for(part, seed)
    part.load(helpers.DictWeights(weights))
    return part, {k: v.double() for k, v in weights.items()}


def tol(dtype):
    return dict(atol=2e-5, rtol=1e-4) if dtype == "float32" else dict(atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rmsnorm_part(dtype):
    from cajeta_llm_b200.parts.plan import PartSpec
    part, w = make("norm", PartSpec("rmsnorm", {"dim": 88, "eps": 3e-5}), "n", dtype, 1)
    x = torch.randn(9, 88, generator=torch.Generator().manual_seed(2)).to(DEV)
    y, y32 = part.forward(x, want_f32=True)
    want = P.rmsnorm(x.double().cpu(), w["n.weight"], 3e-5)
    assert y.dtype == part.runtime.act_dtype and y32.dtype == torch.float32
    assert torch.allclose(y32.double().cpu(), want, atol=1e-5, rtol=1e-5)
    assert torch.allclose(y.double().cpu(), want, **tol(dtype))


def test_position_parts():
    from cajeta_llm_b200.parts.base import make_part
    from cajeta_llm_b200.parts.plan import PartSpec
    rope = make_part("position", PartSpec("rope", {"head_dim": 48, "rotary_dim": 32, "theta": 5e5}), "", runtime("float32"))
    assert rope.rotary_dim == 32
    assert torch.allclose(rope.inv_freq.cpu().double(), P.inv_freq(32, 5e5, torch.float64), rtol=1e-6)
    none = make_part("position", PartSpec("none", {}), "", runtime("float32"))
    assert none.rotary_dim == 0 and none.inv_freq is None
    with pytest.raises(ValueError, match="no position of kind"):
        make_part("position", PartSpec("alibi", {}), "", runtime("float32"))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tied,bias,scale", [(True, False, 0.0), (False, True, 12.0), (False, False, 0.0)])
def test_embedding_and_head_parts(dtype, tied, bias, scale):
    """The two ends of a model as parts: a scaled embedding, a head with and without bias,
    tied to the embedding table or with a matrix of its own (hidden 192: the tensor-core
    product on the bfloat16 path)."""
    from cajeta_llm_b200.parts.plan import PartSpec
    V, H = 333, 192
    emb, w = make("embedding", PartSpec("token_embedding", {"scale": scale}), "", dtype, 3, vocab_size=V, hidden_size=H,
                  weight_name="e.weight")
    ids = torch.tensor([5, 332, 0, 5, 17], dtype=torch.int32, device=DEV)
    hs = emb.forward(ids)
    assert hs.dtype == torch.float32
    assert torch.allclose(hs.double().cpu(), w["e.weight"][ids.long().cpu()] * (scale or 1.0), atol=1e-6, rtol=1e-6)
    if bias and tied:
        return
    head, wh = make("head", PartSpec("linear_head", {"bias": bias}), "", dtype, 4, vocab_size=V, hidden_size=H,
                    weight_name=None if tied else "h.weight", embedding=emb)
    assert set(wh) == (set() if tied else {"h.weight"} | ({"h.bias"} if bias else set()))
    x = (torch.randn(7, H, generator=torch.Generator().manual_seed(5)) * 0.5).to(head.runtime.act_dtype).to(DEV)
    got = head.forward(x)
    assert got.dtype == torch.float32 and tuple(got.shape) == (7, V)
    want = P.linear(x.double().cpu(), w["e.weight"] if tied else wh["h.weight"], wh.get("h.bias"))
    assert torch.allclose(got.double().cpu(), want, **tol(dtype))
    with pytest.raises(ValueError, match="tied"):
        make("head", PartSpec("linear_head", {"bias": True}), "", dtype, 4, vocab_size=V, hidden_size=H, weight_name=None,
             embedding=emb)


def step_context(requests, page, n_pages, device=DEV):
    """requests: [(prior_len, n_new)] -> a context like the step function builds, with a
    scrambled block table."""
    g = torch.Generator().manual_seed(5)
    perm = torch.randperm(n_pages, generator=g).tolist()
    width = max(-(-(p + n) // page) for p, n in requests)
    table = torch.full((len(requests), width), -1, dtype=torch.int32)
    nxt = 0
    pos, req = [], []
    for r, (prior, n) in enumerate(requests):
        for j in range(-(-(prior + n) // page)):
            table[r, j] = perm[nxt]
            nxt += 1
        pos += list(range(prior, prior + n))
        req += [r] * n
    ctx = SimpleNamespace(positions=torch.tensor(pos, dtype=torch.int32, device=device),
                          row_req=torch.tensor(req, dtype=torch.int32, device=device), n_rows=len(pos))
    return ctx, table.to(device)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,kv,hd,window,rot", [(6, 2, 40, 0, 40), (5, 5, 16, 7, 16), (8, 1, 64, 0, 32)])
def test_attention_mixer_part_in_two_steps(dtype, heads, kv, hd, window, rot):
    """A prompt in two steps (a portion, then the rest beside another request's portion)
    equals the plain attention layer over the whole sequences."""
    from cajeta_llm_b200.engine.step import EntryContext
    from cajeta_llm_b200.parts.plan import PartSpec
    H, page = 72, 4
    spec = PartSpec("attention", {"hidden_size": H, "num_heads": heads, "num_kv_heads": kv, "head_dim": hd,
                                  "window": window, "qkv_bias": True, "out_bias": False, "scale": None,
                                  "position": PartSpec("rope", {"head_dim": hd, "rotary_dim": rot, "theta": 1e4})})
    part, w = make("mixer", spec, "a", dtype, 3)
    rt = part.runtime
    g = torch.Generator().manual_seed(4)
    xa, xb = torch.randn(21, H, generator=g), torch.randn(10, H, generator=g)
    n_pages = 12
    kp = torch.zeros(n_pages, kv, page, hd, dtype=rt.cache_dtype, device=DEV)
    vp = torch.zeros_like(kp)
    res = {}

    def run(requests, xs, table_rows):
        ctx, table = step_context(requests, page, n_pages)
        if table_rows is not None:
            table = table_rows
        x = torch.cat(xs).to(rt.act_dtype).to(DEV)
        out = torch.zeros(x.shape[0], H, device=DEV)
        entry = EntryContext(index=0, writes_cache=True, k_plane=kp, v_plane=vp, block_table=table, page_tokens=page, state=None)
        part.forward(x, out, ctx, entry)
        return out.cpu().double(), table

    # step 1: the first 13 rows of a;  step 2: the remaining 8 of a beside all 10 of b
    ctx_all, table_all = step_context([(0, 21), (0, 10)], page, n_pages)
    o1, _ = run([(0, 13)], [xa[:13]], table_all[:1].contiguous())
    o2, _ = run([(13, 8), (0, 10)], [xa[13:], xb], table_all)
    got = {"a": torch.cat([o1, o2[:8]]), "b": o2[8:]}
    for name, x in (("a", xa), ("b", xb)):
        xd = x.to(rt.act_dtype).double()
        T = xd.shape[0]
        q = P.linear(xd, w["a.q_proj.weight"], w["a.q_proj.bias"]).reshape(T, heads, hd)
        k = P.linear(xd, w["a.k_proj.weight"], w["a.k_proj.bias"]).reshape(T, kv, hd)
        v = P.linear(xd, w["a.v_proj.weight"], w["a.v_proj.bias"]).reshape(T, kv, hd)
        inv = P.inv_freq(rot, 1e4, torch.float64)
        pos = torch.arange(T)
        q = torch.cat([P.rope(q[..., :rot], pos, inv), q[..., rot:]], -1)
        k = torch.cat([P.rope(k[..., :rot], pos, inv), k[..., rot:]], -1)
        ao = P.attention(q, k, v, window, 1.0 / math.sqrt(hd)).reshape(T, heads * hd)
        want = P.linear(ao, w["a.o_proj.weight"])
        assert torch.allclose(got[name], want, **tol(dtype)), name


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_dense_feed_forward_part(dtype):
    from cajeta_llm_b200.parts.plan import PartSpec
    part, w = make("feed_forward", PartSpec("dense_swiglu", {"hidden_size": 72, "intermediate_size": 100}), "m", dtype, 6)
    x = torch.randn(13, 72, generator=torch.Generator().manual_seed(7)).to(part.runtime.act_dtype)
    res = torch.ones(13, 72, device=DEV)
    part.forward(x.to(DEV), None, res, None)
    want = 1.0 + P.swiglu_mlp(x.double(), w["m.gate_proj.weight"], w["m.up_proj.weight"], w["m.down_proj.weight"])
    assert torch.allclose(res.cpu().double(), want, **tol(dtype))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("E,k,I,S,gate,norm", [(7, 3, 36, 52, True, False), (5, 1, 20, 0, False, True), (9, 9, 24, 40, False, True)])
def test_sparse_moe_part(dtype, E, k, I, S, gate, norm):
    from cajeta_llm_b200.parts.plan import PartSpec
    spec = PartSpec("sparse_moe", {"hidden_size": 56, "num_experts": E, "top_k": k, "expert_intermediate_size": I,
                                   "shared_intermediate_size": S, "shared_gate": gate, "norm_topk_prob": norm})
    part, w = make("feed_forward", spec, "m", dtype, 8)
    x32 = torch.randn(17, 56, generator=torch.Generator().manual_seed(9))
    x = x32.to(part.runtime.act_dtype)
    res = torch.zeros(17, 56, device=DEV)
    part.forward(x.to(DEV), x.float().to(DEV), res, None)
    if S > 0 and not gate:
        # the plain mixture always reads a gate row; an ungated shared expert is a gate of +inf -> sigma = 1
        w["m.shared_expert_gate.weight"] = torch.zeros(1, 56, dtype=torch.float64)
        want = P.sparse_moe(x.double(), w, "m", E, k, norm, True)
        s = P.swiglu_mlp(x.double(), w["m.shared_expert.gate_proj.weight"], w["m.shared_expert.up_proj.weight"],
                         w["m.shared_expert.down_proj.weight"])
        want = want + 0.5 * s                                   # sigma(0) = 0.5 was applied; the part applies 1
    else:
        want = P.sparse_moe(x.double(), w, "m", E, k, norm, S > 0)
    assert torch.allclose(res.cpu().double(), want, **tol(dtype))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_block_part(dtype):
    from cajeta_llm_b200.engine.step import EntryContext
    from cajeta_llm_b200.parts.plan import LayerSpec, PartSpec
    H, heads, kv, hd, page = 48, 3, 1, 16, 8
    norm = PartSpec("rmsnorm", {"dim": H, "eps": 1e-6})
    layer = LayerSpec(
        prefix="L", block=PartSpec("prenorm", {"mixer_norm_name": "n1", "feed_forward_norm_name": "n2", "mixer_name": "att",
                                               "feed_forward_name": "ff"}),
        mixer=PartSpec("attention", {"hidden_size": H, "num_heads": heads, "num_kv_heads": kv, "head_dim": hd, "window": 0,
                                     "qkv_bias": True, "position": PartSpec("rope", {"head_dim": hd, "theta": 1e4})}),
        feed_forward=PartSpec("dense_swiglu", {"hidden_size": H, "intermediate_size": 80}),
        mixer_norm=norm, feed_forward_norm=norm)
    part, w = make("block", layer.block, "L", dtype, 10, layer=layer)
    T = 19
    hs0 = torch.randn(T, H, generator=torch.Generator().manual_seed(11))
    hs = hs0.clone().to(DEV)
    ctx, table = step_context([(0, T)], page, 4)
    rt = part.runtime
    kp = torch.zeros(4, kv, page, hd, dtype=rt.cache_dtype, device=DEV)
    entry = EntryContext(index=0, writes_cache=True, k_plane=kp, v_plane=torch.zeros_like(kp), block_table=table,
                         page_tokens=page, state=None)
    part.forward(hs, ctx, entry)
    x = hs0.double()
    xn = P.rmsnorm(x, w["L.n1.weight"], 1e-6)
    q = P.linear(xn, w["L.att.q_proj.weight"], w["L.att.q_proj.bias"]).reshape(T, heads, hd)
    k = P.linear(xn, w["L.att.k_proj.weight"], w["L.att.k_proj.bias"]).reshape(T, kv, hd)
    v = P.linear(xn, w["L.att.v_proj.weight"], w["L.att.v_proj.bias"]).reshape(T, kv, hd)
    inv = P.inv_freq(hd, 1e4, torch.float64)
    q, k = P.rope(q, torch.arange(T), inv), P.rope(k, torch.arange(T), inv)
    x = x + P.linear(P.attention(q, k, v, 0, 1 / math.sqrt(hd)).reshape(T, heads * hd), w["L.att.o_proj.weight"])
    x = x + P.swiglu_mlp(P.rmsnorm(x, w["L.n2.weight"], 1e-6), w["L.ff.gate_proj.weight"], w["L.ff.up_proj.weight"],
                         w["L.ff.down_proj.weight"])
    assert torch.allclose(hs.cpu().double(), x, **tol(dtype))


@pytest.mark.parametrize("E,k,gate,norm,T", [(60, 4, True, False, 150), (7, 2, False, True, 64), (130, 3, True, True, 300)])
def test_router_on_tensor_cores_is_float32_grade(E, k, gate, norm, T):
    """Many rows route through a bfloat16 tensor-core product over the three-term form of the
    float32 normed row.  The norm's three terms add up to its float32 result, and the
    selection and weights equal those of the float32 router kernel (and the plain router)."""
    from cajeta_llm_b200.parts.plan import PartSpec
    from cajeta_llm_b200.csrc import kernels as K
    H = 264
    norm_part, nw = make("norm", PartSpec("rmsnorm", {"dim": H, "eps": 1e-5}), "n", "bfloat16", 21)
    hs = (torch.randn(T, H, generator=torch.Generator().manual_seed(22)) * 3).to(DEV)
    out, split = norm_part.forward(hs, want_split=True)
    out2, x32 = norm_part.forward(hs, want_f32=True)
    assert torch.equal(out, out2) and split.shape == (T, 3 * H) and split.dtype == torch.bfloat16
    assert torch.equal(split[:, :H], out)
    back = split[:, :H].double() + split[:, H:2 * H].double() + split[:, 2 * H:].double()
    assert float((back - x32.double()).abs().max()) <= 2.0 ** -23 * float(x32.abs().max())

    spec = PartSpec("sparse_moe", {"hidden_size": H, "num_experts": E, "top_k": k, "expert_intermediate_size": 32,
                                   "shared_intermediate_size": 64 if gate else 0, "shared_gate": gate, "norm_topk_prob": norm})
    part, w = make("feed_forward", spec, "m", "bfloat16", 23)
    assert part.wants_split_input(T) and not part.wants_split_input(8)
    sel = [torch.empty((T, k), dtype=torch.int32, device=DEV) for _ in range(2)]
    wts = [torch.empty((T, k), dtype=torch.float32, device=DEV) for _ in range(2)]
    sc = [torch.empty((T,), dtype=torch.float32, device=DEV) if gate else None for _ in range(2)]
    part._route(split, sel[0], wts[0], sc[0])
    part._route(x32, sel[1], wts[1], sc[1])
    assert K.gemm_tc_error() == 0
    same = (sel[0] == sel[1]).all(dim=1)
    assert int((~same).sum()) <= 1                     # an exact near-tie may fall either way
    assert torch.allclose(wts[0][same], wts[1][same], atol=1e-6, rtol=1e-5)
    if gate:
        assert torch.allclose(sc[0], sc[1], atol=1e-6, rtol=1e-5)
    # and against the plain router on a few rows
    for t in (0, T // 2, T - 1):
        logits = x32[t].double().cpu() @ w["m.gate.weight"].t()
        psel, pw = P.route(logits, k, norm)
        assert sel[0][t].tolist() == psel
        assert torch.allclose(wts[0][t].double().cpu(), pw, atol=1e-6, rtol=1e-5)
