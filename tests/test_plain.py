"""The plain implementation itself: held to the reference's asserted routing constants
and to direct restatements of the formulas (no GPU)."""
import json
import math
import os

import numpy as np
import pytest
import torch

import helpers
import plain_qwen2moe as P

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "router_oracle.json")


def oracle_inputs():
    with open(GOLDEN) as f:
        o = json.load(f)
    H, E = o["hidden"], o["experts"]
    j = np.arange(H)
    rr, pr, gr = o["router_row"], o["probe_row"], o["gate_row"]
    router = np.stack([(((j + rr["row_shift"] * r) % rr["modulus"]) - rr["offset"]).astype(np.float32) / np.float32(rr["divisor"])
                       * np.float32(rr["scale"]) for r in range(E)])
    probe = ((j * pr["multiplier"] % pr["modulus"]) - pr["offset"]).astype(np.float32) / np.float32(pr["divisor"])
    gate = ((j % gr["modulus"]) - gr["offset"]).astype(np.float32) / np.float32(gr["divisor"]) * np.float32(gr["scale"])
    return o, torch.from_numpy(router), torch.from_numpy(probe), torch.from_numpy(gate)


def test_router_matches_the_constants_the_reference_asserts():
    o, router, probe, gate = oracle_inputs()
    tol = o["tolerance"]
    sel, w = P.route(P.linear(probe, router), o["top_k"], False)
    assert sel == o["probe"]["sel"] and np.allclose(w.numpy(), o["probe"]["w_raw"], atol=tol)
    sel, w = P.route(P.linear(probe, router), o["top_k"], True)
    assert sel == o["probe"]["sel"] and np.allclose(w.numpy(), o["probe"]["w_norm"], atol=tol)
    sel, w = P.route(P.linear(-probe, router), o["top_k"], False)
    assert sel == o["probe_negated"]["sel"] and np.allclose(w.numpy(), o["probe_negated"]["w_raw"], atol=tol)
    z = float((gate * probe).sum())
    assert abs(1.0 / (1.0 + math.exp(-z)) - o["shared_gate_sigmoid"]) < tol


def test_router_ties_go_to_the_lower_index_and_nan_is_refused():
    sel, w = P.route(torch.tensor([1.0, 2.0, 2.0, 0.5, 2.0]), 2, False)
    assert sel == [1, 2]
    with pytest.raises(ValueError):
        P.route(torch.tensor([float("nan")] * 4), 2, False)


def test_rmsnorm_and_rope_and_silu_restate_the_formulas():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(3, 10, generator=g, dtype=torch.float64)
    w = torch.randn(10, generator=g, dtype=torch.float64)
    y = P.rmsnorm(x, w, 1e-5)
    for r in range(3):
        ss = sum(float(v) ** 2 for v in x[r])
        scale = 1.0 / math.sqrt(ss / 10 + 1e-5)
        assert np.allclose(y[r].numpy(), [float(x[r, i]) * scale * float(w[i]) for i in range(10)])
    inv = P.inv_freq(8, 10000.0, torch.float64)
    assert np.allclose(inv.numpy(), [10000.0 ** (-2 * d / 8) for d in range(4)], rtol=1e-6)
    t = torch.randn(2, 1, 8, generator=g, dtype=torch.float64)
    r = P.rope(t, torch.tensor([0, 5]), inv)
    assert torch.equal(r[0], t[0])                                    # position 0 rotates nothing
    for d in range(4):
        ang = float(np.float32(5.0) * np.float32(inv[d]))
        a, b = float(t[1, 0, d]), float(t[1, 0, d + 4])
        assert abs(float(r[1, 0, d]) - (a * math.cos(ang) - b * math.sin(ang))) < 1e-12
        assert abs(float(r[1, 0, d + 4]) - (a * math.sin(ang) + b * math.cos(ang))) < 1e-12
    assert abs(float(P.silu(torch.tensor(0.7, dtype=torch.float64))) - 0.7 / (1 + math.exp(-0.7))) < 1e-15


def test_attention_is_causal_grouped_and_windowed():
    g = torch.Generator().manual_seed(1)
    T, H, KV, D = 9, 4, 2, 6
    q = torch.randn(T, H, D, generator=g, dtype=torch.float64)
    k = torch.randn(T, KV, D, generator=g, dtype=torch.float64)
    v = torch.randn(T, KV, D, generator=g, dtype=torch.float64)
    for window in (0, 4):
        out = P.attention(q, k, v, window, 0.3)
        for p in (0, 3, 8):
            lo = max(0, p + 1 - window) if window else 0
            for h in range(H):
                s = torch.tensor([float(q[p, h] @ k[t, h // 2]) * 0.3 for t in range(lo, p + 1)], dtype=torch.float64)
                pr = torch.softmax(s, 0)
                want = sum(pr[i] * v[lo + i, h // 2] for i in range(len(pr)))
                assert torch.allclose(out[p, h], want, atol=1e-12)
    # a later token never changes an earlier row
    out_short = P.attention(q[:5], k[:5], v[:5], 0, 0.3)
    assert torch.allclose(out_short, P.attention(q, k, v, 0, 0.3)[:5])


def test_whole_model_prefix_property_and_layer_choices(model_dirs):
    for name in ("A", "B", "C"):
        cfg = helpers.CONFIGS[name]
        toks = helpers.random_tokens(cfg["vocab_size"], 14, seed=4)
        full = helpers.plain_logits(model_dirs[name], toks)
        part = helpers.plain_logits(model_dirs[name], toks[:9])
        assert full.shape == (14, cfg["vocab_size"])
        assert torch.allclose(full[:9], part, atol=1e-6)              # causal: a prefix gives the same logits
    assert [P.layer_is_sparse(helpers.TINY_B, l) for l in range(3)] == [False, True, False]
    assert [P.layer_window(helpers.TINY_B, l) for l in range(3)] == [0, 8, 8]
    assert [P.layer_window(helpers.TINY_C, l) for l in range(2)] == [20, 20]


def test_window_matters_in_the_plain_model(model_dirs):
    cfg = dict(helpers.TINY_B)
    toks = helpers.random_tokens(cfg["vocab_size"], 20, seed=9)
    config, weights = P.read_model(model_dirs["B"])
    with_window = P.forward(config, weights, toks)
    no_window = P.forward({**config, "use_sliding_window": False}, weights, toks)
    assert torch.allclose(with_window[:8], no_window[:8], atol=1e-9)   # the first 8 positions see everything either way
    assert not torch.allclose(with_window[12:], no_window[12:], atol=1e-4)


def test_plain_sampler_arithmetic():
    logits = torch.tensor([1.0, 3.0, 2.0, 3.0, -1.0, 0.5])
    assert P.argmax_first(logits) == 1
    d = P.prepared_distribution(logits, 0.0, 0, 0.0, 1.0, [])
    assert d.tolist() == [0, 1, 0, 0, 0, 0]
    d = P.prepared_distribution(logits, 0.5, 0, 0.0, 1.0, [])
    assert torch.allclose(d, torch.softmax(logits / 0.5, 0), atol=1e-6)
    d = P.prepared_distribution(logits, 1.0, 3, 0.0, 1.0, [])
    assert (d > 0).tolist() == [False, True, True, True, False, False]
    d = P.prepared_distribution(logits, 1.0, 0, 0.6, 1.0, [])
    assert (d > 0).tolist() == [False, True, False, True, False, False]      # 0.36 + 0.36 >= 0.6
    d = P.prepared_distribution(logits, 1.0, 0, 0.0, 2.0, [1, 4])
    e = logits.clone()
    e[1], e[4] = 1.5, -2.0
    assert torch.allclose(d, torch.softmax(e, 0), atol=1e-6)
    d = P.prepared_distribution(logits, 1.0, 0, 0.0, 1.0, [])
    assert P.draw(d, 0.0) == 1 and P.draw(d, 0.999999) == 4
    order = [1, 3, 2, 0, 5, 4]
    cum = 0.0
    for i in order:
        assert P.draw(d, cum + 1e-4) == i
        cum += float(d[i])


@pytest.mark.parametrize("name", sorted(helpers.CONFIGS))
def test_vectorised_restatement_equals_the_row_by_row_implementation(name, tmp_path):
    """tests/plain_vectorised.py (whole tensors, used against the full-size models) against
    tests/plain_qwen2moe.py (Python loops) on every small configuration: logits, the experts
    each row picks in every sparse layer, and the routing margins."""
    import plain_vectorised as PV
    raw = helpers.CONFIGS[name]
    d = str(tmp_path)
    helpers.write_model(d, raw, seed=helpers.SEEDS[name])
    config, weights = P.read_model(d)
    n = 70 if name in helpers.LONG_REQUESTS else 45             # beyond the small windows; W's window is 40
    tokens = helpers.random_tokens(raw["vocab_size"], n, seed=3)
    m_rows, m_vec, picked = [1.0] * n, [1.0] * n, {}
    want = P.forward(config, weights, tokens, margins=m_rows)
    got = PV.forward(config, weights.__getitem__, tokens, margins=m_vec, selections=picked)
    assert torch.allclose(got, want, atol=1e-11, rtol=1e-9), float((got - want).abs().max())
    assert np.allclose(m_rows, m_vec, atol=1e-9)
    sparse = [l for l in range(config["num_hidden_layers"]) if P.layer_is_sparse(config, l)]
    assert sorted(picked) == sparse and all(tuple(s.shape) == (n, config["num_experts_per_tok"]) for s in picked.values())
    # ties go to the lower index here as there
    sel, w, margin = PV.route(torch.tensor([[1.0, 2.0, 2.0, 0.5, 2.0]], dtype=torch.float64), 2, False)
    assert sel.tolist() == [[1, 2]] and abs(float(margin[0])) < 1e-12


def _filled2(rows, cols, seed):
    i = np.arange(rows * cols, dtype=np.int64)
    return torch.from_numpy((np.float32(0.0625) * (((i + seed) * 7 + 3) % 15).astype(np.float32) - np.float32(0.4375))
                            .reshape(rows, cols)).double()


def test_plain_parts_meet_the_cases_of_the_reference_tests():
    """tests/golden/reference_cases.json holds the cases of the reference's own unit tests for
    RMSNorm, the rotation, SwiGLU and attention (grouped heads, causal rows, a window whose
    out-of-window values are 10^6) with the values those tests hold the reference to.  The plain
    implementation's part functions meet them within the reference's tolerances."""
    with open(os.path.join(os.path.dirname(GOLDEN), "reference_cases.json")) as f:
        cases = json.load(f)

    c = cases["rmsnorm"]
    i = np.arange(c["rows"] * c["dim"])
    x = torch.from_numpy((np.float32(0.25) * ((3 * i + 1) % 11).astype(np.float32) - np.float32(1.0)).reshape(c["rows"], c["dim"])).double()
    w = torch.from_numpy(np.float32(0.125) * (np.arange(c["dim"]) + 1).astype(np.float32)).double()
    assert np.allclose(P.rmsnorm(x, w, c["eps"]).numpy(), c["want"], atol=c["tolerance"], rtol=0)

    c = cases["rope"]
    hd = c["head_dim"]
    xv = torch.from_numpy(np.float32(0.25) * (np.arange(hd) + 1).astype(np.float32) - np.float32(1.0)).double().reshape(1, 1, hd)
    for theta, want in c["want"].items():
        got = P.rope(xv, torch.tensor([c["position"]]), P.inv_freq(hd, float(theta), torch.float64))
        assert np.allclose(got.reshape(-1).numpy(), want, atol=c["tolerance"], rtol=0), theta

    c = cases["swiglu"]
    g = torch.from_numpy(np.float32(0.75) * (np.arange(8) - 4).astype(np.float32)).double()
    u = torch.from_numpy(np.float32(0.5) * (np.arange(8) + 1).astype(np.float32) - np.float32(2.0)).double()
    assert np.allclose((P.silu(g) * u).numpy(), c["want"], atol=c["tolerance"], rtol=0)

    c = cases["attention_gqa"]
    nH, nKv, hd, T = c["heads"], c["kv_heads"], c["head_dim"], c["keys"]
    q = torch.zeros(T, nH, hd, dtype=torch.float64)
    q[T - 1] = _filled2(1, nH * hd, c["seeds"][0]).reshape(nH, hd)
    k, v = (_filled2(T, nKv * hd, s).reshape(T, nKv, hd) for s in c["seeds"][1:])
    assert np.allclose(P.attention(q, k, v, 0, c["scale"])[T - 1].numpy(), c["want"], atol=c["tolerance"], rtol=0)

    c = cases["attention_causal"]
    nH, nKv, hd, T = c["heads"], c["kv_heads"], c["head_dim"], c["rows_total"]
    q = _filled2(T, nH * hd, c["seeds"][0]).reshape(T, nH, hd)
    k, v = (_filled2(T, nKv * hd, s).reshape(T, nKv, hd) for s in c["seeds"][1:])
    got = P.attention(q, k, v, 0, c["scale"])
    assert np.allclose(got[c["rows"]].numpy(), c["want"], atol=c["tolerance"], rtol=0)

    c = cases["attention_window"]
    hd, T = c["head_dim"], c["keys"]
    k = _filled2(T, hd, c["seeds"]["k"]).reshape(T, 1, hd)
    v = torch.tensor([[1000000.0 if t < c["poison_before"] else float(np.float32(0.125) * np.float32(t % 5) - np.float32(0.25))] * hd
                      for t in range(T)], dtype=torch.float64).reshape(T, 1, hd)
    q = torch.zeros(T, 1, hd, dtype=torch.float64)
    q[20, 0] = _filled2(1, hd, c["seeds"]["q20"])[0]
    q[5, 0] = _filled2(1, hd, c["seeds"]["q5"])[0]
    got = P.attention(q, k, v, c["window"], c["scale"])
    assert float(got[20].abs().max()) < 1000.0                       # nothing of the values behind the window
    assert np.allclose(got[20, 0].numpy(), c["row_20"], atol=c["tolerance"], rtol=0)
    assert np.allclose(got[5, 0].numpy(), c["row_5"], atol=c["tolerance"], rtol=0)
