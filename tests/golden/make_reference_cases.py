"""Writes ``reference_cases.json``: the cases of the reference's own unit tests for the parts
of a layer, with the values those tests hold the reference to.

The reference's model code is cajeta source and cannot be compiled or imported here.  Its unit
tests, however, build their inputs from small integer formulas and check the engine against
an oracle written out in the test itself, in float64, element by element.  This script
restates those inputs and oracles in plain Python (no tensor library, one scalar at a time, as
the tests do) and records inputs' parameters and expected outputs; ``tests/test_plain.py``
rebuilds the inputs and holds the plain implementation's part functions to the outputs, within
the tolerance the reference's test uses.  What this pins are the conventions a misreading would
bend: eps inside the root of RMSNorm, the half-split pairs and the frequency formula of the
rotation, SiLU times up, the kv head of a query head, causality, and the first key of a window.

Cases (paths under src/test/cajeta/dev/cajeta/llm/selftest/):
  rmsnorm          PrimTest.cajeta:63-108   x = 0.25 ((3i + 1) % 11) - 1, w = 0.125 (i + 1), eps 1e-6
  rope             PrimTest.cajeta:187-232  head of 8, x = 0.25 (j + 1) - 1, position 7, theta 10000 and 500
  swiglu           PrimTest.cajeta:489-512  g = 0.75 (j - 4), u = 0.5 (j + 1) - 2
  attention_gqa    AttentionTest.cajeta:124-166   8 heads over 2 kv heads of 16, 512 keys, scale 0.25, last row
  attention_causal AttentionTest.cajeta:172-222   4 heads over 2 kv heads of 8, 64 rows, scale 1/sqrt(8), rows 0, 8, ...
  attention_window AttentionTest.cajeta:228-293   1 head of 4, 24 keys, window 8: row 20 sees keys [13, 20]
                                                   (values before 13 are 10^6), row 5 sees [0, 5]
Inputs of the attention cases: filled2(rows, cols, seed)[i] = 0.0625 (((i + seed) 7 + 3) % 15) - 0.4375
(AttentionTest.cajeta:98-110).

Run from the repository root:  python tests/golden/make_reference_cases.py
"""
import json
import math
import os
import struct


def f32(x):
    return struct.unpack("<f", struct.pack("<f", x))[0]


def filled2(rows, cols, seed):
    return [[f32(0.0625 * (((r * cols + c + seed) * 7 + 3) % 15) - 0.4375) for c in range(cols)] for r in range(rows)]


def head_oracle(q_row, k, v, kvh, hd, first, p, scale):
    """One query head over keys [first, p] of kv head kvh (AttentionTest.cajeta:38-92)."""
    scores = [sum(q_row[d] * k[t][kvh * hd + d] for d in range(hd)) * scale for t in range(first, p + 1)]
    mx = max(scores)
    e = [math.exp(s - mx) for s in scores]
    total = sum(e)
    return [sum(e[i] * v[first + i][kvh * hd + d] for i in range(len(e))) / total for d in range(hd)]


def build():
    cases = {}
    # RMSNorm
    rows, dim, eps = 3, 8, f32(0.000001)
    x = [[f32(0.25 * ((3 * (r * dim + d) + 1) % 11) - 1.0) for d in range(dim)] for r in range(rows)]
    w = [f32(0.125 * (d + 1)) for d in range(dim)]
    want = []
    for r in range(rows):
        rms = math.sqrt(sum(v * v for v in x[r]) / dim + eps)
        want.append([x[r][d] / rms * w[d] for d in range(dim)])
    cases["rmsnorm"] = {"rows": rows, "dim": dim, "eps": eps, "want": want, "tolerance": 1e-5}
    # rotation
    hd, pos = 8, 7
    xv = [f32(0.25 * (j + 1) - 1.0) for j in range(hd)]
    rope = {}
    for theta in (10000.0, 500.0):
        out = [0.0] * hd
        for d in range(hd // 2):
            ang = pos * math.pow(theta, -(2.0 * d) / hd)
            c, s = math.cos(ang), math.sin(ang)
            a, b = xv[d], xv[d + hd // 2]
            out[d], out[d + hd // 2] = a * c - b * s, a * s + b * c
        rope[str(int(theta))] = out
    cases["rope"] = {"head_dim": hd, "position": pos, "want": rope, "tolerance": 1e-5}
    # SwiGLU
    g = [f32(0.75 * (j - 4)) for j in range(8)]
    u = [f32(0.5 * (j + 1) - 2.0) for j in range(8)]
    cases["swiglu"] = {"want": [gv / (1.0 + math.exp(-gv)) * uv for gv, uv in zip(g, u)], "tolerance": 1e-5}
    # attention, grouped heads, one decode row over 512 keys
    nH, nKv, hd, T, scale = 8, 2, 16, 512, 0.25
    q, k, v = filled2(1, nH * hd, 1), filled2(T, nKv * hd, 2), filled2(T, nKv * hd, 3)
    cases["attention_gqa"] = {"heads": nH, "kv_heads": nKv, "head_dim": hd, "keys": T, "scale": scale, "seeds": [1, 2, 3],
                              "want": [head_oracle(q[0][h * hd:(h + 1) * hd], k, v, h // (nH // nKv), hd, 0, T - 1, scale)
                                       for h in range(nH)], "tolerance": 1e-4}
    # causal prompt
    nH, nKv, hd, T = 4, 2, 8, 64
    scale = f32(1.0 / f32(math.sqrt(f32(hd))))
    q, k, v = filled2(T, nH * hd, 5), filled2(T, nKv * hd, 6), filled2(T, nKv * hd, 7)
    rows = list(range(0, T, 8))
    cases["attention_causal"] = {"heads": nH, "kv_heads": nKv, "head_dim": hd, "rows_total": T, "scale": scale, "seeds": [5, 6, 7],
                                 "rows": rows, "want": [[head_oracle(q[r][h * hd:(h + 1) * hd], k, v, h // (nH // nKv), hd, 0, r, scale)
                                                         for h in range(nH)] for r in rows], "tolerance": 1e-4}
    # window
    hd, T, wnd, scale = 4, 24, 8, 0.5
    k = filled2(T, hd, 10)
    v = [[(1000000.0 if t < 13 else f32(0.125 * (t % 5) - 0.25))] * hd for t in range(T)]
    q20, q5 = filled2(1, hd, 9)[0], filled2(1, hd, 11)[0]
    cases["attention_window"] = {"head_dim": hd, "keys": T, "window": wnd, "scale": scale, "poison_before": 13,
                                 "row_20": head_oracle(q20, k, v, 0, hd, 13, 20, scale), "row_5": head_oracle(q5, k, v, 0, hd, 0, 5, scale),
                                 "seeds": {"q20": 9, "k": 10, "q5": 11}, "tolerance": 1e-4}
    return cases


if __name__ == "__main__":
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_cases.json")
    with open(path, "w", encoding="utf-8") as f:
        json.dump(build(), f, indent=1)
    print("wrote", path)
