"""Writes ``router_oracle.json``: the routing constants the reference's own test asserts.

The reference's model code is cajeta source and cannot be compiled or imported here, so
the plain implementation under ``tests/`` rests on the reference's formulas.  For the
router and the shared expert's gate there is more: the reference's self-test asserts
numbers that its fixture generator computed offline
(src/test/cajeta/dev/cajeta/llm/selftest/MoeForwardTest.cajeta:116-126 raw arm,
:143-146 renormalised arm, :191 sigmoid gate), for inputs that are plain formulas
(tools/gguf/gen_moe_fixture.py: router rows ``((j + 7r) % 25 - 12) / 64 * 1.28`` for
expert ``r``; probe row ``x[j] = ((3j % 25) - 12) / 64`` and its negation; gate vector
``((j % 25) - 12) / 64 * 1.28``; 4 experts, top-2, width 512).  This script records
those asserted constants and the formulas' parameters; ``tests/test_plain.py`` rebuilds
the inputs and holds the plain router to them, and the GPU test holds the router
kernel to them.

Run from the repository root:  python tests/golden/make_router_oracle.py
"""
import json
import os

ORACLE = {
    "source": "selftest/MoeForwardTest.cajeta:116-126,143-146,191; tools/gguf/gen_moe_fixture.py",
    "hidden": 512,
    "experts": 4,
    "top_k": 2,
    "router_row": {"modulus": 25, "row_shift": 7, "offset": 12, "divisor": 64.0, "scale": 1.28},
    "probe_row": {"multiplier": 3, "modulus": 25, "offset": 12, "divisor": 64.0},
    "gate_row": {"modulus": 25, "offset": 12, "divisor": 64.0, "scale": 1.28},
    "tolerance": 1e-4,
    "probe": {"sel": [0, 1], "w_raw": [0.71762824, 0.22958289], "w_norm": [0.75762224, 0.24237773]},
    "probe_negated": {"sel": [3, 2], "w_raw": [0.87409478, 0.09893262]},
    "shared_gate_sigmoid": 0.92898820,
}

if __name__ == "__main__":
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "router_oracle.json")
    with open(path, "w", encoding="utf-8") as f:
        json.dump(ORACLE, f, indent=2)
    print("wrote", path)
