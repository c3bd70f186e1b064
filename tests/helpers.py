"""Shared by the tests: the tiny configurations, model folders, the plain reference."""
import functools
import json
import os
import subprocess
import sys
from typing import Dict, List, Sequence

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# Two tiny configurations that differ in every size and option, and a third whose
# explicit head_dim is not hidden / heads.
TINY_A = {
    "architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe",
    "hidden_size": 64, "intermediate_size": 128, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "vocab_size": 256,
    "max_position_embeddings": 4096, "rms_norm_eps": 1e-6, "rope_theta": 10000.0,
    "num_experts": 4, "num_experts_per_tok": 2, "moe_intermediate_size": 32,
    "shared_expert_intermediate_size": 64, "norm_topk_prob": True,
    "decoder_sparse_step": 1, "mlp_only_layers": [], "tie_word_embeddings": False,
    "use_sliding_window": False, "sliding_window": 4096, "max_window_layers": 2, "eos_token_id": 255,
}
TINY_B = {
    "architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe",
    "hidden_size": 96, "intermediate_size": 160, "num_hidden_layers": 3,
    "num_attention_heads": 4, "num_key_value_heads": 1, "head_dim": 24, "vocab_size": 320,
    "max_position_embeddings": 4096, "rms_norm_eps": 1e-5, "rope_theta": 1000000.0,
    "num_experts": 6, "num_experts_per_tok": 3, "moe_intermediate_size": 48,
    "shared_expert_intermediate_size": 80, "norm_topk_prob": False,
    "decoder_sparse_step": 2, "mlp_only_layers": [0], "tie_word_embeddings": True,
    "use_sliding_window": True, "sliding_window": 8, "max_window_layers": 1, "eos_token_id": [318, 319],
}
TINY_C = {
    "architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe",
    "hidden_size": 80, "intermediate_size": 112, "num_hidden_layers": 2,
    "num_attention_heads": 6, "num_key_value_heads": 3, "head_dim": 32, "vocab_size": 200,
    "max_position_embeddings": 4096, "rms_norm_eps": 1e-6, "rope_theta": 50000.0,
    "num_experts": 5, "num_experts_per_tok": 1, "moe_intermediate_size": 40,
    "shared_expert_intermediate_size": 0, "norm_topk_prob": True,
    "decoder_sparse_step": 1, "mlp_only_layers": [1], "tie_word_embeddings": False,
    "use_sliding_window": True, "sliding_window": 20, "max_window_layers": 0,
}
# Wide enough for the tensor-core kernels of the bfloat16 path (every product has K >= 128
# and >= 128 output features); widths are still no power of two where the kernels allow.
MEDIUM = {
    "architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe",
    "hidden_size": 384, "intermediate_size": 512, "num_hidden_layers": 2,
    "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 64, "vocab_size": 1000,
    "max_position_embeddings": 4096, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
    "num_experts": 8, "num_experts_per_tok": 2, "moe_intermediate_size": 192,
    "shared_expert_intermediate_size": 320, "norm_topk_prob": False,
    "decoder_sparse_step": 1, "mlp_only_layers": [1], "tie_word_embeddings": False,
    "use_sliding_window": False,
}
# The layer sizes of Qwen1.5-MoE-A2.7B (hidden 2048, 16 heads of 128, experts of 1408, shared
# expert of 5632) with fewer layers, fewer experts and a small vocabulary, so that the kernels
# are checked against the plain implementation at the shapes the benchmark runs.
REAL_SIZES = {
    "architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe",
    "hidden_size": 2048, "intermediate_size": 5632, "num_hidden_layers": 2,
    "num_attention_heads": 16, "num_key_value_heads": 16, "head_dim": 128, "vocab_size": 3000,
    "max_position_embeddings": 4096, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
    "num_experts": 12, "num_experts_per_tok": 4, "moe_intermediate_size": 1408,
    "shared_expert_intermediate_size": 5632, "norm_topk_prob": False,
    "decoder_sparse_step": 1, "mlp_only_layers": [], "tie_word_embeddings": False,
    "use_sliding_window": False,
}
# Windowed layers on the fast bfloat16 kernels: head sizes 128 and 64 (split-KV decode, the
# tcgen05 and the mma.sync prompt kernels), windows that are no multiple of a page (16) or of
# a key chunk (128), one group of full layers beside one of windowed layers, every product
# wide enough for the tensor cores.  Replayed with requests several windows long, so that the
# windowed group gives pages back (table entries turn -1) while the request goes on.
WINDOW_128 = {
    "architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe",
    "hidden_size": 256, "intermediate_size": 384, "num_hidden_layers": 3,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 128, "vocab_size": 520,
    "max_position_embeddings": 4096, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
    "num_experts": 6, "num_experts_per_tok": 2, "moe_intermediate_size": 128,
    "shared_expert_intermediate_size": 256, "norm_topk_prob": True,
    "decoder_sparse_step": 1, "mlp_only_layers": [1], "tie_word_embeddings": False,
    "use_sliding_window": True, "sliding_window": 40, "max_window_layers": 1,
}
WINDOW_64 = {
    "architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe",
    "hidden_size": 320, "intermediate_size": 256, "num_hidden_layers": 3,
    "num_attention_heads": 6, "num_key_value_heads": 3, "head_dim": 64, "vocab_size": 777,
    "max_position_embeddings": 4096, "rms_norm_eps": 1e-5, "rope_theta": 10000.0,
    "num_experts": 5, "num_experts_per_tok": 3, "moe_intermediate_size": 192,
    "shared_expert_intermediate_size": 192, "norm_topk_prob": False,
    "decoder_sparse_step": 1, "mlp_only_layers": [], "tie_word_embeddings": True,
    "use_sliding_window": True, "sliding_window": 150, "max_window_layers": 2,
}
CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "M": MEDIUM, "W": WINDOW_128, "X": WINDOW_64}
SEEDS = {"A": 11, "B": 23, "C": 37, "M": 41, "W": 43, "X": 47}
LONG_REQUESTS = ("W", "X")     # configurations replayed with requests of 200-400 tokens


def write_model(model_dir: str, raw_config: dict, seed: int, store_dtype=torch.bfloat16) -> None:
    """A model folder through the engine's random-weights mode."""
    import cajeta_llm_b200  # noqa: F401
    from cajeta_llm_b200.config import parse_config_dict
    from cajeta_llm_b200.engine.model import build_model
    from cajeta_llm_b200.parts.base import Runtime
    from cajeta_llm_b200.weights.sources import write_model_folder

    cfg = parse_config_dict(raw_config)
    schema = build_model(cfg, Runtime("float32", device="cpu")).params()
    write_model_folder(model_dir, cfg, schema, seed, store_dtype)


def random_tokens(vocab: int, n: int, seed: int) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


_plain_cache: Dict = {}


def plain_logits(model_dir: str, tokens: Sequence[int]) -> torch.Tensor:
    """Logits [T, vocab] of the plain implementation (float64 arithmetic), cached."""
    import plain_qwen2moe as P

    return _plain(model_dir, tokens)[0]


def plain_margins(model_dir: str, tokens: Sequence[int]) -> torch.Tensor:
    """Each position's smallest routing margin over the layers (see plain_qwen2moe.routing_margin)."""
    return _plain(model_dir, tokens)[1]


def plain_selections(model_dir: str, tokens: Sequence[int]) -> Dict[int, List[List[int]]]:
    """Per sparse layer, the experts each position picks in the plain implementation."""
    return _plain(model_dir, tokens)[2]


def _plain(model_dir, tokens):
    import plain_qwen2moe as P

    key = (model_dir, tuple(tokens))
    if key not in _plain_cache:
        if model_dir not in _plain_cache:
            _plain_cache[model_dir] = P.read_model(model_dir)
        config, weights = _plain_cache[model_dir]
        margins, selections = [1.0] * len(tokens), {}
        logits = P.forward(config, weights, list(tokens), margins=margins, selections=selections).to(torch.float32)
        _plain_cache[key] = (logits, torch.tensor(margins), selections)
    return _plain_cache[key]


# Tolerances.  float32: the engine differs from the float64 plain implementation by the
# rounding of float32 sums (measured ~3e-7 on logits of size ~1).  bfloat16: activations
# between kernels and the cache are rounded to 8 bits of mantissa; on these models the
# logits differ by ~1e-2 at most (measured), against logits of size ~1.
#
# A mixture of experts is discontinuous where two experts are nearly tied for the last
# pick: rounding upstream of the router can then swap one expert for another, and the row
# changes by a finite amount (the reference met this too and measures the gap behind each
# flip, model/MoeFfn.cajeta:135-149).  Two comparisons deal with it:
#  * routing pinned (``assert_close`` without ``margins``): the engine is given the plain
#    implementation's experts for every row (the step function's ``routing_pin``, the replay
#    tool's ``--pin-routing``); then nothing is discontinuous and EVERY row must meet the
#    element-wise bound.  This is the comparison that proves the arithmetic.
#  * routing free (``assert_close`` with ``margins``): a bfloat16 row may miss the bound only
#    if its routing margin in the plain implementation is below NEAR_TIE in some layer; such a
#    row must still point the same way as the plain row (cosine >= TIE_COSINE) unless the
#    caller says that a pinned run holds it (``pinned_elsewhere``).  These rows are counted
#    and must stay the exception.  float32 rows get no allowance at all.
TOL = {"float32": dict(atol=2e-5, rtol=1e-4), "bfloat16": dict(atol=4e-2, rtol=4e-2)}
NEAR_TIE = 0.02
TIE_COSINE = 0.995
near_tie_rows = {"seen": 0, "rows": 0}


def assert_close(got: torch.Tensor, want: torch.Tensor, dtype: str, what: str = "", margins=None,
                 pinned_elsewhere: bool = False, scale: float = 1.0) -> None:
    """``scale``: the absolute part of the bound was set for logits of size ~1; a model whose
    logits are larger (the real layer widths: sums over thousands of terms, logits up to 5-7)
    passes its largest |logit| here, since rounding errors grow with the magnitudes summed."""
    tol = TOL[dtype]
    diff = (got.double() - want.double()).abs()
    bound = tol["atol"] * max(1.0, scale) + tol["rtol"] * want.double().abs()
    if dtype == "bfloat16" and margins is not None:
        near_tie_rows["rows"] += int(margins.numel())
        bad_rows = (diff > bound).any(dim=-1)
        excusable = bad_rows & (margins.to(torch.float64) < NEAR_TIE)
        if bool(excusable.any()):
            if not pinned_elsewhere:
                cos = torch.nn.functional.cosine_similarity(got.double()[excusable], want.double()[excusable], dim=-1)
                assert bool((cos >= TIE_COSINE).all()), f"{what}: a near-tie row strays from the plain row (cosine {float(cos.min()):.4f})"
            near_tie_rows["seen"] += int(excusable.sum())
            bound = torch.where(excusable[:, None], torch.full_like(bound, float("inf")), bound)
    if bool((diff > bound).any()):
        i = int(torch.argmax(diff - bound))
        r, c = divmod(i, got.shape[-1])
        raise AssertionError(f"{what}: {int((diff > bound).sum())} of {got.numel()} logits differ; worst at row {r} "
                             f"col {c}: got {got.reshape(-1)[i]:.6f} want {want.reshape(-1)[i]:.6f}; "
                             f"first bad row {int(torch.nonzero((diff > bound).any(dim=-1))[0])}")


def run_trace(model_dir: str, dtype: str, steps: List[dict], out_dir: str, max_tokens: int, extra: Sequence[str] = ()) -> Dict[int, np.ndarray]:
    """Replay ``steps`` through ``bin/trace_run`` as a child process, one step at a time
    (the next step is written only after ``done <step>`` came back)."""
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
           "--out", out_dir, "--max-tokens", str(max_tokens)] + list(extra)
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, bufsize=1)
    try:
        for s in steps:
            proc.stdin.write(json.dumps(s) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline().strip()
            assert line == f"done {s['step']}", f"trace_run answered {line!r} to step {s['step']}"
        proc.stdin.close()
        assert proc.wait(timeout=120) == 0
    finally:
        if proc.poll() is None:
            proc.kill()
    with open(os.path.join(model_dir, "config.json")) as f:
        vocab = json.load(f)["vocab_size"]
    out = {}
    for s in steps:
        n = sum(len(e.get("want", [])) for e in s["entries"])
        path = os.path.join(out_dir, f"{s['step']}.f32")
        if n:
            out[s["step"]] = np.fromfile(path, dtype="<f4").reshape(n, vocab)
        else:
            assert not os.path.exists(path)
    return out


class DictWeights:
    """A weight source over a dict of host tensors (tests build parts from it)."""

    def __init__(self, tensors):
        self.tensors = tensors

    def check(self, schema):
        from cajeta_llm_b200.weights.sources import check_schema
        check_schema(schema, {n: tuple(t.shape) for n, t in self.tensors.items()}, "test weights")

    def get(self, name, spec):
        return self.tensors[name]

    def close(self):
        pass


def random_weights_for(part, seed, store_dtype=torch.bfloat16):
    """Random host tensors for everything ``part.params()`` declares (stored dtype rounding applied)."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, spec in part.params().items():
        if spec.init == "ones":
            t = 1.0 + 0.1 * torch.randn(spec.shape, generator=g)
        else:
            t = torch.randn(spec.shape, generator=g) * 0.08
        out[name] = t.to(store_dtype)
    return out
