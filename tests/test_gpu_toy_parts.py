"""Generality of the parts, continued: a toy feed-forward with routing of its own, a toy
position encoding (half of each head rotated, stretched frequencies), a toy norm, a toy
embedding (scaled) and a toy head (bias and a soft cap), all defined here, registered, and run
inside the framework's own attention mixer, block, cache, step function and loader without a
change to the package.  Layers differ: one has the toy feed-forward, the other the
framework's dense one."""
from dataclasses import dataclass

import numpy as np
import pytest
import torch

import helpers
import plain_qwen2moe as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
HEADS, KV, HD, ROT, STRETCH, THETA = 3, 1, 32, 16, 4.0, 500.0
EMBED_SCALE, LOGIT_CAP = 1.75, 0.5


def define_toys():
    import cajeta_llm_b200  # noqa: F401
    from cajeta_llm_b200.config import ModelConfig, register_architecture
    from cajeta_llm_b200.parts.base import Part, register_part
    from cajeta_llm_b200.parts.plan import LayerSpec, ModelPlan, ParamSpec, PartSpec, ScheduleEntry

    class StretchedHalfRotary(Part):
        """Rotates only the first ``rotary_dim`` dims of a head, at frequencies divided by
        ``stretch`` (positions count ``stretch`` times slower)."""

        def __init__(self, spec, prefix, runtime):
            super().__init__(spec, prefix, runtime)
            self.rotary_dim = int(spec["rotary_dim"])
            d = np.arange(self.rotary_dim // 2, dtype=np.float32)
            inv = np.power(np.float32(spec["theta"]), -2.0 * d / np.float32(self.rotary_dim)).astype(np.float32)
            self.inv_freq = torch.from_numpy((inv / np.float32(spec["stretch"])).astype(np.float32)).to(runtime.device)

    class PickOneFeedForward(Part):
        """Each row goes to ONE of ``n`` square maps, the one whose score row gives the largest
        dot with the row (ties to the lower index), and is scaled by tanh of that score."""

        def __init__(self, spec, prefix, runtime):
            super().__init__(spec, prefix, runtime)
            self.hidden, self.n = int(spec["hidden_size"]), int(spec["n"])
            self.score = self.maps = None

        def params(self):
            p = {self.name("score.weight"): ParamSpec((self.n, self.hidden), role="vector")}
            for e in range(self.n):
                p[self.name(f"maps.{e}.weight")] = ParamSpec((self.hidden, self.hidden))
            return p

        def load(self, source):
            self.score = self.fetch(source, self.name("score.weight"))
            self.maps = torch.stack([self.fetch(source, self.name(f"maps.{e}.weight")) for e in range(self.n)])

        needs_f32_input = True

        def forward(self, x, x_f32, residual, ctx):
            s = x_f32 @ self.score.t()                                  # [rows, n] float32
            pick = s.argmax(dim=1)                                      # first maximum
            gate = torch.tanh(s.gather(1, pick[:, None]))
            y = torch.einsum("rh,rkh->rk", x.float(), self.maps[pick].float())
            residual += gate * y

    class MeanNorm(Part):
        """y = (x - mean x) * w: a norm that cannot fold anything owed into its read."""

        def __init__(self, spec, prefix, runtime):
            super().__init__(spec, prefix, runtime)
            self.dim = int(spec["dim"])
            self.weight = None

        def params(self):
            return {self.name("weight"): ParamSpec((self.dim,), role="vector", init="ones")}

        def load(self, source):
            self.weight = self.fetch(source, self.name("weight"))

        def forward(self, x, want_f32=False, row_index=None, out_dtype=None, pending=None, want_split=False):
            if pending is not None:
                for s in range(pending.shape[0]):
                    x += pending[s]
            rows = x if row_index is None else x[row_index.long()]
            y = (rows - rows.mean(dim=1, keepdim=True)) * self.weight
            return y.to(out_dtype or self.runtime.act_dtype), (y if want_f32 else None)

    class ScaledEmbedding(Part):
        """hs = table[token] * scale: only the interface of an embedding, nothing of the package's."""

        def __init__(self, spec, prefix, runtime, vocab_size, hidden_size, weight_name):
            super().__init__(spec, prefix, runtime)
            self.shape, self.weight_name, self.scale = (vocab_size, hidden_size), weight_name, float(spec["scale"])
            self.table = None

        def params(self):
            return {self.weight_name: ParamSpec(self.shape)}

        def load(self, source):
            self.table = self.fetch(source, self.weight_name)

        def forward(self, token_ids):
            return self.table[token_ids.long()].float() * self.scale

    class CappedHead(Part):
        """logits = cap * tanh((x W^T + b) / cap)."""

        def __init__(self, spec, prefix, runtime, vocab_size, hidden_size, weight_name, embedding):
            super().__init__(spec, prefix, runtime)
            self.shape, self.weight_name, self.cap = (vocab_size, hidden_size), weight_name, float(spec["cap"])
            self.weight = self.bias = None

        def params(self):
            return {self.weight_name: ParamSpec(self.shape),
                    self.weight_name.replace("weight", "bias"): ParamSpec(self.shape[:1], role="vector")}

        def load(self, source):
            self.weight = self.fetch(source, self.weight_name)
            self.bias = self.fetch(source, self.weight_name.replace("weight", "bias"))

        def forward(self, x):
            return self.cap * torch.tanh((x.float() @ self.weight.float().t() + self.bias) / self.cap)

    register_part("embedding", "toy_scaled", ScaledEmbedding, replace=True)
    register_part("head", "toy_capped", CappedHead, replace=True)
    register_part("position", "toy_stretched_half", StretchedHalfRotary, replace=True)
    register_part("feed_forward", "toy_pick_one", PickOneFeedForward, replace=True)
    register_part("norm", "toy_mean", MeanNorm, replace=True)

    @dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        hidden_size: int = 0
        vocab_size: int = 0
        n_maps: int = 0

        @classmethod
        def from_reader(cls, r):
            return cls(architecture=r.raw["architectures"][0], hidden_size=r.integer("hidden_size"),
                       vocab_size=r.integer("vocab_size"), n_maps=r.integer("n_maps"))

        def to_json_dict(self):
            return {"architectures": [self.architecture], "hidden_size": self.hidden_size, "vocab_size": self.vocab_size,
                    "n_maps": self.n_maps}

    def build_plan(cfg):
        h = cfg.hidden_size
        rms = PartSpec("rmsnorm", {"dim": h, "eps": 1e-5})
        mean = PartSpec("toy_mean", {"dim": h})
        block = PartSpec("prenorm", {"mixer_norm_name": "n1", "feed_forward_norm_name": "n2", "mixer_name": "att",
                                     "feed_forward_name": "ff"})
        att = PartSpec("attention", {"hidden_size": h, "num_heads": HEADS, "num_kv_heads": KV, "head_dim": HD, "window": 0,
                                     "qkv_bias": True,
                                     "position": PartSpec("toy_stretched_half", {"rotary_dim": ROT, "theta": THETA,
                                                                                 "stretch": STRETCH})})
        layers = (
            LayerSpec("t.0", block, att, PartSpec("toy_pick_one", {"hidden_size": h, "n": cfg.n_maps}), rms, mean),
            LayerSpec("t.1", block, att, PartSpec("dense_swiglu", {"hidden_size": h, "intermediate_size": 3 * h}), mean, rms),
        )
        return ModelPlan(architecture=cfg.architecture, hidden_size=h, vocab_size=cfg.vocab_size,
                         embedding_name="t.embed.weight", layers=layers, schedule=(ScheduleEntry(0), ScheduleEntry(1)),
                         final_norm=rms, final_norm_prefix="t.norm", lm_head_name="t.head.weight",
                         embedding=PartSpec("toy_scaled", {"scale": EMBED_SCALE}), head=PartSpec("toy_capped", {"cap": LOGIT_CAP}))

    register_architecture("ToyPickOneForCausalLM", ToyConfig, build_plan, replace=True)
    return ToyConfig


def plain(weights, tokens, n_maps):
    """The toy model over one whole sequence in float64, from the formulas in the docstrings above."""
    W = {k: v.double() for k, v in weights.items()}
    T = len(tokens)
    hs = W["t.embed.weight"][torch.tensor(tokens)] * EMBED_SCALE
    inv = torch.tensor((np.power(np.float32(THETA), -2.0 * np.arange(ROT // 2, dtype=np.float32) / np.float32(ROT))
                        .astype(np.float32) / np.float32(STRETCH)).astype(np.float32)).double()

    def mean_norm(x, w):
        return (x - x.mean(dim=1, keepdim=True)) * w

    def rotate(t):                      # only the first ROT dims of each head turn
        return torch.cat([P.rope(t[..., :ROT], torch.arange(T), inv), t[..., ROT:]], dim=-1)

    for layer in (0, 1):
        p = f"t.{layer}"
        xn = P.rmsnorm(hs, W[f"{p}.n1.weight"], 1e-5) if layer == 0 else mean_norm(hs, W[f"{p}.n1.weight"])
        q = rotate(P.linear(xn, W[f"{p}.att.q_proj.weight"], W[f"{p}.att.q_proj.bias"]).reshape(T, HEADS, HD))
        k = rotate(P.linear(xn, W[f"{p}.att.k_proj.weight"], W[f"{p}.att.k_proj.bias"]).reshape(T, KV, HD))
        v = P.linear(xn, W[f"{p}.att.v_proj.weight"], W[f"{p}.att.v_proj.bias"]).reshape(T, KV, HD)
        ao = P.attention(q, k, v, 0, HD ** -0.5).reshape(T, HEADS * HD)
        hs = hs + P.linear(ao, W[f"{p}.att.o_proj.weight"])
        if layer == 0:
            xn = mean_norm(hs, W[f"{p}.n2.weight"])
            s = xn @ W[f"{p}.ff.score.weight"].t()
            out = torch.zeros_like(hs)
            for t in range(T):
                e = int(s[t].argmax())
                out[t] = torch.tanh(s[t, e]) * (W[f"{p}.ff.maps.{e}.weight"] @ xn[t])
            hs = hs + out
        else:
            hs = hs + P.swiglu_mlp(P.rmsnorm(hs, W[f"{p}.n2.weight"], 1e-5), W[f"{p}.ff.gate_proj.weight"],
                                   W[f"{p}.ff.up_proj.weight"], W[f"{p}.ff.down_proj.weight"])
    y = P.linear(P.rmsnorm(hs, W["t.norm.weight"], 1e-5), W["t.head.weight"], W["t.head.bias"])
    return (LOGIT_CAP * torch.tanh(y / LOGIT_CAP)).float()


def test_toy_feed_forward_position_and_norm_run_in_the_framework(tmp_path):
    ToyConfig = define_toys()
    from cajeta_llm_b200.engine.model import build_model, load_model
    from cajeta_llm_b200.engine.step import ModelRunner, StepEntry
    from cajeta_llm_b200.parts.base import Runtime
    from cajeta_llm_b200.weights.sources import write_model_folder

    cfg = ToyConfig(architecture="ToyPickOneForCausalLM", hidden_size=56, vocab_size=77, n_maps=3)
    schema = build_model(cfg, Runtime("float32", device="cpu")).params()
    assert "t.0.ff.maps.2.weight" in schema and "t.1.ff.gate_proj.weight" in schema and "t.0.n2.weight" in schema
    assert tuple(schema["t.head.bias"].shape) == (77,) and tuple(schema["t.embed.weight"].shape) == (77, 56)
    write_model_folder(str(tmp_path), cfg, schema, seed=9, store_dtype=torch.float32)
    model, _ = load_model(str(tmp_path), Runtime("float32", device=DEV))
    runner = ModelRunner(model, page_tokens=4, max_seqs=2, max_tokens_per_seq=40, num_pages=16)
    weights = P.read_safetensors(str(tmp_path / "model.safetensors"))
    seqs = {"a": helpers.random_tokens(77, 21, seed=5), "b": helpers.random_tokens(77, 13, seed=6)}
    want = {n: plain(weights, t, 3) for n, t in seqs.items()}
    slots = {n: runner.admit() for n in seqs}
    got = {n: [] for n in seqs}

    def step(parts):
        out = runner.step([StepEntry(slots[n], seqs[n][a:b], list(range(b - a))) for n, a, b in parts]).cpu()
        i = 0
        for n, a, b in parts:
            got[n].append(out[i:i + b - a])
            i += b - a

    step([("a", 0, 9)])
    step([("a", 9, 11), ("b", 0, 13)])         # a portion of two beside a whole prompt
    step([("a", 11, 12)])
    step([("a", 12, 21)])
    for n in seqs:
        helpers.assert_close(torch.cat(got[n]), want[n], "float32", f"toy request {n}")
    # routing did use more than one map (the test would pass trivially otherwise)
    W = {k: v.double() for k, v in weights.items()}
    assert len({int((W["t.embed.weight"][t] @ W["t.0.ff.score.weight"].t()).argmax()) for t in seqs["a"]}) > 1
