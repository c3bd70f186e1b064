"""Generality of the parts: a toy mixer with state of its own, a toy architecture that
runs a layer twice and lets one entry read another entry's cache -- all defined here,
registered, built from a model folder and stepped without touching the package."""
import math
from dataclasses import dataclass

import pytest
import torch

import helpers
import plain_qwen2moe as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def define_toy():
    """Registers the toy mixer and the toy architecture (idempotent)."""
    import cajeta_llm_b200  # noqa: F401
    from cajeta_llm_b200.config import ModelConfig, register_architecture
    from cajeta_llm_b200.parts.base import Part, StateNeed, register_part
    from cajeta_llm_b200.parts.plan import LayerSpec, ModelPlan, ParamSpec, PartSpec, ScheduleEntry

    class DecayMixer(Part):
        """s_t = decay * s_{t-1} + W x_t;  out_t = s_t.  The state s is per request and is
        carried from one step to the next in the request's state slot."""

        def __init__(self, spec, prefix, runtime):
            super().__init__(spec, prefix, runtime)
            self.hidden, self.decay = int(spec["hidden_size"]), float(spec["decay"])
            self.w = None

        def params(self):
            return {self.name("w_in.weight"): ParamSpec((self.hidden, self.hidden))}

        def load(self, source):
            self.w = self.fetch(source, self.name("w_in.weight"))

        def cache_need(self):
            return None

        def state_need(self):
            return StateNeed((self.hidden,), torch.float32)

        def forward(self, x, residual, ctx, entry):
            u = x.float() @ self.w.float().t()
            for r, slot in enumerate(ctx.h_req_slot):
                s = entry.state[slot]
                for row in range(ctx.h_req_start[r], ctx.h_req_start[r + 1]):
                    s.mul_(self.decay).add_(u[row])
                    residual[row] += s

    class DecayMixerOnDevice(DecayMixer):
        """The same mixer written so that a step which runs it can be captured as a CUDA graph and
        replayed: it finds slots, rows and request boundaries in the step's device metadata only,
        with shapes that depend on nothing but the step's numbers of rows and (laid-out) requests.
        s after row j of a request = decay^(j+1) s_before + sum_{m <= j} decay^(j-m) u_m: one
        masked triangular product instead of a loop over rows."""

        graph_safe = True

        def forward(self, x, residual, ctx, entry):
            u = x.float() @ self.w.float().t()                                  # [rows, hidden]
            rows = torch.arange(u.shape[0], device=u.device)
            req = ctx.row_req.long()
            start, slot = ctx.req_start.long(), ctx.req_slot.long()
            j = rows - start[req]                                               # index of the row within its request's rows
            same = req[:, None] == req[None, :]
            ahead = rows[:, None] - rows[None, :]
            m = torch.where(same & (ahead >= 0), torch.pow(self.decay, ahead.clamp(min=0).float()), 0.0)
            before = entry.state[slot.clamp(min=0)[req]]                        # each row's request's state before the step
            s = m @ u + torch.pow(self.decay, (j + 1).float())[:, None] * before
            residual += s
            # new state of every request that brought rows: s at its last row; the others (and the
            # requests the layout was filled up with, slot -1) keep theirs
            has = start[1:] > start[:-1]
            last = (start[1:] - 1).clamp(min=0)
            onehot = (torch.arange(entry.state.shape[0], device=u.device)[:, None] == slot[None, :]) & has[None, :]
            onehot = onehot.float()                                             # [slots, requests]
            entry.state.copy_(onehot @ s[last] + (1.0 - onehot.sum(dim=1, keepdim=True)) * entry.state)

    register_part("mixer", "toy_decay", DecayMixer, replace=True)
    register_part("mixer", "toy_decay_device", DecayMixerOnDevice, replace=True)

    @dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        hidden_size: int = 0
        vocab_size: int = 0
        decay: float = 0.5
        mixer_kind: str = "toy_decay"

        @classmethod
        def from_reader(cls, r):
            return cls(architecture=r.raw["architectures"][0], hidden_size=r.integer("hidden_size"),
                       vocab_size=r.integer("vocab_size"), decay=r.number("decay"), mixer_kind=r.raw.get("mixer_kind", "toy_decay"))

        def to_json_dict(self):
            return {"architectures": [self.architecture], "hidden_size": self.hidden_size, "vocab_size": self.vocab_size,
                    "decay": self.decay, "mixer_kind": self.mixer_kind}

    def build_plan(cfg):
        h = cfg.hidden_size
        norm = PartSpec("rmsnorm", {"dim": h, "eps": 1e-5})
        ff = PartSpec("dense_swiglu", {"hidden_size": h, "intermediate_size": 2 * h})
        block = PartSpec("prenorm", {"mixer_norm_name": "n1", "feed_forward_norm_name": "n2", "mixer_name": "mix",
                                     "feed_forward_name": "ff"})
        att = PartSpec("attention", {"hidden_size": h, "num_heads": 2, "num_kv_heads": 1, "head_dim": 16, "window": 0,
                                     "qkv_bias": False, "position": PartSpec("rope", {"head_dim": 16, "theta": 1e4})})
        layers = (
            LayerSpec("toy.0", block, PartSpec(cfg.mixer_kind, {"hidden_size": h, "decay": cfg.decay}), ff, norm, norm),
            LayerSpec("toy.1", block, att, ff, norm, norm),
        )
        # run order: the state layer, the attention layer, the state layer AGAIN (its own
        # state), then the attention layer again reading the cache its first run wrote
        schedule = (ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0), ScheduleEntry(1, cache_from=1))
        return ModelPlan(architecture=cfg.architecture, hidden_size=h, vocab_size=cfg.vocab_size,
                         embedding_name="toy.embed.weight", layers=layers, schedule=schedule, final_norm=norm,
                         final_norm_prefix="toy.norm", lm_head_name=None)

    register_architecture("ToyDecayForCausalLM", ToyConfig, build_plan, replace=True)
    return ToyConfig


def plain_toy(weights, tokens, hidden, decay):
    """The toy model over one whole sequence, in float64."""
    W = {k: v.double() for k, v in weights.items()}
    hs = W["toy.embed.weight"][torch.tensor(tokens)]
    T = len(tokens)
    inv = P.inv_freq(16, 1e4, torch.float64)
    first_k = first_v = None
    for entry, (layer, reads) in enumerate([(0, False), (1, False), (0, False), (1, True)]):
        p = f"toy.{layer}"
        xn = P.rmsnorm(hs, W[f"{p}.n1.weight"], 1e-5)
        if layer == 0:
            u = xn @ W[f"{p}.mix.w_in.weight"].t()
            s = torch.zeros(hidden, dtype=torch.float64)
            out = torch.zeros_like(hs)
            for t in range(T):
                s = decay * s + u[t]
                out[t] = s
            hs = hs + out
        else:
            q = P.rope(P.linear(xn, W[f"{p}.mix.q_proj.weight"]).reshape(T, 2, 16), torch.arange(T), inv)
            if not reads:
                first_k = P.rope(P.linear(xn, W[f"{p}.mix.k_proj.weight"]).reshape(T, 1, 16), torch.arange(T), inv)
                first_v = P.linear(xn, W[f"{p}.mix.v_proj.weight"]).reshape(T, 1, 16)
            ao = P.attention(q, first_k, first_v, 0, 0.25).reshape(T, 32)
            hs = hs + P.linear(ao, W[f"{p}.mix.o_proj.weight"])
        hs = hs + P.swiglu_mlp(P.rmsnorm(hs, W[f"{p}.n2.weight"], 1e-5), W[f"{p}.ff.gate_proj.weight"],
                               W[f"{p}.ff.up_proj.weight"], W[f"{p}.ff.down_proj.weight"])
    return P.linear(P.rmsnorm(hs, W["toy.norm.weight"], 1e-5), W["toy.embed.weight"]).float()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_mixer_with_state_is_registered_built_and_stepped(dtype, tmp_path):
    ToyConfig = define_toy()
    from cajeta_llm_b200.config import load_config
    from cajeta_llm_b200.engine.model import build_model, load_model
    from cajeta_llm_b200.engine.step import ModelRunner, StepEntry
    from cajeta_llm_b200.parts.base import Runtime
    from cajeta_llm_b200.weights.sources import write_model_folder

    cfg = ToyConfig(architecture="ToyDecayForCausalLM", hidden_size=40, vocab_size=90, decay=0.6)
    schema = build_model(cfg, Runtime("float32", device="cpu")).params()
    assert "toy.0.mix.w_in.weight" in schema and "toy.1.mix.k_proj.weight" in schema
    write_model_folder(str(tmp_path), cfg, schema, seed=3)
    assert load_config(str(tmp_path)) == cfg                                  # chosen by config.json's architecture name
    model, _ = load_model(str(tmp_path), Runtime(dtype, device=DEV))
    runner = ModelRunner(model, page_tokens=4, max_seqs=3, max_tokens_per_seq=48, num_pages=14)
    cache = runner.cache
    assert cache.num_groups == 1 and cache.entry_plane == [None, 0, None, 0]  # entry 3 reads entry 1's plane
    assert sorted(cache.state) == [0, 2] and cache.state[0].shape == (3, 40)  # one state slot array per run of the layer

    weights = P.read_safetensors(str(tmp_path / "model.safetensors"))
    seqs = {n: helpers.random_tokens(90, L, seed=70 + L) for n, L in (("x", 23), ("y", 9), ("z", 17))}
    want = {n: plain_toy(weights, t, 40, 0.6) for n, t in seqs.items()}
    got = {n: [] for n in seqs}
    slots = {n: runner.admit() for n in ("x", "y")}

    def step(parts):
        out = runner.step([StepEntry(slots[n], seqs[n][a:b], list(range(b - a))) for n, a, b in parts]).cpu()
        i = 0
        for n, a, b in parts:
            got[n].append(out[i:i + b - a])
            i += b - a

    step([("x", 0, 5)])
    step([("x", 5, 7), ("y", 0, 9)])          # a portion of two beside a whole prompt
    runner.release(slots.pop("y"))
    slots["z"] = runner.admit()               # z takes y's slot: its state must start from zero
    step([("z", 0, 6), ("x", 7, 8)])          # a portion beside a single token
    step([("x", 8, 20), ("z", 6, 7)])
    step([("z", 7, 17), ("x", 20, 23)])
    for n in seqs:
        helpers.assert_close(torch.cat(got[n]), want[n], dtype, f"toy request {n}")
    cache.books.check()


def test_a_state_mixer_that_says_it_is_graph_safe_is_captured_and_replayed(tmp_path):
    """The same toy model with the mixer that works from device metadata only (``graph_safe``):
    on the bfloat16 path its steps are captured as CUDA graphs like any other model's - decode
    steps and steps of one size with changing requests - give the bits of the same steps launched
    kernel by kernel, and match the plain model.  (The mixer that walks host-side slot lists is
    left uncaptured: the runner asks.)"""
    ToyConfig = define_toy()
    from cajeta_llm_b200.engine.model import build_model, load_model
    from cajeta_llm_b200.engine.step import ModelRunner, StepEntry
    from cajeta_llm_b200.parts.base import Runtime
    from cajeta_llm_b200.weights.sources import write_model_folder

    hidden = 136                                               # wide enough for the bfloat16 path's fast kernels
    cfg = ToyConfig(architecture="ToyDecayForCausalLM", hidden_size=hidden, vocab_size=200, decay=0.6, mixer_kind="toy_decay_device")
    schema = build_model(cfg, Runtime("float32", device="cpu")).params()
    write_model_folder(str(tmp_path), cfg, schema, seed=4)
    weights = P.read_safetensors(str(tmp_path / "model.safetensors"))
    seqs = [helpers.random_tokens(200, n, seed=90 + n) for n in (40, 33, 27)]
    want = [plain_toy(weights, t, hidden, 0.6) for t in seqs]
    # 12 rows a step among two or three requests (two shapes: the requests count rounded up), then everybody decodes
    plan = [{0: 6, 1: 6}, {0: 2, 1: 2, 2: 8}, {1: 11, 2: 1}, {0: 5, 1: 5, 2: 2}, {0: 4, 1: 4, 2: 4}, {0: 5, 2: 7}]
    outs = {}
    for graphs in (False, True):
        model, _ = load_model(str(tmp_path), Runtime("bfloat16", device=DEV))
        runner = ModelRunner(model, page_tokens=4, max_seqs=3, max_tokens_per_seq=48, cuda_graphs=graphs)
        assert runner.cuda_graphs == graphs
        slots = [runner.admit() for _ in seqs]
        at, got = [0, 0, 0], [[], [], []]
        for counts in plan:
            out = runner.step([StepEntry(slots[i], seqs[i][at[i]:at[i] + n], list(range(n))) for i, n in counts.items()])
            lo = 0
            for i, n in counts.items():
                got[i].append(out[lo:lo + n].clone())
                lo, at[i] = lo + n, at[i] + n
        while min(len(seqs[i]) - at[i] for i in range(3)) > 0:
            out = runner.step([StepEntry(slots[i], [seqs[i][at[i]]], [0]) for i in range(3)])
            for i in range(3):
                got[i].append(out[i:i + 1].clone())
                at[i] += 1
        outs[graphs] = [torch.cat(g).cpu() for g in got]
        if graphs:
            assert len(runner._mixed_graphs) == 2 and runner.graph_replays >= 2 + 4
    for i in range(3):
        assert torch.equal(outs[True][i], outs[False][i])
        helpers.assert_close(outs[True][i], want[i][:at[i]], "bfloat16", f"graph-safe toy request {i}")
    # the mixer that reads host-side lists is not captured
    plain_cfg = ToyConfig(architecture="ToyDecayForCausalLM", hidden_size=hidden, vocab_size=200, decay=0.6)
    model = build_model(plain_cfg, Runtime("bfloat16", device=DEV))
    assert not getattr(model.blocks[0].mixer, "graph_safe", False)
