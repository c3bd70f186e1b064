"""The engine in one process: the first tokens of a sequence, long decoding, greedy and
sampled generation through the entry point, scarce pages, and the command line."""
import subprocess
import sys

import pytest
import torch

import helpers
import plain_qwen2moe as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def runner_for(model_dir, dtype, **kw):
    import cajeta_llm_b200  # noqa: F401
    from cajeta_llm_b200.engine.model import load_model
    from cajeta_llm_b200.engine.step import ModelRunner
    from cajeta_llm_b200.parts.base import Runtime
    model, _ = load_model(model_dir, Runtime(dtype, device=DEV))
    return ModelRunner(model, **kw)


def engine_for(model_dir, dtype="float32", **kw):
    from cajeta_llm_b200.engine.llm_engine import LlmEngine
    from cajeta_llm_b200.engine.options import EngineOptions
    return LlmEngine.load(EngineOptions(model=model_dir, dtype=dtype, **kw))


def plain_greedy(model_dir, prompt, n, stop=()):
    toks = list(prompt)
    out = []
    for _ in range(n):
        t = P.argmax_first(helpers.plain_logits(model_dir, toks)[-1])
        toks.append(t)
        out.append(t)
        if t in stop:
            break
    return out


class PlainXorshift:
    """The request's random stream, restated: x ^= x << 13; x ^= x >> 7; x ^= x << 17 on 64
    bits; the uniform number is the top 24 bits over 2^24."""

    def __init__(self, seed):
        self.x = seed & (2 ** 64 - 1) or 0x9E3779B97F4A7C15

    def unit(self):
        x = self.x
        x ^= (x << 13) & (2 ** 64 - 1)
        x ^= x >> 7
        x ^= (x << 17) & (2 ** 64 - 1)
        self.x = x
        return (x >> 40) / 2.0 ** 24


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_first_tokens_of_a_sequence(name, dtype, model_dirs):
    from cajeta_llm_b200.engine.step import StepEntry
    r = runner_for(model_dirs[name], dtype, page_tokens=16, max_seqs=4, max_tokens_per_seq=64)
    vocab = helpers.CONFIGS[name]["vocab_size"]
    for n in (1, 2, 3):
        toks = helpers.random_tokens(vocab, n, seed=n)
        s = r.admit()
        got = r.step([StepEntry(s, toks, list(range(n)))]).cpu()
        helpers.assert_close(got, helpers.plain_logits(model_dirs[name], toks), dtype, f"{n} tokens")
        r.release(s)
    # token by token from the very first one
    toks = helpers.random_tokens(vocab, 5, seed=9)
    s = r.admit()
    got = torch.cat([r.step([StepEntry(s, [t], [0])]) for t in toks]).cpu()
    helpers.assert_close(got, helpers.plain_logits(model_dirs[name], toks), dtype, "one by one")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_across_many_pages(dtype, model_dirs):
    from cajeta_llm_b200.engine.step import StepEntry
    name = "B"                                              # a full layer and two windowed ones
    vocab = helpers.CONFIGS[name]["vocab_size"]
    toks = helpers.random_tokens(vocab, 230, seed=21)
    r = runner_for(model_dirs[name], dtype, page_tokens=16, max_seqs=2, max_tokens_per_seq=256)
    s = r.admit()
    outs = [r.step([StepEntry(s, toks[:6], [5])])]
    for t in toks[6:]:
        outs.append(r.step([StepEntry(s, [t], [0])]))
    got = torch.cat(outs).cpu()
    want = helpers.plain_logits(model_dirs[name], toks)[5:]
    helpers.assert_close(got, want, dtype, "long decoding")
    books = r.cache.books
    assert len(books.groups[0].held_pages(s)) == 15         # 230 tokens in pages of 16
    assert len(books.groups[1].held_pages(s)) <= 2          # the windowed layers gave their pages back
    books.check()


def test_greedy_generation_through_the_entry_point(model_dirs):
    """configs[0]'s workload: prompts of 5, 9 and 17 tokens, 8 greedy steps each."""
    from cajeta_llm_b200.sampling.params import SamplingParams
    eng = engine_for(model_dirs["A"], "float32", ctx=64, max_seqs=4)
    vocab = helpers.TINY_A["vocab_size"]
    prompts = [helpers.random_tokens(vocab, n, seed=30 + n) for n in (5, 9, 17)]
    got = eng.generate(prompts, SamplingParams(max_new_tokens=8, stop_token_ids=()))
    for p, g in zip(prompts, got):
        assert g == plain_greedy(model_dirs["A"], p, 8)
    assert eng.eog_tokens() == (255,) and eng.is_eog(255) and not eng.is_eog(3)
    # the end-of-generation set is the default stop set
    first = got[0][2]
    rid = eng.submit_tokens(prompts[0], 8, SamplingParams(stop_token_ids=(first,)))
    eng.run_all()
    req = eng.request(rid)
    assert req.generated == got[0][:got[0].index(first) + 1] and req.finish_reason.value == "eos"
    eng.close()


def test_sampled_generation_in_a_mixed_batch_follows_the_plain_sampler(model_dirs):
    """configs[1]'s workload: 4 requests with prompts of 3, 12, 20 and 31 tokens, prefill
    portions of 7, temperature 0.8, 10 steps; each request has its own random stream."""
    from cajeta_llm_b200.sampling.params import SamplingParams
    eng = engine_for(model_dirs["B"], "float32", ctx=64, max_seqs=4, chunk=7)
    vocab = helpers.TINY_B["vocab_size"]
    prompts = [helpers.random_tokens(vocab, n, seed=40 + n) for n in (3, 12, 20, 31)]
    params = [SamplingParams(temperature=0.8, seed=100 + i, max_new_tokens=10, stop_token_ids=(),
                             top_k=(0, 30, 0, 12)[i], top_p=(0.0, 0.0, 0.9, 0.95)[i],
                             repeat_penalty=(1.0, 1.0, 1.0, 1.2)[i]) for i in range(4)]
    got = eng.generate(prompts, params)
    steps = eng.scheduler().counters.steps
    assert steps >= 10 + 4 and eng.scheduler().counters.preempted == 0
    for p, sp, g in zip(prompts, params, got):
        rng = PlainXorshift(sp.seed)
        toks, out = list(p), []
        for _ in range(10):
            dist = P.prepared_distribution(helpers.plain_logits(model_dirs["B"], toks)[-1], sp.temperature, sp.top_k,
                                           sp.top_p, sp.repeat_penalty, out)
            t = P.draw(dist, rng.unit())
            toks.append(t)
            out.append(t)
        assert g == out
    eng.close()


def test_scarce_pages_preempt_recompute_and_match_solo(model_dirs):
    from cajeta_llm_b200.sampling.params import SamplingParams
    vocab = helpers.TINY_A["vocab_size"]
    prompts = [helpers.random_tokens(vocab, n, seed=50 + n) for n in (20, 26, 9)]
    sp = SamplingParams(max_new_tokens=24, stop_token_ids=())
    solo = []
    for p in prompts:
        eng = engine_for(model_dirs["A"], "float32", ctx=64, max_seqs=1)
        solo.append(eng.generate([p], sp)[0])
        eng.close()
    eng = engine_for(model_dirs["A"], "float32", ctx=64, max_seqs=3, block_tokens=4, num_blocks=22, max_batch_tokens=16)
    got = eng.generate(prompts, sp)
    c = eng.scheduler().counters
    assert c.preempted >= 1 and c.resumed == c.preempted and c.recomputed_tokens > 0
    assert got == solo
    assert eng.runner.cache.free_pages() == [22]
    eng.runner.cache.books.check()
    eng.close()


def test_step_refuses_bad_input_without_touching_the_cache(model_dirs):
    from cajeta_llm_b200.engine.step import OutOfPages, StepEntry, StepError
    r = runner_for(model_dirs["A"], "float32", page_tokens=16, max_seqs=2, max_tokens_per_seq=64, num_pages=2)
    s = r.admit()
    with pytest.raises(StepError, match="vocabulary"):
        r.step([StepEntry(s, [1, 256], [])])
    with pytest.raises(StepError, match="want"):
        r.step([StepEntry(s, [1, 2], [2])])
    with pytest.raises(OutOfPages):
        r.step([StepEntry(s, list(range(40)), [])])
    assert r.cache.free_pages() == [2] and r.cache.length(s) == 0
    r.step([StepEntry(s, list(range(32)), [])])
    with pytest.raises(OutOfPages):
        r.step([StepEntry(s, [5], [0])])
    assert r.cache.length(s) == 32


def test_command_line(model_dirs, tmp_path):
    vocab = helpers.TINY_A["vocab_size"]
    prompt = helpers.random_tokens(vocab, 6, seed=60)
    cmd = [sys.executable, "-m", "cajeta_llm_b200", "run", "--model", model_dirs["A"], "--prompt",
           " ".join(map(str, prompt)), "-n", "5", "--dtype", "float32", "--ctx", "64", "--block-size", "16", "--verbose"]
    out = subprocess.run(cmd, capture_output=True, text=True, cwd=helpers.ROOT, timeout=300)
    assert out.returncode == 0, out.stderr
    lines = out.stdout.strip().splitlines()
    want = plain_greedy(model_dirs["A"], prompt, 5, stop=(255,))
    assert lines[0].split() == [str(t) for t in want if t != 255]
    assert lines[1] == f"[{len(want)} tokens, {'eos' if want[-1] == 255 else 'budget'}]"
    bad = subprocess.run([sys.executable, "-m", "cajeta_llm_b200", "run", "--model", model_dirs["A"], "--frobnicate"],
                         capture_output=True, text=True, cwd=helpers.ROOT, timeout=300)
    assert bad.returncode == 2 and "unknown flag '--frobnicate'" in bad.stderr


def test_captured_decode_steps_give_the_same_logits_as_uncaptured_ones(model_dirs):
    """Pure decode steps are replayed from a CUDA graph; they must equal, bit for bit, the
    same steps launched kernel by kernel, also when the batch changes and pages move."""
    from cajeta_llm_b200.engine.step import StepEntry
    vocab = helpers.MEDIUM["vocab_size"]
    seqs = [helpers.random_tokens(vocab, n, seed=80 + n) for n in (40, 23, 31)]
    outs = {}
    for graphs in (False, True):
        r = runner_for(model_dirs["M"], "bfloat16", page_tokens=16, max_seqs=4, max_tokens_per_seq=64, cuda_graphs=graphs)
        slots = [r.admit() for _ in seqs]
        r.step([StepEntry(s, t[:6], []) for s, t in zip(slots, seqs)])
        # one step of two rows first: its graph is captured before the wider ones, whose
        # larger scratch must not move anything the first graph points to
        r.step([StepEntry(slots[0], [seqs[0][6]], []), StepEntry(slots[2], [seqs[2][6]], [])])
        r.step([StepEntry(slots[1], [seqs[1][6]], [])])
        got = []
        for i in range(7, 23):                       # three rows at a time
            got.append(r.step([StepEntry(s, [t[i]], [0]) for s, t in zip(slots, seqs)]).clone())
        r.release(slots[1])                          # then two, one of them wanting nothing
        for i in range(23, 31):
            got.append(r.step([StepEntry(slots[0], [seqs[0][i]], [0]), StepEntry(slots[2], [seqs[2][i]], [])]).clone())
        outs[graphs] = torch.cat(got).cpu()
        if graphs:
            assert r.graph_replays >= 20
    assert torch.equal(outs[True], outs[False])
    want = torch.cat([torch.stack([helpers.plain_logits(model_dirs["M"], t)[i] for t in seqs]) for i in range(7, 23)]
                     + [helpers.plain_logits(model_dirs["M"], seqs[0])[23:31]])
    margins = torch.cat([torch.stack([helpers.plain_margins(model_dirs["M"], t)[i] for t in seqs]) for i in range(7, 23)]
                        + [helpers.plain_margins(model_dirs["M"], seqs[0])[23:31]])
    helpers.assert_close(outs[True], want, "bfloat16", "captured decode", margins)


def test_captured_steps_with_prompt_portions_give_the_same_logits_as_uncaptured_ones(model_dirs):
    """A step shape (rows, requests, wanted rows) that comes again is captured and replayed.  The
    replays must equal, bit for bit, the same steps launched kernel by kernel: with the rows shared
    out differently among the requests, at other positions, on other pages, beside decode steps."""
    from cajeta_llm_b200.engine.step import StepEntry
    vocab = helpers.MEDIUM["vocab_size"]
    seqs = [helpers.random_tokens(vocab, 150, seed=300 + i) for i in range(3)]
    # every step: 24 rows, 3 requests, 4 wanted; the split of the rows changes from step to step
    splits = [(10, 13, 1), (1, 22, 1), (8, 8, 8), (20, 2, 2), (3, 1, 20), (12, 11, 1)]
    outs = {}
    for graphs in (False, True):
        r = runner_for(model_dirs["M"], "bfloat16", page_tokens=16, max_seqs=4, max_tokens_per_seq=160, cuda_graphs=graphs)
        slots = [r.admit() for _ in seqs]
        at = [0, 0, 0]
        got = []
        for n in splits:
            entries = []
            for i in range(3):
                want = [0, n[i] - 1] if i == 0 and n[i] > 1 else [n[i] - 1]
                entries.append(StepEntry(slots[i], seqs[i][at[i]:at[i] + n[i]], want))
                at[i] += n[i]
            if n[0] == 1:                          # four wanted rows in every step
                entries[1] = StepEntry(entries[1].slot, entries[1].tokens, [0, n[1] - 1])
            got.append(r.step(entries).clone())
            # a decode step in between (a graph of its own)
            got.append(r.step([StepEntry(slots[i], [seqs[i][at[i]]], [0]) for i in range(3)]).clone())
            at = [a + 1 for a in at]
        outs[graphs] = torch.cat(got).cpu()
        if graphs:
            assert len(r._mixed_graphs) == 1 and r.graph_replays >= len(splits) - 2 + len(splits) - 1
    assert torch.equal(outs[True], outs[False])
    # and against the plain implementation: the last wanted row of each request in the last portion step
    at = [sum(n[i] for n in splits) + len(splits) for i in range(3)]
    want = torch.stack([helpers.plain_logits(model_dirs["M"], seqs[i][:at[i]])[at[i] - 1] for i in range(3)])
    margins = torch.stack([helpers.plain_margins(model_dirs["M"], seqs[i][:at[i]])[at[i] - 1] for i in range(3)])
    helpers.assert_close(outs[True][-3:], want, "bfloat16", "captured mixed steps", margins)


@pytest.mark.parametrize("name", ["W", "X"])
def test_windowed_layers_on_the_fast_kernels_give_pages_back_and_match_the_plain_implementation(name, model_dirs):
    """Head sizes 128 and 64 with a window (40 and 150 tokens: no multiple of a page or of a
    128-key chunk), bfloat16: two requests are fed in portions that cross the window, then
    decode side by side past several page trims - launched kernel by kernel and replayed from
    graphs, with the same bits - and every position is held to the plain implementation.  The
    windowed group must have given back all pages behind the window, and get them again."""
    from cajeta_llm_b200.engine.step import StepEntry
    cfg = helpers.CONFIGS[name]
    vocab, w, page = cfg["vocab_size"], cfg["sliding_window"], 16
    seqs = [helpers.random_tokens(vocab, n, seed=400 + n) for n in (330, 241)]
    portions = [(57, 100, 73), (130, 31)]                      # then one by one
    outs = {}
    for graphs in (False, True):
        r = runner_for(model_dirs[name], "bfloat16", page_tokens=page, max_seqs=2, max_tokens_per_seq=336,
                       num_pages=2 * 21, cuda_graphs=graphs)
        slots = [r.admit(), r.admit()]
        at, got = [0, 0], [[], []]
        for k in range(3):
            entries = []
            for i in range(2):
                if k < len(portions[i]):
                    n = portions[i][k]
                    entries.append((i, StepEntry(slots[i], seqs[i][at[i]:at[i] + n], list(range(n)))))
                    at[i] += n
            out = r.step([e for _, e in entries])
            lo = 0
            for i, e in entries:
                got[i].append(out[lo:lo + len(e.tokens)].clone())
                lo += len(e.tokens)
        books = r.cache.books
        full = [g for g, spec in enumerate(r.cache.group_specs) if spec.window == 0]
        windowed = [g for g, spec in enumerate(r.cache.group_specs) if spec.window > 0]
        assert len(full) == 1 and len(windowed) == 1
        while at[1] < len(seqs[1]):                            # both decode, then the longer one alone
            out = r.step([StepEntry(slots[i], [seqs[i][at[i]]], [0]) for i in range(2)])
            for i in range(2):
                got[i].append(out[i:i + 1].clone())
                at[i] += 1
            for i in range(2):
                held = books.groups[windowed[0]].held_pages(slots[i])
                assert len(held) <= -(-w // page) + 1, (at[i], len(held))
                assert len(books.groups[full[0]].held_pages(slots[i])) == -(-at[i] // page)
        r.release(slots[1])
        while at[0] < len(seqs[0]):
            got[0].append(r.step([StepEntry(slots[0], [seqs[0][at[0]]], [0])]).clone())
            at[0] += 1
        books.check()
        table = books.groups[windowed[0]].table[slots[0]]
        first_live = (len(seqs[0]) + 1 - w) // page
        assert (table[:first_live] == -1).all() and (table[first_live:-(-len(seqs[0]) // page)] >= 0).all()
        outs[graphs] = [torch.cat(g).cpu() for g in got]
        if graphs:
            assert r.graph_replays >= 90
    for i in range(2):
        assert torch.equal(outs[True][i], outs[False][i])
        helpers.assert_close(outs[True][i], helpers.plain_logits(model_dirs[name], seqs[i]), "bfloat16",
                             f"{name} windowed request {i}", helpers.plain_margins(model_dirs[name], seqs[i]))


def test_real_layer_sizes_match_the_plain_implementation(tmp_path):
    """Layers of the benchmark's sizes (fewer of them): a prompt in one step, in portions
    beside another request's decode tokens, and token by token, in float32 and bfloat16."""
    from cajeta_llm_b200.engine.step import StepEntry
    d = str(tmp_path)
    helpers.write_model(d, helpers.REAL_SIZES, seed=77)
    vocab = helpers.REAL_SIZES["vocab_size"]
    a = helpers.random_tokens(vocab, 150, seed=1)
    b = helpers.random_tokens(vocab, 40, seed=2)
    want_a, want_b = helpers.plain_logits(d, a), helpers.plain_logits(d, b)
    m_a, m_b = helpers.plain_margins(d, a), helpers.plain_margins(d, b)
    for dtype in ("float32", "bfloat16"):
        r = runner_for(d, dtype, page_tokens=16, max_seqs=2, max_tokens_per_seq=256)
        sa, sb = r.admit(), r.admit()
        got_a = [r.step([StepEntry(sa, a[:97], list(range(97)))])]                       # a long portion alone
        got_b = [r.step([StepEntry(sb, b[:30], list(range(30)))])]
        for i in range(30, 40):                                                            # b decodes beside a's portions
            n = 5 if i < 39 else 8
            lo = 97 + (i - 30) * 5
            out = r.step([StepEntry(sb, [b[i]], [0]), StepEntry(sa, a[lo:lo + n], list(range(n)))])
            got_b.append(out[:1])
            got_a.append(out[1:])
        r.release(sb)
        assert 97 + 9 * 5 + 8 == 150
        helpers.assert_close(torch.cat(got_b).cpu(), want_b, dtype, f"real sizes {dtype} b", m_b)
        helpers.assert_close(torch.cat(got_a).cpu(), want_a, dtype, f"real sizes {dtype} a", m_a)
        # and a pure decode tail (captured as a graph on the bfloat16 path)
        sc = r.admit()
        r.step([StepEntry(sc, b[:20], [])])
        tail = torch.cat([r.step([StepEntry(sc, [t], [0])]) for t in b[20:]]).cpu()
        helpers.assert_close(tail, want_b[20:], dtype, f"real sizes {dtype} decode", m_b[20:])


def test_layer_sizes_of_the_larger_configuration_match_the_plain_implementation(tmp_path):
    """One layer of Qwen2-57B-A14B's sizes (hidden 3,584, 28 heads over 4 kv heads, 8 of the experts
    of 2,560 per token; fewer experts, a smaller shared expert and vocabulary): a prompt of 530
    tokens in one step (above 512 rows the shared expert runs as dense products), the same prompt in
    portions of changing size, and a decoded tail, against the plain implementation.

    float32: the usual bound.  bfloat16: the usual bound's absolute part (0.04) was set for logits of
    size ~1; here they have a standard deviation of 1.2 and reach 7.4, the mean error of bfloat16
    rounding is 0.008 (0.7 % of that), and its tail crosses 0.04 for about one logit in 10^5
    (measured: 11 of 1,060,000, in rows whose routing is far from a tie).  So the bound must hold
    for all but one logit in 10^4, the mean error must stay below two bfloat16 steps (2^-7) of the
    logits' standard deviation (measured 1.7 steps, the same on the tensor-core kernels and on the
    float32-arithmetic kernels with bfloat16 storage: it is the storage's rounding), and every row
    that is not near a routing tie must point the same way as the plain row to a cosine of 0.9995
    - a misplaced tile or head moves rows far more."""
    from cajeta_llm_b200.engine.step import StepEntry
    cfg = dict(helpers.REAL_SIZES, hidden_size=3584, intermediate_size=18944, num_hidden_layers=1, num_attention_heads=28,
               num_key_value_heads=4, num_experts=9, num_experts_per_tok=8, moe_intermediate_size=2560,
               shared_expert_intermediate_size=5120, vocab_size=2000)
    d = str(tmp_path)
    helpers.write_model(d, cfg, seed=91)
    toks = helpers.random_tokens(cfg["vocab_size"], 530, seed=3)
    want, margins = helpers.plain_logits(d, toks), helpers.plain_margins(d, toks)

    def check(got, what, dtype):
        if dtype == "float32":
            helpers.assert_close(got, want, dtype, what, margins)
            return
        tol = helpers.TOL["bfloat16"]
        diff = (got.double() - want.double()).abs()
        clear = margins.to(torch.float64) >= helpers.NEAR_TIE
        outside = (diff > tol["atol"] + tol["rtol"] * want.double().abs())[clear]
        assert int(outside.sum()) <= 1e-4 * outside.numel(), (what, int(outside.sum()))
        assert float(diff[clear].mean()) <= 2.0 ** -7 * float(want.std()), (what, float(diff[clear].mean()))
        cosine = torch.nn.functional.cosine_similarity(got.double(), want.double(), dim=1)
        assert float(cosine[clear].min()) >= 0.9995, (what, float(cosine[clear].min()))
        assert float(cosine.min()) >= helpers.TIE_COSINE, (what, float(cosine.min()))

    for dtype in ("float32", "bfloat16"):
        r = runner_for(d, dtype, page_tokens=16, max_seqs=2, max_tokens_per_seq=544)
        s = r.admit()
        check(r.step([StepEntry(s, toks, list(range(530)))]).cpu(), f"larger sizes {dtype}, whole", dtype)
        r.release(s)
        s = r.admit()
        got, at = [], 0
        for n in (300, 129, 2, 67, 16):                   # 514 tokens in portions, then 16 one by one
            got.append(r.step([StepEntry(s, toks[at:at + n], list(range(n)))]))
            at += n
        got += [r.step([StepEntry(s, [t], [0])]) for t in toks[514:]]
        check(torch.cat(got).cpu(), f"larger sizes {dtype}, portions and decode", dtype)
        del r
        torch.cuda.empty_cache()


@pytest.mark.parametrize("name", ["A", "M"])
def test_decoding_one_step_ahead_of_the_host_changes_no_token(name, model_dirs):
    """While all requests decode the scheduler launches the next step before it has seen the
    tokens of the one in flight.  Budgets that end at different steps, a stop token that ends a
    request in the middle (its row rides along for one step and is dropped), greedy and sampled
    rows: every request's tokens equal those of the scheduler that waits for each step."""
    from cajeta_llm_b200.sampling.params import SamplingParams
    cfg = helpers.CONFIGS[name]
    vocab = cfg["vocab_size"]
    prompts = [helpers.random_tokens(vocab, n, seed=60 + n) for n in (6, 11, 19, 4)]

    def run(lookahead, stop_for_second=()):
        eng = engine_for(model_dirs[name], "bfloat16", ctx=96, max_seqs=4, lookahead=lookahead)
        params = [SamplingParams(max_new_tokens=14, stop_token_ids=()),
                  SamplingParams(max_new_tokens=20, stop_token_ids=tuple(stop_for_second)),
                  SamplingParams(max_new_tokens=9, stop_token_ids=(), temperature=0.7, top_k=20, seed=5),
                  SamplingParams(max_new_tokens=3, stop_token_ids=())]
        ids = [eng.submit_tokens(p, sp.max_new_tokens, sp) for p, sp in zip(prompts, params)]
        eng.run_all()
        out = [(list(eng.request(i).generated), eng.request(i).finish_reason.value) for i in ids]
        steps = eng.scheduler().counters.steps
        eng.close()
        return out, steps

    base, _ = run(False)
    stop = base[1][0][7]                         # the second request will end on this token, in the middle
    want, steps_wait = run(False, (stop,))
    got, steps_ahead = run(True, (stop,))
    assert got == want
    assert want[1][1] == "eos" and len(want[1][0]) <= 8 and [r[1] for r in want[:1] + want[2:]] == ["budget"] * 3
    assert steps_ahead <= steps_wait + 1         # at most the one step a stopped request rode along


def test_full_size_float32_path_gives_the_same_logits_however_the_work_is_cut():
    """The whole model at Qwen1.5-MoE-A2.7B sizes (24 layers, 60 experts, vocabulary 151,936,
    ~64 GB) on the true 32-bit path: a mixed workload of 8 requests with prompts of 64 to 1,024
    tokens, prefill portions of 256 beside decode tokens, runs through the scheduler; one
    request's logits are the same to the bit whole, in portions and token by token (the 32-bit
    kernels sum in an order that does not depend on the batch), and its greedy tokens inside
    the mixed batch equal those it gives alone."""
    from cajeta_llm_b200.engine.llm_engine import LlmEngine
    from cajeta_llm_b200.engine.options import EngineOptions
    from cajeta_llm_b200.engine.step import StepEntry
    from cajeta_llm_b200.sampling.params import SamplingParams
    if torch.cuda.mem_get_info()[0] < 80e9:
        pytest.skip("needs 80 GB of free device memory")
    cfg = dict(helpers.REAL_SIZES, num_hidden_layers=24, num_experts=60, vocab_size=151936)
    eng = LlmEngine.load(EngineOptions(config=cfg, random_weights=True, seed=1, dtype="float32", ctx=1280, max_seqs=8,
                                       block_tokens=16, max_batch_tokens=2048, chunk=256))
    vocab = cfg["vocab_size"]
    prompts = [helpers.random_tokens(vocab, n, seed=200 + n) for n in (64, 1024, 300, 517, 129, 800, 256, 999)]
    new = 24
    ids = [eng.submit_tokens(p, new, SamplingParams(max_new_tokens=new, stop_token_ids=())) for p in prompts]
    eng.run_all()
    mixed = [list(eng.request(i).generated) for i in ids]
    assert all(len(g) == new for g in mixed)
    r = eng.runner

    def last_logits(cuts):
        s, pos, lg = r.admit(), 0, None
        for n in cuts:
            lg = r.step([StepEntry(s, prompts[1][pos:pos + n], [n - 1])])
            pos += n
        r.release(s)
        return lg[-1].clone()

    whole = last_logits([1024])
    assert torch.isfinite(whole).all() and float(whole.abs().max()) > 0.1
    assert torch.equal(whole, last_logits([256, 256, 256, 256]))
    assert torch.equal(whole, last_logits([1000] + [1] * 24))
    rid = eng.submit_tokens(prompts[1], new, SamplingParams(max_new_tokens=new, stop_token_ids=()))
    eng.run_all()
    assert list(eng.request(rid).generated) == mixed[1]
    eng.close()


def test_full_size_bfloat16_path_agrees_with_itself_however_the_work_is_cut():
    """The same at serving precision (tensor-core kernels at the benchmark's shapes): all 1,024
    positions of a prompt, whole, in portions of 256 and with the last tokens one by one (captured
    decode steps).  Different cuts take different kernels (a step of 512 rows or more runs the
    shared expert as dense products of its own, a smaller one as extra groups of the experts'
    products) and different tile shapes, so rounding differs between cuts as much as bfloat16
    rounding differs from exact arithmetic: through 24 layers and with logits up to 5 that is more
    than the element-wise bound of the small models for some rows.  The measure is therefore the
    model's own 32-bit path on the same prompt: every cut must agree with it equally well (every
    row points the same way, the mean error is below one bfloat16 step of the largest logit), and
    two cuts must not differ from each other in more rows than they differ from the 32-bit path."""
    from cajeta_llm_b200.engine.llm_engine import LlmEngine
    from cajeta_llm_b200.engine.options import EngineOptions
    from cajeta_llm_b200.engine.step import StepEntry
    if torch.cuda.mem_get_info()[0] < 120e9:
        pytest.skip("needs 120 GB of free device memory")
    cfg = dict(helpers.REAL_SIZES, num_hidden_layers=24, num_experts=60, vocab_size=151936)
    prompt = helpers.random_tokens(cfg["vocab_size"], 1024, seed=1224)

    def all_logits(r, cuts):
        s, pos, outs = r.admit(), 0, []
        for n in cuts:
            outs.append(r.step([StepEntry(s, prompt[pos:pos + n], list(range(n)))]).clone())
            pos += n
        r.release(s)
        return torch.cat(outs)

    exact_engine = LlmEngine.load(EngineOptions(config=cfg, random_weights=True, seed=1, dtype="float32", ctx=1280,
                                                max_seqs=4, block_tokens=16, max_batch_tokens=2048))
    exact = all_logits(exact_engine.runner, [1024])
    exact_engine.close()
    del exact_engine
    torch.cuda.empty_cache()
    eng = LlmEngine.load(EngineOptions(config=cfg, random_weights=True, seed=1, dtype="bfloat16", ctx=1280, max_seqs=4,
                                       block_tokens=16, max_batch_tokens=2048))
    r = eng.runner
    tol = helpers.TOL["bfloat16"]

    def rows_apart(a, b):
        return int(((a - b).abs() > tol["atol"] + tol["rtol"] * a.abs()).any(dim=1).sum())

    results = {}
    for cuts in ([1024], [512, 512], [256, 256, 256, 256], [700, 2, 61, 237] + [1] * 24):
        got = all_logits(r, cuts)
        assert torch.isfinite(got).all() and float(got.abs().max()) > 0.1
        cosine = torch.nn.functional.cosine_similarity(exact, got, dim=1)
        assert float(cosine.min()) >= helpers.TIE_COSINE, (cuts[:4], float(cosine.min()))
        assert float((exact - got).abs().mean()) <= 2.0 ** -8 * float(exact.abs().max()), cuts[:4]
        results[tuple(cuts)] = (got, rows_apart(exact, got))
    whole, whole_apart = results[(1024,)]
    for cuts, (got, apart) in results.items():
        assert rows_apart(whole, got) <= max(whole_apart, apart), (cuts[:4], rows_apart(whole, got), whole_apart, apart)
    r.check_waits()
    eng.close()
