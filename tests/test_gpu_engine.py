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


def test_a_windowed_group_gets_a_pool_of_its_own_size_through_the_entry_point(model_dirs):
    """Configuration W (one layer keeps every key, two a window of 40) through LlmEngine with
    steps of at most 48 tokens: the windowed group's pool is sized by window + step, not by the
    context; three requests run side by side in it and generate what the plain implementation
    generates (float32, greedy)."""
    from cajeta_llm_b200.sampling.params import SamplingParams
    eng = engine_for(model_dirs["W"], "float32", ctx=320, max_seqs=3, max_batch_tokens=48)
    cache = eng.runner.cache
    sizes = {spec.window: pages for spec, pages in zip(cache.group_specs, cache.group_pages)}
    assert sizes == {0: 3 * 20, 40: 3 * (-(-(40 + 48) // 16) + 1)}
    vocab = helpers.CONFIGS["W"]["vocab_size"]
    prompts = [helpers.random_tokens(vocab, n, seed=600 + n) for n in (150, 90, 201)]
    got = eng.generate(prompts, SamplingParams(max_new_tokens=4, stop_token_ids=()))
    assert eng.scheduler().counters.preempted == 0
    for p, g in zip(prompts, got):
        assert g == plain_greedy(model_dirs["W"], p, 4)
    assert cache.free_pages() == [60, 21]
    cache.books.check()
    eng.close()


def test_steps_of_one_size_replay_one_graph_whatever_their_requests(model_dirs):
    """What a scheduler that fills a token budget produces: the same number of rows step after
    step, shared among two, three or four requests of which one, two or all want logits.  Steps
    whose requests round up to the same power of two replay ONE captured graph (the per-request
    arrays are laid out for that many requests, the wanted rows filled up to it), with the bits
    of the same steps launched kernel by kernel."""
    from cajeta_llm_b200.engine.step import StepEntry
    vocab = helpers.MEDIUM["vocab_size"]
    seqs = [helpers.random_tokens(vocab, 140, seed=700 + i) for i in range(4)]
    # (request -> number of its next tokens, requests that want their last row); 20 rows each
    plan = [({0: 5, 1: 5, 2: 10}, [0, 2]), ({0: 1, 1: 1, 2: 9, 3: 9}, [0, 1, 2, 3]), ({0: 4, 1: 4, 2: 4, 3: 8}, [0, 1]),
            ({1: 10, 2: 5, 3: 5}, [3]), ({0: 3, 1: 3, 2: 3, 3: 11}, [1, 2, 3]),                # three or four requests: one shape
            ({0: 10, 1: 10}, [1]), ({1: 19, 3: 1}, [3]), ({0: 7, 3: 13}, [0, 3]), ({2: 2, 3: 18}, [2]),     # two requests: another
            ({0: 20}, [0]), ({2: 20}, [2]), ({0: 20}, [0])]                                    # one request: a third
    outs = {}
    for graphs in (False, True):
        r = runner_for(model_dirs["M"], "bfloat16", page_tokens=16, max_seqs=4, max_tokens_per_seq=144, cuda_graphs=graphs)
        slots = [r.admit() for _ in seqs]
        at, got = [0] * 4, []
        for counts, wanting in plan:
            entries = [StepEntry(slots[i], seqs[i][at[i]:at[i] + n], [n - 1] if i in wanting else []) for i, n in counts.items()]
            for i, n in counts.items():
                at[i] += n
            got.append(r.step(entries).clone())
            assert got[-1].shape[0] == len(wanting)
        outs[graphs] = torch.cat(got).cpu()
        if graphs:
            # a shape's first step is launched kernel by kernel, its second captured, the others replayed
            assert len(r._mixed_graphs) == 3 and r.graph_replays == (5 - 2) + (4 - 2) + (3 - 2)
    assert torch.equal(outs[True], outs[False])
    # the last step's rows against the plain implementation
    want = torch.stack([helpers.plain_logits(model_dirs["M"], seqs[i][:at[i]])[at[i] - 1] for i in (0,)])
    margins = torch.stack([helpers.plain_margins(model_dirs["M"], seqs[i][:at[i]])[at[i] - 1] for i in (0,)])
    helpers.assert_close(outs[True][-1:], want, "bfloat16", "steps of one size", margins)


@pytest.mark.parametrize("trial", range(6))
def test_random_workloads_with_and_without_graphs_and_alone(model_dirs, trial):
    """Random requests (prompts of 1 to 250 tokens, 1 to 30 new tokens) through the scheduler with random
    limits (live requests, token budget, pages down to one more than the longest request needs, so that
    some runs preempt): with CUDA graphs the schedule and the kernels are those of the run without, so every
    request generates the same tokens; and in float32, whose kernels do not depend on the batch, the same
    tokens as the request alone."""
    import random
    from cajeta_llm_b200.sampling.params import SamplingParams
    rnd = random.Random(100 + trial)
    name = rnd.choice(["M", "W", "X"])
    vocab = helpers.CONFIGS[name]["vocab_size"]
    reqs = [([rnd.randrange(vocab) for _ in range(rnd.choice([1, 2, 3, 17, 40, 64, 65, 130, 250]))], rnd.randint(1, 30))
            for _ in range(rnd.randint(6, 14))]
    max_seqs = rnd.choice([2, 3, 4, 6, 8])
    budget = rnd.choice([32, 48, 96, 200])
    need = max((len(p) + n + 15) // 16 + 1 for p, n in reqs)
    blocks = rnd.choice([need + 1, need + 2, need + need // 2, need * 2, need * max_seqs])

    def run(dtype, graphs, requests, seqs, pages):
        eng = engine_for(model_dirs[name], dtype, ctx=512, max_seqs=seqs, block_tokens=16, num_blocks=pages,
                         max_batch_tokens=budget, cuda_graphs=graphs, warmup=False)
        ids = [eng.submit_tokens(p, n, SamplingParams(max_new_tokens=n, stop_token_ids=())) for p, n in requests]
        eng.run_all()
        out = [list(eng.request(i).generated) for i in ids]
        replays = eng.runner.graph_replays
        eng.close()
        return out, replays

    with_graphs, replays = run("bfloat16", True, reqs, max_seqs, blocks)
    without, _ = run("bfloat16", False, reqs, max_seqs, blocks)
    assert replays > 0 and with_graphs == without
    if trial % 2 == 0:
        batched, _ = run("float32", False, reqs, max_seqs, blocks)
        alone = [run("float32", False, [r], 1, need + 2)[0][0] for r in reqs]
        assert batched == alone


def routing_pins(model_dir, rows):
    """The plain implementation's experts for the rows [(tokens, position)] of one step, as the
    step function's ``routing_pin``: a routed feed-forward's prefix -> int32 [rows, k]."""
    first = helpers.plain_selections(model_dir, rows[0][0])
    return {f"model.layers.{l}.mlp": torch.tensor([helpers.plain_selections(model_dir, toks)[l][pos] for toks, pos in rows],
                                                   dtype=torch.int32, device=DEV) for l in first}


def test_real_layer_sizes_match_the_plain_implementation(tmp_path):
    """Layers of the benchmark's sizes (fewer of them): a prompt in one step, in portions
    beside another request's decode tokens, and token by token, in float32 and bfloat16.  In
    bfloat16 everything runs twice: with the routing free (a row at a near-tie may pick another
    expert than the plain implementation and is then excused, counted), and with every row's
    experts pinned to the plain implementation's, where every logit must meet the bound."""
    from cajeta_llm_b200.engine.step import StepEntry
    d = str(tmp_path)
    helpers.write_model(d, helpers.REAL_SIZES, seed=77)
    vocab = helpers.REAL_SIZES["vocab_size"]
    a = helpers.random_tokens(vocab, 150, seed=1)
    b = helpers.random_tokens(vocab, 40, seed=2)
    want_a, want_b = helpers.plain_logits(d, a), helpers.plain_logits(d, b)
    m_a, m_b = helpers.plain_margins(d, a), helpers.plain_margins(d, b)
    for dtype, pinned in (("float32", False), ("bfloat16", False), ("bfloat16", True)):
        r = runner_for(d, dtype, page_tokens=16, max_seqs=2, max_tokens_per_seq=256)

        def step(parts):
            """parts: [(slot, tokens of the request, lo, hi)] -> logits of all their rows"""
            entries = [StepEntry(s, t[lo:hi], list(range(hi - lo))) for s, t, lo, hi in parts]
            if not pinned:
                return r.step(entries)
            return r.step(entries, routing_pin=routing_pins(d, [(t, p) for _, t, lo, hi in parts for p in range(lo, hi)]))

        sa, sb = r.admit(), r.admit()
        got_a = [step([(sa, a, 0, 97)])]                                                   # a long portion alone
        got_b = [step([(sb, b, 0, 30)])]
        for i in range(30, 40):                                                            # b decodes beside a's portions
            n = 5 if i < 39 else 8
            lo = 97 + (i - 30) * 5
            out = step([(sb, b, i, i + 1), (sa, a, lo, lo + n)])
            got_b.append(out[:1])
            got_a.append(out[1:])
        r.release(sb)
        assert 97 + 9 * 5 + 8 == 150
        what = f"real sizes {dtype}{' pinned' if pinned else ''}"

        def hold(got, want, margins, which):
            if pinned:
                helpers.assert_close(got, want, dtype, f"{what} {which}")                  # no allowance at all
            else:
                helpers.assert_close(got, want, dtype, f"{what} {which}", margins, pinned_elsewhere=dtype == "bfloat16")

        hold(torch.cat(got_b).cpu(), want_b, m_b, "b")
        hold(torch.cat(got_a).cpu(), want_a, m_a, "a")
        # and a pure decode tail (captured as a graph on the bfloat16 path when the routing is free)
        sc = r.admit()
        r.step([StepEntry(sc, b[:20], [])])
        tail = torch.cat([step([(sc, b, i, i + 1)]) for i in range(20, 40)]).cpu()
        hold(tail, want_b[20:], m_b[20:], "decode")


def test_layer_sizes_of_the_larger_configuration_match_the_plain_implementation(tmp_path):
    """One layer of Qwen2-57B-A14B's sizes (hidden 3,584, 28 heads over 4 kv heads, 8 of the experts
    of 2,560 per token; fewer experts, a smaller shared expert and vocabulary): a prompt of 530
    tokens in one step (above 512 rows the shared expert runs as dense products), the same prompt in
    portions of changing size, and a decoded tail, against the plain implementation.

    float32: the usual bound, its absolute part taken relative to the largest logit (7.4; sums over
    3,584 to 20,480 terms).  bfloat16: the usual bound's absolute part (0.04) was set for logits of
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
            helpers.assert_close(got, want, dtype, what, margins, scale=float(want.abs().max()))
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


FULL_SIZE = dict(helpers.REAL_SIZES, num_hidden_layers=24, num_experts=60, vocab_size=151936)


def need_free_memory(n_bytes, what):
    """Skips a full-size test on a device with too little free memory - and says so where the
    log shows it (a warning in pytest's summary), so that a skip is never a silent pass."""
    import warnings
    free = torch.cuda.mem_get_info()[0]
    if free < n_bytes:
        reason = f"{what} SKIPPED: needs {n_bytes / 1e9:.0f} GB of free device memory, {free / 1e9:.0f} GB are free"
        warnings.warn(reason)
        print("\n" + reason)
        pytest.skip(reason)


def oracle_for(engine, cfg, tokens):
    """Float64 logits, routing margins and picked experts of the whole-tensor plain
    implementation over the very tensors the engine holds (no second copy of the weights)."""
    import plain_vectorised as PV
    margins, picked = [1.0] * len(tokens), {}
    logits = PV.forward(cfg, PV.engine_views(engine.runner.model), tokens, margins=margins, selections=picked)
    return logits, torch.tensor(margins), picked


def check_drawn_tensors(model, seed):
    """A model drawn in place on the device holds what the generator gives for (seed, tensor
    name, element): single elements of stacked and sliced tensors against the restatement
    with Python integers (bfloat16 values rounded to nearest even)."""
    import plain_random as PR
    import plain_vectorised as PV
    get = PV.engine_views(model)
    names = ["model.embed_tokens.weight", "lm_head.weight", "model.layers.0.self_attn.k_proj.weight",
             "model.layers.7.self_attn.v_proj.bias", "model.layers.23.self_attn.o_proj.weight",
             "model.layers.5.mlp.gate.weight", "model.layers.11.mlp.experts.59.up_proj.weight",
             "model.layers.2.mlp.experts.0.down_proj.weight", "model.layers.19.mlp.shared_expert.down_proj.weight",
             "model.layers.19.mlp.shared_expert.gate_proj.weight", "model.layers.3.mlp.shared_expert_gate.weight"]
    for name in names:
        t = get(name)
        flat_size = t.numel()
        for i in (0, flat_size // 3 + 1, flat_size - 1):
            idx = []
            rest = i
            for n in reversed(t.shape):
                idx.append(rest % n)
                rest //= n
            got = float(t[tuple(reversed(idx))])
            want = PR.value(seed, name, i, 0.02)
            # matrices keep the stored bfloat16 value on either path; vectors too (a bfloat16 file)
            assert got == PR.to_bfloat16(want), (name, i, got, want)


def test_full_size_float32_path_against_the_plain_implementation_however_the_work_is_cut():
    """The whole model at Qwen1.5-MoE-A2.7B sizes (24 layers, 60 experts, vocabulary 151,936,
    ~64 GB) on the true 32-bit path, held to the whole-tensor plain implementation in float64
    over the same weight tensors: all 1,024 positions of a prompt in one step, in four portions
    of 256, with the last 32 tokens one by one, and inside a mixed batch (portions of 256 beside
    other requests' portions and decode tokens).  The cuts also agree with each other to the bit
    (the 32-bit kernels sum in an order that does not depend on the batch).  Then the scheduler's
    mixed workload of 8 requests: a request's greedy tokens equal those it gives alone and the
    plain implementation's."""
    import plain_vectorised as PV
    from cajeta_llm_b200.engine.llm_engine import LlmEngine
    from cajeta_llm_b200.engine.options import EngineOptions
    from cajeta_llm_b200.engine.step import StepEntry
    from cajeta_llm_b200.sampling.params import SamplingParams
    need_free_memory(80e9, "full-size float32 test")
    cfg = FULL_SIZE
    eng = LlmEngine.load(EngineOptions(config=cfg, random_weights=True, seed=1, dtype="float32", ctx=1280, max_seqs=8,
                                       block_tokens=16, max_batch_tokens=2048, chunk=256))
    check_drawn_tensors(eng.runner.model, seed=1)
    vocab = cfg["vocab_size"]
    prompts = [helpers.random_tokens(vocab, n, seed=200 + n) for n in (64, 1024, 300, 517, 129, 800, 256, 999)]
    r = eng.runner
    main = prompts[1]
    want, margins, _ = oracle_for(eng, cfg, main)
    scale = float(want.abs().max())
    assert scale > 0.5

    def all_logits(cuts):
        s, pos, outs = r.admit(), 0, []
        for n in cuts:
            outs.append(r.step([StepEntry(s, main[pos:pos + n], list(range(n)))]).clone())
            pos += n
        r.release(s)
        return torch.cat(outs)

    def held_to_the_oracle(got, what):
        d = (got.double() - want).abs()
        bad = (d > 2e-5 * scale + 1e-4 * want.abs()).any(dim=1)
        # a row within 1e-5 of a routing tie may legitimately pick the other expert in float32
        assert not bool((bad & (margins.to(bad.device) > 1e-5)).any()), (what, float(d.max()), int(bad.sum()))
        print(f"\nfull size float32, {what}: worst |diff| {float(d.max()):.3e} of logits up to {scale:.2f}; "
              f"smallest routing margin {float(margins.min()):.2e}; rows off at a near-tie {int(bad.sum())}")
        assert int(bad.sum()) <= 1

    whole = all_logits([1024])
    held_to_the_oracle(whole, "whole")
    assert torch.equal(whole, all_logits([256, 256, 256, 256]))
    assert torch.equal(whole, all_logits([992] + [1] * 32))
    # inside a mixed batch: its portions beside another prompt's portions and a third request's decode tokens
    sa, sb, sc = r.admit(), r.admit(), r.admit()
    b, c = prompts[3], prompts[2]
    r.step([StepEntry(sc, c[:200], [])])
    got, at_b, at_c = [], 0, 200
    for k in range(4):
        entries = [StepEntry(sc, [c[at_c]], [0]), StepEntry(sa, main[256 * k:256 * (k + 1)], list(range(256)))]
        if at_b < len(b):
            entries.append(StepEntry(sb, b[at_b:at_b + 173], []))
            at_b += 173
        out = r.step(entries)
        got.append(out[1:257].clone())
        at_c += 1
    for s in (sa, sb, sc):
        r.release(s)
    mixed = torch.cat(got)
    assert torch.equal(whole, mixed)
    del whole, mixed, got
    # the scheduler's workload (configs[4]: 8 requests, prompts of 64-1,024 tokens, portions of 256 beside decode tokens)
    new = 24
    ids = [eng.submit_tokens(p, new, SamplingParams(max_new_tokens=new, stop_token_ids=())) for p in prompts]
    eng.run_all()
    batch = [list(eng.request(i).generated) for i in ids]
    assert all(len(g) == new for g in batch)
    rid = eng.submit_tokens(prompts[1], new, SamplingParams(max_new_tokens=new, stop_token_ids=()))
    eng.run_all()
    assert list(eng.request(rid).generated) == batch[1]
    # and the plain implementation's greedy choice at every one of those steps (request 4: 129 + 24 tokens)
    seq = prompts[4] + batch[4]
    plain = PV.forward(cfg, PV.engine_views(r.model), seq)[len(prompts[4]) - 1:-1]
    for i, tok in enumerate(batch[4]):
        best = int(plain[i].argmax())
        assert tok == best or float(plain[i, best] - plain[i, tok]) < 2e-5 * scale, (i, tok, best)
    eng.close()


def test_full_size_bfloat16_path_against_the_plain_implementation_however_the_work_is_cut():
    """The same at serving precision (tensor-core kernels at the benchmark's shapes): all 1,024
    positions of a prompt, whole, in portions of 512 and of 256, and in ragged portions with the
    last tokens one by one (captured decode steps), each held to the whole-tensor plain
    implementation in float64 over the engine's own weight tensors.  Different cuts take
    different kernels (a step of 512 rows or more runs the shared expert as dense products of its
    own, a smaller one as extra groups of the experts' products) and different tile shapes, so
    rounding differs between cuts as much as bfloat16 rounding differs from exact arithmetic:
    through 24 layers and with logits up to 5 that is more than the element-wise bound of the
    small models for some rows.  Every cut must therefore agree with the exact logits equally
    well - every row points the same way, the mean error is below one bfloat16 step of the
    largest logit - and two cuts
    must not differ from each other in more rows than they differ from the exact logits."""
    from cajeta_llm_b200.engine.llm_engine import LlmEngine
    from cajeta_llm_b200.engine.options import EngineOptions
    from cajeta_llm_b200.engine.step import StepEntry
    need_free_memory(60e9, "full-size bfloat16 test")
    cfg = FULL_SIZE
    prompt = helpers.random_tokens(cfg["vocab_size"], 1024, seed=1224)
    eng = LlmEngine.load(EngineOptions(config=cfg, random_weights=True, seed=1, dtype="bfloat16", ctx=1280, max_seqs=4,
                                       block_tokens=16, max_batch_tokens=2048))
    check_drawn_tensors(eng.runner.model, seed=1)
    r = eng.runner
    exact, margins, _ = oracle_for(eng, cfg, prompt)
    exact = exact.float()

    def all_logits(cuts):
        s, pos, outs = r.admit(), 0, []
        for n in cuts:
            outs.append(r.step([StepEntry(s, prompt[pos:pos + n], list(range(n)))]).clone())
            pos += n
        r.release(s)
        return torch.cat(outs)

    tol = helpers.TOL["bfloat16"]

    def rows_apart(a, b):
        return int(((a - b).abs() > tol["atol"] + tol["rtol"] * a.abs()).any(dim=1).sum())

    results = {}
    for cuts in ([1024], [512, 512], [256, 256, 256, 256], [700, 2, 61, 237] + [1] * 24):
        got = all_logits(cuts)
        assert torch.isfinite(got).all() and float(got.abs().max()) > 0.1
        cosine = torch.nn.functional.cosine_similarity(exact, got, dim=1)
        assert float(cosine.min()) >= helpers.TIE_COSINE, (cuts[:4], float(cosine.min()))
        err = float((exact - got).abs().mean())
        assert err <= 2.0 ** -8 * float(exact.abs().max()), cuts[:4]
        top, best = got.argmax(dim=1), exact.argmax(dim=1)
        results[tuple(cuts)] = (got, rows_apart(exact, got))
        print(f"\nfull size bfloat16, cuts {cuts[:4]}...: mean |diff| {err:.4f}, smallest cosine {float(cosine.min()):.5f}, "
              f"rows outside the small models' bound {results[tuple(cuts)][1]} of 1024, top choice differs in {int((top != best).sum())}")
    whole, whole_apart = results[(1024,)]
    for cuts, (got, apart) in results.items():
        assert rows_apart(whole, got) <= max(whole_apart, apart), (cuts[:4], rows_apart(whole, got), whole_apart, apart)
    r.check_waits()
    eng.close()
