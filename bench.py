#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at Qwen1.5-MoE-A2.7B sizes on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference]

A "step" is one decode step of a batch of 8 requests (each holding a 512-token prompt
in a 4096-token context, 16-token pages), random weights, random token ids.  One JSON
line is printed:

* ``value``: decoded tokens a second, timed on the device over K steps after W warm-up
  steps (the step function plus the greedy pick).  The K-step region is repeated, every
  repeat from 512-token contexts again, until at least ``--min-seconds`` of device time have
  been timed; ``value`` and ``ms_per_step`` are the median repeat, ``repeats`` says how many
  there were and how far apart the fastest and the slowest lie;
* ``e2e``: the same through ``LlmEngine`` (host token ids in, host token ids out every
  step, scheduler included);
* ``prefill``: one step of 2,048 prompt tokens, with the fraction of the bf16 peak, the
  compute floor and the floor of streaming every weight once;
* ``roofline``: bytes a decode step must read (every weight it uses once, the cache of
  the live requests) over its time, against the measured copy bandwidth; ``rooflines`` has
  the same for the other points;
* ``points``: decode tokens a second at batch 1 and 64, at batch 8 with contexts of 2,048 and
  4,096 tokens, prefill tokens a second at 512, 4,096 and 8,192 tokens;
* ``kernels``: where a decode step's and the 2,048-token prefill's time goes by class of work
  (launches serialised, each followed by an event on the stream behind a queue that was
  filled while the device was kept waiting), with each class's bytes or flops and its
  fraction of the measured peak.

Every timed region reads far more than the 126 MB of L2 (a decode step reads the
model's weights, GBs), so no L2 flush is needed between iterations.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# the headline configuration: Qwen1.5-MoE-A2.7B sizes
A27B = {
    "architectures": ["Qwen2MoeForCausalLM"], "hidden_size": 2048, "intermediate_size": 5632, "num_hidden_layers": 24,
    "num_attention_heads": 16, "num_key_value_heads": 16, "head_dim": 128, "vocab_size": 151936,
    "max_position_embeddings": 8192, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "num_experts": 60,
    "num_experts_per_tok": 4, "moe_intermediate_size": 1408, "shared_expert_intermediate_size": 5632,
    "norm_topk_prob": False, "decoder_sparse_step": 1, "mlp_only_layers": [], "tie_word_embeddings": False,
    "use_sliding_window": False,
}
# the larger configuration: Qwen2-57B-A14B sizes (about 115 GB of bf16 weights); not the default run
Q57B = {
    "architectures": ["Qwen2MoeForCausalLM"], "hidden_size": 3584, "intermediate_size": 18944, "num_hidden_layers": 28,
    "num_attention_heads": 28, "num_key_value_heads": 4, "head_dim": 128, "vocab_size": 151936,
    "max_position_embeddings": 8192, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "num_experts": 64,
    "num_experts_per_tok": 8, "moe_intermediate_size": 2560, "shared_expert_intermediate_size": 20480,
    "norm_topk_prob": False, "decoder_sparse_step": 1, "mlp_only_layers": [], "tie_word_embeddings": False,
    "use_sliding_window": False,
}
MODELS = {"a2.7b": ("Qwen1.5-MoE-A2.7B sizes", A27B), "57b-a14b": ("Qwen2-57B-A14B sizes", Q57B)}
CTX, PROMPT, PAGE, BATCH, PREFILL_TOKENS = 4096, 512, 16, 8, 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                p = json.load(f)
            return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]), "source": "measured"}
        except (OSError, ValueError, KeyError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def model_numbers(cfg, n_layers):
    """Bytes and flops from the configuration (bf16 weights), whole and by class of work."""
    H, V = cfg["hidden_size"], cfg["vocab_size"]
    heads, hd = cfg["num_attention_heads"], cfg["head_dim"]
    qd = heads * hd
    kvd = cfg["num_key_value_heads"] * hd
    E, k, Ie, Is = cfg["num_experts"], cfg["num_experts_per_tok"], cfg["moe_intermediate_size"], cfg["shared_expert_intermediate_size"]
    per_layer_fixed = 2 * (H * (qd + 2 * kvd) + qd * H + 3 * H * Is) + 4 * (E * H + H + (qd + 2 * kvd) + 2 * H)
    per_expert = 2 * 3 * H * Ie
    head = 2 * V * H + 4 * H
    kv_per_token = 2 * 2 * kvd * n_layers

    def prefill_flops(T):
        lin = 2 * T * (H * (qd + 2 * kvd) + qd * H + E * H + k * 3 * H * Ie + 3 * H * Is + H)
        att = 4 * heads * hd * T * (T + 1) // 2
        return n_layers * (lin + att) + 2 * V * H

    def prefill_weight_bytes(T):
        """Every weight a prefill of T tokens touches, once (all experts from a few hundred tokens on)."""
        touched = E if T * k >= 4 * E else min(E, T * k)
        return n_layers * (per_layer_fixed + touched * per_expert) + head

    def classes(T, ctx_tokens, experts_touched):
        """Per layer (head and embedding: per step): bytes that must move and flops, by class of
        work, for a step of T rows whose requests hold ``ctx_tokens`` cached tokens in all and
        touch ``experts_touched`` routed experts a layer.  Weights bf16, the residual stream and
        the products' float32 results 4 bytes, activations between kernels 2."""
        slots = T * k
        return {
            "rmsnorm": (2 * (T * H * 4 + T * H * 2) + 2 * H * 4, 2 * 4 * T * H),
            "qkv": (2 * H * (qd + 2 * kvd) + T * H * 2 + T * (qd + 2 * kvd) * 4, 2 * T * H * (qd + 2 * kvd)),
            "rope + cache write": (T * (qd + 2 * kvd) * 4 + T * (qd + 2 * kvd) * 2, 6 * T * (qd + kvd)),
            "attention": (2 * 2 * kvd * ctx_tokens + 2 * T * qd * 2, 0),          # flops depend on the shape of the step: see below
            "o": (2 * qd * H + T * qd * 2 + T * H * 4, 2 * T * qd * H),
            "router": (4 * (E + 1) * H + T * H * 4, 2 * T * (E + 1) * H),
            "grouping": (3 * slots * 4, 0),
            "row gather": (2 * slots * H * 2, 0),
            "experts gate/up": (experts_touched * 2 * 2 * H * Ie + slots * H * 2 + slots * Ie * 2, 2 * 2 * slots * H * Ie),
            "experts down": (experts_touched * 2 * H * Ie + slots * Ie * 2 + slots * H * 4, 2 * slots * H * Ie),
            "shared gate/up": (2 * 2 * H * Is + T * H * 2 + T * Is * 2, 2 * 2 * T * H * Is),
            "shared down": (2 * H * Is + T * Is * 2 + T * H * 4, 2 * T * H * Is),
            "combine": (slots * H * 4 + 2 * T * H * 4, 2 * slots * H),
            "head": (head, 2 * V * H),
            "embedding": (H * 2 + H * 4, 0),
        }

    return dict(per_layer_fixed=per_layer_fixed, per_expert=per_expert, head=head, kv_per_token=kv_per_token,
                prefill_flops=prefill_flops, prefill_weight_bytes=prefill_weight_bytes, classes=classes, H=H,
                attention_flops=lambda T: 4 * heads * hd * T * (T + 1) // 2)


def timeline(runner, batch, prompts, rng, vocab, n_layers) -> int:
    """One replayed decode step of ``batch`` requests under the profiler: launches overlap (a kernel's
    blocks are set up while the one before drains), so a kernel's duration contains its wait; what
    adds up to the step is how much later each kernel ENDS than every kernel before it."""
    import collections

    import torch
    from torch.profiler import ProfilerActivity, profile

    from cajeta_llm_b200.engine.step import StepEntry
    slots = [runner.admit() for _ in range(batch)]
    for i in range(0, batch, 8):
        runner.step([StepEntry(s, p, []) for s, p in zip(slots[i:i + 8], prompts(len(slots[i:i + 8]), PROMPT))])

    def one():
        return runner.step([StepEntry(s, [int(rng.integers(0, vocab))], [0]) for s in slots])

    for _ in range(6):
        one()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(3):
            one()
        torch.cuda.synchronize()
    events = sorted((e for e in prof.events() if e.device_type is not None and "Memcpy" not in e.name and "Memset" not in e.name
                     and e.device_time_total > 0 and e.time_range is not None), key=lambda e: e.time_range.start)
    first = [i for i, e in enumerate(events) if "embed_gather" in e.name]
    if not first:
        print("no kernel of a step was recorded")
        return 1
    step = events[first[-1]:]
    t0 = step[0].time_range.start

    def short(name):
        for junk in ("void ", "(anonymous namespace)::", "cj::"):
            name = name.replace(junk, "")
        return name.split("(")[0][:56]

    spent, prev_end = collections.OrderedDict(), t0
    for e in step:
        end = e.time_range.end
        a = spent.setdefault(short(e.name), [0, 0.0])
        a[0] += 1
        a[1] += max(0.0, end - prev_end)
        prev_end = max(prev_end, end)
    print(f"decode step, batch {batch}, {n_layers} layers, {PROMPT}-token contexts: {len(step)} kernels, {prev_end - t0:.1f} us")
    for name, (n, us) in spent.items():
        print(f"  {name:58s} x{n:4d}  ends {us:8.1f} us later than what ran before it ({us / max(1, n):6.2f} a launch)")
    for s in slots:
        runner.release(s)
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration has (0 = all)")
    ap.add_argument("--quick", action="store_true", help="the headline and the 2,048-token prefill only")
    ap.add_argument("--no-graphs", action="store_true", help="launch decode steps kernel by kernel (for profilers)")
    ap.add_argument("--model", default="a2.7b", choices=sorted(MODELS), help="layer sizes (default: the headline configuration)")
    ap.add_argument("--min-seconds", type=float, default=2.0,
                    help="device time over which the K-step region is repeated at the headline point (half of it at the other points)")
    ap.add_argument("--batch", type=int, default=BATCH, help="requests of the headline decode run (default 8: the headline)")
    ap.add_argument("--timeline", action="store_true",
                    help="instead of the bench line: where one replayed decode step of --batch requests spends its time, kernel by "
                         "kernel, from the device's own timestamps (how much later each kernel ends than the one before it)")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "jklappenbach/cajeta-llm is cajeta-language source with no Python or C++ build (pip: 'neither setup.py "
                          "nor pyproject.toml found') and the cajeta toolchain is not on this machine"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    warmup = max(3, args.warmup)
    steps = max(1, args.steps)

    import numpy as np
    import torch

    import cajeta_llm_b200  # noqa: F401
    from cajeta_llm_b200.csrc import kernels as K
    from cajeta_llm_b200.engine.llm_engine import LlmEngine
    from cajeta_llm_b200.engine.options import EngineOptions
    from cajeta_llm_b200.engine.step import StepEntry
    from cajeta_llm_b200.sampling.params import SamplingParams

    model_name, model_cfg = MODELS[args.model]
    cfg = dict(model_cfg)
    full_layers = cfg["num_hidden_layers"]
    if args.layers > 0:
        cfg["num_hidden_layers"] = min(args.layers, full_layers)
    n_layers = cfg["num_hidden_layers"]
    pk = peaks()
    nums = model_numbers(cfg, n_layers)
    max_b = 64 if not args.quick else max(BATCH, args.batch)
    longest_prefill = 8192 if not args.quick else PREFILL_TOKENS
    ctx = max(CTX, longest_prefill + 64)
    # pool: 64 requests of 512 + generated tokens, 8 at the full context, or the longest prompt, whichever is largest
    tokens_needed = max(max_b * (PROMPT + warmup + steps + 64), BATCH * (CTX + 64), longest_prefill + 64)
    opts = EngineOptions(config=cfg, random_weights=True, seed=1234, dtype="bfloat16", ctx=ctx, max_seqs=max_b,
                         block_tokens=PAGE, num_blocks=-(-tokens_needed // PAGE) + max_b, max_batch_tokens=8192,
                         cuda_graphs=not args.no_graphs)
    t0 = time.time()
    engine = LlmEngine.load(opts)
    torch.cuda.synchronize()
    load_s = time.time() - t0
    runner = engine.runner
    vocab = cfg["vocab_size"]
    rng = np.random.default_rng(7)

    def prompts(n, length):
        return [rng.integers(0, vocab, size=length).tolist() for _ in range(n)]

    def event_ms(fn, reps=1):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b)

    def decode_run(batch, n_warm, n_steps, min_seconds, prompt_len=PROMPT):
        """Prefill ``batch`` prompts and time ``n_steps`` decode steps on the device after
        ``n_warm`` untimed ones; again from fresh prompts until ``min_seconds`` were timed."""
        picks = torch.empty((batch,), dtype=torch.int32, device=runner.runtime.device)
        per_step = max(1, 8192 // prompt_len)
        times, launches, step_bytes, distinct = [], 0, 0, 0
        while not times or (sum(times) < min_seconds * 1e3 and len(times) < 200):
            slots = [runner.admit() for _ in range(batch)]
            ps = prompts(batch, prompt_len)
            for i in range(0, batch, per_step):
                runner.step([StepEntry(s, p, []) for s, p in zip(slots[i:i + per_step], ps[i:i + per_step])])
            toks = rng.integers(0, vocab, size=(n_warm + n_steps, batch))

            def one(i):
                logits = runner.step([StepEntry(s, [int(toks[i, j])], [0]) for j, s in enumerate(slots)])
                K.argmax(logits, picks)

            for i in range(n_warm):
                one(i)
            launches0 = K.launches
            it = iter(range(n_warm, n_warm + n_steps))
            times.append(event_ms(lambda: one(next(it)), reps=n_steps))
            launches = K.launches - launches0
            if not step_bytes:
                # bytes a step like the timed ones has to read: one more step, launched kernel by kernel
                # so that it can say which experts its rows picked (a replayed graph keeps that to itself)
                dump = {}
                extra = rng.integers(0, vocab, size=batch)
                runner.step([StepEntry(s, [int(extra[j])], [0]) for j, s in enumerate(slots)], routing_dump=dump)
                distinct = sum(int(torch.unique(sel).numel()) for sel, _ in dump.values())
                ctx_len = prompt_len + n_warm + n_steps
                step_bytes = (n_layers * nums["per_layer_fixed"] + distinct * nums["per_expert"] + nums["head"]
                              + batch * ctx_len * nums["kv_per_token"] + batch * nums["H"] * 2)
            for s in slots:
                runner.release(s)
        ms = statistics.median(times)
        gbs = step_bytes / (ms / n_steps / 1e3) / 1e9
        return dict(ms_per_step=ms / n_steps, tok_s=batch * n_steps / (ms / 1e3), step_bytes=step_bytes, launches=launches,
                    distinct_experts=distinct, repeats=len(times), fastest_ms_per_step=min(times) / n_steps,
                    slowest_ms_per_step=max(times) / n_steps,
                    roofline={"bound": "hbm", "achieved": gbs, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": gbs / pk["hbm_gbs"]})

    def prefill_run(tokens, reps=5):
        def once():
            s = runner.admit()
            p = prompts(1, tokens)[0]
            ms = event_ms(lambda: runner.step([StepEntry(s, p, [tokens - 1])]))
            runner.release(s)
            return ms

        for _ in range(3):
            once()
        ms = statistics.median(once() for _ in range(reps))
        flops = nums["prefill_flops"](tokens)
        wbytes = nums["prefill_weight_bytes"](tokens)
        return {"value": tokens / (ms / 1e3), "tokens": tokens, "ms": ms,
                "frac": flops / (ms / 1e3) / (pk["bf16_tflops"] * 1e12),
                "compute_floor_ms": flops / (pk["bf16_tflops"] * 1e12) * 1e3,
                "weight_stream_floor_ms": wbytes / (pk["hbm_gbs"] * 1e9) * 1e3}

    def breakdown(entries_of, rows, ctx_tokens, prefill_rows=0):
        """Device time of one step by class of work, launches serialised.  The step is launched
        kernel by kernel with an event behind each launch, into a queue that is filled while the
        device is kept waiting (so that the host's launch cost is not in the figures)."""
        for _ in range(2):
            slots, entries = entries_of()
            runner.step(entries, routing_dump={})          # kernel by kernel; also warms what this shape needs
            for s in slots:
                runner.release(s)
        slots, entries = entries_of()
        torch.cuda.synchronize()
        torch.cuda._sleep(60_000_000)                      # ~30 ms: longer than the host needs to queue the step
        first = torch.cuda.Event(enable_timing=True)
        first.record()
        K.start_trace()
        dump = {}
        runner.step(entries, routing_dump=dump)
        trace = K.stop_trace()
        torch.cuda.synchronize()
        touched = sum(int(torch.unique(sel).numel()) for sel, _ in dump.values()) / max(1, n_layers)
        for s in slots:
            runner.release(s)
        spent, prev = {}, first
        for label, ev in trace:
            spent[label] = spent.get(label, 0.0) + prev.elapsed_time(ev) * 1e3
            prev = ev
        need = nums["classes"](rows, ctx_tokens, touched)
        out = {}
        for label, us in sorted(spent.items(), key=lambda kv: -kv[1]):
            per_step = label in ("head", "embedding")
            n = 1 if per_step else n_layers
            by, fl = need.get(label, (0, 0))
            if label == "attention" and prefill_rows:
                fl = nums["attention_flops"](prefill_rows)
            if label == "head":
                fl = fl * 1                                     # one wanted row
            t = us / n * 1e-6
            entry = {"us": round(us / n, 2), "per": "step" if per_step else "layer", "bytes": int(by), "flops": int(fl)}
            if by:
                entry["hbm_frac"] = round(by / t / (pk["hbm_gbs"] * 1e9), 3)
            if fl:
                entry["bf16_frac"] = round(fl / t / (pk["bf16_tflops"] * 1e12), 3)
            out[label] = entry
        out["_sum_us_per_step"] = round(sum(spent.values()), 1)
        return out

    if args.timeline:
        return timeline(runner, args.batch, prompts, rng, vocab, n_layers)

    # ---- headline: batch 8 -------------------------------------------------------------
    clocks = ClockSampler()
    clocks.start()                      # from before the warm-up on, so that a short region has samples too
    time.sleep(0.3)                     # nvidia-smi needs a moment to come up
    main_run = decode_run(args.batch, warmup, steps, args.min_seconds)
    clock_info = clocks.stop()
    if clock_info.get("sm_mhz"):
        clock_info["ms_per_step_x_sm_mhz"] = main_run["ms_per_step"] * clock_info["sm_mhz"]

    # ---- prefill of 2,048 tokens -------------------------------------------------------
    prefill = prefill_run(PREFILL_TOKENS)

    points, rooflines, kernels = {}, {}, {}
    e2e = None
    if not args.quick:
        short = max(8, steps // 2)
        for name, b, plen in (("decode_b1", 1, PROMPT), ("decode_b64", 64, PROMPT), ("decode_b8_ctx2048", BATCH, 2048 - warmup - short),
                              ("decode_b8_ctx4096", BATCH, 4096 - warmup - short)):
            r = decode_run(b, warmup, short, args.min_seconds / 2, prompt_len=plen)
            points[name] = r["tok_s"]
            rooflines[name] = dict(r["roofline"], ms_per_step=r["ms_per_step"])
        for tokens in (512, 4096, 8192):
            r = prefill_run(tokens, reps=3)
            points[f"prefill_{tokens}"] = r["value"]
            rooflines[f"prefill_{tokens}"] = {"bound": "bf16 tensor", "frac": r["frac"], "ms": r["ms"],
                                              "compute_floor_ms": r["compute_floor_ms"],
                                              "weight_stream_floor_ms": r["weight_stream_floor_ms"]}

        # ---- where the time goes, by class of work ----------------------------------------
        def decode_entries():
            slots = [runner.admit() for _ in range(BATCH)]
            runner.step([StepEntry(s, p, []) for s, p in zip(slots, prompts(BATCH, PROMPT))])
            return slots, [StepEntry(s, [int(rng.integers(0, vocab))], [0]) for s in slots]

        def prefill_entries():
            s = runner.admit()
            return [s], [StepEntry(s, prompts(1, PREFILL_TOKENS)[0], [PREFILL_TOKENS - 1])]

        kernels["decode_b8"] = breakdown(decode_entries, BATCH, BATCH * (PROMPT + 1))
        kernels["prefill_2048"] = breakdown(prefill_entries, PREFILL_TOKENS, PREFILL_TOKENS, prefill_rows=PREFILL_TOKENS)

        # ---- end to end through the Python entry point -------------------------------------
        eng_steps = steps
        sched = engine.scheduler()

        def through_the_engine(lookahead: bool) -> float:
            """Tokens a second of ``run_all`` over ``eng_steps`` decode steps of BATCH requests."""
            sched.lookahead = lookahead
            rates = []
            while not rates or (sum(r[1] for r in rates) < args.min_seconds / 2 and len(rates) < 100):
                sp = SamplingParams(max_new_tokens=warmup + eng_steps + 4, stop_token_ids=())
                ids = [engine.submit_tokens(p, sp.max_new_tokens, sp) for p in prompts(BATCH, PROMPT)]
                while any(engine.request(i).generated_count() < warmup for i in ids):
                    engine.step_once()
                torch.cuda.synchronize()
                before = sum(engine.request(i).generated_count() for i in ids)
                t1 = time.perf_counter()
                engine.run_all(max_steps=eng_steps)
                torch.cuda.synchronize()
                dt = time.perf_counter() - t1
                made = sum(engine.request(i).generated_count() for i in ids) - before
                for i in ids:
                    engine.cancel(i)
                rates.append((made / dt, dt))
            return statistics.median(r[0] for r in rates)

        # the scheduler that waits for every step's tokens before it launches the next, then the
        # default one, which launches the next decode step before it has read this step's tokens
        # (they stay on the device for the next step; the host still reads every one of them)
        waited = through_the_engine(False)
        ahead = through_the_engine(True)
        # per step: the pinned int32 metadata buffer up (tokens, positions, row->request, request tables, wanted rows,
        # block-table rows) and one int32 token per request down
        width = runner.cache.books.max_pages_per_seq
        h2d = 4 * (3 * BATCH + (BATCH + 1) + 2 * BATCH + BATCH + BATCH * width)
        e2e = {"value": ahead, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * BATCH,
               "value_waiting_for_each_step": waited}

    line = {
        "metric": f"decode tokens/s at batch {args.batch} ({model_name}, bf16, random weights)",
        "value": main_run["tok_s"], "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": main_run["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded random weights (bell-shaped, std 0.02), uniform random token ids",
        "config": {
            "model": model_name, "global_batch": args.batch, "seq_len": CTX, "prompt_len": PROMPT,
            "parallelism": "single GPU", "layers": n_layers, "layers_in_config": full_layers, "hidden": cfg["hidden_size"],
            "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
            "experts": cfg["num_experts"], "top_k": cfg["num_experts_per_tok"], "moe_inter": cfg["moe_intermediate_size"],
            "shared_inter": cfg["shared_expert_intermediate_size"], "vocab": vocab, "page_tokens": PAGE,
            "l2": "inputs larger than L2 (a step reads GBs of weights)", "peaks": pk["source"],
        },
        "repeats": {"n": main_run["repeats"], "fastest_ms_per_step": main_run["fastest_ms_per_step"],
                    "slowest_ms_per_step": main_run["slowest_ms_per_step"], "value_is": "the median repeat of K steps"},
        "prefill": prefill,
        "roofline": main_run["roofline"],
        "rooflines": rooflines,
        "points": points,
        "kernels": kernels,
        "clocks": clock_info,
        "gpu_launches": main_run["launches"],
        "load_s": load_s,
    }
    if e2e is not None:
        line["e2e"] = e2e
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
