"""Command line, in the reference's manner.

The reference's CLI (cli/Main.cajeta:21-31, cli/CliArgs.cajeta:77-217) has the verbs
``run`` and ``chat`` and maps each flag onto an engine option or a sampling parameter;
an unknown flag and a missing value are errors.  This engine keeps the names and
meanings of the flags it has a counterpart for:

    python -m cajeta_llm_b200 run --model DIR --prompt "1 2 3" [-n 128 --temp 0.7
        --top-k 40 --top-p 0.95 --seed 42 --repeat-penalty 1.1 --ctx 4096
        --max-seqs 4 --block-size 16 --chunk 128 --device cuda:0 --verbose]

It works on token ids (there is no tokenizer): ``--prompt`` takes the ids separated by
spaces or commas, and the generated ids are printed, followed by
``[N tokens, budget | eos | stop | cancel]`` as the reference prints it
(cli/Main.cajeta:83-122).  ``--prompt`` may be given several times; the prompts are then
served together.  ``chat`` needs a chat template and a tokenizer and is not offered.
Added flags: ``--dtype bfloat16|float32``, ``--max-batch-tokens N``, ``--num-blocks N``,
``--no-warmup`` (skip the throw-away steps at load).

A second verb writes a random-weights model folder from a configuration and a seed:

    python -m cajeta_llm_b200 random-weights --config config.json --seed 1 --out DIR
        [--store-dtype bfloat16|float32]
"""
from __future__ import annotations

import json
import sys
from typing import List, Optional, Sequence


class CliError(Exception):
    pass


def _need_val(args: Sequence[str], i: int, flag: str) -> int:
    if i + 1 >= len(args):
        raise CliError(f"cajeta-llm: {flag} needs a value")
    return i + 1


def _ids(text: str) -> List[int]:
    try:
        return [int(t) for t in text.replace(",", " ").split()]
    except ValueError:
        raise CliError(f"cajeta-llm: --prompt takes token ids separated by spaces or commas, found '{text}'") from None


def parse_run(args: Sequence[str]):
    from .engine.options import EngineOptions
    from .sampling.params import SamplingParams

    o = EngineOptions()
    prompts: List[List[int]] = []
    max_new = 128
    sp = dict(temperature=0.0, top_k=0, top_p=0.0, repeat_penalty=1.0, seed=0)
    i = 0
    while i < len(args):
        a = args[i]
        if a == "--model":
            i = _need_val(args, i, a); o.model = args[i]
        elif a == "--prompt":
            i = _need_val(args, i, a); prompts.append(_ids(args[i]))
        elif a == "--device":
            i = _need_val(args, i, a); o.device = args[i]
        elif a == "--ctx":
            i = _need_val(args, i, a); o.ctx = int(args[i])
        elif a == "-n":
            i = _need_val(args, i, a); max_new = int(args[i])
        elif a == "--temp":
            i = _need_val(args, i, a); sp["temperature"] = float(args[i])
        elif a == "--top-k":
            i = _need_val(args, i, a); sp["top_k"] = int(args[i])
        elif a == "--top-p":
            i = _need_val(args, i, a); sp["top_p"] = float(args[i])
        elif a == "--seed":
            i = _need_val(args, i, a); sp["seed"] = int(args[i])
        elif a == "--repeat-penalty":
            i = _need_val(args, i, a); sp["repeat_penalty"] = float(args[i])
        elif a == "--max-seqs":
            i = _need_val(args, i, a); o.max_seqs = int(args[i])
        elif a == "--block-size":
            i = _need_val(args, i, a); o.block_tokens = int(args[i])
        elif a == "--chunk":
            i = _need_val(args, i, a); o.chunk = int(args[i])
        elif a == "--dtype":
            i = _need_val(args, i, a); o.dtype = args[i]
        elif a == "--max-batch-tokens":
            i = _need_val(args, i, a); o.max_batch_tokens = int(args[i])
        elif a == "--num-blocks":
            i = _need_val(args, i, a); o.num_blocks = int(args[i])
        elif a == "--no-warmup":
            o.warmup = False      # a bare toggle: the first request then pays for cold kernels and graph capture
        elif a == "--verbose":
            o.verbose = True      # a bare toggle: it takes no value
        else:
            raise CliError(f"cajeta-llm: unknown flag '{a}'")
        i += 1
    if not o.model:
        raise CliError("cajeta-llm: --model is required")
    if not prompts:
        raise CliError("cajeta-llm: --prompt is required (token ids)")
    params = SamplingParams(max_new_tokens=max_new, **sp)
    return o, prompts, params


def cmd_run(args: Sequence[str]) -> int:
    from .engine.llm_engine import LlmEngine

    o, prompts, params = parse_run(args)
    engine = LlmEngine.load(o)
    if o.verbose:
        print(f"[cajeta-llm] {engine.config.architecture}: {engine.model().weight_bytes() / 1e6:.1f} MB of weights, "
              f"dtype {o.dtype}, eog {list(engine.eog_tokens())}", file=sys.stderr)
    ids = [engine.submit_tokens(p, params.max_new_tokens, params) for p in prompts]
    engine.run_all()
    for rid in ids:
        r = engine.request(rid)
        shown = [t for t in r.generated if not engine.is_eog(t)]      # end markers are not printed
        print(" ".join(str(t) for t in shown))
        print(f"[{len(r.generated)} tokens, {r.finish_reason.value}]")
    if o.verbose:
        c = engine.scheduler().counters
        print(f"[cajeta-llm] steps {c.steps}, admitted {c.admitted}, preempted {c.preempted}, "
              f"prefill rows {c.prefill_rows}, decode rows {c.decode_rows}", file=sys.stderr)
    engine.close()
    return 0


def cmd_random_weights(args: Sequence[str]) -> int:
    import torch

    from .config.base import parse_config_dict
    from .engine.model import build_model
    from .parts.base import Runtime
    from .weights.sources import write_model_folder

    config_path, out, seed, store = None, None, 0, "bfloat16"
    i = 0
    while i < len(args):
        a = args[i]
        if a == "--config":
            i = _need_val(args, i, a); config_path = args[i]
        elif a == "--out":
            i = _need_val(args, i, a); out = args[i]
        elif a == "--seed":
            i = _need_val(args, i, a); seed = int(args[i])
        elif a == "--store-dtype":
            i = _need_val(args, i, a); store = args[i]
        else:
            raise CliError(f"cajeta-llm: unknown flag '{a}'")
        i += 1
    if not config_path or not out:
        raise CliError("cajeta-llm: random-weights needs --config and --out")
    if store not in ("bfloat16", "float32"):
        raise CliError(f"cajeta-llm: --store-dtype takes bfloat16 or float32, not '{store}'")
    with open(config_path, "r", encoding="utf-8") as f:
        config = parse_config_dict(json.load(f), config_path)
    schema = build_model(config, Runtime("float32", device="cpu")).params()
    write_model_folder(out, config, schema, seed, torch.bfloat16 if store == "bfloat16" else torch.float32)
    print(f"wrote {out} ({len(schema)} tensors, seed {seed}, {store})")
    return 0


def main(argv: Optional[Sequence[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] in ("-h", "--help"):
        print(__doc__)
        return 0
    verb, rest = argv[0], argv[1:]
    try:
        if verb == "run":
            return cmd_run(rest)
        if verb == "random-weights":
            return cmd_random_weights(rest)
        if verb == "chat":
            raise CliError("cajeta-llm: chat needs a tokenizer and a chat template; this engine works on token ids (use run)")
        raise CliError(f"cajeta-llm: unknown verb '{verb}'; verbs: run, random-weights")
    except CliError as e:
        print(str(e), file=sys.stderr)
        return 2


if __name__ == "__main__":
    sys.exit(main())
