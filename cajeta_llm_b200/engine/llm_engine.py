"""The engine's public face, in the manner of the reference's ``LlmEngine``.

LlmEngine.cajeta:165-547: ``load(opts)`` opens the checkpoint, reads the configuration,
builds the model, binds the weights and creates the scheduler; then
``submit_tokens`` / ``run_all`` / ``step_once`` / ``request`` / ``eog_tokens`` /
``is_eog`` / ``cancel`` / ``set_sink`` / ``close``.  This engine works on token ids:
there is no tokenizer, so ``submit_text`` and stop strings are not offered.  The
end-of-generation set is the configuration's ``eos_token_id`` (and that of
``generation_config.json`` when the folder has one); it is the default stop set
(LlmEngine.cajeta:388-475).
"""
from __future__ import annotations

import json
import os
from typing import Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import torch

from ..config.base import ModelConfig, load_config, parse_config_dict
from ..parts.base import Runtime
from ..sampling.params import SamplingParams
from ..sampling.sampler import BatchSampler
from .model import Model, build_model, load_model, random_model
from .options import EngineOptions
from .scheduler import FinishReason, Request, Scheduler
from .step import ModelRunner


class LlmEngine:
    def __init__(self, options: EngineOptions, model: Model, config: ModelConfig, eog: Tuple[int, ...]):
        self.options = options
        self._model = model
        self.config = config
        self._eog = tuple(sorted(set(eog)))
        self.runner = ModelRunner(model, page_tokens=options.block_tokens, max_seqs=options.max_seqs,
                                  max_tokens_per_seq=options.ctx,
                                  num_pages=options.num_blocks if options.num_blocks > 0 else None,
                                  cuda_graphs=options.cuda_graphs,
                                  max_step_tokens=min(options.max_batch_tokens, options.chunk or options.max_batch_tokens))
        self.sampler = BatchSampler(model.runtime.device, model.vocab)
        self._scheduler = Scheduler(self.runner, self.sampler, max_batch_tokens=options.max_batch_tokens,
                                    chunk=options.chunk, eog_token_ids=self._eog, lookahead=options.lookahead)
        self._closed = False
        if options.warmup:
            self._warm_up()

    def _warm_up(self) -> None:
        """A throw-away prompt portion and decode steps right after load, as the reference does
        (LlmEngine.cajeta:294-324): kernels are loaded and configured, and on the bfloat16 path
        the decode graphs of the batch sizes 1, 2, 4, ... up to ``max_seqs`` are captured, before
        the first request arrives.  Everything it held is given back."""
        from .step import OutOfPages, StepEntry
        r = self.runner
        n = min(16, self.options.ctx - 8)
        if n < 1:
            return
        sizes = sorted({b for b in (1, 2, 4, 8, 16, 32, 64, 128, 256) if b <= self.options.max_seqs} | {self.options.max_seqs})
        if not r.cuda_graphs:
            sizes = sizes[:1]
        slots: List[int] = []
        try:
            for size in sizes:
                fresh = []
                while len(slots) + len(fresh) < size:
                    s = r.admit()
                    if s is None:
                        break
                    fresh.append(s)
                if fresh:
                    r.step([StepEntry(s, [0] * n, []) for s in fresh])
                    slots += fresh
                if any(r.cache.length(s) + 2 > self.options.ctx for s in slots):
                    break
                for _ in range(2):                     # the first captures this batch size's graph, the second replays it
                    r.step([StepEntry(s, [0], [0]) for s in slots])
        except OutOfPages:
            pass                                       # a pool too small for all sizes: what fitted is warm
        finally:
            for s in slots:
                r.release(s)
            torch.cuda.synchronize()

    # -- loading ---------------------------------------------------------------------
    @classmethod
    def load(cls, options: EngineOptions) -> "LlmEngine":
        options.validate()
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device: this engine runs on a B200 and has no CPU path")
        runtime = Runtime(dtype=options.dtype, device=options.device)
        eog: List[int] = []
        if options.random_weights or not options.model:
            config = options.config
            if config is None:
                config = load_config(options.model)
            elif isinstance(config, dict):
                config = parse_config_dict(config)
            model = random_model(config, runtime, options.seed)
        else:
            model, config = load_model(options.model, runtime)
            gen = os.path.join(options.model, "generation_config.json")
            if os.path.isfile(gen):
                with open(gen, "r", encoding="utf-8") as f:
                    e = json.load(f).get("eos_token_id")
                if isinstance(e, int):
                    eog.append(e)
                elif isinstance(e, list):
                    eog.extend(int(x) for x in e)
        eog.extend(model.plan.eog_token_ids)
        return cls(options, model, config, tuple(eog))

    # -- requests --------------------------------------------------------------------
    def submit_tokens(self, ids: Sequence[int], max_new: int = 128, params: Optional[SamplingParams] = None) -> int:
        """Queue a request of prompt token ids; returns its id."""
        p = params or SamplingParams()
        if p.max_new_tokens != max_new:
            p = SamplingParams(temperature=p.temperature, top_k=p.top_k, top_p=p.top_p, repeat_penalty=p.repeat_penalty,
                               seed=p.seed, stop_token_ids=p.stop_token_ids, max_new_tokens=max_new)
        if len(ids) + max_new > self.options.ctx:
            raise ValueError(f"prompt of {len(ids)} tokens plus {max_new} new ones exceeds ctx {self.options.ctx}")
        return self._scheduler.submit(ids, p)

    def submit_text(self, prompt: str, *args, **kwargs) -> int:
        raise NotImplementedError("this engine works on token ids and has no tokenizer; use submit_tokens")

    def run_all(self, max_steps: int = 0) -> int:
        return self._scheduler.run_all(max_steps)

    def step_once(self) -> int:
        return self._scheduler.step_once()

    def request(self, request_id: int) -> Request:
        return self._scheduler.request(request_id)

    def cancel(self, request_id: int) -> bool:
        return self._scheduler.cancel(request_id)

    def set_sink(self, sink: Optional[Callable[[int, int], None]]) -> None:
        """``sink(request_id, token)`` is called for every emitted token, before the next step."""
        self._scheduler.sink = sink

    def eog_tokens(self) -> Tuple[int, ...]:
        return self._eog

    def is_eog(self, token: int) -> bool:
        return token in self._eog

    def scheduler(self) -> Scheduler:
        return self._scheduler

    def model(self) -> Model:
        return self._model

    def generate(self, prompts: Sequence[Sequence[int]], params: Optional[SamplingParams | Sequence[SamplingParams]] = None
                 ) -> List[List[int]]:
        """Host token ids in, generated token ids out, for a batch of prompts."""
        if params is None or isinstance(params, SamplingParams):
            plist = [params or SamplingParams()] * len(prompts)
        else:
            plist = list(params)
        ids = [self.submit_tokens(p, sp.max_new_tokens, sp) for p, sp in zip(prompts, plist)]
        self.run_all()
        return [list(self.request(i).generated) for i in ids]

    def close(self) -> None:
        if self._closed:
            return
        self._closed = True
        self._scheduler = None
        self.runner = None
        self._model = None
        torch.cuda.empty_cache()
