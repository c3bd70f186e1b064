"""Engine options, with the reference's names, meanings and defaults where it has them.

EngineOptions.cajeta:98-122: ``ctx`` 4096 (most tokens one request may hold),
``max_seqs`` 4 (requests live at a time), ``block_tokens`` 16 (tokens per cache page,
``--block-size``), ``chunk`` 0 (0 = portions are cut by the token budget alone, N pins
the largest portion), ``device``.  This engine adds ``dtype`` (``bfloat16`` serving
path or the true ``float32`` path), ``max_batch_tokens`` (token budget of one mixed
step), ``num_blocks`` (cache pages per layer group; 0 = enough for ``max_seqs``
requests of ``ctx`` tokens), the random-weights mode (``random_weights``, ``seed``) and
``warmup`` (the reference always warms at load with one throw-away prefill and decode step,
LlmEngine.cajeta:294-324; here it can be switched off).
The reference's tuning pins, KV store and per-backend switches have no counterpart.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass
class EngineOptions:
    model: str = ""                    # folder with config.json and model.safetensors
    ctx: int = 4096
    max_seqs: int = 4
    block_tokens: int = 16
    chunk: int = 0
    device: str = "cuda:0"
    dtype: str = "bfloat16"
    max_batch_tokens: int = 2048
    num_blocks: int = 0
    random_weights: bool = False       # draw the weights from ``seed`` instead of reading them
    seed: int = 0
    config: Optional[object] = None    # a ModelConfig (or config.json dict) for random weights without a folder
    verbose: bool = False
    cuda_graphs: bool = True           # replay pure decode steps of the bfloat16 path from CUDA graphs
    lookahead: bool = True             # while all requests decode, launch the next step before the host has seen this step's tokens
    warmup: bool = True                # at load: a throw-away prompt portion and decode steps, so that the first request meets warm kernels and captured graphs

    def validate(self) -> None:
        if self.ctx < 1:
            raise ValueError(f"ctx must be >= 1, found {self.ctx}")
        if self.max_seqs < 1:
            raise ValueError(f"max_seqs must be >= 1, found {self.max_seqs}")
        if self.block_tokens < 1:
            raise ValueError(f"block_tokens must be >= 1, found {self.block_tokens}")
        if self.chunk < 0:
            raise ValueError(f"chunk must be >= 0, found {self.chunk}")
        if self.dtype not in ("bfloat16", "float32"):
            raise ValueError(f"dtype must be bfloat16 or float32, found '{self.dtype}'")
        if not self.model and self.config is None:
            raise ValueError("either a model folder or a configuration is required")
