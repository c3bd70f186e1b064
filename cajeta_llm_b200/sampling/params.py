"""Per-request sampling parameters, with the reference's names and meanings.

gen/SampleParams.cajeta:26-41: ``temperature`` 0 = greedy argmax, otherwise the logits
are divided by it; ``top_k`` 0 = off; ``top_p`` <= 0 or >= 1 = off; ``repeat_penalty``
1 = off (a previously EMITTED token's logit is divided by it when positive, multiplied
otherwise); ``seed`` starts the request's own random stream; ``stop_token_ids`` None
means the engine's end-of-generation set.  Stop strings need a tokenizer and are not
part of this engine (it works on token ids).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 0.0
    repeat_penalty: float = 1.0
    seed: int = 0
    stop_token_ids: Optional[Tuple[int, ...]] = None
    max_new_tokens: int = 128

    def __post_init__(self):
        if self.temperature < 0.0:
            raise ValueError(f"temperature must be >= 0, found {self.temperature}")
        if self.top_k < 0:
            raise ValueError(f"top_k must be >= 0, found {self.top_k}")
        if self.repeat_penalty <= 0.0:
            raise ValueError(f"repeat_penalty must be > 0, found {self.repeat_penalty}")
        if self.max_new_tokens < 1:
            raise ValueError(f"max_new_tokens must be >= 1, found {self.max_new_tokens}")
        if self.stop_token_ids is not None:
            object.__setattr__(self, "stop_token_ids", tuple(int(t) for t in self.stop_token_ids))

    @property
    def is_greedy(self) -> bool:
        """The choice is the argmax of the raw logits (gen/Sampler.cajeta:44-47)."""
        return self.temperature == 0.0 and self.repeat_penalty == 1.0
