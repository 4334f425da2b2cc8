"""Sampling options of a request, with the reference's names and defaults (fusezap/serve/engine.py:39-50)."""
from __future__ import annotations
from dataclasses import dataclass, field


@dataclass
class SamplingParams:
    max_tokens: int = 16                 # new tokens; the request ends with reason "length" when it has them
    temperature: float = 0.0             # 0: greedy
    top_k: int = 0                       # 0: off; 1: greedy
    top_p: float = 1.0                   # 1: off
    repetition_penalty: float = 1.0      # 1: off
    seed: int | None = None              # one random stream per request: its draws do not depend on the batch
    stop_token_ids: list[int] = field(default_factory=list)   # a stop token ends the request and stays in the output
    ignore_eos: bool = False

    def __post_init__(self) -> None:
        if self.max_tokens <= 0:
            raise ValueError(f"max_tokens must be positive, got {self.max_tokens}")
        if self.temperature < 0 or not 0 < self.top_p <= 1 or self.repetition_penalty <= 0 or self.top_k < 0:
            raise ValueError(f"bad sampling params {self}")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0 or self.top_k == 1

    @property
    def on_device(self) -> bool:
        """The device kernels pick the token (greedy, temperature, top-k, top-p); a repetition penalty, which needs the
        request's history, goes to the host."""
        return self.repetition_penalty == 1.0

    @property
    def filtered(self) -> bool:
        """Sampled after a top-k or top-p filter."""
        return not self.greedy and (self.top_k > 0 or self.top_p < 1.0)
