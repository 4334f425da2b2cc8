"""Engine options: the arguments of the reference's `LLMEngine` (fusezap/serve/engine.py:367-369) and `SchedulerConfig`
(fusezap/serve/scheduler.py:56-74) as one validated dataclass. Names follow the reference's: `num_blocks`, `block_size`,
`max_num_seqs`, `max_prefill_tokens`, `max_model_len`, `max_num_batched_tokens`, `prefill_first`."""
from __future__ import annotations
from dataclasses import dataclass

DTYPES = ("float32", "bfloat16")


@dataclass
class EngineConfig:
    dtype: str = "bfloat16"
    num_blocks: int = 1024                       # pages of the full-attention group (window groups are sized from it)
    block_size: int = 16                         # tokens per page
    max_num_seqs: int = 32                       # live requests = decode rows per step
    max_prefill_tokens: int = 2048               # prompt tokens per step
    max_num_batched_tokens: int | None = None    # all tokens per step; default max_num_seqs + max_prefill_tokens
    max_model_len: int = 2048                    # positions per request (prompt + generated)
    prefill_first: int = 0                       # up to this many consecutive steps of prompt portions alone while
                                                 # others decode (0: portions and decoded tokens share every step)
    cuda_graphs: bool = True                     # replay decode steps from captured CUDA graphs
    graph_rows: int = 256                        # other steps of at most this many rows are captured too, by their sizes
    lookahead: bool = True                       # launch the next decode step before reading the last one's tokens
    seed: int = 0

    def __post_init__(self) -> None:
        if self.dtype not in DTYPES:
            raise ValueError(f"dtype {self.dtype!r} is not one of {DTYPES}")
        for k in ("num_blocks", "block_size", "max_num_seqs", "max_prefill_tokens", "max_model_len"):
            v = getattr(self, k)
            if not isinstance(v, int) or v <= 0:
                raise ValueError(f"{k} must be a positive integer, got {v!r}")
        if self.max_num_batched_tokens is not None and self.max_num_batched_tokens <= 0:
            raise ValueError(f"max_num_batched_tokens must be positive, got {self.max_num_batched_tokens}")
        if self.prefill_first < 0:
            raise ValueError("prefill_first must be >= 0")
        if not isinstance(self.graph_rows, int) or self.graph_rows < 0:
            raise ValueError(f"graph_rows must be an integer >= 0, got {self.graph_rows!r}")

    @property
    def token_budget(self) -> int:
        return self.max_num_batched_tokens or (self.max_num_seqs + self.max_prefill_tokens)
