"""Engine options, in one place.

`EngineConfig` is the single object that `LLMEngine`, the scheduler and the command line read. Every option is a field
with its default, its meaning and (where it has one) its command-line flag in the field's metadata; the command line is
generated from these fields, so there is no second copy of a default anywhere. The names and meanings are those of the
reference's `LLMEngine` arguments (fusezap/serve/engine.py:367-369), of its `SchedulerConfig`
(fusezap/serve/scheduler.py:56-74) and of `fusezap serve` (fusezap/serve/cli.py:8-41).

An engine is made with `LLMEngine(model, config)` or with the options as keywords, `LLMEngine(model, num_blocks=...,
max_num_seqs=...)`, which builds the same object.
"""
from __future__ import annotations
import argparse
import dataclasses
from dataclasses import dataclass, field
from typing import Any

DTYPES = ("float32", "bfloat16")
DEFAULT_MODEL_LEN = 2048       # positions a model is loaded for when nothing says otherwise (`fusezap serve`'s default)
DEFAULT_PREFILL_TOKENS = 2048  # prompt tokens per step when max_prefill_tokens is not given


def _opt(default: Any, help: str, flag: str | None = None, **kw: Any) -> Any:
    return field(default=default, metadata={"help": help, "flag": flag, **kw})


@dataclass
class EngineConfig:
    dtype: str = _opt("bfloat16", "compute dtype: bfloat16 (the serving kernels) or float32 (true 32-bit everywhere); "
                                  "auto means bfloat16", "--dtype", choices=("auto",) + DTYPES)
    device: str = _opt("cuda:0", "the GPU", "--device")
    max_model_len: int | None = _opt(None, f"positions per request, prompt and generated (default: what the model was "
                                           f"loaded for; {DEFAULT_MODEL_LEN} on the command line)", "--max-model-len")
    max_num_seqs: int = _opt(32, "requests running at once = decoded rows per step", "--max-num-seqs")
    max_prefill_tokens: int | None = _opt(None, f"prompt tokens per step (default {DEFAULT_PREFILL_TOKENS}, at most "
                                                f"max-model-len)", "--max-prefill-tokens")
    num_blocks: int = _opt(1024, "cache pages, shared by all requests", "--num-blocks")
    block_size: int = _opt(16, "tokens per cache page", "--block-size")
    max_num_batched_tokens: int | None = _opt(None, "all tokens of a step, decoded and prompt (default max-num-seqs + "
                                                    "max-prefill-tokens)", "--max-num-batched-tokens")
    max_prefill_seqs: int | None = _opt(None, "requests that may have a prompt portion in one step (default "
                                              "max-num-seqs)", "--max-prefill-seqs")
    mixed_prefill_tokens: int | None = _opt(None, "prompt tokens per step while some request decodes (default: "
                                                  "max-prefill-tokens)", "--mixed-prefill-tokens")
    prefill_every: int = _opt(1, "while some request decodes, prompt portions only on every n-th step", "--prefill-every")
    prefill_first: int = _opt(0, "up to this many consecutive steps of prompt portions alone while others wait to "
                                 "decode (0: portions and decoded tokens share every step)", "--prefill-first")
    cuda_graphs: bool = _opt(True, "replay captured CUDA graphs instead of launching kernel by kernel", "--no-cuda-graphs")
    graph_rows: int = _opt(256, "steps of at most this many rows that are not pure decode steps replay graphs "
                                "captured by shape (0: off)", "--graph-rows")
    lookahead: bool = _opt(True, "launch the next decode step before reading the last one's tokens", "--no-lookahead")
    profile: bool = _opt(False, "time every kernel class of every step with CUDA events (kernel by kernel, no graphs, "
                                "no lookahead); LLMEngine.profile_report() gives the table", "--profile")

    def __post_init__(self) -> None:
        if self.dtype == "auto":
            self.dtype = "bfloat16"
        if self.dtype not in DTYPES:
            raise ValueError(f"dtype {self.dtype!r} is not one of {DTYPES}")
        for k in ("num_blocks", "block_size", "max_num_seqs", "prefill_every"):
            v = getattr(self, k)
            if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
                raise ValueError(f"{k} must be a positive integer, got {v!r}")
        for k in ("max_model_len", "max_prefill_tokens", "max_num_batched_tokens", "max_prefill_seqs", "mixed_prefill_tokens"):
            v = getattr(self, k)
            if v is not None and (not isinstance(v, int) or isinstance(v, bool) or v <= 0):
                raise ValueError(f"{k} must be a positive integer or None, got {v!r}")
        for k in ("prefill_first", "graph_rows"):
            v = getattr(self, k)
            if not isinstance(v, int) or isinstance(v, bool) or v < 0:
                raise ValueError(f"{k} must be an integer >= 0, got {v!r}")

    # ---- what the options come to for a given model
    def resolved(self, model_max_len: int) -> "EngineConfig":
        """A copy with every `None` replaced by its value for a model loaded for `model_max_len` positions."""
        mml = self.max_model_len if self.max_model_len is not None else model_max_len
        if mml > model_max_len:
            raise ValueError(f"max_model_len {mml} exceeds the length the model was loaded for ({model_max_len})")
        mpt = self.max_prefill_tokens if self.max_prefill_tokens is not None else min(DEFAULT_PREFILL_TOKENS, mml)
        return dataclasses.replace(self, max_model_len=mml, max_prefill_tokens=mpt,
                                   max_prefill_seqs=self.max_prefill_seqs or self.max_num_seqs)

    @property
    def token_budget(self) -> int:
        """Rows of the largest step."""
        if self.max_num_batched_tokens:
            return self.max_num_batched_tokens
        return self.max_num_seqs + (self.max_prefill_tokens or DEFAULT_PREFILL_TOKENS)

    # ---- the command line, generated from the fields
    @classmethod
    def add_arguments(cls, parser: argparse.ArgumentParser) -> None:
        """One flag per field that names one. A flag that is not given leaves the field at its default."""
        for f in dataclasses.fields(cls):
            flag = f.metadata.get("flag")
            if flag is None:
                continue
            kw: dict[str, Any] = {"dest": f.name, "default": argparse.SUPPRESS, "help": f.metadata["help"]}
            if isinstance(f.default, bool):
                kw["action"] = "store_false" if flag.startswith("--no-") else "store_true"
            elif f.metadata.get("choices"):
                kw["choices"] = f.metadata["choices"]
            else:
                kw["type"] = str if isinstance(f.default, str) else int
            parser.add_argument(flag, **kw)

    @classmethod
    def from_arguments(cls, args: argparse.Namespace) -> "EngineConfig":
        names = {f.name for f in dataclasses.fields(cls)}
        return cls(**{k: v for k, v in vars(args).items() if k in names})
