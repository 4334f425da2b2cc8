"""Typed configuration of the dense Llama / Qwen2.5 decoder, read from the architecture's own config.json keys.

Keys and defaults follow the reference's `LlamaConfig.from_hf` (fusezap/serve/models/llama.py:78-100): `rms_norm_eps`
defaults to 1e-6, `max_position_embeddings` to 4096, `head_dim` to hidden_size // num_attention_heads,
`num_key_value_heads` to num_attention_heads; `rope_theta` and the scaling dict may live under `rope_parameters`
(llama.py:86-88); `eos_token_id` may be an int or a list (llama.py:85,93). A sliding window applies only when
`use_sliding_window` is set (llama.py:94, default false for llama / qwen2); with `layer_types` present the window
applies to the layers it names "sliding_attention" (swa.py:24-30), else to every layer (llama.py:99).
Whether q/k/v projections carry a bias is decided by the checkpoint's tensors, not by a key (llama.py:293-295);
`attention_bias` only tells the random-weights writer what to write.
"""
from __future__ import annotations
from dataclasses import dataclass, field, asdict
from typing import Any

from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

ROPE_KINDS = ("default", "linear", "llama3")


@dataclass(frozen=True)
class RopeScaling:
    kind: str = "default"
    factor: float = 1.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    original_max_position_embeddings: int = 0

    @staticmethod
    def from_hf(d: dict | None) -> "RopeScaling":
        if not d:
            return RopeScaling()
        kind = d.get("rope_type", d.get("type")) or "default"
        if kind not in ROPE_KINDS:
            raise NotImplementedError(f"rope_scaling {d!r}: rope type {kind!r} is not supported (have {list(ROPE_KINDS)})")
        if kind == "default":
            return RopeScaling()
        if "factor" not in d:
            raise ValueError(f"rope_scaling {d!r} has no 'factor'")
        if kind == "linear":
            return RopeScaling("linear", float(d["factor"]))
        if "original_max_position_embeddings" not in d:
            raise ValueError(f"rope_scaling {d!r} has no 'original_max_position_embeddings'")
        return RopeScaling("llama3", float(d["factor"]), float(d.get("low_freq_factor", 1.0)),
                           float(d.get("high_freq_factor", 4.0)), int(d["original_max_position_embeddings"]))

    def to_hf(self) -> dict | None:
        if self.kind == "default":
            return None
        if self.kind == "linear":
            return {"rope_type": "linear", "factor": self.factor}
        return {"rope_type": "llama3", "factor": self.factor, "low_freq_factor": self.low_freq_factor,
                "high_freq_factor": self.high_freq_factor,
                "original_max_position_embeddings": self.original_max_position_embeddings}


@dataclass(frozen=True)
class DenseDecoderConfig:
    model_type: str
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    rope_scaling: RopeScaling = field(default_factory=RopeScaling)
    tie_word_embeddings: bool = False
    max_position_embeddings: int = 4096
    eos_token_ids: tuple[int, ...] = ()
    bos_token_id: int | None = None
    layer_windows: tuple[int, ...] = ()      # per layer: 0 = all keys, W = the last W keys; () = all layers full
    attention_bias: bool | None = None       # random-weights writer only; loading goes by tensor presence
    hidden_act: str = "silu"

    def __post_init__(self) -> None:
        for k in ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                  "num_key_value_heads", "head_dim", "vocab_size", "max_position_embeddings"):
            v = getattr(self, k)
            if not isinstance(v, int) or v <= 0:
                raise ValueError(f"config: {k} must be a positive integer, got {v!r}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ValueError(f"config: num_attention_heads {self.num_attention_heads} is not a multiple of "
                             f"num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2:
            raise ValueError(f"config: head_dim {self.head_dim} must be even (rotate-half pairs j, j + head_dim/2)")
        if self.hidden_act != "silu":
            raise NotImplementedError(f"config: hidden_act {self.hidden_act!r} is not supported (have ['silu'])")
        if not self.rms_norm_eps > 0:
            raise ValueError(f"config: rms_norm_eps must be positive, got {self.rms_norm_eps!r}")
        if self.layer_windows and len(self.layer_windows) != self.num_hidden_layers:
            raise ValueError(f"config: {len(self.layer_windows)} layer windows for {self.num_hidden_layers} layers")
        if any(w < 0 for w in self.layer_windows):
            raise ValueError(f"config: negative sliding window in {self.layer_windows}")

    # ---- config.json -> typed
    @staticmethod
    def from_hf(c: dict) -> "DenseDecoderConfig":
        missing = [k for k in ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads", "vocab_size")
                   if k not in c]
        if missing:
            raise ValueError(f"config.json lacks {missing}")
        rp = c.get("rope_parameters") or {}
        theta = c.get("rope_theta") or rp.get("rope_theta") or 10000.0
        scaling = c.get("rope_scaling") or ({k: v for k, v in rp.items() if k != "rope_theta"}
                                            if rp.get("rope_type", "default") != "default" else None)
        eos = c.get("eos_token_id")
        n_layers = int(c["num_hidden_layers"])
        windows: tuple[int, ...] = ()
        if c.get("use_sliding_window", False) and c.get("sliding_window"):
            w = int(c["sliding_window"])
            types = c.get("layer_types")
            if types:
                if len(types) != n_layers:
                    raise ValueError(f"config.json: {len(types)} layer_types for {n_layers} layers")
                windows = tuple(w if t == "sliding_attention" else 0 for t in types)
            else:
                windows = (w,) * n_layers
            if not any(windows):
                windows = ()
        heads = int(c["num_attention_heads"])
        return DenseDecoderConfig(
            model_type=c.get("model_type", "llama"),
            hidden_size=int(c["hidden_size"]), intermediate_size=int(c["intermediate_size"]), num_hidden_layers=n_layers,
            num_attention_heads=heads, num_key_value_heads=int(c.get("num_key_value_heads") or heads),
            head_dim=int(c.get("head_dim") or int(c["hidden_size"]) // heads), vocab_size=int(c["vocab_size"]),
            rms_norm_eps=float(c.get("rms_norm_eps", 1e-6)), rope_theta=float(theta),
            rope_scaling=RopeScaling.from_hf(scaling), tie_word_embeddings=bool(c.get("tie_word_embeddings", False)),
            max_position_embeddings=int(c.get("max_position_embeddings", 4096)),
            eos_token_ids=(int(eos),) if isinstance(eos, int) else tuple(int(e) for e in (eos or ())),
            bos_token_id=c.get("bos_token_id"), layer_windows=windows,
            attention_bias=c.get("attention_bias"), hidden_act=c.get("hidden_act", "silu"))

    # ---- typed -> config.json (the random-weights writer)
    def to_hf(self) -> dict:
        out: dict[str, Any] = {
            "model_type": self.model_type, "architectures": [_HF_CLASS.get(self.model_type, "LlamaForCausalLM")],
            "hidden_size": self.hidden_size, "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers, "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads, "head_dim": self.head_dim, "vocab_size": self.vocab_size,
            "rms_norm_eps": self.rms_norm_eps, "rope_theta": self.rope_theta, "hidden_act": self.hidden_act,
            "tie_word_embeddings": self.tie_word_embeddings, "max_position_embeddings": self.max_position_embeddings,
        }
        if (rs := self.rope_scaling.to_hf()) is not None:
            out["rope_scaling"] = rs
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        if self.bos_token_id is not None:
            out["bos_token_id"] = self.bos_token_id
        if self.attention_bias is not None:
            out["attention_bias"] = self.attention_bias
        if self.layer_windows:
            w = max(self.layer_windows)
            out.update(use_sliding_window=True, sliding_window=w,
                       layer_types=["sliding_attention" if x else "full_attention" for x in self.layer_windows])
            if any(x not in (0, w) for x in self.layer_windows):
                raise ValueError("config.json can name one sliding window size only")
        return out

    @property
    def writes_qkv_bias(self) -> bool:
        return self.attention_bias if self.attention_bias is not None else self.model_type == "qwen2"

    def random_optional_groups(self, expected: dict) -> set[str]:
        """Which optional tensor groups the random-weights writer writes for this configuration."""
        groups = {p.group for p in expected.values() if p.group}
        out = {g for g in groups if g.endswith("qkv_bias")} if self.writes_qkv_bias else set()
        if not self.tie_word_embeddings:
            out.add("lm_head")
        return out

    # ---- typed -> the description the engine builds from
    def spec(self) -> ModelSpec:
        rope = PartSpec("rope", {"head_dim": self.head_dim, "theta": self.rope_theta, **asdict(self.rope_scaling)})
        norm = PartSpec("rmsnorm", {"size": self.hidden_size, "eps": self.rms_norm_eps})
        ffn = PartSpec("swiglu", {"hidden_size": self.hidden_size, "intermediate_size": self.intermediate_size})
        layers = []
        for i in range(self.num_hidden_layers):
            win = self.layer_windows[i] if self.layer_windows else 0
            mixer = PartSpec("gqa_attention", {
                "hidden_size": self.hidden_size, "num_heads": self.num_attention_heads,
                "num_kv_heads": self.num_key_value_heads, "head_dim": self.head_dim,
                "scale": float(self.head_dim) ** -0.5, "window": win, "position": "rope"})
            layers.append(LayerSpec(f"model.layers.{i}.", PartSpec("pre_norm"), mixer, ffn, norm))
        return ModelSpec(
            architecture=self.model_type, hidden_size=self.hidden_size, vocab_size=self.vocab_size,
            embed_name="model.embed_tokens.weight",
            lm_head_name="lm_head.weight", tie_embeddings=self.tie_word_embeddings,
            final_norm=norm, final_norm_name="model.norm.weight", layers=tuple(layers),
            schedule=tuple(ScheduleEntry(i, i) for i in range(self.num_hidden_layers)),
            positions={"rope": rope}, max_position=self.max_position_embeddings,
            eos_token_ids=self.eos_token_ids, bos_token_id=self.bos_token_id)


_HF_CLASS = {"llama": "LlamaForCausalLM", "qwen2": "Qwen2ForCausalLM"}
