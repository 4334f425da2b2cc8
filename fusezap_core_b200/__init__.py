"""A B200-native inference engine for the dense Llama / Qwen2.5 decoder: model folder in, next tokens out, one GPU.

  from fusezap_core_b200 import load_model, LLMEngine, SamplingParams
"""
__version__ = "0.2.0"

from .engine.model import load_model, DecoderModel
from .engine.llm_engine import LLMEngine, RequestOutput
from .sampling import SamplingParams
from .config import register_architecture, EngineConfig

__all__ = ["load_model", "DecoderModel", "LLMEngine", "RequestOutput", "SamplingParams", "register_architecture", "EngineConfig"]
