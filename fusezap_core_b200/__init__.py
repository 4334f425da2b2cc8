"""A B200-native inference engine for the dense Llama / Qwen2.5 decoder: model folder in, next tokens out, one GPU."""
__version__ = "0.1.0"
