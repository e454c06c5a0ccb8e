"""Model families of the named configurations: Llama-3 (8B / 70B shapes), GPT-2 (small / toy),
Qwen3-MoE (30B-A3B shape)."""
from .gpt2 import GPT2, GPT2Config
from .llama import Llama, LlamaBlock, LlamaConfig
from .qwen3_moe import Qwen3MoE, Qwen3MoEBlock, Qwen3MoEConfig

__all__ = ["GPT2", "GPT2Config", "Llama", "LlamaBlock", "LlamaConfig", "Qwen3MoE", "Qwen3MoEBlock", "Qwen3MoEConfig"]
