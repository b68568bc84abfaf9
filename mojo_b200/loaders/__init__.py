"""Checkpoint loaders: Hugging Face safetensors (bf16, 128x128 block-scaled fp8) and GGUF (Q4_K / Q6_K)."""
from .safetensors_loader import load_safetensors_into, read_safetensors_index  # noqa: F401
from .gguf_loader import GGUFFile, load_gguf_into  # noqa: F401
