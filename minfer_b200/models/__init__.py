"""Architectures that ship with the library, registered under their config.json names."""
from ..config.qwen2 import ARCHITECTURE as QWEN2, Qwen2Config
from ..registry import register_architecture

register_architecture(QWEN2, Qwen2Config.from_dict, replace=True)
