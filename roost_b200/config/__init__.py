from .reader import ConfigError, ConfigReader
from .spec import (AttentionSpec, BlockSpec, FeedForwardSpec, GatedMlpSpec, MixerSpec, ModelSpec, NormSpec,
                   PositionSpec, RunEntry)
from .qwen3 import Qwen3Config

__all__ = ["ConfigError", "ConfigReader", "AttentionSpec", "BlockSpec", "FeedForwardSpec", "GatedMlpSpec", "MixerSpec",
           "ModelSpec", "NormSpec", "PositionSpec", "RunEntry", "Qwen3Config"]
