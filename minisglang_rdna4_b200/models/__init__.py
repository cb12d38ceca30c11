"""Model registry: architecture string → constructor (python/minisgl/models/register.py:5-34)."""
from __future__ import annotations

import torch

from ..utils import Registry
from .config import NAMED_CONFIGS, ModelConfig, RotaryConfig

MODEL_REGISTRY: Registry = Registry("model architecture")


def _register_defaults() -> None:
    from .transformer import CausalLM

    for arch in (
        "LlamaForCausalLM", "MistralForCausalLM", "Qwen2ForCausalLM", "Qwen3ForCausalLM",
        "Qwen2MoeForCausalLM", "Qwen3MoeForCausalLM", "Glm4MoeForCausalLM", "MixtralForCausalLM",
    ):
        if arch not in MODEL_REGISTRY:
            MODEL_REGISTRY.register(arch)(CausalLM)
    from .gemma import GemmaForCausalLM

    for arch in ("Gemma2ForCausalLM", "Gemma3ForCausalLM", "Gemma3ForConditionalGeneration"):
        if arch not in MODEL_REGISTRY:
            MODEL_REGISTRY.register(arch)(GemmaForCausalLM)


    from .gemma4 import DiffusionGemmaForBlockDiffusion, Gemma4ForCausalLM

    if "DiffusionGemmaForBlockDiffusion" not in MODEL_REGISTRY:
        MODEL_REGISTRY.register("DiffusionGemmaForBlockDiffusion")(DiffusionGemmaForBlockDiffusion)

    for arch in ("Gemma4ForCausalLM", "Gemma4ForConditionalGeneration"):
        if arch not in MODEL_REGISTRY:
            MODEL_REGISTRY.register(arch)(Gemma4ForCausalLM)

    from .laguna import LagunaForCausalLM

    if "LagunaForCausalLM" not in MODEL_REGISTRY:
        MODEL_REGISTRY.register("LagunaForCausalLM")(LagunaForCausalLM)
    from .muse_glimmer import MuseGlimmerForConditionalGeneration

    if "MuseGlimmerForConditionalGeneration" not in MODEL_REGISTRY:
        MODEL_REGISTRY.register("MuseGlimmerForConditionalGeneration")(MuseGlimmerForConditionalGeneration)

    from .qwen3_5 import Qwen3_5ForCausalLM

    for arch in ("Qwen3_5ForCausalLM", "Qwen3_5ForConditionalGeneration", "Qwen3_5MoeForCausalLM",
                 "Qwen3_5MoeForConditionalGeneration", "Qwen3NextForCausalLM"):
        if arch not in MODEL_REGISTRY:
            MODEL_REGISTRY.register(arch)(Qwen3_5ForCausalLM)


    from .glm4_moe_lite import Glm4MoeLiteForCausalLM

    for arch in ("Glm4MoeLiteForCausalLM", "DeepseekV2ForCausalLM", "DeepseekV3ForCausalLM"):
        if arch not in MODEL_REGISTRY:
            MODEL_REGISTRY.register(arch)(Glm4MoeLiteForCausalLM)


    from .nemotron_h import NemotronHForCausalLM

    if "NemotronHForCausalLM" not in MODEL_REGISTRY:
        MODEL_REGISTRY.register("NemotronHForCausalLM")(NemotronHForCausalLM)


def create_model(cfg: ModelConfig, dtype: torch.dtype, device):
    """Instantiate the model for ``cfg`` with uninitialised (or meta) parameters."""
    _register_defaults()
    for arch in cfg.architectures:
        if arch in MODEL_REGISTRY:
            return MODEL_REGISTRY[arch](cfg, dtype, device)
    raise KeyError(f"no model registered for architectures {cfg.architectures}; "
                   f"known: {MODEL_REGISTRY.names()}")


__all__ = ["MODEL_REGISTRY", "create_model", "ModelConfig", "RotaryConfig", "NAMED_CONFIGS"]
