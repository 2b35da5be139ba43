"""Model families: tiny test models, LLaMA, OLMo-2, a tiny MoE decoder and a GPT-2-style tiny decoder."""
from .activation_checkpointing import ActivationCheckpointConfig
from .gpt import GPTConfig, TinyGPT
from .llama import LlamaConfig, LlamaForCausalLM, LlamaForCausalLMTp, LlamaForCausalLMTpSp
from .olmo import OlmoConfig, OlmoForCausalLM, OlmoForCausalLMTp, OlmoForCausalLMTpSp
from .tiny_model import TinyModel
from .tiny_moe_transformer import (MoETransformerBlock, TinyMoETransformer, TinyMoETransformerTp, TinyMoETransformerTpSp,
                                   Top1MoE, TopKMoE)
from .tiny_transformer import TinyTransformer, TinyTransformerTp, TinyTransformerTpSp

__all__ = [
    "ActivationCheckpointConfig", "GPTConfig", "LlamaConfig", "LlamaForCausalLM", "LlamaForCausalLMTp",
    "LlamaForCausalLMTpSp", "MoETransformerBlock", "OlmoConfig", "OlmoForCausalLM", "OlmoForCausalLMTp",
    "OlmoForCausalLMTpSp", "TinyGPT", "TinyModel", "TinyMoETransformer", "TinyMoETransformerTp",
    "TinyMoETransformerTpSp", "TinyTransformer", "TinyTransformerTp", "TinyTransformerTpSp", "Top1MoE", "TopKMoE",
]
