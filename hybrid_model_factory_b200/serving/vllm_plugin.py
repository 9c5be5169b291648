"""vLLM out-of-tree plugin shim.  ``register()`` is exposed under the ``vllm.general_plugins`` entry point
so that ``vllm serve <hybrid checkpoint>`` recognises the hybrid architectures when vLLM is installed.
The registered names and config ``model_type``s are the ones the reference plugin registers
(``vllm-inference/src/primed_vllm/register.py:32-73``).  The native engine in this package does not
need vLLM; this module only keeps the reference's launch surface working."""
from __future__ import annotations

ARCHITECTURES = {
    "HybridQwen2ForCausalLM": "hybrid_model_factory_b200.serving.vllm_models:HybridQwen2ForCausalLM",
    "HybridQwen3ForCausalLM": "hybrid_model_factory_b200.serving.vllm_models:HybridQwen3ForCausalLM",
    "HybridQwen3MoeForCausalLM": "hybrid_model_factory_b200.serving.vllm_models:HybridQwen3MoeForCausalLM",
}
MODEL_TYPES = ("hybrid_qwen2", "hybrid_qwen3", "hybrid_qwen3_moe")

_registered = False


def register() -> bool:
    """Registers the hybrid architectures with vLLM's ModelRegistry (lazy ``module:Class`` strings) and the
    config classes with transformers' AutoConfig.  Returns False when vLLM is not importable."""
    global _registered
    if _registered:
        return True
    try:
        from vllm import ModelRegistry
    except Exception:
        return False
    for name, target in ARCHITECTURES.items():
        try:
            if name not in ModelRegistry.get_supported_archs():
                ModelRegistry.register_model(name, target)
        except Exception:
            pass
    try:
        from transformers import AutoConfig, PretrainedConfig
        for mt in MODEL_TYPES:
            cls = type(f"{mt.title().replace('_', '')}Config", (PretrainedConfig,), {"model_type": mt})
            try:
                AutoConfig.register(mt, cls)
            except Exception:
                pass
    except Exception:
        pass
    _registered = True
    return True


def registry() -> dict:
    """Architecture name -> native model class (used by ``hmf serve`` and by tests)."""
    from ..models.modeling_hybrid import (HybridQwen2ForCausalLM, HybridQwen3ForCausalLM, HybridQwen3MoeForCausalLM)
    return {"HybridQwen2ForCausalLM": HybridQwen2ForCausalLM, "HybridQwen3ForCausalLM": HybridQwen3ForCausalLM,
            "HybridQwen3MoeForCausalLM": HybridQwen3MoeForCausalLM}
