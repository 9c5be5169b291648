"""Model classes named like the reference plugin's vLLM models; they resolve to the native model zoo.
Running them *inside* vLLM's worker is not implemented (the native engine replaces vLLM's executor)."""
from ..models.modeling_hybrid import (HybridQwen2ForCausalLM, HybridQwen3ForCausalLM,  # noqa: F401
                                      HybridQwen3MoeForCausalLM)
