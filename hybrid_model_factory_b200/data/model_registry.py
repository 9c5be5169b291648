"""Which chat template a model family speaks.

``template_for_model("Qwen/Qwen3-8B")`` -> ``"qwen3"``: the checkpoint's name (last path component, case-folded) is
matched against family patterns, most specific first.  Used when a run names a model but no ``template``; an explicit
``template`` always wins.  Reference: the model groups of ``extras/constants.py`` (``register_model_group(...,
template=...)``), restated here as patterns instead of an enumeration of every checkpoint."""
from __future__ import annotations

import os
import re
from typing import List, Optional, Tuple

# (regular expression on the lower-cased model name, template); first match wins, so the specific forms come first
_RULES: List[Tuple[str, str]] = [
    # distilled checkpoints carry two family names: the teacher's format is the one they speak
    (r"deepseek.*r1", "deepseekr1"), (r"deepseek.*(v3|v2\.5)", "deepseek3"), (r"deepseek.*coder", "deepseekcoder"),
    (r"deepseek", "deepseek"),
    (r"qwen3.*vl", "qwen3_vl"), (r"qwen3.*omni", "qwen3_omni"), (r"qwen3[._-]?5", "qwen3_5"), (r"qwen3.*next", "qwen3_next"),
    (r"qwen3", "qwen3"), (r"qwen2.*vl|qvq", "qwen2_vl"), (r"qwen2.*audio", "qwen2_audio"), (r"qwen2.*omni", "qwen2_omni"),
    (r"qwq|qwen", "qwen"),
    (r"llama-?4", "llama4"), (r"llama-?3.*vision", "mllama"), (r"llama-?3", "llama3"), (r"chinese.*llama-?2", "llama2_zh"),
    (r"llama-?2", "llama2"),
    (r"ministral-?3", "ministral"), (r"mistral.*small", "mistral_small"), (r"pixtral", "pixtral"),
    (r"mi[sx]tral|ministral", "mistral"),
    (r"gemma-?3n", "gemma3n"), (r"gemma-?3", "gemma3"), (r"gemma-?2", "gemma2"), (r"paligemma", "paligemma"), (r"gemma", "gemma"),
    (r"glm-?4.*moe|glm-?4\.[56]", "glm4_moe"), (r"glm-?4.*v", "glm4v"), (r"glm-?z1", "glmz1"), (r"glm-?4", "glm4"),
    (r"chatglm3", "chatglm3"), (r"chatglm2", "chatglm2"),
    (r"phi-?4", "phi4"), (r"phi-?3.*small", "phi_small"), (r"phi-?3", "phi"),
    (r"yi.*vl", "yi_vl"), (r"\byi\b|yi-", "yi"),
    (r"internvl", "intern_vl"), (r"intern.*s1", "intern_s1"), (r"internlm-?[23]", "intern2"), (r"internlm", "intern"),
    (r"minicpm.*o", "minicpm_o"), (r"minicpm.*v", "minicpm_v"), (r"minicpm-?4", "cpm4"), (r"minicpm-?3", "cpm3"),
    (r"minicpm", "cpm"),
    (r"llava.*next.*mistral", "llava_next_mistral"), (r"llava.*next.*llama-?3", "llava_next_llama3"),
    (r"llava.*next", "llava_next"), (r"video.*llava", "video_llava"), (r"llava", "llava"),
    (r"granite.*4", "granite4"), (r"granite.*vision", "granite3_vision"), (r"granite", "granite3"),
    (r"falcon.*h1", "falcon_h1"), (r"falcon", "falcon"), (r"gpt-?oss", "gpt_oss"), (r"kimi.*vl", "kimi_vl"),
    (r"moonlight", "moonlight"), (r"mimo.*vl", "mimo_vl"), (r"mimo", "mimo"), (r"hunyuan", "hunyuan"),
    (r"seed.*oss", "seed_oss"), (r"seed.*coder", "seed_coder"), (r"smollm-?2", "smollm2"), (r"smollm", "smollm"),
    (r"baichuan-?2", "baichuan2"), (r"baichuan", "baichuan"), (r"command-?r|aya", "cohere"), (r"dbrx", "dbrx"),
    (r"exaone", "exaone"), (r"olmo", "olmo"), (r"openchat", "openchat"), (r"opencoder", "opencoder"),
    (r"solar", "solar"), (r"starchat", "starchat"), (r"telechat-?2", "telechat2"), (r"telechat", "telechat"),
    (r"vicuna", "vicuna"), (r"xverse", "xverse"), (r"xuanyuan", "xuanyuan"), (r"yuan", "yuan"), (r"zephyr", "zephyr"),
    (r"ziya", "ziya"), (r"codegeex-?4", "codegeex4"), (r"codegeex", "codegeex2"), (r"breeze", "breeze"),
    (r"bluelm", "bluelm"), (r"skywork.*o1", "skywork_o1"), (r"sailor", "sailor"), (r"orion", "orion"),
    (r"index", "index"), (r"marco", "marco"), (r"aquila", "aquila"),
]
_COMPILED = [(re.compile(p), t) for p, t in _RULES]


def template_for_model(name_or_path: Optional[str], base_model: bool = False) -> Optional[str]:
    """Template of the family ``name_or_path`` belongs to, or ``None`` when no family matches.  ``base_model``:
    pretrained (non-chat) checkpoints are fine-tuned with the plain ``default`` template."""
    if not name_or_path or name_or_path.lstrip().startswith("{"):      # nothing, or an inline JSON configuration
        return None
    name = os.path.basename(os.path.normpath(name_or_path)).lower()
    if base_model or re.search(r"(^|[-_])base($|[-_])", name):
        return "default"
    for rx, template in _COMPILED:
        if rx.search(name):
            return template
    return None


def families() -> List[str]:
    return sorted({t for _, t in _RULES})
