"""More chat templates, registered on import of ``data.formats`` (``template: <name>`` in a training YAML).

One row per template: the format of the system turn, of a user turn (which ends where the assistant starts to write)
and of the assistant turn, plus flags.  Multimodal variants of a family share the text format of the family; the media
placeholders are expanded by ``data/mm_plugin.py``.  Reference: ``data/template.py`` (the registered names are kept).
"""
from __future__ import annotations

CHATML = dict(system_fmt="<|im_start|>system\n{content}<|im_end|>\n",
              user_fmt="<|im_start|>user\n{content}<|im_end|>\n<|im_start|>assistant\n",
              assistant_fmt="{content}<|im_end|>\n", efficient_eos=False)
LLAMA3 = dict(system_fmt="<|start_header_id|>system<|end_header_id|>\n\n{content}<|eot_id|>",
              user_fmt="<|start_header_id|>user<|end_header_id|>\n\n{content}<|eot_id|>"
                       "<|start_header_id|>assistant<|end_header_id|>\n\n",
              assistant_fmt="{content}<|eot_id|>", add_bos=True, efficient_eos=False, tool_format="llama3")
GEMMA = dict(system_fmt="{content}\n\n", user_fmt="<start_of_turn>user\n{content}<end_of_turn>\n<start_of_turn>model\n",
             assistant_fmt="{content}<end_of_turn>\n", add_bos=True, efficient_eos=False)
MISTRAL = dict(system_fmt="{content}\n\n", user_fmt="[INST] {content}[/INST]", assistant_fmt=" {content}", add_bos=True,
               tool_format="mistral")
VICUNA_SYS = ("A chat between a curious user and an artificial intelligence assistant. "
              "The assistant gives helpful, detailed, and polite answers to the user's questions.")

ZOO = {
    # ChatML family
    "chatml_de": dict(CHATML, default_system="Du bist ein freundlicher und hilfsbereiter KI-Assistent."),
    "dolphin": dict(CHATML, default_system="You are Dolphin, a helpful AI assistant."),
    "qwen2_vl": dict(CHATML, default_system="You are a helpful assistant."),
    "qwen2_audio": dict(CHATML, default_system="You are a helpful assistant."),
    "qwen2_omni": dict(CHATML, default_system="You are a helpful assistant."),
    "qwen3_vl": dict(CHATML), "qwen3_vl_nothink": dict(CHATML), "qwen3_omni": dict(CHATML), "qwen3_5": dict(CHATML),
    "qwen3_next": dict(CHATML), "yi_vl": dict(CHATML), "intern2": dict(CHATML, add_bos=True), "intern_vl": dict(CHATML),
    "intern_s1": dict(CHATML), "minicpm_v": dict(CHATML), "minicpm_o": dict(CHATML), "smollm": dict(CHATML),
    "smollm2": dict(CHATML, default_system="You are a helpful AI assistant named SmolLM, trained by Hugging Face."),
    "marco": dict(CHATML), "opencoder": dict(CHATML, default_system="You are OpenCoder, created by OpenCoder Team."),
    "sailor": dict(CHATML, default_system="You are an AI assistant named Sailor created by Sea AI Lab."),
    "seed_coder": dict(CHATML), "skywork_o1": dict(CHATML), "mimo": dict(CHATML, default_system="You are MiMo, an AI assistant developed by Xiaomi."),
    "mimo_vl": dict(CHATML), "kimi_vl": dict(CHATML), "moonlight": dict(CHATML), "hunyuan": dict(CHATML),
    "exaone": dict(system_fmt="[|system|]{content}[|endofturn|]\n", user_fmt="[|user|]{content}\n[|assistant|]",
                   assistant_fmt="{content}[|endofturn|]\n", efficient_eos=False),
    # Llama family
    "llama3_vl": dict(LLAMA3), "mllama": dict(LLAMA3), "llava_next_llama3": dict(LLAMA3), "skywork_o1_llama": dict(LLAMA3),
    "llama2_zh": dict(system_fmt="<<SYS>>\n{content}\n<</SYS>>\n\n", user_fmt="[INST] {content} [/INST]",
                      assistant_fmt=" {content} ", add_bos=True, default_system="You are a helpful assistant. 你是一个乐于助人的助手。"),
    "llava": dict(system_fmt="{content} ", user_fmt="USER: {content} ASSISTANT:", assistant_fmt="{content}",
                  default_system=VICUNA_SYS),
    "llava_next": dict(system_fmt="{content} ", user_fmt="USER: {content} ASSISTANT:", assistant_fmt="{content}",
                       default_system=VICUNA_SYS),
    "video_llava": dict(system_fmt="{content} ", user_fmt="USER: {content} ASSISTANT:", assistant_fmt="{content}",
                        default_system=VICUNA_SYS),
    # Mistral family
    "mistral_small": dict(system_fmt="[SYSTEM_PROMPT]{content}[/SYSTEM_PROMPT]", user_fmt="[INST]{content}[/INST]",
                          assistant_fmt="{content}", add_bos=True, tool_format="mistral"),
    "pixtral": dict(MISTRAL), "llava_next_mistral": dict(MISTRAL), "breeze": dict(MISTRAL, efficient_eos=True),
    # Gemma family
    "gemma2": dict(GEMMA), "gemma3": dict(GEMMA), "gemma3n": dict(GEMMA), "paligemma": dict(GEMMA),
    # others
    "aquila": dict(system_fmt="{content}###", user_fmt="Human: {content}###Assistant:", assistant_fmt="{content}###",
                   default_system=VICUNA_SYS, efficient_eos=False),
    "atom": dict(system_fmt="{content}", user_fmt="<s>Human: {content}\n</s><s>Assistant:", assistant_fmt="{content}\n</s>",
                 efficient_eos=False),
    "baichuan": dict(system_fmt="{content}", user_fmt="<reserved_102>{content}<reserved_103>", assistant_fmt="{content}"),
    "baichuan2": dict(system_fmt="{content}", user_fmt="<reserved_106>{content}<reserved_107>", assistant_fmt="{content}"),
    "bailing": dict(system_fmt="<role>SYSTEM</role>{content}", user_fmt="<role>HUMAN</role>{content}<role>ASSISTANT</role>",
                    assistant_fmt="{content}"),
    "belle": dict(system_fmt="{content}", user_fmt="Human: {content}\n\nBelle: ", assistant_fmt="{content}\n\n", add_bos=True),
    "bluelm": dict(system_fmt="{content}", user_fmt="[|Human|]:{content}[|AI|]:", assistant_fmt="{content}"),
    "chatglm2": dict(system_fmt="{content}", user_fmt="[Round 1]\n\n问:{content}\n\n答:", assistant_fmt="{content}\n\n"),
    "chatglm3": dict(system_fmt="<|system|>\n{content}", user_fmt="<|user|>\n{content}<|assistant|>\n", assistant_fmt="{content}", tool_format="glm4"),
    "glm4_moe": dict(system_fmt="<|system|>\n{content}", user_fmt="<|user|>\n{content}<|assistant|>\n", assistant_fmt="{content}", tool_format="glm4"),
    "glm4v": dict(system_fmt="<|system|>\n{content}", user_fmt="<|user|>\n{content}<|assistant|>\n", assistant_fmt="{content}", tool_format="glm4"),
    "glmz1": dict(system_fmt="<|system|>\n{content}", user_fmt="<|user|>\n{content}<|assistant|>\n", assistant_fmt="{content}", tool_format="glm4"),
    "codegeex2": dict(system_fmt="{content}", user_fmt="{content}", assistant_fmt="{content}"),
    "codegeex4": dict(system_fmt="<|system|>\n{content}", user_fmt="<|user|>\n{content}<|assistant|>\n", assistant_fmt="{content}",
                      default_system="你是一位智能编程助手，你叫CodeGeeX。"),
    "cohere": dict(system_fmt="<|START_OF_TURN_TOKEN|><|SYSTEM_TOKEN|>{content}<|END_OF_TURN_TOKEN|>",
                   user_fmt="<|START_OF_TURN_TOKEN|><|USER_TOKEN|>{content}<|END_OF_TURN_TOKEN|>"
                            "<|START_OF_TURN_TOKEN|><|CHATBOT_TOKEN|>",
                   assistant_fmt="{content}<|END_OF_TURN_TOKEN|>", add_bos=True, efficient_eos=False),
    "cpm": dict(system_fmt="{content}", user_fmt="<用户>{content}<AI>", assistant_fmt="{content}", add_bos=True),
    "cpm3": dict(CHATML, add_bos=True), "cpm4": dict(CHATML),
    "dbrx": dict(CHATML, default_system="You are DBRX, created by Databricks."),
    "deepseekcoder": dict(system_fmt="{content}", user_fmt="### Instruction:\n{content}\n### Response:",
                          assistant_fmt="\n{content}\n<|EOT|>\n", add_bos=True, efficient_eos=False,
                          default_system="You are an AI programming assistant, utilizing the DeepSeek Coder model."),
    "deepseekr1": dict(system_fmt="{content}", user_fmt="<｜User｜>{content}<｜Assistant｜>",
                       assistant_fmt="{content}", add_bos=True),
    "falcon_h1": dict(CHATML), "gpt_oss": dict(system_fmt="<|start|>system<|message|>{content}<|end|>",
                                               user_fmt="<|start|>user<|message|>{content}<|end|><|start|>assistant",
                                               assistant_fmt="<|channel|>final<|message|>{content}<|return|>", efficient_eos=False),
    "granite3_vision": dict(system_fmt="<|system|>\n{content}\n", user_fmt="<|user|>\n{content}\n<|assistant|>\n",
                            assistant_fmt="{content}\n"),
    "granite4": dict(system_fmt="<|start_of_role|>system<|end_of_role|>{content}<|end_of_text|>\n",
                     user_fmt="<|start_of_role|>user<|end_of_role|>{content}<|end_of_text|>\n<|start_of_role|>assistant<|end_of_role|>",
                     assistant_fmt="{content}<|end_of_text|>\n", efficient_eos=False),
    "index": dict(system_fmt="<unk>{content}", user_fmt="reserved_0{content}reserved_1", assistant_fmt="{content}"),
    "intern": dict(system_fmt="<|System|>:{content}\n", user_fmt="<|User|>:{content}\n<|Bot|>:", assistant_fmt="{content}<eoa>\n",
                   add_bos=True, efficient_eos=False),
    "olmo": dict(system_fmt="<|endoftext|>{content}", user_fmt="<|user|>\n{content}<|assistant|>\n", assistant_fmt="{content}"),
    "orion": dict(system_fmt="{content}", user_fmt="Human: {content}\n\nAssistant: </s>", assistant_fmt="{content}", add_bos=True),
    "phi_small": dict(system_fmt="<|system|>\n{content}<|end|>\n", user_fmt="<|user|>\n{content}<|end|>\n<|assistant|>\n",
                      assistant_fmt="{content}<|end|>\n", add_bos=True, efficient_eos=False),
    "seed_oss": dict(system_fmt="<seed:bos>system\n{content}<seed:eos>", user_fmt="<seed:bos>user\n{content}<seed:eos><seed:bos>assistant\n",
                     assistant_fmt="{content}<seed:eos>", efficient_eos=False),
    "solar": dict(system_fmt="### System:\n{content}\n\n", user_fmt="### User:\n{content}\n\n### Assistant:\n", assistant_fmt="{content}\n\n"),
    "starchat": dict(system_fmt="<|system|>\n{content}<|end|>\n", user_fmt="<|user|>\n{content}<|end|>\n<|assistant|>",
                     assistant_fmt="{content}<|end|>\n", efficient_eos=False),
    "telechat": dict(system_fmt="<_system>{content}<_end>", user_fmt="<_user>{content}<_bot>", assistant_fmt="{content}<_end>",
                     efficient_eos=False),
    "telechat2": dict(system_fmt="<_system>{content}", user_fmt="<_user>{content}<_bot>", assistant_fmt="{content}<_end>",
                      efficient_eos=False),
    "xuanyuan": dict(system_fmt="{content}", user_fmt="Human: {content} Assistant:", assistant_fmt="{content}"),
    "xverse": dict(system_fmt="{content}", user_fmt="Human: {content}\n\nAssistant: ", assistant_fmt="{content}\n\n"),
    "yayi": dict(system_fmt="<|System|>\n{content}\n\n", user_fmt="<|Human|>\n{content}\n\n<|YaYi|>", assistant_fmt="\n{content}\n\n"),
    "yuan": dict(system_fmt="{content}", user_fmt="{content}<sep>", assistant_fmt="{content}<eod>\n", efficient_eos=False),
    "ziya": dict(system_fmt="{content}", user_fmt="<human>:{content}\n<bot>:", assistant_fmt="{content}\n"),
    "fewshot": dict(system_fmt="{content}\n\n", user_fmt="{content}", assistant_fmt="{content}\n\n", efficient_eos=False),
    "qwen3_nothink_pt": dict(CHATML),
}


def register_all(templates: dict, template_cls) -> int:
    n = 0
    for name, fields in ZOO.items():
        if name not in templates:
            templates[name] = template_cls(name, **fields)
            n += 1
    return n
