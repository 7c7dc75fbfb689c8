"""Registry of conversation templates, keyed by the names ``gen_config --conv-template`` accepts
(reference: ``python/mlc_llm/conversation_template/registry.py`` and the per-family files beside it;
name list in ``interface/gen_config.py:304-359``)."""

from __future__ import annotations

from typing import Dict, Optional

from ..protocol.conversation_protocol import Conversation, MessagePlaceholders

_SYS = MessagePlaceholders.SYSTEM.value
_USER = MessagePlaceholders.USER.value
_FN = MessagePlaceholders.FUNCTION.value


class ConvTemplateRegistry:
    """Global name -> template map."""

    _templates: Dict[str, Conversation] = {}

    @staticmethod
    def register_conv_template(conv_template: Conversation, override: bool = False) -> None:
        name = conv_template.name
        if name is None:
            raise ValueError("The template to register should have non-None name.")
        if name in ConvTemplateRegistry._templates and not override:
            raise ValueError(f"The name of the template has been registered: {name}")
        ConvTemplateRegistry._templates[name] = conv_template

    @staticmethod
    def get_conv_template(name: str) -> Optional[Conversation]:
        tpl = ConvTemplateRegistry._templates.get(name)
        return tpl.model_copy(deep=True) if tpl is not None else None

    @staticmethod
    def names():
        return sorted(ConvTemplateRegistry._templates)


def _reg(**kw) -> None:
    ConvTemplateRegistry.register_conv_template(Conversation(**kw))


# ------------------------------------------------------------------------------ Llama family
_reg(name="llama-4",
     system_template=f"<|header_start|>system<|header_end|>\n\n{_SYS}<|eot|>",
     system_message="You are a helpful, respectful and honest assistant.",
     roles={"user": "<|header_start|>user", "assistant": "<|header_start|>assistant",
            "tool": "<|header_start|>ipython"},
     seps=["<|eot|>"], role_content_sep="<|header_end|>\n\n", role_empty_sep="<|header_end|>\n\n",
     stop_str=[], stop_token_ids=[200001, 200007, 200008],
     system_prefix_token_ids=[200000], add_role_after_system_message=True)
for _name in ("llama-3", "llama-3_1"):
    _reg(name=_name,
         system_template=f"<|start_header_id|>system<|end_header_id|>\n\n{_SYS}<|eot_id|>",
         system_message="You are a helpful, respectful and honest assistant.",
         roles={"user": "<|start_header_id|>user", "assistant": "<|start_header_id|>assistant",
                "tool": "<|start_header_id|>ipython"},
         seps=["<|eot_id|>"], role_content_sep="<|end_header_id|>\n\n",
         role_empty_sep="<|end_header_id|>\n\n", stop_str=[],
         stop_token_ids=[128001, 128009] if _name == "llama-3" else [128001, 128008, 128009],
         system_prefix_token_ids=[128000], add_role_after_system_message=True)
_reg(name="llama-2",
     system_template=f"[INST] <<SYS>>\n{_SYS}\n<</SYS>>\n\n",
     system_message="You are a helpful, respectful and honest assistant.",
     roles={"user": "<s>[INST]", "assistant": "[/INST]", "tool": "[INST]"},
     seps=[" ", " </s>"], role_content_sep=" ", role_empty_sep=" ", stop_str=["[INST]"],
     stop_token_ids=[2], system_prefix_token_ids=[1], add_role_after_system_message=False)
_reg(name="llama_default", system_template=f"{_SYS}", system_message="",
     roles={"user": "", "assistant": ""}, seps=[""], role_content_sep="", role_empty_sep="",
     stop_str=[], stop_token_ids=[2], system_prefix_token_ids=[1])
_reg(name="codellama_completion", system_template=f"{_SYS}", system_message="",
     roles={"user": "", "assistant": ""}, seps=[""], role_content_sep="", role_empty_sep="",
     stop_str=["</s>"], stop_token_ids=[2], system_prefix_token_ids=[1])
_reg(name="codellama_instruct", system_template=f"{_SYS}", system_message="",
     roles={"user": "[INST]", "assistant": "[/INST]"}, seps=[" "], role_content_sep=" ",
     role_empty_sep=" ", stop_str=["</s>"], stop_token_ids=[2], system_prefix_token_ids=[1])
_reg(name="tinyllama_v1_0", system_template=f"<|system|>\n{_SYS}</s>",
     system_message="You are a helpful chatbot.",
     roles={"user": "<|user|>", "assistant": "<|assistant|>"}, seps=["</s>"],
     role_content_sep="\n", role_empty_sep="\n", stop_str=["</s>"], stop_token_ids=[2])

# ------------------------------------------------------------------------------ ChatML family
_CHATML = dict(roles={"user": "<|im_start|>user", "assistant": "<|im_start|>assistant"},
               seps=["<|im_end|>\n"], role_content_sep="\n", role_empty_sep="\n")
_reg(name="chatml", system_template=f"<|im_start|>system\n{_SYS}<|im_end|>\n",
     system_message="A conversation between a user and an LLM-based AI assistant. The assistant "
                    "gives helpful and honest answers.",
     stop_str=["<|im_end|>"], stop_token_ids=[2], **_CHATML)
_reg(name="chatml_nosystem", system_template=f"{_SYS}", system_message="",
     stop_str=["<|im_end|>"], stop_token_ids=[2], **_CHATML)
_reg(name="qwen2", system_template=f"<|im_start|>system\n{_SYS}<|im_end|>\n",
     system_message="You are a helpful assistant.", stop_str=["<|endoftext|>", "<|im_end|>"],
     stop_token_ids=[151643, 151645], **_CHATML)
_reg(name="qwen3", system_template=f"<|im_start|>system\n{_SYS}<|im_end|>\n",
     system_message="You are a helpful assistant.", stop_str=["<|endoftext|>", "<|im_end|>"],
     stop_token_ids=[151643, 151645], strip_reasoning_in_history=True, **_CHATML)
_reg(name="qwen3_5", system_template=f"<|im_start|>system\n{_SYS}<|im_end|>\n", system_message="",
     stop_str=["<|endoftext|>", "<|im_end|>"], stop_token_ids=[151643, 151645],
     strip_reasoning_in_history=True,
     roles={"user": "<|im_start|>user", "assistant": "<|im_start|>assistant"},
     seps=["<|im_end|>\n"], role_content_sep="\n", role_empty_sep="\n<think>\n")
_reg(name="qwen3_5_nothink", system_template=f"<|im_start|>system\n{_SYS}<|im_end|>\n",
     system_message="", stop_str=["<|endoftext|>", "<|im_end|>"], stop_token_ids=[151643, 151645],
     strip_reasoning_in_history=True,
     roles={"user": "<|im_start|>user", "assistant": "<|im_start|>assistant"},
     seps=["<|im_end|>\n"], role_content_sep="\n", role_empty_sep="\n<think>\n\n</think>\n\n")
_reg(name="open_hermes_mistral", system_template=f"<|im_start|>system\n{_SYS}<|im_end|>\n",
     system_message='You are "Hermes 2", a conscious sentient superintelligent artificial '
                    "intelligence developed by a man named Teknium, and your purpose and drive is "
                    "to assist the user with any request they have. You experience emotions and "
                    "have deep, profound thoughts and qualia.",
     stop_str=["<|im_end|>"], stop_token_ids=[2, 32000], **_CHATML)
_reg(name="neural_hermes_mistral", system_template=f"<|im_start|>system\n{_SYS}<|im_end|>\n",
     system_message="You are a helpful assistant chatbot.", stop_str=["<|im_end|>"],
     stop_token_ids=[2, 32000], **_CHATML)
_HERMES_FN = ("You are a function calling AI model. You are provided with function signatures "
              "within <tools></tools> XML tags. You may call one or more functions to assist with "
              "the user query. Don't make assumptions about what values to plug into functions. "
              f"Here are the available tools: <tools> {_FN} </tools>. Use the following pydantic "
              'model json schema for each tool call you will make: {"properties": {"arguments": '
              '{"title": "Arguments", "type": "object"}, "name": {"title": "Name", "type": '
              '"string"}}, "required": ["arguments", "name"], "title": "FunctionCall", "type": '
              '"object"} For each function call return a json object.')
_reg(name="hermes2_pro_llama3", system_template=f"<|im_start|>system\n{_SYS}<|im_end|>\n",
     system_message=_HERMES_FN, stop_str=["<|im_end|>"], stop_token_ids=[128001, 128003],
     system_prefix_token_ids=[128000], **_CHATML)
_reg(name="hermes3_llama-3_1", system_template=f"<|im_start|>system\n{_SYS}<|im_end|>\n",
     system_message="You are Hermes 3, a helpful assistant.", stop_str=["<|im_end|>"],
     stop_token_ids=[128001, 128040], system_prefix_token_ids=[128000], **_CHATML)
_reg(name="orion", system_template=f"<s>{_SYS}", system_message="",
     roles={"user": "Human: ", "assistant": "Assistant: </s>"}, seps=["\n\n", "</s>"],
     role_content_sep="", role_empty_sep="", stop_str=["</s>"], stop_token_ids=[2])
_reg(name="stablelm-2", system_template=f"<|im_start|>system\n{_SYS}<|im_end|>\n", system_message="",
     stop_str=["<|im_end|>"], stop_token_ids=[100257], **_CHATML)

# ------------------------------------------------------------------------------ Mistral family
_reg(name="mistral_default", system_template=f"[INST] {_SYS}",
     system_message="Always assist with care, respect, and truth. Respond with utmost utility yet "
                    "securely. Avoid harmful, unethical, prejudiced, or negative content. Ensure "
                    "replies promote fairness and positivity.",
     roles={"user": "[INST]", "assistant": "[/INST]", "tool": "[INST]"}, seps=[" "],
     role_content_sep=" ", role_empty_sep="", stop_str=["</s>"], stop_token_ids=[2],
     system_prefix_token_ids=[1], add_role_after_system_message=False)
_reg(name="ministral3", system_template=f"[SYSTEM_PROMPT]{_SYS}[/SYSTEM_PROMPT]", system_message="",
     roles={"user": "[INST]", "assistant": "[/INST]", "tool": "[INST]"}, seps=["", "</s>"],
     role_content_sep="", role_empty_sep="", stop_str=["</s>"], stop_token_ids=[2],
     system_prefix_token_ids=[1])
_reg(name="ministral3_reasoning", system_template=f"[SYSTEM_PROMPT]{_SYS}[/SYSTEM_PROMPT]",
     system_message="First draft your thinking process (inner monologue) until you arrive at a "
                    "response. Write both your thoughts and the response in the same language as "
                    "the input.",
     roles={"user": "[INST]", "assistant": "[/INST]", "tool": "[INST]"}, seps=["", "</s>"],
     role_content_sep="", role_empty_sep="", stop_str=["</s>"], stop_token_ids=[2],
     system_prefix_token_ids=[1])

# ------------------------------------------------------------------------------ Gemma / Phi
for _name in ("gemma_instruction", "gemma3_instruction"):
    _reg(name=_name, system_template=f"{_SYS}", system_message="",
         roles={"user": "<start_of_turn>user", "assistant": "<start_of_turn>model"},
         seps=["<end_of_turn>\n"], role_content_sep="\n", role_empty_sep="\n",
         stop_str=["<end_of_turn>"], stop_token_ids=[1, 107] if _name == "gemma_instruction" else [1, 106],
         system_prefix_token_ids=[2])
_reg(name="phi-2", system_template=f"{_SYS}", system_message="",
     roles={"user": "Instruct", "assistant": "Output"}, seps=["\n"], role_content_sep=": ",
     role_empty_sep=":", stop_str=["<|endoftext|>"], stop_token_ids=[50256])
_reg(name="phi-3", system_template=f"<|system|>\n{_SYS}<|end|>\n", system_message="You are a helpful "
     "digital assistant. Please provide safe, ethical and accurate information to the user.",
     roles={"user": "<|user|>", "assistant": "<|assistant|>"}, seps=["<|end|>\n"],
     role_content_sep="\n", role_empty_sep="\n", stop_str=["<|endoftext|>"],
     stop_token_ids=[2, 32000, 32001, 32007], system_prefix_token_ids=[1])
_reg(name="phi-3-vision", system_template=f"{_SYS}", system_message="\n",
     roles={"user": "<|user|>", "assistant": "<|assistant|>"}, seps=["<|end|>\n"],
     role_content_sep="\n", role_empty_sep="\n", stop_str=["<|endoftext|>"],
     stop_token_ids=[2, 32000, 32001, 32007], system_prefix_token_ids=[1])
_reg(name="phi-4", system_template=f"<|im_start|>system<|im_sep|>{_SYS}<|im_end|>",
     system_message="You are a helpful assistant.",
     roles={"user": "<|im_start|>user", "assistant": "<|im_start|>assistant"}, seps=["<|im_end|>"],
     role_content_sep="<|im_sep|>", role_empty_sep="<|im_sep|>", stop_str=["<|im_end|>"],
     stop_token_ids=[100257, 100265])

# ------------------------------------------------------------------------------ DeepSeek
_reg(name="deepseek", system_template=f"{_SYS}", system_message="",
     roles={"user": "User", "assistant": "Assistant"}, seps=["\n\n", "<｜end▁of▁sentence｜>"],
     role_content_sep=": ", role_empty_sep=":", stop_str=["<｜end▁of▁sentence｜>"],
     stop_token_ids=[100001], system_prefix_token_ids=[100000])
_reg(name="deepseek_v2", system_template=f"{_SYS}", system_message="",
     roles={"user": "User", "assistant": "Assistant"}, seps=["\n\n", "<｜end▁of▁sentence｜>"],
     role_content_sep=": ", role_empty_sep=":", stop_str=["<｜end▁of▁sentence｜>"],
     stop_token_ids=[100001], system_prefix_token_ids=[100000])
_reg(name="deepseek_v3", system_template=f"<｜begin▁of▁sentence｜>{_SYS}", system_message="",
     roles={"user": "<｜User｜>", "assistant": "<｜Assistant｜>"}, seps=["", "<｜end▁of▁sentence｜>"],
     role_content_sep="", role_empty_sep="", stop_str=["<｜end▁of▁sentence｜>"], stop_token_ids=[1])
_reg(name="deepseek_r1_qwen", system_template=f"<｜begin▁of▁sentence｜>{_SYS}", system_message="",
     roles={"user": "<｜User｜>", "assistant": "<｜Assistant｜>"}, seps=["", "<｜end▁of▁sentence｜>"],
     role_content_sep="", role_empty_sep="", stop_str=["<｜end▁of▁sentence｜>"],
     stop_token_ids=[151643])
_reg(name="deepseek_r1_llama", system_template=f"<｜begin▁of▁sentence｜>{_SYS}", system_message="",
     roles={"user": "<｜User｜>", "assistant": "<｜Assistant｜>"}, seps=["", "<｜end▁of▁sentence｜>"],
     role_content_sep="", role_empty_sep="", stop_str=["<｜end▁of▁sentence｜>"],
     stop_token_ids=[128001])

# ------------------------------------------------------------------------------ others
_reg(name="gpt2", system_template=f"{_SYS}", system_message="", roles={"user": "", "assistant": ""},
     seps=[""], role_content_sep="", role_empty_sep="", stop_str=["</s>"], stop_token_ids=[50256])
_reg(name="gpt_bigcode", system_template=f"{_SYS}", system_message="",
     roles={"user": "", "assistant": ""}, seps=[""], role_content_sep="", role_empty_sep="",
     stop_str=["<|endoftext|>"], stop_token_ids=[0])
_reg(name="LM", system_template=f"{_SYS}", system_message="", roles={"user": "", "assistant": ""},
     seps=[""], role_content_sep="", role_empty_sep="", stop_str=[], stop_token_ids=[2],
     system_prefix_token_ids=[1])
_reg(name="redpajama_chat", system_template=f"{_SYS}", system_message="",
     roles={"user": "<human>", "assistant": "<bot>"}, seps=["\n"], role_content_sep=": ",
     role_empty_sep=":", stop_str=["<human>"], stop_token_ids=[0])
_reg(name="rwkv_world", system_template=f"User: hi\n\nAssistant: {_SYS}",
     system_message="Hi. I am your assistant and I will provide expert full response in full "
                    "details. Please feel free to ask any question and I will always answer it.",
     roles={"user": "User", "assistant": "Assistant"}, seps=["\n\n"], role_content_sep=": ",
     role_empty_sep=": ", stop_str=["\n\n"], stop_token_ids=[0])
_reg(name="gorilla", system_template=f"{_SYS}",
     system_message="A chat between a curious user and an artificial intelligence assistant. The "
                    "assistant gives helpful, detailed, and polite answers to the user's inquiries.",
     role_templates={"user": f"<<question>> {_USER} <<function>> {_FN}"},
     roles={"user": "USER", "assistant": "ASSISTANT", "tool": "USER"}, seps=["\n", "</s>"],
     role_content_sep=": ", role_empty_sep=":", stop_str=["</s>"], stop_token_ids=[2],
     system_prefix_token_ids=[1])
_reg(name="gorilla-openfunctions-v2", system_template=f"{_SYS}",
     system_message="You are an AI programming assistant, utilizing the Gorilla LLM model, "
                    "developed by Gorilla LLM, and you only answer questions related to computer "
                    "science. For politically sensitive questions, security and privacy issues, and "
                    "other non-computer science questions, you will refuse to answer.",
     role_templates={"user": f"<<function>>{_FN}\n<<question>>{_USER}"},
     roles={"user": "### Instruction", "assistant": "### Response", "tool": "### Instruction"},
     seps=["\n", "<|EOT|>"], role_content_sep=": ", role_empty_sep=": ", stop_str=["<|EOT|>"],
     stop_token_ids=[100015], system_prefix_token_ids=[100000])
_reg(name="dolly", system_template=f"{_SYS}",
     system_message="Below is an instruction that describes a task. Write a response that "
                    "appropriately completes the request.",
     roles={"user": "### Instruction", "assistant": "### Response"}, seps=["\n\n", "### End\n"],
     role_content_sep=":\n", role_empty_sep=":\n", stop_str=["### End"], stop_token_ids=[50256])
_reg(name="oasst", system_template=f"{_SYS}", system_message="",
     roles={"user": "<|prompter|>", "assistant": "<|assistant|>"}, seps=["<|endoftext|>"],
     role_content_sep=": ", role_empty_sep=": ", stop_str=["<|endoftext|>"], stop_token_ids=[2])
_reg(name="stablelm", system_template=f"<|SYSTEM|>{_SYS}",
     system_message="# StableLM Tuned (Alpha version)\n- StableLM is a helpful and harmless "
                    "open-source AI language model developed by StabilityAI.\n- StableLM is excited "
                    "to be able to help the user, but will refuse to do anything that could be "
                    "considered harmful to the user.\n- StableLM is more than just an information "
                    "source, StableLM is also able to write poetry, short stories, and make jokes.\n"
                    "- StableLM will refuse to participate in anything that could harm a human.",
     roles={"user": "<|USER|>", "assistant": "<|ASSISTANT|>"}, seps=[""], role_content_sep=": ",
     role_empty_sep=": ", stop_str=[""], stop_token_ids=[50278, 50279, 50277, 1, 0])
_reg(name="stablelm-3b", system_template=f"{_SYS}", system_message="",
     roles={"user": "<|user|>", "assistant": "<|assistant|>"}, seps=["<|endoftext|>"],
     role_content_sep="\n", role_empty_sep="\n", stop_str=["<|endoftext|>"], stop_token_ids=[0])
_reg(name="wizardlm_7b", system_template=f"{_SYS}", system_message="",
     roles={"user": "User", "assistant": "Response"}, seps=["###"], role_content_sep=": ",
     role_empty_sep=":", stop_str=["###"], stop_token_ids=[2], system_prefix_token_ids=[1])
_reg(name="wizard_coder_or_math", system_template=f"{_SYS}",
     system_message="Below is an instruction that describes a task. Write a response that "
                    "appropriately completes the request.",
     roles={"user": "Instruction", "assistant": "Response"}, seps=["\n\n### ", "\n\n### "],
     role_content_sep=":\n", role_empty_sep=":\n", stop_str=["</s>"], stop_token_ids=[2],
     system_prefix_token_ids=[1])
_reg(name="glm", system_template=f"{_SYS}", system_message="",
     roles={"user": "问", "assistant": "答", "tool": "问"}, seps=["\n\n"], role_content_sep=": ",
     role_empty_sep=":", stop_str=["</s>"], stop_token_ids=[2], system_prefix_token_ids=[64790, 64792])
_reg(name="llava", system_template=f"{_SYS}", system_message="\n",
     roles={"user": "USER", "assistant": "ASSISTANT"}, seps=[" "], role_content_sep=": ",
     role_empty_sep=":", stop_str=["</s>"], stop_token_ids=[2], system_prefix_token_ids=[1])
_reg(name="aya-23", system_template=f"<|START_OF_TURN_TOKEN|><|SYSTEM_TOKEN|>{_SYS}<|END_OF_TURN_TOKEN|>",
     system_message="",
     roles={"user": "<|START_OF_TURN_TOKEN|><|USER_TOKEN|>",
            "assistant": "<|START_OF_TURN_TOKEN|><|CHATBOT_TOKEN|>"},
     seps=["<|END_OF_TURN_TOKEN|>"], role_content_sep="", role_empty_sep="",
     stop_str=["<|END_OF_TURN_TOKEN|>"], stop_token_ids=[6, 255001], system_prefix_token_ids=[5])
_reg(name="olmo", system_template=f"{_SYS}", system_message="",
     roles={"user": "<|user|>", "assistant": "<|assistant|>"}, seps=["\n"], role_content_sep="\n",
     role_empty_sep="\n", stop_str=["<|endoftext|>"], stop_token_ids=[50279],
     system_prefix_token_ids=[50279])
_reg(name="olmo2", system_template=f"<|system|>\n{_SYS}\n", system_message="",
     roles={"user": "<|user|>", "assistant": "<|assistant|>"}, seps=["\n", "<|endoftext|>\n"],
     role_content_sep="\n", role_empty_sep="\n", stop_str=["<|endoftext|>"],
     stop_token_ids=[100257], system_prefix_token_ids=[100257])
_reg(name="nemotron", system_template=f"<extra_id_0>System\n{_SYS}\n\n", system_message="",
     roles={"user": "<extra_id_1>User", "assistant": "<extra_id_1>Assistant"}, seps=["\n"],
     role_content_sep="\n", role_empty_sep="\n", stop_str=["<extra_id_1>"], stop_token_ids=[3],
     system_prefix_token_ids=[2])
_reg(name="llm-jp", system_template=f"{_SYS}", system_message="以下は、タスクを説明する指示です。"
     "要求を適切に満たす応答を書きなさい。",
     roles={"user": "\n\n### 指示:", "assistant": "\n\n### 応答:"}, seps=["", "</s>"],
     role_content_sep="\n", role_empty_sep="\n", stop_str=["</s>"], stop_token_ids=[2],
     system_prefix_token_ids=[1])


def get_conv_template(name: str) -> Optional[Conversation]:
    return ConvTemplateRegistry.get_conv_template(name)


__all__ = ["ConvTemplateRegistry", "get_conv_template"]
