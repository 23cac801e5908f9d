"""Chat templates: turn a list of role-tagged messages into token ids with a training mask.

The registry plays the role of paddleformers/datasets/template/template.py (``Template`` :58, ``register_template``
:518): every template knows how to render the system prompt, user / assistant / tool turns, function calls and tool
observations, which end-of-turn tokens to use and whether only assistant turns are trained on. Encoding returns, per
turn pair, the prompt ids (masked out of the loss) and the response ids (trained).
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple


@dataclass
class Template:
    name: str
    format_user: str = "{content}"
    format_assistant: str = "{content}"
    format_system: str = "{content}"
    format_function: str = "{content}"          # assistant turn that calls tools
    format_observation: str = "{content}"       # tool results fed back to the model
    format_tools: str = "{content}"             # tool catalogue appended to the system prompt
    format_prefix: str = ""                     # emitted once at the very start (bos etc.)
    default_system: str = ""
    stop_words: List[str] = field(default_factory=list)
    efficient_eos: bool = False                 # append eos after each assistant turn
    thought_words: Tuple[str, str] = ("<think>", "</think>")
    replace_eos: bool = False

    # ------------------------------------------------------------------ rendering
    def render_tools(self, tools: Optional[Sequence[dict]]) -> str:
        if not tools:
            return ""
        lines = []
        for t in tools:
            fn = t.get("function", t)
            lines.append(json.dumps(fn, ensure_ascii=False))
        return self.format_tools.format(content="\n".join(lines))

    def render_function_call(self, calls) -> str:
        if isinstance(calls, str):
            try:
                calls = json.loads(calls)
            except json.JSONDecodeError:
                return self.format_function.format(content=calls)
        if isinstance(calls, dict):
            calls = [calls]
        body = "\n".join(json.dumps({"name": c.get("name"), "arguments": c.get("arguments", {})}, ensure_ascii=False) for c in calls)
        return self.format_function.format(content=body)

    def render_turns(self, messages: Sequence[dict], system: Optional[str] = None, tools=None) -> List[Tuple[str, str]]:
        """Returns [(prompt text, response text)] pairs; the first prompt carries prefix + system (+ tools)."""
        msgs = list(messages)
        if msgs and msgs[0]["role"] == "system":
            system = msgs.pop(0)["content"]
        system = system if system is not None else self.default_system
        sys_text = ""
        tool_text = self.render_tools(tools)
        if system or tool_text:
            sys_text = self.format_system.format(content=(system or "") + tool_text)
        pairs: List[Tuple[str, str]] = []
        prompt = self.format_prefix + sys_text
        for m in msgs:
            role, content = m["role"], m.get("content", "")
            if role == "user":
                prompt += self.format_user.format(content=content)
            elif role in ("observation", "tool"):
                prompt += self.format_observation.format(content=content)
            elif role in ("assistant", "function", "function_call"):
                if role != "assistant" or m.get("tool_calls"):
                    resp = self.render_function_call(m.get("tool_calls") or content)
                else:
                    resp = self.format_assistant.format(content=content)
                pairs.append((prompt, resp))
                prompt = ""
            else:
                raise ValueError(f"unknown role {role!r}")
        if prompt:
            pairs.append((prompt, ""))  # trailing user turn: inference prompt
        return pairs

    # ------------------------------------------------------------------ tokenisation
    def encode_multiturn(self, tokenizer, messages, system=None, tools=None) -> List[Tuple[List[int], List[int]]]:
        eos = tokenizer.eos_token or ""
        out = []
        for prompt, resp in self.render_turns(messages, system, tools):
            if resp and self.efficient_eos:
                resp = resp + eos
            p_ids = tokenizer.encode(prompt, add_special_tokens=False) if prompt else []
            r_ids = tokenizer.encode(resp, add_special_tokens=False) if resp else []
            out.append((p_ids, r_ids))
        return out

    def encode_oneturn(self, tokenizer, messages, system=None, tools=None) -> Tuple[List[int], List[int]]:
        pairs = self.encode_multiturn(tokenizer, messages, system, tools)
        prompt: List[int] = []
        for p, r in pairs[:-1]:
            prompt += p + r
        prompt += pairs[-1][0]
        return prompt, pairs[-1][1]

    def remove_thought(self, text: str) -> str:
        a, b = self.thought_words
        if a in text and b in text:
            return text.split(b, 1)[1].lstrip("\n")
        return text


TEMPLATES: Dict[str, Template] = {}


def register_template(name: str, **kw) -> Template:
    t = Template(name=name, **kw)
    TEMPLATES[name] = t
    return t


def get_template(name: Optional[str]) -> Template:
    if not name:
        return TEMPLATES["empty"]
    if name not in TEMPLATES:
        raise ValueError(f"unknown template {name!r}; registered: {sorted(TEMPLATES)}")
    return TEMPLATES[name]


_TOOLS_GENERIC = ("\n\n# Tools\n\nYou may call one or more functions to assist with the user query.\n<tools>\n{content}\n</tools>\n\n"
                  "For each function call, return a json object with function name and arguments within "
                  "<tool_call></tool_call> XML tags.")

register_template("empty", efficient_eos=True)
register_template("default", format_user="Human: {content}\nAssistant: ", format_assistant="{content}\n",
                  format_system="System: {content}\n", efficient_eos=True)
register_template("alpaca", format_user="### Instruction:\n{content}\n\n### Response:\n", format_assistant="{content}\n\n",
                  default_system="Below is an instruction that describes a task. Write a response that appropriately completes the request.\n\n",
                  efficient_eos=True)
register_template("chatml", format_user="<|im_start|>user\n{content}<|im_end|>\n<|im_start|>assistant\n",
                  format_assistant="{content}<|im_end|>\n", format_system="<|im_start|>system\n{content}<|im_end|>\n",
                  format_observation="<|im_start|>user\n<tool_response>\n{content}\n</tool_response><|im_end|>\n<|im_start|>assistant\n",
                  format_function="<tool_call>\n{content}\n</tool_call><|im_end|>\n", format_tools=_TOOLS_GENERIC,
                  stop_words=["<|im_end|>"], replace_eos=True)
register_template("qwen", format_user="<|im_start|>user\n{content}<|im_end|>\n<|im_start|>assistant\n",
                  format_assistant="{content}<|im_end|>\n", format_system="<|im_start|>system\n{content}<|im_end|>\n",
                  format_observation="<|im_start|>user\n<tool_response>\n{content}\n</tool_response><|im_end|>\n<|im_start|>assistant\n",
                  format_function="<tool_call>\n{content}\n</tool_call><|im_end|>\n", format_tools=_TOOLS_GENERIC,
                  default_system="You are a helpful assistant.", stop_words=["<|im_end|>"], replace_eos=True)
register_template("qwen3", format_user="<|im_start|>user\n{content}<|im_end|>\n<|im_start|>assistant\n",
                  format_assistant="{content}<|im_end|>\n", format_system="<|im_start|>system\n{content}<|im_end|>\n",
                  format_observation="<|im_start|>user\n<tool_response>\n{content}\n</tool_response><|im_end|>\n<|im_start|>assistant\n",
                  format_function="<tool_call>\n{content}\n</tool_call><|im_end|>\n", format_tools=_TOOLS_GENERIC,
                  stop_words=["<|im_end|>"], replace_eos=True)
register_template("llama3", format_prefix="<|begin_of_text|>",
                  format_user="<|start_header_id|>user<|end_header_id|>\n\n{content}<|eot_id|><|start_header_id|>assistant<|end_header_id|>\n\n",
                  format_assistant="{content}<|eot_id|>",
                  format_system="<|start_header_id|>system<|end_header_id|>\n\n{content}<|eot_id|>",
                  format_observation="<|start_header_id|>ipython<|end_header_id|>\n\n{content}<|eot_id|><|start_header_id|>assistant<|end_header_id|>\n\n",
                  format_function="{content}<|eot_id|>", format_tools="\n\nYou have access to the following functions:\n{content}",
                  stop_words=["<|eot_id|>", "<|eom_id|>"], replace_eos=True)
register_template("deepseek3", format_prefix="<｜begin▁of▁sentence｜>", format_user="<｜User｜>{content}<｜Assistant｜>",
                  format_assistant="{content}<｜end▁of▁sentence｜>", format_system="{content}",
                  format_observation="<｜tool▁outputs▁begin｜><｜tool▁output▁begin｜>{content}<｜tool▁output▁end｜><｜tool▁outputs▁end｜>",
                  format_function="<｜tool▁calls▁begin｜>{content}<｜tool▁calls▁end｜><｜end▁of▁sentence｜>")
register_template("glm4", format_prefix="[gMASK]<sop>", format_user="<|user|>\n{content}<|assistant|>",
                  format_assistant="\n{content}", format_system="<|system|>\n{content}",
                  format_observation="<|observation|>\n{content}<|assistant|>", format_function="\n{content}",
                  format_tools="\n\n# 可用工具\n{content}", stop_words=["<|user|>", "<|observation|>"], efficient_eos=True)
register_template("glm4_moe", format_prefix="[gMASK]<sop>", format_user="<|user|>\n{content}<|assistant|>",
                  format_assistant="\n{content}", format_system="<|system|>\n{content}",
                  format_observation="<|observation|>\n<tool_response>\n{content}\n</tool_response><|assistant|>",
                  format_function="\n<tool_call>{content}</tool_call>", format_tools=_TOOLS_GENERIC,
                  stop_words=["<|user|>", "<|observation|>"], efficient_eos=True)
register_template("mistral", format_prefix="<s>", format_user="[INST] {content}[/INST]", format_assistant=" {content}</s>",
                  format_system="{content}\n\n")
register_template("gemma", format_prefix="<bos>", format_user="<start_of_turn>user\n{content}<end_of_turn>\n<start_of_turn>model\n",
                  format_assistant="{content}<end_of_turn>\n", format_system="{content}\n\n", stop_words=["<end_of_turn>"])
register_template("phi4", format_user="<|im_start|>user<|im_sep|>{content}<|im_end|><|im_start|>assistant<|im_sep|>",
                  format_assistant="{content}<|im_end|>", format_system="<|im_start|>system<|im_sep|>{content}<|im_end|>",
                  stop_words=["<|im_end|>"])
register_template("ernie", format_prefix="<|begin_of_sentence|>", format_user="User: {content}\nAssistant: ",
                  format_assistant="{content}<|end_of_sentence|>", format_system="{content}\n")

# ---- further public chat formats (as published on the respective model cards) -------------------------------------------
_CHATML = dict(format_user="<|im_start|>user\n{content}<|im_end|>\n<|im_start|>assistant\n", format_assistant="{content}<|im_end|>\n",
               format_system="<|im_start|>system\n{content}<|im_end|>\n", stop_words=["<|im_end|>"], replace_eos=True)
register_template("llama2", format_prefix="<s>", format_user="[INST] {content} [/INST]", format_assistant=" {content} </s><s>",
                  format_system="<<SYS>>\n{content}\n<</SYS>>\n\n")
register_template("llama4", format_prefix="<|begin_of_text|>",
                  format_user="<|header_start|>user<|header_end|>\n\n{content}<|eot|><|header_start|>assistant<|header_end|>\n\n",
                  format_assistant="{content}<|eot|>", format_system="<|header_start|>system<|header_end|>\n\n{content}<|eot|>",
                  format_observation="<|header_start|>ipython<|header_end|>\n\n{content}<|eot|><|header_start|>assistant<|header_end|>\n\n",
                  format_function="{content}<|eot|>", stop_words=["<|eot|>", "<|eom|>"], replace_eos=True)
register_template("vicuna", format_user="USER: {content} ASSISTANT:", format_assistant=" {content}</s>", format_system="{content} ",
                  default_system="A chat between a curious user and an artificial intelligence assistant. The assistant gives "
                                 "helpful, detailed, and polite answers to the user's questions.")
register_template("zephyr", format_user="<|user|>\n{content}</s>\n<|assistant|>\n", format_assistant="{content}</s>\n",
                  format_system="<|system|>\n{content}</s>\n")
register_template("yi", **_CHATML)
register_template("qwen2_vl", default_system="You are a helpful assistant.", **_CHATML)
register_template("qwen3_nothink", format_user="<|im_start|>user\n{content}<|im_end|>\n<|im_start|>assistant\n<think>\n\n</think>\n\n",
                  format_assistant="{content}<|im_end|>\n", format_system="<|im_start|>system\n{content}<|im_end|>\n",
                  stop_words=["<|im_end|>"], replace_eos=True)
register_template("minicpm", **_CHATML)
register_template("internlm2", format_prefix="<s>", format_observation="<|im_start|>environment\n{content}<|im_end|>\n<|im_start|>assistant\n",
                  **_CHATML)
register_template("internlm3", format_prefix="<s>", **_CHATML)
register_template("seed_oss", format_prefix="<seed:bos>", format_user="user\n{content}<seed:eos><seed:bos>assistant\n",
                  format_assistant="{content}<seed:eos>", format_system="system\n{content}<seed:eos><seed:bos>", stop_words=["<seed:eos>"])
register_template("baichuan2", format_user="<reserved_106>{content}<reserved_107>", format_assistant="{content}", format_system="{content}",
                  efficient_eos=True)
register_template("deepseek", format_prefix="<｜begin▁of▁sentence｜>", format_user="User: {content}\n\nAssistant:",
                  format_assistant=" {content}<｜end▁of▁sentence｜>", format_system="{content}\n\n")
register_template("deepseek_coder", format_prefix="<｜begin▁of▁sentence｜>", format_user="### Instruction:\n{content}\n### Response:\n",
                  format_assistant="{content}\n<|EOT|>\n", format_system="{content}\n", stop_words=["<|EOT|>"],
                  default_system="You are an AI programming assistant, utilizing the DeepSeek Coder model, developed by DeepSeek "
                                 "Company, and you only answer questions related to computer science.")
register_template("deepseek_r1", format_prefix="<｜begin▁of▁sentence｜>", format_user="<｜User｜>{content}<｜Assistant｜>",
                  format_assistant="{content}<｜end▁of▁sentence｜>", format_system="{content}")
register_template("gemma3", format_prefix="<bos>", format_user="<start_of_turn>user\n{content}<end_of_turn>\n<start_of_turn>model\n",
                  format_assistant="{content}<end_of_turn>\n", format_system="{content}\n\n", stop_words=["<end_of_turn>"], replace_eos=True)
register_template("phi3", format_user="<|user|>\n{content}<|end|>\n<|assistant|>\n", format_assistant="{content}<|end|>\n",
                  format_system="<|system|>\n{content}<|end|>\n", stop_words=["<|end|>"], replace_eos=True)
register_template("cohere", format_prefix="<BOS_TOKEN>",
                  format_user="<|START_OF_TURN_TOKEN|><|USER_TOKEN|>{content}<|END_OF_TURN_TOKEN|><|START_OF_TURN_TOKEN|><|CHATBOT_TOKEN|>",
                  format_assistant="{content}<|END_OF_TURN_TOKEN|>",
                  format_system="<|START_OF_TURN_TOKEN|><|SYSTEM_TOKEN|>{content}<|END_OF_TURN_TOKEN|>", stop_words=["<|END_OF_TURN_TOKEN|>"])
register_template("falcon", format_user="User: {content}\nFalcon:", format_assistant=" {content}\n", format_system="{content}\n",
                  efficient_eos=True)
register_template("olmo", format_user="<|user|>\n{content}\n<|assistant|>\n", format_assistant="{content}<|endoftext|>\n",
                  format_system="<|system|>\n{content}\n")
register_template("granite3", format_user="<|start_of_role|>user<|end_of_role|>{content}<|end_of_text|>\n<|start_of_role|>assistant<|end_of_role|>",
                  format_assistant="{content}<|end_of_text|>\n", format_system="<|start_of_role|>system<|end_of_role|>{content}<|end_of_text|>\n",
                  stop_words=["<|end_of_text|>"])
register_template("hunyuan", format_prefix="<|startoftext|>", format_user="{content}<|extra_0|>", format_assistant="{content}<|eos|>",
                  format_system="{content}<|extra_4|>", stop_words=["<|eos|>"])
register_template("kimi", format_user="<|im_user|>user<|im_middle|>{content}<|im_end|><|im_assistant|>assistant<|im_middle|>",
                  format_assistant="{content}<|im_end|>", format_system="<|im_system|>system<|im_middle|>{content}<|im_end|>",
                  stop_words=["<|im_end|>"])
register_template("gpt_oss", format_user="<|start|>user<|message|>{content}<|end|><|start|>assistant",
                  format_assistant="<|channel|>final<|message|>{content}<|end|>", format_system="<|start|>system<|message|>{content}<|end|>",
                  stop_words=["<|return|>", "<|end|>"], thought_words=("<|channel|>analysis<|message|>", "<|end|><|start|>assistant"))
register_template("ernie_nothink", format_prefix="<|begin_of_sentence|>", format_user="User: {content}\nAssistant: <think>\n\n</think>\n\n",
                  format_assistant="{content}<|end_of_sentence|>", format_system="{content}\n")
register_template("mistral_small", format_prefix="<s>", format_user="[INST]{content}[/INST]", format_assistant="{content}</s>",
                  format_system="[SYSTEM_PROMPT]{content}[/SYSTEM_PROMPT]")
register_template("minimax", format_user="<beginning_of_sentence>user name=user\n{content}<end_of_sentence>\n<beginning_of_sentence>ai name=assistant\n",
                  format_assistant="{content}<end_of_sentence>\n", format_system="<beginning_of_sentence>system ai_setting=assistant\n{content}<end_of_sentence>\n",
                  stop_words=["<end_of_sentence>"])
register_template("xverse", format_user="Human: {content}\n\nAssistant: ", format_assistant="{content}", efficient_eos=True)
register_template("openchat", format_user="GPT4 Correct User: {content}<|end_of_turn|>GPT4 Correct Assistant:",
                  format_assistant=" {content}<|end_of_turn|>", format_system="{content}<|end_of_turn|>", stop_words=["<|end_of_turn|>"])
register_template("solar", format_user="### User:\n{content}\n\n### Assistant:\n", format_assistant="{content}\n\n",
                  format_system="### System:\n{content}\n\n", efficient_eos=True)
register_template("starchat", format_user="<|user|>\n{content}<|end|>\n<|assistant|>", format_assistant="\n{content}<|end|>\n",
                  format_system="<|system|>\n{content}<|end|>\n", stop_words=["<|end|>"])
