"""Chat templates by name.

Same names and rendered text as the ``CHAT_TEMPLATES`` table of the reference
(``open_instruct/dataset_transformation.py:152-641``) so that tokenised datasets and label masks are
interchangeable, but the Jinja sources are assembled here from small building blocks: a template
is described by how each role is framed, what closes an assistant turn, and what the generation
prompt is.  ``render(name, messages, ...)`` renders without a tokenizer (tests, tools).
"""

from __future__ import annotations

import jinja2


def _role_block(role: str, body: str) -> str:
    return "{% if message['role'] == '" + role + "' %}" + body


def _tagged(sys_fmt: str, user_fmt: str, asst_open: str, asst_mid_close: str, asst_last_close: str, gen: str,
            content_setup: str = "", preamble: str = "") -> str:
    """Role-tag families (tulu, zephyr): per-role framing, assistant turns closed differently when last."""
    return (
        preamble
        + "{% for message in messages %}"
        + "{% if message['role'] == 'system' %}{{ " + sys_fmt + " }}"
        + "{% elif message['role'] == 'user' %}{{ " + user_fmt + " }}"
        + "{% elif message['role'] == 'assistant' %}"
        + content_setup
        + "{% if not loop.last %}{{ " + asst_open + " + " + asst_mid_close + " }}"
        + "{% else %}{{ " + asst_open + " + " + asst_last_close + " }}{% endif %}"
        + "{% endif %}"
        + "{% if loop.last and add_generation_prompt %}{{ " + gen + " }}{% endif %}"
        + "{% endfor %}"
    )


def _concat(sep: str, body: str) -> str:
    """Plain concatenation families: separator between messages, eos after the last one."""
    return (
        "{% for message in messages %}"
        "{{ " + repr(sep) + " if not loop.first else '' }}"
        "{{ " + body + " }}"
        "{% if loop.last and not add_generation_prompt %}{{ eos_token }}{% endif %}"
        "{% endfor %}"
    )


_FUNCS_NONE = " You do not currently have access to any functions. <functions></functions><|im_end|>\n"


def _olmo(default_system: str, gen: str, strip_thinking: bool = False) -> str:
    """``<|im_start|>role`` families with optional function-calling fields."""
    content = (
        "{% if message.get('content', none) is not none %}{{ message['content'] }}{% endif %}"
        if not strip_thinking
        else "{% set content = message.get('content', none) %}{% if content is not none %}"
             "{% set content = content | string %}"
             "{% if '</think>' in content and not loop.last %}"
             "{% set content = content.split('</think>')[-1].lstrip('\\n') %}{% endif %}"
             "{{ content }}{% endif %}"
    )
    return (
        "{% set has_system = messages|selectattr('role', 'equalto', 'system')|list|length > 0 %}"
        "{% if not has_system %}{{ " + repr("<|im_start|>system\n" + default_system + "<|im_end|>\n") + " }}{% endif %}"
        "{% for message in messages %}"
        "{% if message['role'] == 'system' %}{{ '<|im_start|>system\n' + message['content'] }}"
        "{% if message.get('functions', none) is not none %}"
        "{{ ' <functions>' + message['functions'] + '</functions><|im_end|>\n' }}"
        "{% else %}{{ " + repr(_FUNCS_NONE) + " }}{% endif %}"
        "{% elif message['role'] == 'user' %}"
        "{% if message.get('functions', none) is not none %}"
        "{{ '<|im_start|>user\n' + message['content'] + '\n' + '<functions>' + message['functions'] + '</functions><|im_end|>\n' }}"
        "{% else %}{{ '<|im_start|>user\n' + message['content'] + '<|im_end|>\n' }}{% endif %}"
        "{% elif message['role'] == 'assistant' %}{{ '<|im_start|>assistant\n' }}"
        + content
        + "{% if message.get('function_calls', none) is not none %}"
        "{{ '<function_calls>' + message['function_calls'] + '</function_calls>' }}{% endif %}"
        "{% if not loop.last %}{{ '<|im_end|>' + '\n' }}{% else %}{{ eos_token }}{% endif %}"
        "{% elif message['role'] == 'environment' %}"
        "{{ '<|im_start|>environment\n' + message['content'] + '<|im_end|>\n' }}"
        "{% endif %}"
        "{% if loop.last and add_generation_prompt %}{{ " + repr(gen) + " }}{% endif %}"
        "{% endfor %}"
    )


_R1_PREAMBLE = (
    "A conversation between User and Assistant. The user asks a question, and the Assistant solves it. "
    "The assistant first thinks about the reasoning process in the mind and then provides the user with the answer. "
    "The reasoning process and answer are enclosed within <think> </think> and <answer> </answer> tags, respectively, "
    "i.e., <think> reasoning process here </think> <answer> answer here </answer>."
    "\n\n"
)


def _r1(gen: str, body: str = "message['role'].capitalize() + ': ' + message['content'] + '\n'",
        preamble: str = _R1_PREAMBLE) -> str:
    return (
        preamble
        + "{% for message in messages %}"
        "{{ '\n\n' if not loop.first else '' }}"
        "{{ " + body + " }}"
        "{% if loop.last and add_generation_prompt %}{{ " + repr(gen) + " }}{% endif %}"
        "{% endfor %}"
    )


_OLMO_FC_SYSTEM = ("You are OLMo, a helpful function-calling AI assistant built by Ai2. Your date cutoff is November 2024, "
                   "and your model weights are available at https://huggingface.co/allenai. You do not currently have "
                   "access to any functions. <functions></functions>")
_OLMO_7B_SYSTEM = ("You are Olmo, a helpful AI assistant built by Ai2. Your date cutoff is December 2024, and your model "
                   "weights are available at https://huggingface.co/allenai.")
_TOOL_PREAMBLE = (
    "A conversation between User and Assistant. The User asks a question, and the Assistant solves it. "
    "The Assistant first thinks about the reasoning process in the mind and then provides the User with the answer. "
    "\n\n"
    "When given a question, the Assistant must conduct reasoning inside the <think> and </think> tags. "
    "During reasoning, the Assistant may write and execute python code using the <code> </code> tag, in order to solve "
    "the problem or verify the answer. Then the Assistant will get the stdout and stderr in the <output> and </output> tags. "
    "For example, the code could be\n<code>\nx, y = 1, 2\nresult = x + y\nprint(result)\n</code>\nor\n<code>\n"
    "import sympy as sp\nfrom sympy import Symbol\nx = Symbol('x')\ny = Symbol('y')\n"
    "solution = sp.solve(x**2 + y**2 - 1, (x, y))\nprint(solution)\n</code>\n"
    "The Assistant will always `print` the result of the code execution in order to see it in the <output> tag. "
    "The Assistant may use the <code> </code> tag multiple times. "
    "When the Assistant is done reasoning, it should provide the answer inside the <answer> and </answer> tag."
    "\n\n"
)

_ORZ_BODY = ("message['role'].capitalize() + ': You must put your answer inside <answer> </answer> tags, i.e., "
             "<answer> answer here </answer>. And your final answer will be extracted automatically by the \\\\boxed{} tag. "
             "This is the problem: ' + message['content'] + '\n'")

CHAT_TEMPLATES: dict[str, str] = {
    "simple_concat_with_space": _concat(" ", "message['content']"),
    "simple_concat_with_new_line": _concat("\n", "message['content']"),
    "simple_chat": _concat("\n\n", "message['role'].capitalize() + ': ' + message['content']"),
    "assistant_message_only": "{% for message in messages %}{% if message['role'] == 'assistant' %}"
                              "{{ message['content'] }}{% endif %}{% endfor %}",
    "zephyr": (
        "{% for message in messages %}"
        "{% if message['role'] in ('user', 'system', 'assistant') %}"
        "{{ '<|' + message['role'] + '|>\n' + message['content'] + eos_token + '\n' }}{% endif %}"
        "{% if loop.last and add_generation_prompt %}{{ '<|assistant|>\n' }}{% endif %}"
        "{% endfor %}"
    ),
    "tulu": _tagged("'<|system|>\n' + message['content'] + '\n'", "'<|user|>\n' + message['content'] + '\n'",
                    "'<|assistant|>\n' + message['content']", "eos_token + '\n'", "eos_token", "'<|assistant|>\n'"),
    "tulu_thinker": _tagged("'<|system|>\n' + message['content'] + '\n'", "'<|user|>\n' + message['content'] + '\n'",
                            "'<|assistant|>\n' + message['content']", "eos_token + '\n'", "eos_token",
                            "'<|assistant|>\n<think>'"),
    "tulu_thinker_r1_style": _tagged(
        "'<|system|>\n' + message['content'] + '\n'", "'<|user|>\n' + message['content'] + '\n'",
        "'<|assistant|>\n' + content", "eos_token + '\n'", "eos_token", "'<|assistant|>\n<think>'",
        content_setup="{% set content = message['content'] %}{% if '</think>' in content %}"
                      "{% set content = content.split('</think>')[-1] %}{% endif %}",
        preamble=_R1_PREAMBLE),
    "olmo": _olmo(_OLMO_FC_SYSTEM, "<|im_start|>assistant\n"),
    "olmo_old": _olmo(_OLMO_FC_SYSTEM, "<|im_start|>assistant\n"),
    "olmo_thinker": _olmo("You are a helpful AI assistant.", "<|im_start|>assistant\n<think>"),
    "olmo_thinker_no_think_7b": _olmo(_OLMO_7B_SYSTEM, "<|im_start|>assistant\n"),
    "olmo_thinker_remove_intermediate_thinking": _olmo("You are a helpful AI assistant.", "<|im_start|>assistant\n<think>",
                                                       strip_thinking=True),
    "olmo_thinker_no_think_sft_tokenization": _olmo("You are a helpful AI assistant.", "<|im_start|>assistant\n"),
    "olmo_thinker_rlzero": _r1(
        "\nRemember to put your answer on its own line after \"Answer:\"", body="message['content'] + '\n'",
        preamble="Solve the following problem step by step. The last line of your response should be the answer to the "
                 "problem in form Answer: $Answer (without quotes) where $Answer is the answer to the problem.\n\n"),
    "olmo_thinker_code_rlzero": _r1(
        "\nRemember to put your solution inside the ```\npython\nCODE\n``` tags", body="message['content'] + '\n'",
        preamble="Solve the following code problem step by step. The last part of your response should be the solution "
                 "to the problem in form ```\npython\nCODE\n``` where CODE is the solution for the problem.\n\n"),
    "r1_simple_chat": _r1("Assistant:"),
    "r1_simple_chat_postpend_think": _r1("Assistant: <think>"),
    "r1_simple_chat_postpend_think_orz_style": _r1("Assistant: <think>", body=_ORZ_BODY),
    "r1_simple_chat_postpend_think_tool_vllm": _r1("Assistant: <think>", body=_ORZ_BODY, preamble=_TOOL_PREAMBLE),
    "qwen_instruct_user_boxed_math": (
        "{% for message in messages %}"
        "{% if message['role'] == 'user' %}"
        "{{ '<|im_start|>user\n' + message['content'] + '\n\nPlease reason step by step, and put your final answer within \\\\boxed{}<|im_end|>\n' }}"
        "{% elif message['role'] == 'assistant' %}{{ '<|im_start|>assistant\n' + message['content'] + '<|im_end|>\n' }}{% endif %}"
        "{% if loop.last and add_generation_prompt %}{{ '<|im_start|>assistant\n' }}{% endif %}"
        "{% endfor %}"
    ),
}

_env = jinja2.Environment(keep_trailing_newline=True)


def render(template: str, messages: list[dict], add_generation_prompt: bool = False, eos_token: str = "</s>",
           bos_token: str = "<s>") -> str:
    """Render a named (or literal) chat template without a tokenizer."""
    src = CHAT_TEMPLATES.get(template, template)
    return _env.from_string(src).render(messages=messages, add_generation_prompt=add_generation_prompt,
                                        eos_token=eos_token, bos_token=bos_token)
