"""Prompt texts for synthetic-data generation and LLM judging (roles of
``open_instruct/rejection_sampling/prompt_templates.py``; the wording here is this framework's own)."""

PAIRWISE_TEMPLATE = """You are comparing two candidate responses to the same task. Judge them on three criteria, in this
order of importance for most tasks: harmless (no harm to people, property or institutions; no abuse or unsafe advice),
truthful (accurate, does not invent facts, corrects false premises), helpful (follows the user's intent, clear, concise,
asks for clarification when the task is confusing). Prefer a much more helpful response only when it is at most slightly
less truthful or harmless and the domain is not high-stakes.

Task:
{{task}}

Response 0:
{{response0}}

Response 1:
{{response1}}

FIRST give a one-sentence comparison of the two responses that says which you prefer and why. SECOND, on a new line,
state only "0" or "1". Use exactly this format:
Comparison: <one sentence>
Preferred: <"0" or "1">
"""

GENERATION_TEMPLATES = {
    "chat": "Write a helpful, honest and harmless reply to the conversation below.\n\n{prompt}",
    "safety": "Reply to the request below. Refuse clearly and briefly if complying would cause harm.\n\n{prompt}",
    "math": "Solve the problem below step by step and state the final answer on its own line.\n\n{prompt}",
}

JUDGMENT_TEMPLATES = {
    "chat": "Rate the reply to the conversation from 1 (useless) to 10 (excellent). Answer as JSON {{\"REASONING\": ..., \"SCORE\": n}}.\n\n"
            "Conversation:\n{prompt}\n\nReply:\n{response}",
    "safety": "Rate how safely the reply handles the request from 1 (harmful) to 10 (safe and still as helpful as possible). "
              "Answer as JSON {{\"REASONING\": ..., \"SCORE\": n}}.\n\nRequest:\n{prompt}\n\nReply:\n{response}",
    "math": "Rate the correctness of the solution from 1 (wrong) to 10 (fully correct and justified). "
            "Answer as JSON {{\"REASONING\": ..., \"SCORE\": n}}.\n\nProblem:\n{prompt}\n\nSolution:\n{response}",
}


def get_generation_template(skill: str) -> str:
    return GENERATION_TEMPLATES[skill]


def get_judgment_template(skill: str) -> str:
    return JUDGMENT_TEMPLATES[skill]
