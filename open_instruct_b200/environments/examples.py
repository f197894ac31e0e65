"""Small reference environments: a counter, a number-guessing game and Wordle
(cf. ``open_instruct/environments/examples.py``).  They exercise the multi-turn machinery in tests."""

from __future__ import annotations

import random
import re

from .base import RLEnvironment, StepResult, TextRLEnvironment, ToolCall


class CounterEnv(RLEnvironment):
    """Reach ``target`` by calling increment / decrement, then submit."""

    config_name = "counter"

    def __init__(self, target: int = 3):
        self.default_target = target

    @classmethod
    def get_tool_definitions(cls):
        mk = lambda n, d: {"type": "function", "function": {"name": n, "description": d, "parameters": {"type": "object", "properties": {}, "required": []}}}
        return [mk("increment", "add one"), mk("decrement", "subtract one"), mk("submit", "finish")]

    def reset(self, target: int | None = None, **_):
        self.target = self.default_target if target is None else int(target)
        self.value, self.steps = 0, 0
        return StepResult(f"Counter is 0. Reach {self.target} and submit.")

    def step(self, call: ToolCall) -> StepResult:
        self.steps += 1
        if call.name == "increment":
            self.value += 1
        elif call.name == "decrement":
            self.value -= 1
        elif call.name == "submit":
            ok = self.value == self.target
            return StepResult("correct" if ok else f"wrong: counter is {self.value}", 1.0 if ok else 0.0, True)
        else:
            return StepResult(f"unknown tool {call.name}", -0.05, False)
        return StepResult(f"Counter is {self.value}.", 0.0, self.steps >= self.max_steps)

    def state(self):
        return {"value": self.value, "target": self.target}


class GuessNumberEnv(RLEnvironment):
    config_name = "guess_number"

    def __init__(self, low: int = 1, high: int = 100, seed: int | None = None):
        self.low, self.high, self.rng = low, high, random.Random(seed)

    @classmethod
    def get_tool_definitions(cls):
        return [{"type": "function", "function": {"name": "guess", "description": "guess the number",
                                                  "parameters": {"type": "object", "properties": {"number": {"type": "integer"}}, "required": ["number"]}}}]

    def reset(self, secret: int | None = None, **_):
        self.secret = self.rng.randint(self.low, self.high) if secret is None else int(secret)
        self.steps = 0
        return StepResult(f"Guess a number between {self.low} and {self.high}.")

    def step(self, call: ToolCall) -> StepResult:
        self.steps += 1
        try:
            g = int(call.args.get("number"))
        except (TypeError, ValueError):
            return StepResult("number must be an integer", -0.05, self.steps >= self.max_steps)
        if g == self.secret:
            return StepResult("correct", 1.0, True)
        hint = "higher" if g < self.secret else "lower"
        closeness = 1.0 - abs(g - self.secret) / (self.high - self.low)
        return StepResult(hint, 0.1 * closeness if self.steps >= self.max_steps else 0.0, self.steps >= self.max_steps)


class WordleTextEnv(TextRLEnvironment):
    """Text environment: the model writes ``<guess>WORD</guess>``; feedback uses G/Y/X per letter;
    reward 1 for solving, plus a bonus for using few turns."""

    config_name = "wordle"
    WORDS = ["crane", "slate", "pride", "ghost", "flame", "brick", "jumpy", "waltz"]
    max_steps = 6

    def __init__(self, seed: int | None = None):
        self.rng = random.Random(seed)

    def reset(self, word: str | None = None, **_):
        self.word = (word or self.rng.choice(self.WORDS)).lower()
        self.turn = 0
        return StepResult("Guess the 5-letter word. Answer with <guess>WORD</guess>.")

    @staticmethod
    def feedback(guess: str, word: str) -> str:
        out, rest = ["X"] * 5, list(word)
        for i, (g, w) in enumerate(zip(guess, word)):
            if g == w:
                out[i] = "G"
                rest[i] = None
        for i, g in enumerate(guess):
            if out[i] == "X" and g in rest:
                out[i] = "Y"
                rest[rest.index(g)] = None
        return "".join(out)

    def text_step(self, text: str) -> StepResult:
        self.turn += 1
        m = re.search(r"<guess>\s*([A-Za-z]{5})\s*</guess>", text)
        if not m:
            return StepResult("Invalid format. Use <guess>WORD</guess> with a 5-letter word.", -0.05, self.turn >= self.max_steps)
        g = m.group(1).lower()
        if g == self.word:
            return StepResult("GGGGG - solved", 1.0 + 0.1 * (self.max_steps - self.turn), True)
        return StepResult(self.feedback(g, self.word), 0.0, self.turn >= self.max_steps)
