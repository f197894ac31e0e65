"""Verifier behaviour on input/output pairs (puzzle matcher, F1, GSM8K) that a user migrating from the reference relies on."""

import pytest

from open_instruct_b200 import ground_truth_utils as gtu

PUZZLE = [
    ("The answer is 42", "answer is 42", 1.0), ("<think>Let me solve this</think>Paris", "paris", 1.0),
    ("<answer>New York City!</answer>", "new york city", 1.0), ("Wrong answer", "correct answer", 0.0),
    ("<think>This is about geography</think><answer>The capital of France is Paris.</answer>", "capital of france is paris", 1.0),
    ("42", "42", 1.0), ("Hello World", "hello world", 1.0), ("<think>Analysis...</think>Wrong Answer", "42", 0.0),
    ("<answer>wrong</answer>", "42", 0.0), ("<think>Thinking...</think><answer>42</answer>", "42", 1.0),
    ("A simple test.", "simple test", 1.0), ("Hello, world!", "hello world", 1.0), ("  hello   world  ", "hello world", 1.0),
    ("hello\tworld\n", "hello world", 1.0), ("42", "43", 0.0), ("", "42", 0.0), ("<think>Animal question</think>The elephant", "elephant", 1.0),
    ("Romeo and Juliet by Shakespeare", "romeo and juliet by shakespeare", 1.0),
]
F1 = [
    ("hello world", "hello world", 1.0), ("hello world", "hello", 2 / 3), ("hello world", "goodbye", 0.0),
    ("<think>Let me think...</think>hello world", "hello world", 1.0), ("<think>Analysis</think>hello world", "hello", 2 / 3),
    ("<answer>hello world</answer>", "hello world", 1.0), ("<think>Thinking...</think><answer>hello world</answer>", "hello world", 1.0),
    ("hello world", ["hello world", "goodbye"], 1.0), ("hello world", ["goodbye", "hello world"], 1.0), ("hello world", ["hello", "world"], 2 / 3),
    ("hello world", ["foo", "bar", "baz"], 0.0), ("<think>hmm</think>hello world", ["goodbye", "hello world"], 1.0),
]
GSM = [
    ("Therefore the answer is -3", "-3", 1.0), ("Therefore the answer is +7", "+7", 1.0), ("Final answer: -3.5", "-3.5", 1.0),
    (r"The result is \\boxed{-3}", "-3", 1.0), ("Therefore the answer is 3", "-3", 0.0),
]


@pytest.mark.parametrize("pred,label,want", PUZZLE)
def test_puzzle_matcher(pred, label, want):
    assert gtu.PuzzleMatcherVerifier()([], pred, label).score == want


@pytest.mark.parametrize("pred,label,want", F1)
def test_f1(pred, label, want):
    assert abs(gtu.F1Verifier()([], pred, label).score - want) < 1e-5


@pytest.mark.parametrize("pred,label,want", GSM)
def test_gsm8k_signed_numbers(pred, label, want):
    assert gtu.GSM8KVerifier()([], pred, label).score == want


# ------------------------------------------------------------------ instruction-following constraint functions
@pytest.mark.parametrize("text,n,quant,want", [
    ("AAA BBB CCC DDD EEE", 5, "around", True),
    ("AAA BBB CCC DDD", 5, "around", True),
    ("AAA BBB CCC DDD EEE FFF", 5, "around", True),
    ("AAA BBB", 5, "around", False),
    ("AAA BBB CCC", 2, "at least", True),
    ("AAA BBB CCC DDD", 2, "at most", False),
    ("AAA BBB", 2, "no such quantifier", False),
])
def test_capital_word_frequency(text, n, quant, want):
    from open_instruct_b200 import if_functions
    assert if_functions.validate_frequency_capital_words(text, n, quant) is want


@pytest.mark.parametrize("text,options,want", [
    ("I believe the answer is B", ["A", "B", "C", "D"], True),
    ("I choose red", ["red", "blue"], True),
    ("I choose green", ["red", "blue"], False),
    ("red", ["red", "blue"], True),
])
def test_validate_choice(text, options, want):
    from open_instruct_b200 import if_functions
    assert if_functions.validate_choice(text, options) is want


def test_around_tolerances():
    from open_instruct_b200 import if_functions
    words = " ".join(["w"] * 112)
    assert if_functions.validate_word_constraint(words, 100, "around") is False
    assert if_functions.validate_word_constraint(" ".join(["w"] * 91), 100, "around") is True
    assert if_functions.verify_sentence_constraint("One. Two. Three.", 4, "around") is True
    assert if_functions.verify_sentence_constraint("One. Two.", 4, "around") is False
