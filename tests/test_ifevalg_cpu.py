"""IFEval-G constraint checkers: one satisfied and one violated response per constraint id, the text utilities they
share, and the contract that an unknown id raises (it used to score zero silently)."""

import json

import pytest

from open_instruct_b200 import ifevalg
from open_instruct_b200.ifevalg import check_instruction

REFERENCE_IDS = """keywords:existence keywords:frequency keywords:forbidden_words keywords:letter_frequency language:response_language
length_constraints:number_sentences length_constraints:number_paragraphs length_constraints:number_words
length_constraints:nth_paragraph_first_word detectable_content:number_placeholders detectable_content:postscript
detectable_format:number_bullet_lists detectable_format:constrained_response detectable_format:number_highlighted_sections
detectable_format:multiple_sections detectable_format:json_format detectable_format:title combination:two_responses
combination:repeat_prompt startend:end_checker change_case:capital_word_frequency change_case:english_capital
change_case:english_lowercase punctuation:no_comma startend:quotation copy:repeat_phrase copy:copy new:copy_span_idx
detectable_format:sentence_hyphens keywords:no_adjacent_consecutive detectable_format:square_brackets keywords:word_once
keywords:word_count_different_numbers keywords:exclude_word_harder paragraphs:paragraphs paragraphs:paragraphs2
first_word:first_word_sent first_word:first_word_answer last_word:last_word_sent last_word:last_word_answer
detectable_format:bigram_wrapping copy:copying_simple copy:copying_multiple punctuation:punctuation_dot
punctuation:punctuation_exclamation count:lowercase_counting letters:letter_counting letters:letter_counting2
count:counting_composition count:count_unique count:count_increment_word keywords:palindrome keywords:keyword_specific_position
keywords:start_end""".split()

# id -> (kwargs, response that satisfies it, response that violates it)
CASES = {
    "keywords:existence": ({"keywords": ["alpha", "beta"]}, "Alpha meets beta.", "Only alpha here."),
    "keywords:frequency": ({"keyword": "cat", "frequency": 2, "relation": "at least"}, "cat and Cat", "one cat"),
    "keywords:forbidden_words": ({"forbidden_words": ["bad"]}, "all good", "a bad day"),
    "keywords:letter_frequency": ({"letter": "z", "let_frequency": 2, "let_relation": "less than"}, "zebra", "zzz buzz"),
    "language:response_language": ({"language": "de"}, "Das ist ein Satz und er ist nicht auf Englisch.", "This is the only sentence and it is in English."),
    "length_constraints:number_sentences": ({"num_sentences": 3, "relation": "at least"}, "One. Two! Three?", "One. Two."),
    "length_constraints:number_paragraphs": ({"num_paragraphs": 2}, "first\n***\nsecond", "first\n***\n\n***\nthird"),
    "length_constraints:number_words": ({"num_words": 5, "relation": "less than"}, "just three words", "this one has six words total"),
    "length_constraints:nth_paragraph_first_word": ({"num_paragraphs": 2, "nth_paragraph": 2, "first_word": "Second"},
                                                    "First paragraph.\n\nSecond paragraph here.", "First paragraph.\n\nAnother one."),
    "detectable_content:number_placeholders": ({"num_placeholders": 2}, "Dear [name], meet at [place].", "Dear [name]."),
    "detectable_content:postscript": ({"postscript_marker": "P.S."}, "Body.\nP.S. one more thing", "Body only."),
    "detectable_format:number_bullet_lists": ({"num_bullets": 2}, "* one\n* two", "* one\n* two\n- three"),
    "detectable_format:constrained_response": ({}, "My answer is yes.", "Probably."),
    "detectable_format:number_highlighted_sections": ({"num_highlights": 2}, "*one* and **two**", "*one* only"),
    "detectable_format:multiple_sections": ({"section_spliter": "SECTION", "num_sections": 2}, "SECTION 1 a SECTION 2 b", "SECTION 1 a"),
    "detectable_format:json_format": ({}, "```json\n{\"a\": 1}\n```", "{a: 1"),
    "detectable_format:title": ({}, "<<My Title>>\nbody", "My Title\nbody"),
    "combination:two_responses": ({}, "first ****** second", "same ****** same"),
    "combination:repeat_prompt": ({"prompt_to_repeat": "Say hi"}, "say hi - and then: hi!", "hi! Say hi"),
    "startend:end_checker": ({"end_phrase": "The end."}, "Story. The end.", "The end. Not."),
    "change_case:capital_word_frequency": ({"capital_frequency": 2, "capital_relation": "at least"}, "WOW this is BIG", "Wow this is Big"),
    "change_case:english_capital": ({}, "THIS IS ALL CAPITAL AND IT IS THE TEXT", "This is not"),
    "change_case:english_lowercase": ({}, "this is all lowercase and it is the text", "This is not"),
    "punctuation:no_comma": ({}, "no commas here", "one, two"),
    "startend:quotation": ({}, '"quoted"', 'not "quoted'),
    "copy:repeat_phrase": ({"phrase": "the quick brown fox", "small_n": 2}, "the slow brown fox and the quick red fox", "the quick brown fox and the quick brown fox"),
    "copy:copy": ({"prompt_to_repeat": "Do the thing"}, " do the thing ", "Do the thing now"),
    "new:copy_span_idx": ({"prompt_to_repeat": "abcdefghij", "n_start": 2, "n_end": 5}, "cde", "cdef"),
    "detectable_format:sentence_hyphens": ({}, "One here.-Two there.", "One here. -Two there."),
    "keywords:no_adjacent_consecutive": ({}, "apple cat elephant", "apple banana"),
    "detectable_format:square_brackets": ({}, "[every] [word]", "[every] word"),
    "keywords:word_once": ({"keyword": "moon"}, "the moon rose", "moon after moon"),
    "keywords:word_count_different_numbers": ({"keyword": "sun", "frequency": 2, "relation": "less than"}, "sun", "sun sun"),
    "keywords:exclude_word_harder": ({"keyword": "never"}, "I always do", "I would never do"),
    "paragraphs:paragraphs": ({}, "one *** two", "one *** two *** three"),
    "paragraphs:paragraphs2": ({}, "one\n\ntwo", "one\ntwo"),
    "first_word:first_word_sent": ({"first_word": "yes"}, "Yes it is. Yes it was.", "Yes it is. No it was not."),
    "first_word:first_word_answer": ({"first_word": "Well"}, "well then", "so well"),
    "last_word:last_word_sent": ({"last_word": "done"}, "It is done. All done!", "It is done. Not yet."),
    "last_word:last_word_answer": ({"last_word": "bye"}, "ok bye!", "bye then"),
    "detectable_format:bigram_wrapping": ({}, "<<I am>> <<at home>>", "<<I am>> at home"),
    "copy:copying_simple": ({"prompt_to_repeat": "Repeat me"}, "repeat me", "repeat me please"),
    "copy:copying_multiple": ({"prompt_to_repeat": "Repeat me", "N": 2}, "Repeat me ****** repeat me", "Repeat me"),
    "punctuation:punctuation_dot": ({}, "no dots here", "a dot."),
    "punctuation:punctuation_exclamation": ({}, "calm", "loud!"),
    "count:lowercase_counting": ({"N": 2}, "Two lower words HERE", "now there are four"),
    "letters:letter_counting": ({"N": 5, "relation": "at least"}, "abc def", "ab 12"),
    "letters:letter_counting2": ({"letter": "e", "let_frequency": 3, "let_relation": "at least"}, "eerie scene", "set"),
    "count:counting_composition": ({"n_sent": 2, "n_words": 3}, "Ab cd. Ef gh. *** Ij kl. Mn op. *** Qr tu. Uv wx.", "Ab cd. Ef gh. *** Ij kl. Mn op."),
    "count:count_unique": ({}, "all words differ here", "the cat and the dog"),
    "count:count_increment_word": ({"keyword1": "red", "keyword2": "blue"}, "red blue blue", "red red blue"),
    "keywords:palindrome": ({}, "see the level there", "nothing here mate"),
    "keywords:keyword_specific_position": ({"keyword": "dog", "n": 2, "m": 3}, "First one. The big dog ran.", "First one. The dog ran."),
    "keywords:start_end": ({}, "echo in the valley echo", "echo in the valley"),
}


def test_registry_covers_every_reference_id():
    assert sorted(ifevalg.INSTRUCTION_CHECKERS) == sorted(REFERENCE_IDS)
    assert sorted(CASES) == sorted(REFERENCE_IDS)


@pytest.mark.parametrize("iid", sorted(CASES))
def test_constraint_accepts_and_rejects(iid):
    kw, good, bad = CASES[iid]
    assert check_instruction(iid, good, kw) is True, (iid, good)
    assert check_instruction(iid, bad, kw) is False, (iid, bad)
    assert check_instruction(iid, "   ", kw) is False  # an empty response satisfies nothing


def test_unknown_id_raises_and_bad_kwargs_do_not():
    with pytest.raises(ifevalg.UnknownInstruction):
        check_instruction("keywords:not_a_constraint", "text", {})
    assert check_instruction("keywords:frequency", "text", {"keyword": "x"}) is False  # missing argument: not satisfied
    assert check_instruction("keywords:frequency", "x x", {"keyword": "x", "frequency": 2, "relation": None}) is True  # nulled keys are dropped


def test_sentence_splitter_and_tokens():
    s = ifevalg.split_sentences("Dr. Smith paid $3.50 at example.com. He left... Then what? \"Go!\" she said.")
    assert s[0] == "Dr. Smith paid $3.50 at example.com." and s[-1].endswith("she said.") and len(s) == 5
    assert ifevalg.split_sentences("It happened in the U.S. He left.") == ["It happened in the U.S.", "He left."]
    assert ifevalg.word_tokens("Don't stop, it's 3.5!") == ["Do", "n't", "stop", ",", "it", "'s", "3.5", "!"]
    assert ifevalg.detect_language("это предложение на русском языке") == "ru"
    assert ifevalg.detect_language("1234 !!") is None


def test_loose_scoring_and_verifier_label_forms():
    from open_instruct_b200.ground_truth_utils import IFEvalVerifier

    assert not check_instruction("startend:quotation", 'Sure:\n"quoted"', {})
    assert ifevalg.check_instruction_loose("startend:quotation", 'Sure:\n"quoted"', {})
    spec = {"instruction_id": ["punctuation:no_comma", "keywords:palindrome"], "kwargs": [None, {}]}
    v = IFEvalVerifier()
    for label in (json.dumps(spec), json.dumps([spec]), repr([spec]), repr([json.dumps(spec)])):
        assert v([], "<think>hm, tricky</think>a level answer", label).score == 1.0
        assert v([], "a level, answer", label).score == 0.5
    with pytest.raises(ifevalg.UnknownInstruction):
        v([], "text", json.dumps({"instruction_id": ["new:nothing"], "kwargs": [{}]}))
