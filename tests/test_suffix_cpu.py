"""Suffix drafter: every draft is a true continuation of the history (reference: tests/test_suffix.py)."""
import random

import pytest

from coffin_b200.utils.suffix import SuffixDrafter


def _follows(history, draft):
    """``draft`` is what followed an earlier occurrence of some suffix of ``history`` (2..4 tokens)."""
    if not draft:
        return True
    for m in range(4, 1, -1):
        suf = history[-m:]
        for end in range(m, len(history)):
            if history[end - m:end] == suf and history[end:end + len(draft)] == draft:
                return True
    return False


def test_repeated_phrase_drafts_the_continuation_and_disjoint_history_nothing():
    d = SuffixDrafter()
    d.observe([1, 2, 3, 4, 5, 6, 1, 2, 3])
    assert d.draft(4) == [4, 5, 6, 1]
    e = SuffixDrafter()
    e.observe(list(range(100, 120)))
    assert e.draft(4) == []


def test_bounds_empty_history_and_non_positive_k():
    d = SuffixDrafter()
    assert d.draft(4) == []
    d.observe([7])
    assert d.draft(4) == []                                    # shorter than the shortest match
    d.observe([8, 7, 8])
    assert d.draft(0) == [] and d.draft(-3) == []
    assert len(d.draft(1)) <= 1
    with pytest.raises(ValueError):
        SuffixDrafter(max_match=2, min_match=3)


def test_suffix_does_not_match_itself_and_longest_match_wins():
    d = SuffixDrafter()
    d.observe([1, 2, 3])
    assert d.draft(3) == []                                    # the only occurrence of (2, 3) is the suffix itself
    # (9, 1, 2) was followed by 5; the shorter (1, 2) was followed by 7 more recently and more often
    d = SuffixDrafter()
    d.observe([9, 1, 2, 5, 0, 1, 2, 7, 0, 1, 2, 7, 9, 1, 2])
    assert d.draft(1) == [5]


def test_draft_does_not_change_the_history_and_observe_matches_reset_plus_replay():
    d = SuffixDrafter()
    hist = [3, 1, 4, 1, 5, 9, 2, 6, 3, 1, 4]
    d.observe(hist)
    before = list(d.history)
    first = d.draft(5)
    assert d.history == before and d.draft(5) == first
    e = SuffixDrafter()
    for t in hist:                                             # token by token == all at once
        e.observe([t])
    assert e.draft(5) == first
    d.reset()
    d.observe(hist)
    assert d.draft(5) == first


def test_random_histories_only_ever_draft_true_continuations():
    rng = random.Random(0)
    for _ in range(200):
        hist = [rng.randrange(6) for _ in range(rng.randrange(0, 60))]
        d = SuffixDrafter()
        d.observe(hist)
        k = rng.randrange(1, 9)
        draft = d.draft(k)
        assert len(draft) <= k
        assert _follows(hist, draft), (hist, draft)
