"""Host-side suffix-match drafter for speculative decoding.

Keeps the token history of one sequence and proposes the continuation that followed the most
recent earlier occurrence of the current suffix (longest suffix first, ``min_match`` ..
``max_match`` tokens).  Every draft is therefore a true continuation of something already seen;
repetitive outputs (code, lists, quoted context) accept long drafts at zero model cost.
Reference: ``ops/suffix.py`` (``SuffixDrafter(max_match=4, min_match=2).reset/observe/draft``).
"""
from __future__ import annotations


class SuffixDrafter:
    def __init__(self, max_match: int = 4, min_match: int = 2) -> None:
        if not 1 <= min_match <= max_match:
            raise ValueError("need 1 <= min_match <= max_match")
        self.max_match, self.min_match = max_match, min_match
        self.reset()

    def reset(self) -> None:
        self.history: list[int] = []
        self._index: dict[tuple[int, ...], int] = {}     # n-gram -> end position of its latest earlier occurrence

    def observe(self, tokens) -> None:
        for t in tokens:
            self.history.append(int(t))
            n = len(self.history)
            # index the n-grams that end just before the new token, so that a lookup never
            # returns the suffix's own occurrence
            for k in range(self.min_match, self.max_match + 1):
                if n - 1 >= k:
                    self._index[tuple(self.history[n - 1 - k:n - 1])] = n - 1

    def draft(self, k: int) -> list[int]:
        """Up to ``k`` proposed next tokens (possibly none; none for ``k <= 0``)."""
        if k <= 0:
            return []
        h = self.history
        for m in range(min(self.max_match, len(h)), self.min_match - 1, -1):
            end = self._index.get(tuple(h[-m:]))
            if end is not None and end < len(h):
                return h[end:end + k]
        return []
