"""Stop strings over a streamed text.

Text arrives in fragments (one per sampled token), so a stop string can be split across fragments. What the
caller sees follows the reference's rule (src/provider/local/engine/stop.rs:1-110): text is released as soon as it
can no longer become part of a stop string, the tail that still could is held back, and when a stop string
completes, the text before its first occurrence is released and generation ends there. (The reference counts
bytes and cuts on UTF-8 boundaries; Python strings are code points already.)

The matching itself is done one character at a time over the set of stop strings: for every stop string the
matcher keeps how many of its leading characters the text seen so far ends with (the classic failure-function
walk of string matching), so a fragment costs its length times the number of stop strings, whatever was held
before, and the held tail is simply the longest of these partial matches.
"""
from __future__ import annotations

from typing import Iterable, Tuple


def _failure(pattern: str) -> list:
    """fail[i]: length of the longest proper prefix of pattern[:i + 1] that is also its suffix."""
    fail, k = [0] * len(pattern), 0
    for i in range(1, len(pattern)):
        while k and pattern[i] != pattern[k]:
            k = fail[k - 1]
        if pattern[i] == pattern[k]:
            k += 1
        fail[i] = k
    return fail


class StopMatcher:
    def __init__(self, stop: Iterable[str] = ()):
        self.patterns = [s for s in stop if s]  # an empty string is no stop string
        self._fail = [_failure(p) for p in self.patterns]
        self._matched = [0] * len(self.patterns)  # per stop string: how much of it the text ends with
        self._pending = ""  # characters not yet released: the longest partial match (or less, never more)

    @property
    def held(self) -> str:
        """What is held back: the longest tail of the text so far that a stop string begins with."""
        return self._pending

    @property
    def passthrough(self) -> bool:
        return not self.patterns

    def push(self, text: str) -> Tuple[str, bool]:
        """Append `text`; returns (text safe to emit now, whether a stop string occurred). After a stop string the
        emitted text ends right before its first occurrence and nothing is held."""
        if not self.patterns:
            return text, False
        seen = self._pending + text
        base = len(self._pending)
        hit_start = None  # of all stop strings that complete inside this fragment, the earliest start wins
        for offset, ch in enumerate(text):
            end = base + offset + 1  # characters of `seen` consumed so far
            for j, pattern in enumerate(self.patterns):
                k, fail = self._matched[j], self._fail[j]
                while k and ch != pattern[k]:
                    k = fail[k - 1]
                if ch == pattern[k]:
                    k += 1
                if k == len(pattern):
                    hit_start = end - k if hit_start is None else min(hit_start, end - k)
                    k = fail[k - 1]
                self._matched[j] = k
        if hit_start is not None:
            self._pending = ""
            self._matched = [0] * len(self.patterns)
            return seen[:hit_start], True
        keep = max(self._matched)
        cut = len(seen) - keep
        self._pending = seen[cut:]
        return seen[:cut], False

    def flush(self) -> str:
        """Generation ended without completing a stop string: what was held back."""
        held, self._pending = self._pending, ""
        self._matched = [0] * len(self.patterns)
        return held
