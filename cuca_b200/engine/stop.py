"""Stop strings over a streamed text.

Text arrives in fragments (one per sampled token), so a stop string can be split across fragments. The matcher
releases everything that can no longer become part of a stop string, holds back the longest tail that is still a
proper prefix of one (never more than the longest stop string less one character), and, when a stop string is
complete, releases the text before its first occurrence and says that generation ends there
(src/provider/local/engine/stop.rs:1-110; the reference counts bytes and cuts on UTF-8 boundaries, Python strings
are code points already). Without stop strings nothing is held.
"""
from __future__ import annotations

from typing import Iterable, Tuple


class StopMatcher:
    def __init__(self, stop: Iterable[str] = ()):
        self.stops = [s for s in stop if s]  # an empty stop string would match everywhere
        self.longest = max((len(s) for s in self.stops), default=0)
        self.held = ""

    @property
    def passthrough(self) -> bool:
        return not self.stops

    def push(self, text: str) -> Tuple[str, bool]:
        """Append `text`; returns (text safe to emit now, whether a stop string occurred). After a stop string the
        emitted text ends right before it and nothing is held."""
        if not self.stops:
            return text, False
        self.held += text
        found = [at for at in (self.held.find(s) for s in self.stops) if at >= 0]
        if found:
            emit, self.held = self.held[:min(found)], ""
            return emit, True
        keep = 0
        for n in range(min(len(self.held), self.longest - 1), 0, -1):
            tail = self.held[len(self.held) - n:]
            if any(s.startswith(tail) for s in self.stops):
                keep = n
                break
        cut = len(self.held) - keep
        emit, self.held = self.held[:cut], self.held[cut:]
        return emit, False

    def flush(self) -> str:
        """Generation ended without completing a stop string: what was held back."""
        held, self.held = self.held, ""
        return held
