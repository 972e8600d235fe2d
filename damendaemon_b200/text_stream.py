"""Text that is safe to hand out while tokens still arrive, and stopping on a string.

A generated token may end in the middle of a UTF-8 sequence (the decoder then shows U+FFFD until the rest
arrives) or in the middle of a stop string; neither may be shown before it is certain. The rules are the
reference's (damendaemon/stopping.py:4-41): one to four stop strings of 1 to 256 characters; text up to the first
occurrence of a stop string is shown and nothing after it; a trailing piece that could still grow into a stop
string, and trailing replacement characters, are held back until the next token or the end decides. The code is this
project's: a small object that is fed the whole decoded text after every token and answers with what is new.
"""
from __future__ import annotations

REPLACEMENT = "�"
MAX_STOPS, MAX_STOP_LENGTH = 4, 256


def checked_stops(stop) -> tuple:
    """None, one string or a list of strings -> a tuple of stop strings, or ValueError."""
    if stop is None:
        return ()
    items = [stop] if isinstance(stop, str) else stop
    if not isinstance(items, (list, tuple)) or not 1 <= len(items) <= MAX_STOPS:
        raise ValueError(f"stop: one string or a list of 1 to {MAX_STOPS} strings is expected")
    for item in items:
        if not isinstance(item, str) or not 1 <= len(item) <= MAX_STOP_LENGTH:
            raise ValueError(f"stop: every stop string has 1 to {MAX_STOP_LENGTH} characters")
        try:
            item.encode("utf-8")
        except UnicodeError:
            raise ValueError("stop: a stop string cannot be encoded as UTF-8 (a lone surrogate?)") from None
    return tuple(items)


class TextStream:
    """``push(decoded, final)`` takes everything decoded so far and returns (new text to show, stopped)."""

    def __init__(self, stops=()):
        self.stops = tuple(stops)
        self.shown = ""
        self.stopped = False

    def _held_back(self, text: str) -> int:
        """Characters at the end of text that may still turn into something else."""
        settled = text.rstrip(REPLACEMENT)
        held = len(text) - len(settled)             # an incomplete UTF-8 sequence shows as replacement characters
        longest = 0
        for stop in self.stops:                     # the longest proper beginning of a stop string that ends the text
            for n in range(min(len(stop) - 1, len(settled)), longest, -1):
                if settled.endswith(stop[:n]):
                    longest = n
                    break
        return held + longest

    def push(self, decoded: str, final: bool = False):
        if self.stopped:
            return "", True
        # a replacement character at the very end may still become a real one, so it cannot complete a stop string yet
        searchable = decoded if final else decoded.rstrip(REPLACEMENT)
        cuts = [at for at in (searchable.find(stop) for stop in self.stops) if at >= 0]
        if cuts:
            visible, self.stopped = decoded[:min(cuts)], True
        elif final:
            visible = decoded
        else:
            visible = decoded[:len(decoded) - self._held_back(decoded)]
        if len(visible) < len(self.shown):
            visible = self.shown                    # never take back what was shown (only ever shorter while holding back)
        if not visible.startswith(self.shown):
            raise RuntimeError("the tokenizer changed text that had been handed out already")
        delta, self.shown = visible[len(self.shown):], visible
        return delta, self.stopped
