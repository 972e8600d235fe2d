"""Incremental text and stop strings (the rules of damendaemon/stopping.py:4-41)."""
import pytest

from damendaemon_b200.text_stream import TextStream, checked_stops


def test_stop_arguments():
    assert checked_stops(None) == () and checked_stops("END") == ("END",) and checked_stops(["a", "bc"]) == ("a", "bc")
    for bad in ("", [], ["a"] * 5, [""], ["x" * 257], [3], {"a"}, 5, ["\ud800"]):
        with pytest.raises(ValueError, match="stop"):
            checked_stops(bad)


def feed(stream, pieces):
    text, out = "", []
    for i, piece in enumerate(pieces):
        text += piece
        out.append(stream.push(text, final=i == len(pieces) - 1))
    return out


def test_plain_streaming_shows_everything_once():
    assert feed(TextStream(), ["Hel", "lo ", "world"]) == [("Hel", False), ("lo ", False), ("world", False)]


def test_a_stop_string_split_over_tokens_is_never_shown():
    s = TextStream(("<END>",))
    out = feed(s, ["abc <", "EN", "D> tail", " more"])
    assert out == [("abc ", False), ("", False), ("", True), ("", True)]
    assert s.shown == "abc " and s.stopped


def test_a_beginning_that_does_not_grow_into_the_stop_is_released():
    out = feed(TextStream(("<END>",)), ["a<", "EX", "b"])
    assert out == [("a", False), ("<EX", False), ("b", False)]


def test_the_earliest_stop_wins_and_the_end_releases_what_was_held():
    assert feed(TextStream(("yz", "x")), ["wxyz"])[-1] == ("w", True)
    assert feed(TextStream(("stop",)), ["it st"]) == [("it st", False)]          # final: nothing is held back any more
    assert feed(TextStream(("stop",)), ["it st", "ays"]) == [("it ", False), ("stays", False)]


def test_incomplete_utf8_is_held_until_it_completes():
    s = TextStream(("é!",))
    assert s.push("caf�") == ("caf", False)                 # the decoder cannot show the first byte of é yet
    assert s.push("café") == ("", False)                         # é could begin the stop string
    assert s.push("café?") == ("é?", False)
    s = TextStream()
    assert s.push("a��") == ("a", False) and s.push("a��", final=True) == ("��", False)


def test_revised_text_is_an_error():
    s = TextStream()
    s.push("abc")
    with pytest.raises(RuntimeError):
        s.push("abX")
