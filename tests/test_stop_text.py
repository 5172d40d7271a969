"""Stop strings over a streamed text and the tokenizer side (src/provider/local/engine/stop.rs): fragments in,
text safe to emit out; a tail that may still grow into a stop string is held back."""
import json
import random

import pytest

from cuca_b200.engine.stop import StopMatcher
from cuca_b200.engine.text import TextCodec, TextStream


def test_no_stop_strings_hold_nothing():
    m = StopMatcher([])
    assert m.passthrough
    assert m.push("anything") == ("anything", False)
    assert m.flush() == ""
    assert StopMatcher(["", ""]).passthrough  # empty stop strings are ignored


def test_a_stop_string_split_across_fragments_is_cut():
    m = StopMatcher(["bc"])
    assert m.push("ab") == ("a", False)  # "b" may be the start of "bc"
    assert m.push("c") == ("", True)
    assert m.flush() == ""


def test_a_stop_string_inside_one_fragment_cuts_before_it():
    m = StopMatcher(["END"])
    assert m.push("hello END tail") == ("hello ", True)


def test_the_earliest_occurrence_of_any_stop_wins():
    assert StopMatcher(["zz", "b"]).push("abzz") == ("a", True)
    assert StopMatcher(["b", "ab"]).push("xab") == ("x", True)


def test_a_false_start_is_released_and_flush_gives_the_rest():
    m = StopMatcher(["stop"])
    assert m.push("a st") == ("a ", False)
    assert m.push("o") == ("", False)
    assert m.push("ne") == ("stone", False)
    assert m.push(" sto") == (" ", False)
    assert m.flush() == "sto"


def test_never_more_than_the_longest_stop_less_one_is_held():
    m = StopMatcher(["abcd", "xy"])
    out, done = m.push("zzzzabc")
    assert (out, done) == ("zzzz", False) and m.held == "abc"
    out, done = m.push("abc")  # "abcabc": the first "abc" cannot continue any more
    assert (out, done) == ("abc", False) and m.held == "abc"


def test_random_fragmentation_equals_one_cut():
    """However the text is cut into fragments, what comes out is the text before the first stop string."""
    rnd = random.Random(3)
    alphabet = "abc "
    for _ in range(300):
        text = "".join(rnd.choice(alphabet) for _ in range(rnd.randint(0, 40)))
        stops = ["".join(rnd.choice(alphabet) for _ in range(rnd.randint(1, 4))) for _ in range(rnd.randint(1, 3))]
        hits = [text.find(s) for s in stops if text.find(s) >= 0]
        want = text[:min(hits)] if hits else text
        m, got, i, done = StopMatcher(stops), "", 0, False
        while i < len(text) and not done:
            n = rnd.randint(1, 5)
            out, done = m.push(text[i:i + n])
            got += out
            i += n
        if not done:
            got += m.flush()
        assert got == want and done == bool(hits), (text, stops)


@pytest.fixture()
def word_tokenizer(tmp_path):
    tokenizers = pytest.importorskip("tokenizers")
    vocab = {f"w{i}": i for i in range(64)}
    vocab["[UNK]"] = 64
    tok = tokenizers.Tokenizer(tokenizers.models.WordLevel(vocab, unk_token="[UNK]"))
    tok.pre_tokenizer = tokenizers.pre_tokenizers.WhitespaceSplit()
    tok.decoder = tokenizers.decoders.Fuse()
    tok.save(str(tmp_path / "tokenizer.json"))
    (tmp_path / "config.json").write_text(json.dumps({}))
    return tmp_path


def test_codec_round_trip_and_stream(word_tokenizer):
    codec = TextCodec.find(word_tokenizer)
    assert codec is not None and TextCodec.find(None) is None
    ids = codec.encode("w3 w10 w63")
    assert ids == [3, 10, 63]
    stream, seen, out = TextStream(codec), [], ""
    for t in ids:
        seen.append(t)
        out += stream.push(seen)
    assert out == codec.decode(ids)


def test_a_folder_without_tokenizer_has_no_codec(tmp_path):
    assert TextCodec.find(tmp_path) is None


def test_a_character_split_over_two_tokens_is_held_until_it_is_whole(tmp_path):
    """A byte-level vocabulary trained on ASCII alone: "é" is two tokens; the first alone decodes to the
    replacement character, which must not be streamed."""
    tokenizers = pytest.importorskip("tokenizers")
    tok = tokenizers.Tokenizer(tokenizers.models.BPE())
    tok.pre_tokenizer = tokenizers.pre_tokenizers.ByteLevel(add_prefix_space=False)
    tok.decoder = tokenizers.decoders.ByteLevel()
    trainer = tokenizers.trainers.BpeTrainer(vocab_size=300, initial_alphabet=tokenizers.pre_tokenizers.ByteLevel.alphabet(),
                                             show_progress=False)
    tok.train_from_iterator(["plain ascii text only", "more plain text"], trainer)
    tok.save(str(tmp_path / "tokenizer.json"))
    codec = TextCodec.find(tmp_path)
    ids = codec.encode("caf\u00e9 ok")
    assert codec.decode(ids) == "caf\u00e9 ok" and len(ids) >= 5
    stream, seen, pieces = TextStream(codec), [], []
    for t in ids:
        seen.append(t)
        pieces.append(stream.push(seen))
    assert "".join(pieces) == "caf\u00e9 ok"
    assert all("\ufffd" not in piece for piece in pieces)
    assert "" in pieces  # the first half of the character gave nothing
