"""The command line's pieces that need no GPU: the tokenizer reader, the chat template and the
chat session (with a stand-in for the engine)."""

import json

import pytest

from scratch_llm_b200.chat_cli import (ASSISTANT, BOS, EOT, SPECIALS, USER, ChatSession, batch_reply,
                                       render_for_completion, special_id)
from scratch_llm_b200.tokenizer import Tokenizer


@pytest.fixture()
def tokenizer(tmp_path):
    """A byte-level tokenizer with a few merges and the chat specials, in the reference's
    one-file format (src/scratch_llm/tokenizer.py:207-236)."""
    vocab = {str(i): bytes([i]).decode("latin-1") for i in range(256)}
    merges = [["t", "h"], ["th", "e"], [" ", "the"], ["i", "n"], [" ", "c"]]
    for k, (a, b) in enumerate(merges):
        vocab[str(256 + k)] = a + b
    for k, s in enumerate(SPECIALS):
        vocab[str(261 + k)] = s
    path = tmp_path / "tokenizer.json"
    path.write_text(json.dumps({"vocab": vocab, "merges": merges, "special_tokens": SPECIALS}))
    return Tokenizer.load(path)


def test_tokenizer_merges_in_learned_order_and_round_trips(tokenizer):
    ids = tokenizer.encode("the cat in the hat")
    assert ids[0] == 257                      # "the" after t+h, th+e
    assert 258 in ids                         # " the"
    assert 259 in ids and 260 in ids          # "in", " c"
    assert tokenizer.decode(ids) == "the cat in the hat"
    text = "héllo  wörld\n\n 123"
    assert tokenizer.decode(tokenizer.encode(text)) == text
    assert tokenizer.decode([257, 100000]) == "the\ufffd"   # an id the vocabulary does not hold


def test_specials_are_single_ids_and_split_out(tokenizer):
    for s in SPECIALS:
        assert len(tokenizer.encode(s)) == 1
    ids = tokenizer.encode(f"{USER}the{EOT}")
    assert ids == [special_id(tokenizer, USER), 257, special_id(tokenizer, EOT)]
    bare = Tokenizer({i: bytes([i]) for i in range(256)}, [], [])
    with pytest.raises(ValueError, match="expected 1"):
        special_id(bare, EOT)


def test_chat_template(tokenizer):
    ids = render_for_completion([("user", "the"), ("assistant", "in"), ("user", "the")], tokenizer)
    sid = {s: special_id(tokenizer, s) for s in SPECIALS}
    assert ids == [sid[BOS], sid[USER], 257, sid[EOT], sid[ASSISTANT], 259, sid[EOT],
                   sid[USER], 257, sid[EOT], sid[ASSISTANT]]
    with pytest.raises(ValueError, match="unknown role"):
        render_for_completion([("system", "x")], tokenizer)


class FakeLLM:
    """Answers every prompt with "the", the end-of-turn token, and something after it."""

    def __init__(self, tokenizer):
        self.tok, self.calls = tokenizer, []

    def generate(self, prompts, params):
        self.calls.append((prompts, params))
        answer = [257, special_id(self.tok, EOT), 65]
        return answer if isinstance(prompts[0], int) else [list(answer) for _ in prompts]


def test_chat_session_stops_at_end_of_turn_and_keeps_history(tokenizer):
    llm = FakeLLM(tokenizer)
    chat = ChatSession(llm, tokenizer, max_tokens=7)
    assert chat.reply("the hat") == "the"
    assert chat.history == [("user", "the hat"), ("assistant", "the")]
    prompt, params = llm.calls[0]
    assert prompt == render_for_completion([("user", "the hat")], tokenizer)
    assert params.temperature == 0.0 and params.max_tokens == 7
    assert params.stop_ids == (special_id(tokenizer, EOT),)
    chat.reply("in")
    assert len(chat.history) == 4
    assert llm.calls[1][0] == render_for_completion(
        [("user", "the hat"), ("assistant", "the"), ("user", "in")], tokenizer)
    chat.reset()
    assert chat.history == []
    assert batch_reply(llm, tokenizer, ["a", "b"], max_tokens=3) == ["the", "the"]
