"""Decode-loop semantics on the host (CPU only), mirroring the reference's mock-model tests
(crates/llm/tests/mock_decode.rs): the 'model' is a logit table indexed by past_len."""
import pytest

from my_nn_engine_b200.session import GenerateOptions, LlmSession, PromptTooLong, argmax_last

SEQUENCE = [1, 2, 3, 4, 5, 0, 1, 2, 3, 4, 5, 0, 1, 2, 3, 4]  # fixtures/mock_decode/expected_sequence.json
VOCAB = ["<unk>", "a", "b", "c", "d", "e"]


class WordTokenizer:
    def encode(self, text):
        return [VOCAB.index(w) if w in VOCAB else 0 for w in text.split()]

    def decode(self, ids):
        return " ".join(VOCAB[i] for i in ids)


def make_session(prefill_len=None, max_seq_len=16):
    calls = []

    def step(token, past_len):
        calls.append(("step", token, past_len))
        return SEQUENCE[past_len]

    def prefill(ids, past_len):
        calls.append(("prefill", tuple(ids), past_len))
        return SEQUENCE[past_len + len(ids) - 1]

    s = LlmSession(step, max_seq_len, eos_token_id=999, prefill=prefill if prefill_len else None,
                   prefill_len=prefill_len, tokenizer=WordTokenizer())
    return s, calls


def test_generate_ids_follows_logit_table():
    s, _ = make_session()
    assert s.generate_ids("a b c", 5) == [3, 4, 5, 0, 1]


def test_generate_decodes_to_text():
    s, _ = make_session()
    assert s.generate("a b c", 5) == "c d e <unk> a"


def test_past_len_tracks_decode_steps_and_reset():
    s, _ = make_session()
    assert s.past_len() == 0
    s.generate_ids("a b c", 5)
    assert s.past_len() == 7
    s.reset()
    assert s.past_len() == 0


def test_empty_prompt_returns_no_tokens():
    s, calls = make_session()
    assert s.generate_ids("", 5) == [] and not calls


def test_stop_string_truncates_and_rewinds_past_len():
    s, _ = make_session()
    opts = GenerateOptions(max_new_tokens=5, stop_strings=["<unk>"])
    assert s.generate("a b c", opts=opts) == "c d e"
    s2, _ = make_session()
    ids = s2.generate_ids("a b c", opts=opts)
    assert s2.past_len() == 2 + len(ids)


def test_eos_stops_generation():
    s = LlmSession(lambda tok, past: 7, 16, eos_token_id=7)
    assert s.generate_ids([1, 2], 5) == [7]


def test_prompt_too_long_and_cache_limit():
    s, _ = make_session(max_seq_len=4)
    with pytest.raises(PromptTooLong):
        s.generate_ids("a b c d e", 3)
    s, _ = make_session(max_seq_len=4)
    assert len(s.generate_ids("a b c", 10)) == 2  # rows 0..3 only: 3 prompt steps + 1 more


def test_chunked_prefill_matches_decode_only():
    a, _ = make_session()
    b, calls = make_session(prefill_len=2)
    assert a.generate_ids("a b c", 4) == b.generate_ids("a b c", 4)
    assert calls[0] == ("prefill", (1, 2), 0) and calls[1] == ("prefill", (3,), 2)
    assert a.past_len() == b.past_len()
    # prefill pads to a multiple of prefill_len when checking capacity
    c, _ = make_session(prefill_len=4, max_seq_len=6)
    with pytest.raises(PromptTooLong):
        c.generate_ids("a b c d e", 1)


def test_argmax_last_tie_rule():
    assert argmax_last([1.0, 5.0, 5.0, 2.0]) == 2
    with pytest.raises(ValueError):
        argmax_last([1.0, float("nan")])


class FakeStreamingModel:
    """Stands in for DecoderModel(streaming=(sink, window)): records the calls, answers from the logit table."""

    def __init__(self, sink, window):
        self.batch, self.streaming, self.output, self.max_seq_len = 1, (sink, window), "ids", sink + window
        self.calls = []

    def stream(self, tokens, stream_pos):
        toks = tokens[0] if isinstance(tokens[0], (list, tuple)) else tokens
        self.calls.append((tuple(toks), stream_pos))
        return [SEQUENCE[(stream_pos + len(toks) - 1) % len(SEQUENCE)]]


def test_streaming_session_has_no_length_limit_and_never_evicts_inside_a_chunk():
    """LlmSession::for_llama_streaming: the stream position keeps growing past sink + window; prompt chunks are
    prefilled only while they fit into the live rows, afterwards prompt tokens go in one at a time."""
    model = FakeStreamingModel(sink=2, window=6)
    s = LlmSession.for_llama_streaming(model, eos_token_id=999, prefill_len=4)
    out = s.generate_ids(list(range(1, 12)), 9)  # 11 prompt tokens, 8 live rows
    assert len(out) == 9 and s.past_len() == 11 + 8
    sizes = [(len(t), pos) for t, pos in model.calls]
    assert sizes[:2] == [(4, 0), (4, 4)]           # two chunks fill the 8 live rows exactly
    assert sizes[2:5] == [(1, 8), (1, 9), (1, 10)]  # the rest of the prompt would evict: token by token
    assert all(n == 1 for n, _ in sizes[2:]) and [pos for _, pos in sizes[2:]] == list(range(8, 19))
    # without prefill every prompt token is a streaming step
    model2 = FakeStreamingModel(sink=1, window=3)
    s2 = LlmSession.for_llama_streaming(model2, eos_token_id=999)
    s2.generate_ids([1, 2, 3, 4, 5, 1], 3)
    assert [pos for _, pos in model2.calls] == list(range(8))
    with pytest.raises(ValueError):
        LlmSession.for_llama_streaming(type("M", (), {"batch": 2, "streaming": (1, 3)})(), eos_token_id=0)


def test_streaming_chunk_shrinks_to_the_room_left():
    model = FakeStreamingModel(sink=2, window=4)  # 6 live rows
    s = LlmSession.for_llama_streaming(model, eos_token_id=999, prefill_len=4)
    s.generate_ids([1, 2, 3, 4, 5, 1, 2], 1)
    assert [(len(t), pos) for t, pos in model.calls] == [(4, 0), (2, 4), (1, 6)]


def test_engine_literal_streaming_index_math_and_where_it_leaves_the_documented_layout():
    """ref_ops.streaming_state(engine_literal=True) restates the engine's host code line by line
    (crates/llm/src/session.rs:539-635).  While nothing has been evicted it equals the layout this library keeps; from the
    first eviction on the engine derives the ring start and the rank table from the position BEFORE the append and reuses that
    ring start for the write slot: the new row of token P lands in slot sink + 2 * ((P - sink) % window) % window instead of
    sink + (P - sink) % window, and the rank table lags one step behind.  An integrator who needs the engine's exact
    post-eviction behaviour gets it from the literal mode; the library itself keeps the documented layout."""
    import numpy as np
    from oracle import ref_ops as R
    sink, window, cache = 4, 8, 16
    for p in range(sink + window):  # no eviction yet: identical in every field
        a, b = R.streaming_state(p, 1, sink, window, cache), R.streaming_state(p, 1, sink, window, cache, engine_literal=True)
        assert a["slots"] == b["slots"] and a["ring_start"] == b["ring_start"] == 0 and a["active"] == b["active"]
        assert np.array_equal(a["kv_position"], b["kv_position"]) and np.array_equal(a["q_positions"], b["q_positions"])
    for chunk in (2, 5):  # prefill chunks that do not evict: identical too
        a, b = R.streaming_state(3, chunk, sink, window, cache), R.streaming_state(3, chunk, sink, window, cache, engine_literal=True)
        assert a["slots"] == b["slots"] and np.array_equal(a["kv_position"], b["kv_position"])
    for p in range(sink + window, sink + 3 * window):
        a, b = R.streaming_state(p, 1, sink, window, cache), R.streaming_state(p, 1, sink, window, cache, engine_literal=True)
        assert a["slots"] == [sink + (p - sink) % window]
        assert b["slots"] == [sink + (2 * ((p - sink) % window)) % window]
        assert b["ring_start"] == (p - sink) % window and a["ring_start"] == (p + 1 - sink) % window
        assert a["active"] == b["active"] == sink + window
        # documented layout: the slot just written is the newest rank; literal: the table still ranks the rows as before the append
        assert a["kv_position"][a["slots"][0]] == sink + window - 1
        prev = R.streaming_state(p - 1, 1, sink, window, cache)
        assert np.array_equal(b["kv_position"], prev["kv_position"])
