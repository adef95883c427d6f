"""Greedy decode loop: the engine's ``LlmSession`` (crates/llm/src/session.rs) over the B200 decoder.

The loop logic is host code in the engine too; it is kept separate from the device model so that it can be tested
with a stand-in step function, the way the engine tests it with a one-node mock graph
(crates/llm/tests/mock_decode.rs).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Optional, Sequence


class PromptTooLong(ValueError):
    def __init__(self, needed, max_seq_len, past_len):
        super().__init__(f"prompt needs {needed} cache rows, max_seq_len is {max_seq_len} (past_len {past_len})")
        self.needed, self.max_seq_len, self.past_len = needed, max_seq_len, past_len


@dataclass
class GenerateOptions:
    max_new_tokens: int = 16
    stop_strings: list = field(default_factory=list)


def argmax_last(logits) -> int:
    """Index of the maximum, the LAST one among equals (``max_by(partial_cmp)``, crates/llm/src/session.rs:683-690).
    A NaN logit raises, where the engine panics."""
    best, besti = None, -1
    for i, v in enumerate(logits):
        v = float(v)
        if v != v:
            raise ValueError("NaN in logits")
        if best is None or v >= best:
            best, besti = v, i
    return besti


class LlmSession:
    """``decode_step(token, past_len) -> next token`` and optionally ``prefill(ids, past_len) -> next token`` are
    supplied by the device model (batch 1, as the engine wires it).  ``tokenizer`` needs ``encode(str) -> ids`` and
    ``decode(ids) -> str`` only when prompts are strings or stop strings are used."""

    def __init__(self, decode_step: Callable[[int, int], int], max_seq_len: int, eos_token_id: int,
                 prefill: Optional[Callable[[Sequence[int], int], int]] = None, prefill_len: Optional[int] = None,
                 tokenizer=None):
        self._decode_step, self._prefill = decode_step, prefill
        self.max_seq_len, self.eos_token_id = max_seq_len, eos_token_id
        self.prefill_len = prefill_len if prefill is not None else None
        self.tokenizer = tokenizer
        self._past_len = 0
        self.streaming = None  # (sink, window) when bound to a streaming-cache model: the stream has no length limit

    @classmethod
    def for_llama_streaming(cls, model, eos_token_id: int, prefill_len: Optional[int] = None, tokenizer=None):
        """Bind to a ``DecoderModel`` built with ``streaming=(sink, window)`` (``LlmSession::for_llama_streaming``,
        crates/llm/src/session.rs:539-635): ``past_len`` is the absolute stream position and never hits a limit; prompt
        chunks are prefilled while they fit without evicting, later prompt tokens are fed one at a time."""
        if model.batch != 1 or not model.streaming:
            raise ValueError("for_llama_streaming needs a batch-1 model built with streaming=(sink, window)")

        def pick(out):
            return int(out[0]) if model.output == "ids" else argmax_last(out[0].float().tolist())

        def step(token, stream_pos):
            return pick(model.stream([token], stream_pos))

        def prefill(ids, stream_pos):
            return pick(model.stream([list(ids)], stream_pos))

        self = cls(step, model.max_seq_len, eos_token_id, prefill if prefill_len else None, prefill_len, tokenizer)
        self.streaming = model.streaming
        return self

    @classmethod
    def for_llama(cls, model, eos_token_id: int, prefill_len: Optional[int] = None, tokenizer=None):
        """Bind to a ``DecoderModel`` with batch 1 (``LlmSession::for_llama`` / ``for_llama_with_prefill``)."""
        if model.batch != 1:
            raise ValueError("LlmSession drives one sequence; use DecoderModel.step for batched decode")

        def pick(out):
            return int(out[0]) if model.output == "ids" else argmax_last(out[0].float().tolist())

        def step(token, past_len):
            return pick(model.step([token], past_len))

        def prefill(ids, past_len):
            return pick(model.prefill([list(ids)], past_len))

        return cls(step, model.max_seq_len, eos_token_id, prefill if prefill_len else None, prefill_len, tokenizer)

    def past_len(self) -> int:
        return self._past_len

    def reset(self) -> None:
        """Forget the conversation: only ``past_len`` is zeroed, the cache rows are simply overwritten later
        (crates/llm/src/session.rs:303-305)."""
        self._past_len = 0

    def _encode(self, prompt):
        if isinstance(prompt, str):
            if self.tokenizer is None:
                raise ValueError("string prompts need a tokenizer")
            enc = self.tokenizer.encode(prompt)
            return list(getattr(enc, "ids", enc))
        return [int(t) for t in prompt]

    def _text(self, ids):
        return self.tokenizer.decode(list(ids))

    def _hit_stop(self, new_ids, opts):
        if not opts.stop_strings:
            return False
        text = self._text(new_ids)
        return any(s in text for s in opts.stop_strings)

    def _run_prefill(self, prompt_ids):
        """Chunks of at most prefill_len tokens; past_len advances by the real chunk size; the last chunk yields the
        token (crates/llm/src/session.rs:426-480)."""
        pos, tok = 0, None
        while pos < len(prompt_ids):
            size = self.prefill_len
            if self.streaming:  # a chunk must not evict: shrink it to the room left, then go token by token
                size = min(size, sum(self.streaming) - self._past_len)
            if size >= 2:
                chunk = prompt_ids[pos:pos + size]
                tok = self._prefill(chunk, self._past_len)
            else:
                chunk = prompt_ids[pos:pos + 1]
                tok = self._decode_step(chunk[0], self._past_len)
            self._past_len += len(chunk)
            pos += len(chunk)
        return tok

    def _step(self, token):
        nxt = self._decode_step(token, self._past_len)
        self._past_len += 1
        return nxt

    def generate_ids(self, prompt, max_new_tokens: int = 16, opts: Optional[GenerateOptions] = None,
                     on_token: Optional[Callable[[int], None]] = None):
        """``generate_ids_with_callback`` (crates/llm/src/session.rs:333-394)."""
        opts = opts or GenerateOptions(max_new_tokens=max_new_tokens)
        prompt_ids = self._encode(prompt)
        new_ids: list = []
        if not prompt_ids:
            return new_ids
        if self.prefill_len:
            needed = self._past_len + -(-len(prompt_ids) // self.prefill_len) * self.prefill_len
        else:
            needed = self._past_len + len(prompt_ids)
        if not self.streaming and self.max_seq_len < needed:
            raise PromptTooLong(needed, self.max_seq_len, self._past_len)
        for i in range(opts.max_new_tokens):
            if not self.streaming and self.max_seq_len < self._past_len + 1:
                break
            if i == 0:
                if self.prefill_len:
                    token = self._run_prefill(prompt_ids)
                else:
                    for t in prompt_ids:  # every prompt token is a decode step; only the last pick is kept
                        token = self._step(t)
            else:
                token = self._step(new_ids[-1])
            new_ids.append(token)
            if on_token:
                on_token(token)
            if token == self.eos_token_id or self._hit_stop(new_ids, opts):
                # pop tokens until no stop string remains, rewinding past_len with them (:411-424)
                if opts.stop_strings:
                    while new_ids and self._hit_stop(new_ids, opts):
                        new_ids.pop()
                        self._past_len = max(0, self._past_len - 1)
                break
        return new_ids

    def generate(self, prompt, max_new_tokens: int = 16, opts: Optional[GenerateOptions] = None) -> str:
        return self._text(self.generate_ids(prompt, max_new_tokens, opts))
