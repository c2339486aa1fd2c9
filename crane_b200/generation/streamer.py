"""Streamers: receivers of generated tokens, as in the reference
(crane-core/src/generation/streamer.rs:7-107).  ``append`` gets every generated
token except a final EOS; ``finalize`` is always called once, last."""
from __future__ import annotations

import queue
from typing import Callable, List, Optional, Tuple


class TokenStreamer:
    def append(self, token_id: int) -> None:
        raise NotImplementedError

    def finalize(self) -> None:
        raise NotImplementedError


class ListStreamer(TokenStreamer):
    """Collects token ids (no tokenizer needed)."""

    def __init__(self) -> None:
        self.tokens: List[int] = []
        self.finalized = False

    def append(self, token_id: int) -> None:
        self.tokens.append(int(token_id))

    def finalize(self) -> None:
        self.finalized = True


class TextStreamer(TokenStreamer):
    """Decodes every token with ``decode(token_id) -> str`` (for instance a
    ``tokenizers.Tokenizer``'s) into ``buffer`` and prints it as it comes."""

    def __init__(self, decode: Callable[[int], str], echo: bool = True):
        self.decode = decode
        self.buffer = ""
        self.echo = echo

    def append(self, token_id: int) -> None:
        text = self.decode(int(token_id))
        self.buffer += text
        if self.echo:
            print(text, end="", flush=True)

    def finalize(self) -> None:
        if self.echo:
            print()


class AsyncTextStreamer(TokenStreamer):
    """Puts ("token", text) messages and a final ("end",) on a queue that
    another thread reads (the reference's mpsc channel of
    ``StreamerMessage::{Token, End}``)."""

    def __init__(self, decode: Callable[[int], str]):
        self.decode = decode
        self.queue: "queue.Queue[Tuple]" = queue.Queue()

    @staticmethod
    def with_tokenizer(tokenizer) -> "AsyncTextStreamer":
        return AsyncTextStreamer(lambda t: tokenizer.decode([t], skip_special_tokens=True))

    def append(self, token_id: int) -> None:
        self.queue.put(("token", self.decode(int(token_id))))

    def finalize(self) -> None:
        self.queue.put(("end",))
