"""Stop sequences on the worker (`StoppingCriteriaParameters.stop_sequences` of the contract).

The reference carries the field and stops on length only (src/blitz/stopping.h:21).  Here a worker ends a request
when the text of its generated tokens contains one of its stop sequences: after every step the last few tokens of
each such request are turned into text and searched (every token is at least one byte of text, so the longest stop
sequence plus one token bounds the window).  The text comes from the tokenizer the worker was started with; without
one, from the same `<id>` pseudo-text that its generations carry, which is also what a router without a tokenizer
matches against.  With tensor parallelism every shard makes the same decision from the same tokens.
"""
from __future__ import annotations

from typing import Callable, Dict, Iterable, List, Optional, Tuple

FINISH_STOP_SEQUENCE = 2     # proto FinishReason


def pseudo_text(ids: List[int]) -> str:
    return " ".join(f"<{i}>" for i in ids)


class StopSequences:
    MAX_TRACKED = 65536

    def __init__(self, detok: Optional[Callable[[List[int]], str]] = None):
        self.detok = detok or pseudo_text
        self.enabled = True          # False: leave stop sequences to the caller of the worker (a router checks them too)
        self.stops: Dict[int, Tuple[Tuple[str, ...], int]] = {}      # request id -> (texts, token window)

    @classmethod
    def from_tokenizer_file(cls, path: str) -> "StopSequences":
        if not path:
            return cls()
        from ..runtime import core
        tok = core.Tokenizer.from_file(path)
        return cls(lambda ids: tok.decode(list(ids), True))

    def add(self, batch) -> None:
        """Remember the stop sequences of the requests of a `Batch` message (prefill, live prefill, immigrate)."""
        if not self.enabled:
            return
        for r in batch.requests:
            texts = tuple(s for s in r.stopping_parameters.stop_sequences if s)
            if texts:
                self.stops[r.id] = (texts, max(len(s.encode()) for s in texts) + 1)
        if len(self.stops) > self.MAX_TRACKED:
            # entries leave when their request ends here (`check`, `forget`); requests that ended elsewhere (migrated
            # away, length stop) are swept by age so that a long-lived worker does not grow
            for rid in list(self.stops)[:len(self.stops) // 2]:
                del self.stops[rid]

    def check(self, b) -> None:
        """End the requests of native batch `b` whose generated text now contains one of their stop sequences."""
        if not self.stops:
            return
        for rid in b.unfinished_ids():
            ent = self.stops.get(rid)
            if ent is None:
                continue
            try:
                text = self.detok(b.generated_tail(rid, ent[1]))
            except Exception:  # noqa: BLE001 - a detokenizer that fails must not fail the step
                continue
            if any(s in text for s in ent[0]):
                b.finish_request(rid, FINISH_STOP_SEQUENCE)
                del self.stops[rid]

    def forget(self, request_ids: Iterable[int]) -> None:
        if self.stops:
            for rid in request_ids:
                self.stops.pop(rid, None)
