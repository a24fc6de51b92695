"""Pangu reasoning parser (reference: omni/models/pangu/reasoning/*): the model wraps its chain of thought in
``[unused16] ... [unused17]``; everything after the end marker is the answer.  Works on complete strings and on
streamed deltas."""
from __future__ import annotations

from typing import Optional

START, END = "[unused16]", "[unused17]"


class PanguReasoningParser:
    start_token, end_token = START, END

    def extract_reasoning_content(self, text: str) -> tuple:
        """-> (reasoning or None, content or None)."""
        if START in text:
            text = text.split(START, 1)[1]
        elif END not in text:
            return None, text or None
        if END not in text:
            return text or None, None
        reasoning, content = text.split(END, 1)
        return reasoning or None, content or None

    def extract_reasoning_content_streaming(self, previous_text: str, delta_text: str) -> Optional[dict]:
        """Delta message with 'reasoning_content' and/or 'content'; the markers themselves are swallowed, and a
        marker that arrives split over several deltas is held back until it is complete."""
        r0, c0 = self._parts(self._stable(previous_text))
        r1, c1 = self._parts(self._stable(previous_text + delta_text))
        out = {}
        if len(r1) > len(r0):
            out["reasoning_content"] = r1[len(r0):]
        if len(c1) > len(c0):
            out["content"] = c1[len(c0):]
        return out or None

    @staticmethod
    def _stable(text: str) -> str:
        """Text without a trailing fragment that could still grow into a marker."""
        for marker in (START, END):
            for k in range(len(marker) - 1, 0, -1):
                if text.endswith(marker[:k]):
                    return text[:-k]
        return text

    def _parts(self, text: str) -> tuple:
        r, c = self.extract_reasoning_content(text)
        return r or "", c or ""
