"""Pangu tool-call parser (reference: omni/models/pangu/tool_parsers/*): tool calls are emitted as
``[unused11]name|{json arguments}[unused12]`` (several may follow each other); text outside the markers is
ordinary content."""
from __future__ import annotations

import json
import re
import uuid
from dataclasses import dataclass, field
from typing import Optional

START, END, SEP = "[unused11]", "[unused12]", "|"
_CALL = re.compile(re.escape(START) + r"(.*?)" + re.escape(END), re.S)


@dataclass
class ToolCall:
    name: str
    arguments: str
    id: str = field(default_factory=lambda: "call_" + uuid.uuid4().hex[:24])
    type: str = "function"

    def to_dict(self) -> dict:
        return {"id": self.id, "type": self.type, "function": {"name": self.name, "arguments": self.arguments}}


@dataclass
class ExtractedToolCalls:
    tools_called: bool
    tool_calls: list
    content: Optional[str]


class PanguToolParser:
    def extract_tool_calls(self, text: str) -> ExtractedToolCalls:
        calls = []
        for body in _CALL.findall(text):
            # the body may itself be a JSON list of {"name", "arguments"} objects, or "name|{json}"
            body = body.strip()
            parsed = self._parse_body(body)
            if parsed:
                calls.extend(parsed)
        content = _CALL.sub("", text).strip() or None
        if not calls:
            return ExtractedToolCalls(False, [], text or None)
        return ExtractedToolCalls(True, calls, content)

    @staticmethod
    def _parse_body(body: str) -> list:
        if body.startswith("["):
            try:
                items = json.loads(body)
                return [ToolCall(i["name"], json.dumps(i.get("arguments", i.get("parameters", {})), ensure_ascii=False))
                        for i in items if isinstance(i, dict) and "name" in i]
            except (json.JSONDecodeError, TypeError):
                return []
        if SEP in body:
            name, args = body.split(SEP, 1)
            try:
                args = json.dumps(json.loads(args), ensure_ascii=False)
            except json.JSONDecodeError:
                return []
            return [ToolCall(name.strip(), args)]
        return []

    # ---- streaming: emit content as it comes, a tool call once its end marker has arrived
    def extract_tool_calls_streaming(self, previous_text: str, delta_text: str) -> Optional[dict]:
        current = previous_text + delta_text
        open_idx = current.rfind(START)
        closed = open_idx != -1 and current.find(END, open_idx) != -1
        if open_idx != -1 and not closed:
            return None                                      # inside an unfinished call: hold back
        for k in range(1, len(START)):
            if current.endswith(START[:k]):
                return None
        n_before = len(_CALL.findall(previous_text))
        found = _CALL.findall(current)
        if len(found) > n_before:
            calls = []
            for body in found[n_before:]:
                calls.extend(self._parse_body(body.strip()))
            return {"tool_calls": [dict(c.to_dict(), index=n_before + i) for i, c in enumerate(calls)]} if calls else None
        return {"content": delta_text} if delta_text else None
