"""The Pangu parsers as the host engine's parser classes, registered by name ``pangu`` so that its API server accepts
``--reasoning-parser pangu --tool-call-parser pangu`` (reference: omni/models/pangu/reasoning/*, tool_parsers/*, which
register with the same managers).  Imported lazily by the managers: nothing here loads unless the host engine asks."""
from __future__ import annotations

from .reasoning import END as R_END, START as R_START, PanguReasoningParser
from .tool_parser import PanguToolParser

try:
    from vllm.reasoning import ReasoningParser as _ReasoningBase
except Exception:  # noqa: BLE001  (no host engine in this environment)
    _ReasoningBase = object
try:
    from vllm.tool_parsers import ToolParser as _ToolBase
except Exception:  # noqa: BLE001
    _ToolBase = object


class PanguHostReasoningParser(_ReasoningBase):
    def __init__(self, tokenizer=None, *args, **kwargs):
        if _ReasoningBase is not object and tokenizer is not None:
            super().__init__(tokenizer, *args, **kwargs)
        self._impl = PanguReasoningParser()
        vocab = getattr(tokenizer, "get_vocab", lambda: {})() if tokenizer is not None else {}
        self._end_id = vocab.get(R_END)

    @property
    def reasoning_start_str(self) -> str:
        return R_START

    @property
    def reasoning_end_str(self) -> str:
        return R_END

    def is_reasoning_end(self, input_ids) -> bool:
        return self._end_id is not None and self._end_id in input_ids

    def extract_content_ids(self, input_ids) -> list:
        if self._end_id is None or self._end_id not in input_ids:
            return []
        ids = list(input_ids)
        return ids[ids.index(self._end_id) + 1:]

    def extract_reasoning(self, model_output: str, request=None):
        return self._impl.extract_reasoning_content(model_output)

    def extract_reasoning_streaming(self, previous_text, current_text, delta_text, previous_token_ids=(), current_token_ids=(),
                                    delta_token_ids=()):
        d = self._impl.extract_reasoning_content_streaming(previous_text, delta_text)
        if d is None:
            return None
        try:
            from vllm.entrypoints.openai.engine.protocol import DeltaMessage
            return DeltaMessage(reasoning=d.get("reasoning_content"), content=d.get("content"))
        except Exception:  # noqa: BLE001  (protocol class moved or absent: the plain mapping says the same)
            return d


class PanguHostToolParser(_ToolBase):
    def __init__(self, tokenizer=None, *args, **kwargs):
        if _ToolBase is not object and tokenizer is not None:
            super().__init__(tokenizer, *args, **kwargs)
        self._impl = PanguToolParser()

    def extract_tool_calls(self, model_output: str, request=None):
        ex = self._impl.extract_tool_calls(model_output)
        try:
            from vllm.entrypoints.openai.engine.protocol import ExtractedToolCallInformation, FunctionCall, ToolCall
            calls = [ToolCall(id=c.id, type="function", function=FunctionCall(name=c.name, arguments=c.arguments)) for c in ex.tool_calls]
            return ExtractedToolCallInformation(tools_called=ex.tools_called, tool_calls=calls, content=ex.content)
        except Exception:  # noqa: BLE001
            return ex

    def extract_tool_calls_streaming(self, previous_text, current_text, delta_text, previous_token_ids=(), current_token_ids=(),
                                     delta_token_ids=(), request=None):
        return self._impl.extract_tool_calls_streaming(previous_text, delta_text)


def register_with_host_engine() -> dict:
    """Registers both parsers under the name ``pangu``; returns which registrations were possible."""
    done = {"reasoning": False, "tool": False}
    try:
        from vllm.reasoning import ReasoningParserManager
        ReasoningParserManager.register_lazy_module("pangu", __name__, "PanguHostReasoningParser")
        done["reasoning"] = True
    except Exception:  # noqa: BLE001
        pass
    try:
        from vllm.tool_parsers import ToolParserManager
        ToolParserManager.register_lazy_module("pangu", __name__, "PanguHostToolParser")
        done["tool"] = True
    except Exception:  # noqa: BLE001
        pass
    return done
