"""Pangu response parsers (reasoning and tool calls)."""
from .reasoning import PanguReasoningParser  # noqa: F401
from .tool_parser import PanguToolParser  # noqa: F401
