"""Structured output: JSON Schema -> byte automaton -> per-step vocabulary mask."""
from .automaton import Schema  # noqa: F401
from .matcher import Matcher, compile_response_format, compile_schema  # noqa: F401
from .tool_call import tool_call_schema  # noqa: F401
