from astrai_b200.inference.network.anthropic import AnthropicResponseBuilder
from astrai_b200.inference.network.app import (
    AnthropicMessage, ChatCompletionRequest, ChatMessage, CompletionRequest, FunctionDef, MessagesRequest, ToolDef, create_engine, get_app, run_server,
)
from astrai_b200.inference.network.completions import CompletionResponseBuilder
from astrai_b200.inference.network.openai import OpenAIResponseBuilder
from astrai_b200.inference.network.protocol import (
    GenContext, ProtocolHandler, ResponseBuilder, StopChecker, StopInfo, sse_done, sse_event,
)
from astrai_b200.inference.network.tool_parser import BaseToolParser, SimpleJsonToolParser, ToolParserFactory

__all__ = [
    "AnthropicMessage", "AnthropicResponseBuilder", "BaseToolParser", "ChatCompletionRequest", "ChatMessage", "CompletionRequest", "CompletionResponseBuilder", "FunctionDef", "GenContext",
    "MessagesRequest", "OpenAIResponseBuilder", "ProtocolHandler", "ResponseBuilder", "SimpleJsonToolParser", "StopChecker",
    "StopInfo", "ToolDef", "ToolParserFactory", "create_engine", "get_app", "run_server", "sse_done", "sse_event",
]
