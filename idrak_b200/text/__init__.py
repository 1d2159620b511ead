"""Text: tokenizers, chat templates, tool-call parsers."""
from .chat import ChatTemplate, render_chat
from .tokenizer import ByteTokenizer, HfTokenizer, SentencePieceTokenizer, StreamingDecoder, Tokenizer
from .tokenizer_io import load_tokenizer, tokenizer_from_gguf, train_tokenizer
from .tool_calls import (ChatDelta, MarkedToolCallParser, ToolCall, create_parser, detect_format,
                         register_tool_call_format)

__all__ = ["ChatTemplate", "render_chat", "ByteTokenizer", "HfTokenizer", "SentencePieceTokenizer", "StreamingDecoder",
           "Tokenizer", "load_tokenizer", "tokenizer_from_gguf", "train_tokenizer", "ChatDelta", "MarkedToolCallParser",
           "ToolCall", "create_parser", "detect_format", "register_tool_call_format"]
from .conversation import Conversation, Tool  # noqa: E402,F401
