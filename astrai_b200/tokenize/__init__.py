from astrai_b200.tokenize.chat_template import ChatTemplate, MessageType
from astrai_b200.tokenize.tokenizer import AutoTokenizer, Message, Messages

__all__ = ["AutoTokenizer", "ChatTemplate", "Message", "MessageType", "Messages"]
