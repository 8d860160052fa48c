"""Tokenizer front end over the HuggingFace ``tokenizers`` library.

Reference behaviour (``astrai/tokenize/tokenizer.py:20-289``): a directory holds ``tokenizer.json`` and
``tokenizer_config.json`` (``special_tokens`` map and ``chat_template``); ``encode`` takes a string or a list (batch
encode in the Rust backend); ``<name>`` / ``<name>_id`` attributes resolve through the special-token map and
``stop_ids`` is the id of EVERY special token.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, List, Optional, Union

from tokenizers import Tokenizer

from astrai_b200.tokenize.chat_template import ChatTemplate

Message = Dict[str, str]
Messages = List[Message]


class AutoTokenizer:
    def __init__(self, path: Optional[Union[str, Path]] = None, special_token_map: Optional[Dict[str, str]] = None,
                 chat_template: Optional[str] = None):
        self._tokenizer: Optional[Tokenizer] = None
        self._chat_template: Optional[ChatTemplate] = None
        self._special_token_map: Dict[str, str] = dict(special_token_map or {})
        if chat_template:
            self.set_chat_template(chat_template)
        if path:
            self.load(path)

    # -- persistence ------------------------------------------------------------------------------------------------
    def load(self, path: Union[str, Path]):
        root = Path(path)
        self._tokenizer = Tokenizer.from_file(str(root / "tokenizer.json"))
        cfg_file = root / "tokenizer_config.json"
        if cfg_file.exists():
            cfg = json.loads(cfg_file.read_text(encoding="utf-8"))
            self._special_token_map.update(cfg.get("special_tokens") or {})
            if cfg.get("chat_template"):
                self.set_chat_template(cfg["chat_template"])

    @classmethod
    def from_pretrained(cls, path: Union[str, Path]) -> "AutoTokenizer":
        file = Path(path) / "tokenizer.json"
        if not file.exists():
            raise FileNotFoundError(f"Tokenizer file not found: {file}. A valid tokenizer.json is required.")
        tok = cls(path)
        if tok._tokenizer is None:
            raise RuntimeError(f"Failed to load tokenizer from {path}.")
        return tok

    def _need(self) -> Tokenizer:
        if self._tokenizer is None:
            raise RuntimeError("Tokenizer not initialized. Load or create a tokenizer first.")
        return self._tokenizer

    def save_pretrained(self, save_path: str):
        tk = self._need()
        out = Path(save_path)
        out.mkdir(parents=True, exist_ok=True)
        tk.save(str(out / "tokenizer.json"))
        cfg = {"special_tokens": self._special_token_map}
        if self._chat_template is not None:
            cfg["chat_template"] = self._chat_template.template_str
        (out / "tokenizer_config.json").write_text(json.dumps(cfg, ensure_ascii=False, indent=2), encoding="utf-8")

    # -- text <-> ids --------------------------------------------------------------------------------------------------
    def encode(self, tokens: Union[str, List[str]], out_ids: bool = True, is_pretokenized: bool = False,
               add_special_tokens: bool = True) -> List:
        tk = self._need()
        pick = (lambda e: e.ids) if out_ids else (lambda e: e.tokens)
        if isinstance(tokens, str):
            return pick(tk.encode(tokens, is_pretokenized=is_pretokenized, add_special_tokens=add_special_tokens))
        return [pick(e) for e in tk.encode_batch(tokens, is_pretokenized=is_pretokenized, add_special_tokens=add_special_tokens)]

    def decode(self, tokens: List[int], skip_special_tokens: bool = True) -> str:
        return self._need().decode(tokens, skip_special_tokens=skip_special_tokens)

    def __len__(self) -> int:
        return 0 if self._tokenizer is None else self._tokenizer.get_vocab_size()

    @property
    def vocab_size(self) -> int:
        return len(self)

    @property
    def backend(self) -> Optional[Tokenizer]:
        return self._tokenizer

    # -- special tokens ---------------------------------------------------------------------------------------------
    def __getattr__(self, key: str):
        if key.startswith("_"):  # also keeps unpickling from recursing before __dict__ exists
            raise AttributeError(key)
        special = self.__dict__.get("_special_token_map", {})
        tk = self.__dict__.get("_tokenizer")
        if key == "stop_ids":
            if tk is None:
                return []
            ids = (tk.token_to_id(v) for v in special.values())
            return [i for i in ids if i is not None]
        if key.endswith("_id"):
            text = special.get(key[:-3])
            if text is None:
                return None
            if tk is None:
                raise RuntimeError("Tokenizer not loaded, cannot convert token to id.")
            return tk.token_to_id(text)
        if key in special:
            return special[key]
        raise AttributeError(f"'{type(self).__name__}' object has no attribute '{key}'")

    # -- chat templates ------------------------------------------------------------------------------------------------
    def set_chat_template(self, template: Union[str, ChatTemplate]):
        if isinstance(template, ChatTemplate):
            self._chat_template = template
        elif isinstance(template, str):
            self._chat_template = ChatTemplate.from_string(template)
        else:
            raise ValueError("Invalid template type, must be str or ChatTemplate.")

    def apply_chat_template(self, messages: Union[Messages, List[Messages]], system_prompt: Optional[str] = None,
                            tokenize: bool = True, add_generation_prompt: bool = True, **kwargs):
        """One conversation -> ``str`` / ``List[int]``; a list of conversations -> a list of those (batch encode)."""
        if self._chat_template is None:
            raise RuntimeError("Chat template not set. Use set_chat_template() to set a template first.")
        render = lambda msgs: self._chat_template.render(messages=msgs, add_generation_prompt=add_generation_prompt, **kwargs)  # noqa: E731
        if messages and isinstance(messages[0], list):
            texts = [render(m) for m in messages]
            return self.encode(texts) if tokenize else texts
        if system_prompt:
            messages = [{"role": "system", "content": system_prompt}, *messages]
        text = render(messages)
        return self.encode(text) if tokenize else text
