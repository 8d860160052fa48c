"""Jinja2 chat templates (reference ``astrai/tokenize/chat_template.py:9-102``).

Variables visible to a template: ``default_variables`` < ``special_tokens`` < per-call keyword arguments, plus
``messages`` and (if given) ``system_prompt``.  The compiled template is built on first use and dropped when the
object is pickled, so tokenizers travel to spawned data-loader workers.
"""

from __future__ import annotations

from typing import Any, Dict, List, Optional

from jinja2 import Template


MessageType = Dict[str, Any]  # one chat message: {"role": ..., "content": ...} plus whatever the template reads


class ChatTemplate:
    def __init__(self, name: str = "", template_str: str = "", description: str = "",
                 default_variables: Optional[Dict[str, Any]] = None, special_tokens: Optional[Dict[str, str]] = None):
        self.name, self.template_str, self.description = name, template_str, description
        self.default_variables = dict(default_variables or {})
        self.special_tokens = dict(special_tokens or {})
        self._jinja: Optional[Template] = None

    @classmethod
    def from_string(cls, template_str: str, description: str = "", default_variables=None, special_tokens=None):
        return cls("", template_str, description, default_variables, special_tokens)

    def __getstate__(self):
        state = dict(self.__dict__)
        state["_jinja"] = None
        return state

    def __setstate__(self, state):
        self.__dict__.update(state)

    def render(self, messages: List[Dict[str, Any]], system_prompt: Optional[str] = None, **extra: Any) -> str:
        if self._jinja is None:
            self._jinja = Template(self.template_str)
        variables = {**self.default_variables, **self.special_tokens, **extra, "messages": messages}
        if system_prompt is not None:
            variables["system_prompt"] = system_prompt
        return self._jinja.render(**variables)
