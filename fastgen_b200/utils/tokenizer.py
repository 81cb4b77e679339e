"""Tokenizer of a Hugging Face model folder, as the reference wraps it
(fastgen/utils/tokenizer.py:48-118): ``tokenizer.json`` through the
``tokenizers`` library, the chat template of ``tokenizer_config.json`` through
jinja2, and the stop tokens ``[eos_token]``."""

from __future__ import annotations

import json
from pathlib import Path
from typing import List, Optional, TypedDict


class Message(TypedDict):
    role: str
    content: str


class HfTokenizer:
    def __init__(self, directory) -> None:
        from tokenizers import Tokenizer

        directory = Path(directory)
        for name in ("tokenizer.json", "tokenizer_config.json"):
            if not (directory / name).is_file():
                raise RuntimeError(f"Could not find {directory / name}")
        self._tk = Tokenizer.from_file(str(directory / "tokenizer.json"))
        with open(directory / "tokenizer_config.json") as f:
            self._config = json.load(f)

    def encode(self, content: str) -> List[int]:
        return self._tk.encode(content, add_special_tokens=False).ids

    def decode(self, tokens: List[int]) -> str:
        return self._tk.decode(tokens, skip_special_tokens=False)

    def id_to_str(self, id: int) -> Optional[str]:
        return self._tk.id_to_token(id)

    def str_to_id(self, s: str) -> int:
        i = self._tk.token_to_id(s)
        if i is None:
            raise KeyError(f"{s!r} is not a token")
        return i

    @staticmethod
    def _content(token) -> Optional[str]:
        return token["content"] if isinstance(token, dict) else token

    def encode_dialog(self, dialog: List[Message], for_completion: bool = True) -> List[int]:
        from jinja2 import Template

        if "chat_template" not in self._config:
            raise RuntimeError("this tokenizer has no chat template")
        chat = Template(self._config["chat_template"]).render(
            messages=dialog,
            add_generation_prompt=for_completion,
            bos_token=self._content(self._config.get("bos_token")),
            eos_token=self._content(self._config.get("eos_token")),
        )
        return self.encode(chat)

    @property
    def stop_tokens(self) -> List[int]:
        eos = self._content(self._config.get("eos_token"))
        return [self.str_to_id(eos)] if eos else []

    @property
    def vocab_size(self) -> int:
        return self._tk.get_vocab_size()
