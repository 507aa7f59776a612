"""Chat prompts for the command line: what is put around a user's line before it is tokenised.

lite_llama's command line wraps every line in a template chosen by model family and keeps the
conversation so far in it (lite_llama/utils/prompt_templates.py:19-105 the base class with
``insert_prompt`` / ``update_template``, :181-202 the Llama 3 roles, :367-397 the choice by name;
cli.py:26,49-50 their use).  Here a prompt object renders one turn from the turns before it and the
new line, and records the answer afterwards.  The Llama 3 form is the published chat format of the
instruct models: a header per role, ``<|eot_id|>`` after every message, the assistant's header left
open for the model to continue.  The tokenizer adds ``<|begin_of_text|>`` itself.
"""
from __future__ import annotations

from typing import List, Optional, Tuple


class ChatPrompt:
    """One conversation.  ``render(line)`` gives the model's input for the next turn,
    ``record(answer)`` adds the finished turn to the history, ``reset()`` forgets it."""

    def __init__(self) -> None:
        self.turns: List[Tuple[str, str]] = []        # (user line, answer)
        self._pending: Optional[str] = None

    def render(self, line: str) -> str:
        self._pending = line
        return self._render(self.turns, line)

    def record(self, answer: str) -> None:
        if self._pending is None:
            raise RuntimeError("record() without a render() before it")
        self.turns.append((self._pending, answer.strip()))
        self._pending = None

    def reset(self) -> None:
        self.turns.clear()
        self._pending = None

    def _render(self, turns: List[Tuple[str, str]], line: str) -> str:
        raise NotImplementedError


class PlainPrompt(ChatPrompt):
    """No template: the line as it is, no history (base models, and lite_llama's ``EmptyPrompter``,
    prompt_templates.py:127-134)."""

    def _render(self, turns, line):
        return line


class Llama3ChatPrompt(ChatPrompt):
    HEADER = "<|start_header_id|>{role}<|end_header_id|>\n\n"
    END = "<|eot_id|>"

    def __init__(self, system: str = "") -> None:
        super().__init__()
        self.system = system

    def _message(self, role: str, text: str) -> str:
        return self.HEADER.format(role=role) + text + self.END

    def _render(self, turns, line):
        parts = [self._message("system", self.system)] if self.system else []
        for user, answer in turns:
            parts.append(self._message("user", user))
            parts.append(self._message("assistant", answer))
        parts.append(self._message("user", line))
        parts.append(self.HEADER.format(role="assistant"))     # left open: the model writes the answer
        return "".join(parts)


def prompt_for_tokenizer(tokenizer, raw: bool = False, system: str = "") -> ChatPrompt:
    """The Llama 3 chat form when the tokenizer knows its role headers (an instruct checkpoint's
    does), else the plain one; ``raw`` forces the plain one."""
    if raw or tokenizer is None:
        return PlainPrompt()
    try:
        known = tokenizer.convert_tokens_to_ids(["<|start_header_id|>", "<|eot_id|>"])
        unk = getattr(tokenizer, "unk_token_id", None)
        if all(isinstance(t, int) and t >= 0 and t != unk for t in known):
            return Llama3ChatPrompt(system)
    except Exception:
        pass
    return PlainPrompt()
