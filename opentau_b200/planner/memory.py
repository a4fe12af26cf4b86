"""Rolling conversation memory of a planner (reference ``src/opentau/planner/utils/memory.py:20-70``)."""

from __future__ import annotations


class Memory:
    def __init__(self, conversation: list[dict] | None = None, len: int = 1000):  # noqa: A002 - reference signature
        self.max_len = len
        self.conversation: list[dict] = list(conversation or [])

    def add_conversation(self, role: str, message) -> None:
        if role not in ("system", "user", "assistant"):
            raise ValueError(f"unknown role {role!r}")
        self.conversation.append({"role": role, "content": message})
        if builtins_len(self.conversation) > self.max_len:
            # keep the system prompt(s), drop the oldest exchange
            keep = [m for m in self.conversation if m["role"] == "system"]
            rest = [m for m in self.conversation if m["role"] != "system"]
            self.conversation = keep + rest[-(self.max_len - builtins_len(keep)):]

    def get_conversation(self) -> list[dict]:
        return list(self.conversation)

    def clear(self) -> None:
        self.conversation = [m for m in self.conversation if m["role"] == "system"]


def builtins_len(x) -> int:
    return x.__len__()
