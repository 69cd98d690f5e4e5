"""Chat rendering of agent conversations (ChatML-like, JSON tool calls) and a tokenizer wrapper that keeps control
tokens apart from text.

A conversation is {"tools": [schema, ...] (optional), "messages": [{"role": "system" | "user" | "assistant" | "tool",
"content": str, "reasoning": str (assistant, optional), "tool_calls": [{"name", "arguments": {...}}] (assistant)}]}:

    <|im_start|>system\\n{text}[\\n\\n# Tools\\n\\n<tools>\\n{schema}\\n...</tools>]<|im_end|>\\n
    <|im_start|>user\\n{content}<|im_end|>\\n
    <|im_start|>assistant\\n[<think>\\n{reasoning}\\n</think>\\n\\n]{content}[\\n<tool_call>\\n{json}\\n</tool_call>]*<|im_end|>\\n
    <|im_start|>tool\\n<tool_response>\\n{content}\\n</tool_response><|im_end|>\\n

The model generates an assistant message's body and its <|im_end|>; the header and the newline after <|im_end|> come
from the harness. `pieces` returns (text, generated, control) triples built from the structure, never by searching
the text: a control piece is exactly one control token, every other piece is message text encoded on its own, so a
literal "<tool_call>" inside a tool output stays text and generated tokens never share a token with harness text
(reference: tools/data/chat_format.py:1-40; only its version-1 rendering is built).
"""

from __future__ import annotations

import json

IM_START, IM_END, EOT = "<|im_start|>", "<|im_end|>", "<|endoftext|>"
TOOL_CALL, TOOL_CALL_END = "<tool_call>", "</tool_call>"
TOOL_RESPONSE, TOOL_RESPONSE_END = "<tool_response>", "</tool_response>"
THINK, THINK_END, TOOLS, TOOLS_END = "<think>", "</think>", "<tools>", "</tools>"
CONTROL_TOKENS = (EOT, IM_START, IM_END, TOOL_CALL, TOOL_CALL_END, TOOL_RESPONSE, TOOL_RESPONSE_END, THINK, THINK_END,
                  TOOLS, TOOLS_END)
ROLES = ("system", "user", "assistant", "tool")

Piece = tuple[str, bool, bool]      # (text, generated, control)


def call_json(call: dict) -> str:
    return json.dumps({"name": call["name"], "arguments": call.get("arguments", {})}, ensure_ascii=False)


def pieces(conversation: dict) -> list[Piece]:
    out: list[Piece] = []
    text = lambda s, gen=False: out.append((s, gen, False)) if s else None
    ctrl = lambda s, gen=False: out.append((s, gen, True))
    tools = conversation.get("tools") or []
    for i, m in enumerate(conversation["messages"]):
        role = m["role"]
        if role not in ROLES:
            raise ValueError(f"message {i}: role {role!r} is not one of {ROLES}")
        ctrl(IM_START)
        text(role + "\n")
        content = m.get("content") or ""
        if role == "system":
            text(content)
            if tools:
                text("\n\n# Tools\n\n")
                ctrl(TOOLS)
                text("\n" + "\n".join(json.dumps(t, ensure_ascii=False) for t in tools) + "\n")
                ctrl(TOOLS_END)
        elif role == "user":
            text(content)
        elif role == "tool":
            ctrl(TOOL_RESPONSE)
            text("\n" + content + "\n")
            ctrl(TOOL_RESPONSE_END)
        else:
            if m.get("reasoning"):
                ctrl(THINK, True)
                text("\n" + m["reasoning"] + "\n", True)
                ctrl(THINK_END, True)
                text("\n\n", True)
            text(content, True)
            for call in m.get("tool_calls") or []:
                text("\n", True)
                ctrl(TOOL_CALL, True)
                text("\n" + call_json(call) + "\n", True)
                ctrl(TOOL_CALL_END, True)
        ctrl(IM_END, role == "assistant")
        text("\n")
    return out


def render(conversation: dict) -> str:
    return "".join(p[0] for p in pieces(conversation))


class ChatTokenizer:
    """A text tokenizer (`encode(str) -> ids`) with the control tokens at ids of their own, `first_control` upward (the
    byte tokenizer: 256 .. 266). `table[id]` is the bytes of every id, which is all the token-type labeller reads."""

    def __init__(self, base=None, first_control: int = 256, token_bytes=None):
        from .tokenizers import ByteTokenizer

        self.base = base if base is not None else ByteTokenizer()
        self.first_control = first_control
        self.control = {name: first_control + i for i, name in enumerate(CONTROL_TOKENS)}
        if token_bytes is None:
            if not isinstance(self.base, ByteTokenizer):
                raise ValueError("token_bytes (id -> bytes of every text token) is needed for a tokenizer that is not the byte one")
            token_bytes = [bytes([i]) for i in range(256)]
        self.table = list(token_bytes) + [b""] * max(0, first_control - len(token_bytes)) + [c.encode() for c in CONTROL_TOKENS]

    @property
    def vocab_size(self) -> int:
        return self.first_control + len(CONTROL_TOKENS)

    def encode_pieces(self, ps: list[Piece]) -> tuple[list[int], list[bool]]:
        ids, gen = [], []
        for text, generated, control in ps:
            new = [self.control[text]] if control else list(self.base.encode(text))
            ids += new
            gen += [generated] * len(new)
        return ids, gen

    def encode_conversation(self, conversation: dict) -> dict:
        """{"ids", "byte_lens", "scored"}: the eval-set document of a conversation, assistant tokens scored."""
        ids, gen = self.encode_pieces(pieces(conversation))
        return {"ids": ids, "byte_lens": [max(1, len(self.table[t])) for t in ids], "scored": gen}
