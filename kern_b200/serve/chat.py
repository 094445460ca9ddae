"""Chat on top of completions: OpenAI-style messages in (system / user / assistant with tool calls / tool results, an
optional list of tools), and the model's tool-call syntax out as structured `tool_calls`.

    messages_for_template(messages)   what a Hugging Face chat template takes: assistant `tool_calls` with their
                                      arguments as objects (the wire carries them as JSON text), tool results as they are
    select_parser(flag, declared)     which parser reads the output: a flag that says more than `auto` wins, else the
                                      manifest's `chat.tool_parser`, else `auto` (the syntax is recognised from the text)
    parse_tool_calls(text, parser)    -> (content left over, [tool_calls]); parsers: `hermes` — one JSON object
                                      {"name", "arguments"} per <tool_call>…</tool_call> block (Hermes, Qwen2.5 / Qwen3) —
                                      and `qwen3_coder` — <tool_call><function=NAME><parameter=KEY>VALUE</parameter>…
                                      </function></tool_call>, values read as JSON where they parse, else as text
    ToolStream                        the same over a token stream: content is passed on as it comes, except what could
                                      still turn out to be the start of a call; calls are delivered when their block closes

Reference counterpart: crates/kern-run/src/chat.rs:60-160 (message kinds, tool calls and results), crates/kern-serve/src/
lib.rs:60-70,300-315,465-480 (`--tool-call-parser`, the manifest's `chat.tool_parser`).
"""
from __future__ import annotations

import json
import re
import uuid

PARSERS = ("hermes", "qwen3_coder")
OPEN, CLOSE = "<tool_call>", "</tool_call>"


def select_parser(flag: str | None, declared: str | None) -> str:
    """`none` turns parsing off; `auto` (or nothing) defers to the manifest, and without one to recognition by syntax."""
    flag = (flag or "auto").lower()
    if flag != "auto":
        if flag != "none" and flag not in PARSERS:
            raise ValueError(f"unknown tool-call parser `{flag}`; known: auto, none, {', '.join(PARSERS)}")
        return flag
    if declared:
        if declared not in PARSERS:
            raise ValueError(f"the manifest names tool parser `{declared}`, which this server does not have; known: {', '.join(PARSERS)}")
        return declared
    return "auto"


def messages_for_template(messages: list[dict]) -> list[dict]:
    out = []
    for m in messages:
        role = m.get("role")
        if role not in ("system", "user", "assistant", "tool", "developer"):
            raise ValueError(f"message role `{role}`")
        m = dict(m)
        if role == "assistant" and m.get("tool_calls"):
            calls = []
            for c in m["tool_calls"]:
                fn = dict(c.get("function") or {})
                args = fn.get("arguments", {})
                if isinstance(args, str):
                    try:
                        args = json.loads(args) if args.strip() else {}
                    except json.JSONDecodeError as e:
                        raise ValueError(f"tool call `{fn.get('name')}`: arguments are not JSON ({e})") from None
                fn["arguments"] = args
                calls.append({"id": c.get("id", ""), "type": "function", "function": fn})
            m["tool_calls"] = calls
            m["content"] = m.get("content") or ""
        if role == "tool" and not isinstance(m.get("content"), str):
            m["content"] = json.dumps(m.get("content"))
        out.append(m)
    return out


def _call(name: str, arguments) -> dict:
    return {"id": "call_" + uuid.uuid4().hex[:24], "type": "function",
            "function": {"name": name, "arguments": arguments if isinstance(arguments, str) else json.dumps(arguments)}}


def _hermes(block: str) -> dict | None:
    try:
        obj = json.loads(block.strip())
    except json.JSONDecodeError:
        return None
    if not isinstance(obj, dict) or not isinstance(obj.get("name"), str):
        return None
    return _call(obj["name"], obj.get("arguments", obj.get("parameters", {})))


_FN = re.compile(r"<function=([^>\s]+)>(.*?)</function>", re.S)
_PARAM = re.compile(r"<parameter=([^>\s]+)>(.*?)</parameter>", re.S)


def _qwen3_coder(block: str) -> dict | None:
    m = _FN.search(block)
    if m is None:
        return None
    args = {}
    for key, raw in _PARAM.findall(m.group(2)):
        val = raw[1:] if raw.startswith("\n") else raw
        val = val[:-1] if val.endswith("\n") else val
        try:
            args[key] = json.loads(val)
        except json.JSONDecodeError:
            args[key] = val
    return _call(m.group(1), args)


def _block(block: str, parser: str) -> dict | None:
    if parser == "hermes":
        return _hermes(block)
    if parser == "qwen3_coder":
        return _qwen3_coder(block)
    return _hermes(block) or _qwen3_coder(block)            # auto: by syntax


def parse_tool_calls(text: str, parser: str = "auto") -> tuple[str, list[dict]]:
    """Split a completed answer into its content and its tool calls. A block that does not parse stays in the content
    as written (the client sees what the model wrote); an unclosed last block is read to the end of the text."""
    if parser == "none" or OPEN not in text:
        return text, []
    content, calls, at = [], [], 0
    while True:
        i = text.find(OPEN, at)
        if i < 0:
            content.append(text[at:])
            break
        j = text.find(CLOSE, i + len(OPEN))
        end = len(text) if j < 0 else j
        got = _block(text[i + len(OPEN):end], parser)
        content.append(text[at:i])
        if got is None:
            content.append(text[i:end + (len(CLOSE) if j >= 0 else 0)])
        else:
            calls.append(got)
        if j < 0:
            break
        at = j + len(CLOSE)
    return "".join(content).strip() if calls else text, calls


class ToolStream:
    """`feed(piece) -> (content to pass on now, calls that closed)`; `finish() -> (content, calls)` for what is left."""

    def __init__(self, parser: str = "auto"):
        self.parser, self.buf, self.inside = parser, "", False
        self.calls = 0

    def feed(self, piece: str) -> tuple[str, list[dict]]:
        if self.parser == "none":
            return piece, []
        self.buf += piece
        out, calls = [], []
        while True:
            if self.inside:
                j = self.buf.find(CLOSE)
                if j < 0:
                    break
                got = _block(self.buf[:j], self.parser)
                if got is None:
                    out.append(OPEN + self.buf[:j + len(CLOSE)])
                else:
                    got["index"] = self.calls
                    self.calls += 1
                    calls.append(got)
                self.buf, self.inside = self.buf[j + len(CLOSE):], False
            else:
                i = self.buf.find(OPEN)
                if i >= 0:
                    out.append(self.buf[:i])
                    self.buf, self.inside = self.buf[i + len(OPEN):], True
                    continue
                # keep back a tail that could still become the opening tag
                keep = next((k for k in range(min(len(OPEN) - 1, len(self.buf)), 0, -1) if OPEN.startswith(self.buf[-k:])), 0)
                out.append(self.buf[:len(self.buf) - keep])
                self.buf = self.buf[len(self.buf) - keep:]
                break
        return "".join(out), calls

    def finish(self) -> tuple[str, list[dict]]:
        if self.parser == "none":
            return "", []
        if self.inside:
            got = _block(self.buf, self.parser)
            self.buf, self.inside = ("", False) if got is not None else (OPEN + self.buf, False)
            if got is not None:
                got["index"] = self.calls
                self.calls += 1
                return "", [got]
        rest, self.buf = self.buf, ""
        return rest, []
