"""Chat on top of completions: message kinds, parser selection, the two tool-call syntaxes (whole answers and token
streams), and the HTTP surface with `tools` in the request."""
import json
import urllib.request

import pytest

from kern_b200.serve import chat


def test_parser_selection_flag_manifest_auto():
    assert chat.select_parser(None, None) == "auto" and chat.select_parser("auto", "hermes") == "hermes"
    assert chat.select_parser("qwen3_coder", "hermes") == "qwen3_coder" and chat.select_parser("none", "hermes") == "none"
    with pytest.raises(ValueError):
        chat.select_parser("auto", "mystery_parser")
    with pytest.raises(ValueError):
        chat.select_parser("Hermes-2", None)


def test_messages_for_a_template():
    msgs = [{"role": "system", "content": "s"}, {"role": "user", "content": "weather?"},
            {"role": "assistant", "content": None, "tool_calls": [{"id": "c1", "type": "function",
                                                                   "function": {"name": "get_weather", "arguments": "{\"city\": \"Oslo\"}"}}]},
            {"role": "tool", "tool_call_id": "c1", "content": {"temp": 3}}]
    out = chat.messages_for_template(msgs)
    assert out[2]["tool_calls"][0]["function"]["arguments"] == {"city": "Oslo"} and out[2]["content"] == ""
    assert out[3]["content"] == '{"temp": 3}' and out[3]["tool_call_id"] == "c1"
    with pytest.raises(ValueError):
        chat.messages_for_template([{"role": "narrator", "content": "x"}])
    with pytest.raises(ValueError):
        chat.messages_for_template([{"role": "assistant", "tool_calls": [{"function": {"name": "f", "arguments": "{not json"}}]}])


HERMES = 'Let me check.\n<tool_call>\n{"name": "get_weather", "arguments": {"city": "Oslo", "days": 2}}\n</tool_call>\n<tool_call>\n{"name": "now", "arguments": {}}\n</tool_call>'
CODER = ('<tool_call>\n<function=write_file>\n<parameter=path>\n/tmp/a.txt\n</parameter>\n<parameter=lines>\n[1, 2]\n</parameter>\n'
         '<parameter=text>\nhello\nworld\n</parameter>\n</function>\n</tool_call>')


@pytest.mark.parametrize("parser", ["auto", "hermes"])
def test_hermes_blocks(parser):
    content, calls = chat.parse_tool_calls(HERMES, parser)
    assert content == "Let me check." and [c["function"]["name"] for c in calls] == ["get_weather", "now"]
    assert json.loads(calls[0]["function"]["arguments"]) == {"city": "Oslo", "days": 2} and calls[0]["type"] == "function"
    assert calls[0]["id"].startswith("call_") and calls[0]["id"] != calls[1]["id"]


@pytest.mark.parametrize("parser", ["auto", "qwen3_coder"])
def test_qwen3_coder_blocks(parser):
    content, calls = chat.parse_tool_calls(CODER, parser)
    assert content == "" and calls[0]["function"]["name"] == "write_file"
    assert json.loads(calls[0]["function"]["arguments"]) == {"path": "/tmp/a.txt", "lines": [1, 2], "text": "hello\nworld"}


def test_what_does_not_parse_stays_as_written():
    text = "a <tool_call>not a call</tool_call> b"
    assert chat.parse_tool_calls(text, "auto") == (text, [])
    assert chat.parse_tool_calls(HERMES, "none") == (HERMES, [])
    assert chat.parse_tool_calls(HERMES, "qwen3_coder")[1] == []          # the other syntax: nothing is taken
    # an unclosed last block is read to the end of the text
    assert chat.parse_tool_calls('<tool_call>{"name": "f", "arguments": {"x": 1}}', "hermes")[1][0]["function"]["name"] == "f"


@pytest.mark.parametrize("cut", [1, 3, 7, 50])
def test_stream_passes_content_on_and_delivers_calls_when_they_close(cut):
    ts = chat.ToolStream("auto")
    text = "Sure. <not a tag> " + HERMES + " done"
    content, calls = "", []
    for i in range(0, len(text), cut):
        c, k = ts.feed(text[i:i + cut])
        assert "<tool_call>" not in c and "</tool_call>" not in c
        content += c
        calls += k
    c, k = ts.finish()
    content += c
    calls += k
    assert [x["function"]["name"] for x in calls] == ["get_weather", "now"] and [x["index"] for x in calls] == [0, 1]
    assert content.replace("\n", "") == "Sure. <not a tag> Let me check. done"


def test_http_chat_completions_with_tools():
    """A model that answers in the hermes syntax (the byte-level toy decoder cannot; the engine is a stand-in that emits a
    fixed answer) gets `tool_calls` and finish_reason `tool_calls`, whole and streamed; without `tools` the text is left."""
    from kern_b200.serve.scheduler import Request
    from kern_b200.serve.server import ByteTokenizer, Server

    answer = list(HERMES.encode()) + [0]

    class Scripted:
        """The scheduler interface over a script: every request receives `answer`, four tokens a step."""
        stats = type("S", (), {"steps": 0, "step_seconds": 0.0, "prefill_tokens": 0, "decode_tokens": 0, "proposed": 0, "accepted": 0,
                               "prefix_hits": 0, "prefix_queries": 0, "prefix_hit_tokens": 0})()

        def __init__(self):
            self.live: list[Request] = []

        def submit(self, r):
            self.live.append(r)

        def abort(self, rid):
            return False

        def idle(self):
            return not self.live

        def metrics(self):
            return {"kv_used_blocks": 0, "kv_total_blocks": 1, "num_running_reqs": len(self.live), "num_waiting_reqs": 0,
                    "spec_decode": {"accepted": 0, "proposed": 0}, "prefix_cache": {"queries": 0, "hits": 0, "hit_tokens": 0, "entries": 0}}

        def step(self):
            out = []
            for r in list(self.live):
                new = answer[len(r.out):len(r.out) + 4]
                r.out += new
                if r.out[-1:] == [0]:
                    r.finished = "stop"
                    self.live.remove(r)
                out.append((r, new))
            return out

    srv = Server(Scripted(), ByteTokenizer(), model_name="scripted", port=0, tool_parser="auto").start()
    base = f"http://127.0.0.1:{srv.port}"
    try:
        def post(body):
            req = urllib.request.Request(base + "/v1/chat/completions", data=json.dumps(body).encode(), headers={"Content-Type": "application/json"})
            return urllib.request.urlopen(req, timeout=60)

        tools = [{"type": "function", "function": {"name": "get_weather", "parameters": {"type": "object"}}}]
        msgs = [{"role": "user", "content": "weather in Oslo?"}]
        whole = json.load(post({"messages": msgs, "tools": tools, "max_tokens": 400}))["choices"][0]
        assert whole["finish_reason"] == "tool_calls" and whole["message"]["content"] == "Let me check."
        assert [c["function"]["name"] for c in whole["message"]["tool_calls"]] == ["get_weather", "now"]
        plain = json.load(post({"messages": msgs, "max_tokens": 400}))["choices"][0]
        assert plain["finish_reason"] == "stop" and "<tool_call>" in plain["message"]["content"] and "tool_calls" not in plain["message"]
        events = [json.loads(l[6:]) for l in post({"messages": msgs, "tools": tools, "max_tokens": 400, "stream": True}).read().decode().splitlines()
                  if l.startswith("data: {")]
        deltas = [e["choices"][0]["delta"] for e in events]
        assert "".join(d.get("content", "") for d in deltas).strip() == "Let me check."
        assert [c["function"]["name"] for d in deltas for c in d.get("tool_calls", [])] == ["get_weather", "now"]
        assert events[-1]["choices"][0]["finish_reason"] == "tool_calls"
        # a conversation that carries the call and its result back renders (the template sees arguments as objects)
        again = msgs + [{"role": "assistant", "content": None, "tool_calls": whole["message"]["tool_calls"]},
                        {"role": "tool", "tool_call_id": whole["message"]["tool_calls"][0]["id"], "content": "3 C"}]
        assert json.load(post({"messages": again, "tools": tools, "max_tokens": 400}))["choices"][0]["finish_reason"] == "tool_calls"
    finally:
        srv.stop()
