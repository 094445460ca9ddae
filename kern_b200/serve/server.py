"""OpenAI-compatible HTTP front of the scheduler (stdlib only).

Endpoints: POST /v1/completions, POST /v1/chat/completions (optionally streamed as server-sent events),
GET /v1/models, GET /health, GET /kern/metrics (Prometheus text), POST /kern/trace/rotate.
Extras kept from the reference's surface: `return_token_ids`, `usage.prompt_tokens_details.cached_tokens`.

One driver thread owns the scheduler and the device: HTTP threads only enqueue requests and wait on
per-request queues, so nothing but the driver ever touches CUDA.
Reference: crates/kern-serve/src/lib.rs:483-546 (launch), examples/python/server.py:242-334 (minimum surface),
crates/kern-serve/src/kernels.rs:188-222,381-406 (metrics / rotate endpoints).
"""
from __future__ import annotations

import json
import logging
import queue
import threading
import time
import uuid
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer

from ..engine import Sampling
from .scheduler import Request, Scheduler

log = logging.getLogger("kern.serve")


class ByteTokenizer:
    """UTF-8 bytes as token ids (the toy models' tokenizer); id 0 ends a text."""
    eos_token_id = 0

    def encode(self, text: str) -> list[int]:
        return list(text.encode("utf-8"))

    def decode(self, ids) -> str:
        return bytes(int(i) & 0xFF for i in ids if int(i) != 0).decode("utf-8", errors="replace")

    def chat(self, messages, tools=None) -> list[int]:
        text = ("<tools>" + json.dumps(tools) + "\n" if tools else "") + \
            "".join(f"<{m.get('role', 'user')}>{m.get('content', '')}{json.dumps(m['tool_calls']) if m.get('tool_calls') else ''}\n"
                    for m in messages) + "<assistant>"
        return self.encode(text)


class HFTokenizer:
    """A Hugging Face tokenizer directory (tokenizer.json + chat template)."""

    def __init__(self, path: str):
        from transformers import AutoTokenizer

        self.tok = AutoTokenizer.from_pretrained(path)
        self.eos_token_id = self.tok.eos_token_id

    def encode(self, text: str) -> list[int]:
        return self.tok.encode(text, add_special_tokens=False)

    def decode(self, ids) -> str:
        return self.tok.decode(list(ids), skip_special_tokens=True)

    def chat(self, messages, tools=None) -> list[int]:
        return self.tok.apply_chat_template(messages, tools=tools or None, add_generation_prompt=True, tokenize=True)


class Driver(threading.Thread):
    """Owns the scheduler: admits what the HTTP threads queued, steps, fans tokens out."""

    def __init__(self, sched: Scheduler, idle_wait: float = 0.001):
        super().__init__(daemon=True, name="kern-driver")
        self.sched = sched
        self.inbox: queue.Queue = queue.Queue()
        self.streams: dict[str, queue.Queue] = {}
        self.stop_flag = threading.Event()
        self.idle_wait = idle_wait
        self.device_seconds = {"compute": 0.0, "idle": 0.0}
        self.started = time.monotonic()
        self.failed: str | None = None

    def submit(self, req: Request) -> queue.Queue:
        q: queue.Queue = queue.Queue()
        if self.failed:                       # the driver thread is gone: answer at once instead of queueing
            q.put(("error", self.failed))
            return q
        self.inbox.put(("submit", req, q))
        if self.failed:                       # it failed between the check and the put
            self._drain_inbox()
        return q

    def abort(self, req_id: str) -> None:
        self.inbox.put(("abort", req_id, None))

    def run(self) -> None:
        try:
            while not self.stop_flag.is_set():
                try:
                    while True:
                        kind, what, q = self.inbox.get_nowait()
                        if kind == "submit":
                            try:
                                self.sched.submit(what)
                                self.streams[what.id] = q
                            except ValueError as e:
                                q.put(("error", str(e)))
                        else:
                            if self.sched.abort(what):
                                s = self.streams.pop(what, None)
                                if s:
                                    s.put(("done", "abort"))
                except queue.Empty:
                    pass
                if self.sched.idle():
                    t0 = time.monotonic()
                    time.sleep(self.idle_wait)
                    self.device_seconds["idle"] += time.monotonic() - t0
                    continue
                t0 = time.monotonic()
                emitted = self.sched.step()
                self.device_seconds["compute"] += time.monotonic() - t0
                for req, toks in emitted:
                    s = self.streams.get(req.id)
                    if s is None:
                        continue
                    if toks:
                        s.put(("tokens", toks))
                    if req.finished:
                        s.put(("done", req.finished))
                        self.streams.pop(req.id, None)
        except Exception as e:   # a failed step fails every waiting client instead of hanging them
            log.exception("driver failed")
            self.failed = repr(e)
            for s in self.streams.values():
                s.put(("error", self.failed))
            self.streams.clear()
            self._drain_inbox()

    def _drain_inbox(self) -> None:
        """After a failure nothing reads the inbox any more: everyone queued in it gets the error now."""
        while True:
            try:
                kind, _, q = self.inbox.get_nowait()
            except queue.Empty:
                return
            if kind == "submit" and q is not None:
                q.put(("error", self.failed))


def prometheus(driver: Driver, model: str, recorder=None) -> str:
    m = driver.sched.metrics()
    st = driver.sched.stats
    if recorder is not None:          # a traced engine: the board comes from what the recorder saw, step by step
        from ..trace import prometheus_lines

        board = prometheus_lines(recorder)
    else:
        board = None
    lines = [
        "# TYPE kern_device_seconds_total counter",
        f'kern_device_seconds_total{{class="compute"}} {driver.device_seconds["compute"]:.6f}',
        f'kern_device_seconds_total{{class="comm"}} 0',
        f'kern_device_seconds_total{{class="idle"}} {driver.device_seconds["idle"]:.6f}',
        "# TYPE kern_step_compute_seconds_total counter",
        f"kern_step_compute_seconds_total {st.step_seconds:.6f}",
        "# TYPE kern_steps_total counter",
        f'kern_steps_total{{program="step",shape="mixed",kv="paged"}} {st.steps}',
        "# TYPE kern_trace_dropped_records_total counter",
        "kern_trace_dropped_records_total 0",
    ]
    if board is not None:
        lines = board
    lines += [
        "# TYPE kern_kv_used_blocks gauge",
        f"kern_kv_used_blocks {m['kv_used_blocks']}",
        f"kern_kv_total_blocks {m['kv_total_blocks']}",
        f"kern_num_running_reqs {m['num_running_reqs']}",
        f"kern_num_waiting_reqs {m['num_waiting_reqs']}",
        f"kern_prefix_cache_hits_total {m['prefix_cache']['hits']}",
        f"kern_prefix_cache_queries_total {m['prefix_cache']['queries']}",
        f"kern_prefill_tokens_total {st.prefill_tokens}",
        f"kern_decode_tokens_total {st.decode_tokens}",
    ]
    return "\n".join(lines) + "\n"


def make_handler(driver: Driver, tokenizer, model_name: str, on_rotate=None, tool_parser: str = "auto", recorder=None):
    class Handler(BaseHTTPRequestHandler):
        protocol_version = "HTTP/1.1"

        def log_message(self, fmt, *args):
            log.debug("http " + fmt, *args)

        def _json(self, code: int, obj) -> None:
            body = json.dumps(obj).encode()
            self.send_response(code)
            self.send_header("Content-Type", "application/json")
            self.send_header("Content-Length", str(len(body)))
            self.end_headers()
            self.wfile.write(body)

        def _text(self, code: int, text: str, ctype="text/plain; version=0.0.4") -> None:
            body = text.encode()
            self.send_response(code)
            self.send_header("Content-Type", ctype)
            self.send_header("Content-Length", str(len(body)))
            self.end_headers()
            self.wfile.write(body)

        def do_GET(self):
            if self.path == "/health":
                return self._json(503 if driver.failed else 200, {"status": driver.failed or "ok"})
            if self.path == "/v1/models":
                return self._json(200, {"object": "list", "data": [{"id": model_name, "object": "model", "owned_by": "kern_b200"}]})
            if self.path == "/kern/metrics":
                return self._text(200, prometheus(driver, model_name, recorder))
            self._json(404, {"error": {"message": f"no route {self.path}"}})

        def do_POST(self):
            n = int(self.headers.get("Content-Length", "0") or 0)
            try:
                body = json.loads(self.rfile.read(n) or b"{}")
            except json.JSONDecodeError:
                return self._json(400, {"error": {"message": "request body is not JSON"}})
            if self.path == "/kern/trace/rotate":
                if on_rotate:
                    on_rotate()
                return self._json(200, {"rotated": bool(on_rotate)})
            chat = self.path == "/v1/chat/completions"
            if not chat and self.path != "/v1/completions":
                return self._json(404, {"error": {"message": f"no route {self.path}"}})
            if driver.failed:
                return self._json(503, {"error": {"message": f"engine failed: {driver.failed}"}})
            try:
                history = None
                tools = body.get("tools") if chat else None
                if chat:
                    from .chat import messages_for_template

                    msgs = messages_for_template(body["messages"])
                    prompt = tokenizer.chat(msgs, tools) if tools else tokenizer.chat(msgs)
                    # the turn boundary: the rendering of everything before the last message is a prefix of the whole
                    # prompt when the template is prefix-stable; a model with per-sequence state snapshots it there
                    if len(msgs) > 1:
                        try:
                            head = tokenizer.chat(msgs[:-1], tools) if tools else tokenizer.chat(msgs[:-1])
                            n = 0
                            while n < min(len(head), len(prompt)) and head[n] == prompt[n]:
                                n += 1
                            history = n if 0 < n < len(prompt) else None
                        except Exception:
                            history = None
                else:
                    p = body.get("prompt", "")
                    prompt = list(p) if isinstance(p, list) and p and isinstance(p[0], int) else tokenizer.encode(p if isinstance(p, str) else p[0])
                if not prompt:
                    raise ValueError("empty prompt")
                sampling = Sampling(temperature=float(body.get("temperature", 0.0) or 0.0), top_k=int(body.get("top_k", 0) or 0),
                                    top_p=float(body.get("top_p", 1.0) or 1.0), min_p=float(body.get("min_p", 0.0) or 0.0),
                                    seed=int(body.get("seed", 0) or 0))
                stop = tuple(body.get("stop_token_ids") or ()) + (() if body.get("ignore_eos") else
                                                                  ((tokenizer.eos_token_id,) if tokenizer.eos_token_id is not None else ()))
                req = Request(id="cmpl-" + uuid.uuid4().hex[:16], prompt=prompt, max_tokens=int(body.get("max_tokens", 16)),
                              sampling=sampling, stop_ids=stop, history_tokens=history)
            except (KeyError, ValueError, TypeError) as e:
                return self._json(400, {"error": {"message": f"bad request: {e}"}})
            q = driver.submit(req)
            stream = bool(body.get("stream"))
            with_ids = bool(body.get("return_token_ids"))
            created = int(time.time())
            obj = "chat.completion" if chat else "text_completion"

            def usage():
                return {"prompt_tokens": len(prompt), "completion_tokens": len(req.out), "total_tokens": len(prompt) + len(req.out),
                        "prompt_tokens_details": {"cached_tokens": req.cached}}

            if stream:
                self.send_response(200)
                self.send_header("Content-Type", "text/event-stream")
                self.send_header("Cache-Control", "no-cache")
                self.send_header("Connection", "close")
                self.end_headers()
            text_ids: list[int] = []
            # with tools in the request, the model's tool-call syntax becomes structured `tool_calls`
            tstream = None
            if chat and tools and tool_parser != "none":
                from .chat import ToolStream, parse_tool_calls

                tstream = ToolStream(tool_parser)
            called = False
            try:
                while True:
                    try:
                        kind, what = q.get(timeout=600)
                    except queue.Empty:
                        kind, what = "error", "timed out waiting for the engine"
                    if kind == "error":
                        if stream:
                            self.wfile.write(f"data: {json.dumps({'error': {'message': what}})}\n\n".encode())
                            return
                        return self._json(500, {"error": {"message": what}})
                    if kind == "tokens":
                        text_ids.extend(what)
                        if stream:
                            piece = tokenizer.decode(what)
                            calls = []
                            if tstream is not None:
                                piece, calls = tstream.feed(piece)
                                called = called or bool(calls)
                            delta = {"delta": {"content": piece, **({"tool_calls": calls} if calls else {})}} if chat else {"text": piece}
                            chunk = {"id": req.id, "object": obj + ".chunk", "created": created, "model": model_name,
                                     "choices": [{"index": 0, **delta, "finish_reason": None, **({"token_ids": what} if with_ids else {})}]}
                            self.wfile.write(f"data: {json.dumps(chunk)}\n\n".encode())
                            self.wfile.flush()
                    if kind == "done":
                        finish = what
                        break
            except (BrokenPipeError, ConnectionResetError):
                driver.abort(req.id)     # the client left: free its seat
                return
            text = tokenizer.decode(text_ids)
            if stream:
                tail = {}
                if tstream is not None:
                    rest, calls = tstream.finish()
                    called = called or bool(calls)
                    tail = {**({"content": rest} if rest else {}), **({"tool_calls": calls} if calls else {})}
                    if called and finish == "stop":
                        finish = "tool_calls"
                last = {"id": req.id, "object": obj + ".chunk", "created": created, "model": model_name,
                        "choices": [{"index": 0, **({"delta": tail} if chat else {"text": ""}), "finish_reason": finish}], "usage": usage()}
                self.wfile.write(f"data: {json.dumps(last)}\n\ndata: [DONE]\n\n".encode())
                return
            choice = {"index": 0, "finish_reason": finish}
            if chat:
                choice["message"] = {"role": "assistant", "content": text}
                if tstream is not None:
                    content, calls = parse_tool_calls(text, tool_parser)
                    if calls:
                        choice["message"] = {"role": "assistant", "content": content or None, "tool_calls": calls}
                        if finish == "stop":
                            choice["finish_reason"] = "tool_calls"
            else:
                choice["text"] = text
            if with_ids:
                choice["token_ids"] = text_ids
                choice["prompt_token_ids"] = prompt
            self._json(200, {"id": req.id, "object": obj, "created": created, "model": model_name, "choices": [choice], "usage": usage()})

    return Handler


class Server:
    def __init__(self, sched: Scheduler, tokenizer=None, model_name: str = "kern", host: str = "127.0.0.1", port: int = 8000,
                 on_rotate=None, tool_parser: str = "auto", recorder=None):
        """`tool_parser`: `chat.select_parser`'s answer (auto | none | hermes | qwen3_coder): how a chat completion whose
        request carries `tools` has the model's tool-call syntax turned into `tool_calls`."""
        self.driver = Driver(sched)
        if recorder is not None and on_rotate is None:
            on_rotate = recorder.rotate
        self.httpd = ThreadingHTTPServer((host, port), make_handler(self.driver, tokenizer or ByteTokenizer(), model_name, on_rotate,
                                                                    tool_parser, recorder))
        self.httpd.daemon_threads = True
        self.port = self.httpd.server_address[1]
        self._thread = None

    def start(self) -> "Server":
        self.driver.start()
        self._thread = threading.Thread(target=self.httpd.serve_forever, daemon=True, name="kern-http")
        self._thread.start()
        return self

    def serve_forever(self) -> None:
        self.driver.start()
        try:
            self.httpd.serve_forever()
        finally:
            self.stop()

    def stop(self) -> None:
        self.driver.stop_flag.set()
        self.httpd.shutdown()
        self.httpd.server_close()
