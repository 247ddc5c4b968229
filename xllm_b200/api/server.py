"""OpenAI-compatible HTTP service on top of the engine.

Route parity with the reference's APIService / XllmServer (xllm/server/xllm_server.cpp:39-60,
xllm/api_service/*): `/v1/completions`, `/v1/chat/completions` (SSE streaming and plain),
`/v1/models`, `/v1/embeddings`, `/v1/messages` (Anthropic), `/health`, `/metrics` and the admin
endpoints `/sleep`, `/wakeup`, `/pause`, `/resume`, `/start_profile`, `/stop_profile`.
Tool-call and reasoning parsing of chat responses uses the C++ stream parsers; request ids,
`max_concurrent_requests` rate limiting and client-disconnect aborts follow
chat_service_impl.cpp:702-860 / continuous_scheduler.cpp:964-1018.

Transport is the C++ epoll server (`_rt.HttpServer`).  Three stages run concurrently, as in the
reference's master (request thread pool, llm_master.cpp:216-303) and response processor
(async_response_processor.cpp:86-376):
  * request pool (Python threads): JSON parsing, chat template, tokenisation (the C++ tokenizer
    releases the interpreter lock) -> a queue of admitted-to-be requests,
  * engine loop (this thread): drains that queue, steps the engine, hands ALL output events of a step
    to the response stage in one call,
  * response pool (C++ threads, `_rt.ResponseProcessor`): incremental detokenisation, stop strings,
    SSE / JSON formatting and the socket hand-off, without the interpreter.  Calls that need more
    than text (tool-call / reasoning parsers, logprobs, the Anthropic format) are formatted by the
    engine loop in Python instead.
"""
from __future__ import annotations

import json
import os
import queue
import time
import uuid
from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from .. import _rt
from ..engine.llm_engine import LLMEngine


@dataclass
class _Call:
    http_id: int
    request_id: str
    kind: str                      # "completion" | "chat" | "anthropic"
    stream: bool
    model: str
    created: int
    n: int = 1
    prompt_tokens: int = 0
    decoders: List[object] = field(default_factory=list)
    texts: List[str] = field(default_factory=list)
    token_ids: List[List[int]] = field(default_factory=list)
    finish: List[Optional[str]] = field(default_factory=list)
    logprobs: List[List[float]] = field(default_factory=list)
    reasoning: List[object] = field(default_factory=list)
    reasoning_text: List[str] = field(default_factory=list)
    tools: List[object] = field(default_factory=list)
    tool_calls: List[List[dict]] = field(default_factory=list)
    want_logprobs: bool = False
    include_usage: bool = False
    echo_text: str = ""
    t_arrival: float = 0.0
    t_first: float = 0.0
    started: bool = False
    native: int = 0                # handle in the C++ response processor (0: formatted in Python)


class ApiServer:
    def __init__(self, engine: LLMEngine, tokenizer, model_name: str = "xllm_b200", host: str = "", port: int = 8010,
                 max_concurrent_requests: int = 200, tool_call_parser: str = "", reasoning_parser: str = "",
                 request_threads: int = 4, response_threads: int = 4, parent: "ApiServer" = None, backend: str = "llm"):
        self.engine = engine
        self.backend = backend or "llm"   # "rec": /v1/completions answers with the beam_width best items
        self.rec_engine = None
        self.tok = tokenizer
        self.model_name = model_name
        # a forked master (another model served by the same process) shares its parent's transport
        self.parent = parent
        if parent is None:
            self.http = _rt.HttpServer()
            self.port = self.http.start(host, port)
        else:
            self.http, self.port = parent.http, parent.port
        self.forks: Dict[str, "ApiServer"] = {}
        self.pd_prefill = None      # engine/pd_service.PrefillService once linked as the prefill side
        self.pd_decode = None       # engine/pd_service.DecodeService once linked as the decode side
        self._pd_listen = None
        # request stage: a pool of threads that parse, template and tokenise; results queue up for the engine loop
        self.request_pool = ThreadPoolExecutor(max(1, request_threads), thread_name_prefix="xllm-req") \
            if request_threads > 0 else None
        self._ready: "queue.SimpleQueue" = queue.SimpleQueue()
        self._preparing = 0
        # response stage: native worker threads (needs the C++ tokenizer, or none at all)
        self.rp = None
        impl = getattr(tokenizer, "impl", None)
        if response_threads > 0 and (tokenizer is None or isinstance(impl, _rt.BpeTokenizer)):
            self.rp = _rt.ResponseProcessor(self.http, impl, response_threads)
        self._native_by_rid: Dict[str, int] = {}
        self.max_concurrent = max_concurrent_requests
        self.tool_kind = tool_call_parser
        self.reason_kind = reasoning_parser
        self.calls: Dict[str, _Call] = {}
        self.healthy = True
        self.unhealthy_reason = ""
        self.profiler = None
        self._stop = False
        from ..engine.fault import DeviceWatchdog
        self.watchdog = DeviceWatchdog.for_engine(engine, self._set_unhealthy)
        self._next_watch = 0.0
        self.watch_interval_s = 3.0
        from ..utils.tracing import TraceLog
        self.trace = TraceLog(os.environ.get("XLLM_TRACE_LOG", ""))
        from ..utils import metrics_catalog
        if parent is None:
            metrics_catalog.register_all()
        self.metrics = metrics_catalog.EnginePublisher(engine)

    def _set_unhealthy(self, reason: str):
        """/health answers 503 with the reason from now on; an orchestrator is expected to recycle the instance."""
        self.healthy = False
        self.unhealthy_reason = reason

    # ------------------------------------------------------------------ plumbing
    def _json(self, http_id, status, obj):
        self.http.respond(http_id, status, "application/json", json.dumps(obj, ensure_ascii=False))

    def _error(self, http_id, status, message, typ="invalid_request_error"):
        _rt.metric_counter_add("server_request_total_fail")
        _rt.metric_counter_add({400: "request_status_total_invalid_argument", 401: "request_status_total_unauthenticated",
                                404: "request_status_total_unimplemented", 405: "request_status_total_unimplemented",
                                429: "request_status_total_resource_exhausted", 503: "request_status_total_unavailable"}
                               .get(status, "request_status_total_unknown"))
        if status == 429:
            _rt.metric_counter_add("server_request_total_limit")
        self._json(http_id, status, {"error": {"message": message, "type": typ, "code": status}})

    def shutdown(self):
        self._stop = True

    def serve_forever(self, idle_poll_ms: int = 50):
        while not self._stop:
            self.run_once(idle_poll_ms)
        if self.rp is not None:
            self.rp.drain(2000)
            self.rp.stop()
        if self.request_pool is not None:
            self.request_pool.shutdown(wait=False)
        self.http.stop()

    GENERATION_PATHS = ("/v1/completions", "/v1/chat/completions", "/v1/messages")

    def _prepare(self, req):
        """Request stage (pool thread): everything up to the point where the engine is needed."""
        try:
            self._route(req, prepared=True)
        except Exception as e:  # a malformed request must never take a thread down
            self._error(req.id, 500, f"{type(e).__name__}: {e}", "internal_error")
        finally:
            self._ready.put(None)          # one marker per prepared request (this server counts them)

    def _busy(self) -> bool:
        return (self.engine.has_unfinished() or self._preparing > 0 or
                (self.pd_prefill is not None and self.pd_prefill.has_unfinished()) or
                any(f._busy() for f in self.forks.values()))

    def run_once(self, idle_poll_ms: int = 0):
        busy = self._busy()
        for req in self.http.poll(0 if busy else idle_poll_ms):
            try:
                path = req.path.rstrip("/") or "/"
                if self.request_pool is not None and req.method == "POST" and path in self.GENERATION_PATHS:
                    self._preparing += 1
                    self.request_pool.submit(self._prepare, req)
                else:
                    self._route(req)
            except Exception as e:  # a malformed request must never take the loop down
                self._error(req.id, 500, f"{type(e).__name__}: {e}", "internal_error")
        self._after_poll()
        for f in list(self.forks.values()):
            f._after_poll()

    def _after_poll(self):
        """Everything of an iteration that belongs to ONE served model: admit, abort, step, respond."""
        # requests the pool has finished preparing: the engine is only ever touched by this thread
        while True:
            try:
                item = self._ready.get_nowait()
            except queue.Empty:
                break
            if item is None:
                (self.parent or self)._preparing -= 1
                continue
            req, call, ids, sampling, stops = item
            try:
                self._admit(req, call, ids, sampling, stops)
            except Exception as e:
                self._error(req.id, 500, f"{type(e).__name__}: {e}", "internal_error")
        # client went away: abort its request (frees its KV blocks at once)
        self._iter = getattr(self, "_iter", 0) + 1
        if self.calls and self._iter % 8 == 0:           # every few iterations: one native call for all connections
            gone = set(self.http.disconnected_among([c.http_id for c in self.calls.values()]))
            if gone:
                for rid, call in list(self.calls.items()):
                    if call.http_id in gone:
                        (self.pd_prefill or self.engine).abort(rid)
                        self.calls.pop(rid, None)
                        if call.native:
                            self._native_by_rid.pop(rid, None)
                            self.rp.push([call.native], [0], [-1], [4], [""])
        now = time.time()
        if now >= self._next_watch:            # expired bounded waits in kernels -> unhealthy
            self._next_watch = now + self.watch_interval_s
            self.watchdog.check()
        if self._pd_listen is not None:
            self._pd_accept()
        if self.pd_prefill is not None:
            if self.pd_prefill.has_unfinished():
                self._dispatch(self.pd_prefill.step())
        elif self.pd_decode is not None:
            self._dispatch(self.pd_decode.step())
            if self.pd_decode.stopped and not self.engine.has_unfinished():
                self.pd_decode = None          # the peer said bye or went away: plain instance again
        elif self.engine.has_unfinished():
            self._dispatch(self.engine.step())
        self._collect_done()
        self.metrics.tick(len(self.calls))

    def _collect_done(self, wait_ms: int = 0):
        """Forget the calls the response pool has completed."""
        if self.rp is None:
            return
        if wait_ms:
            self.rp.drain(wait_ms)
        for d in self.rp.take_done():
            self.calls.pop(d.request_id, None)
            self._native_by_rid.pop(d.request_id, None)
            self.trace.event(d.request_id, "finished", generated=int(d.generated), ttft_ms=round(d.ttft_ms, 3),
                             e2e_ms=round(d.e2e_ms, 3))

    def _dispatch(self, events):
        """Output events of one step: those of natively formatted calls go to the response pool in
        one call, the others are formatted here."""
        if not self._native_by_rid:
            for ev in events:
                self._on_event(ev)
            return
        if not isinstance(events, list):
            events = list(events)
        h, si, tk, fl, rs = [], [], [], [], []
        for i in self.rp.push_events(events, self._native_by_rid):
            ev = events[i]
            handle = self._native_by_rid.get(ev.request_id)
            if handle is None:
                self._on_event(ev)
                continue
            # an event object of another kind (relayed from a decode instance, a re-labelled first token)
            aborted = ev.finish_reason == "abort" and ev.finished
            h.append(handle)
            si.append(int(ev.seq_index))
            tk.append(int(ev.token))
            fl.append((1 if ev.finished else 0) | (2 if ev.request_finished else 0) | (4 if aborted else 0))
            rs.append(ev.finish_reason if ev.finished else "")
        if h:
            self.rp.push(h, si, tk, fl, rs)

    # ------------------------------------------------------------------ routing
    def _route(self, req, prepared: bool = False):
        path, method = req.path.rstrip("/") or "/", req.method
        _rt.metric_counter_add("server_request_in_total")
        if path == "/health":
            if self.healthy:
                return self._json(req.id, 200, {"status": "ok"})
            return self._json(req.id, 503, {"status": "unhealthy", "reason": self.unhealthy_reason})
        if path == "/metrics":
            return self.http.respond(req.id, 200, "text/plain; version=0.0.4", _rt.metrics_text())
        if path in ("/v1/models", "/models"):
            return self._json(req.id, 200, {"object": "list", "data": [
                {"id": m.model_name, "object": "model", "created": int(time.time()), "owned_by": "xllm_b200"}
                for m in [self] + list(self.forks.values())]})
        if path == "/v2/repository/index":
            return self._json(req.id, 200, [
                {"name": m.model_name, "version": "1", "state": "SLEEPING" if m.engine.asleep else "READY"}
                for m in [self] + list(self.forks.values())])
        if method != "POST":
            return self._error(req.id, 405 if path.startswith("/v1") else 404, f"{method} {path} not supported")
        body = {}
        if req.body:
            try:
                body = json.loads(req.body)
            except json.JSONDecodeError as e:
                return self._error(req.id, 400, f"invalid JSON body: {e}")
        # another model served by this process (fork_master): same routes, its own engine
        target = self.forks.get(str(body.get("model") or body.get("model_id") or ""))
        if target is not None and path in self.GENERATION_PATHS + ("/v1/embeddings", "/v1/rerank", "/v1/sample",
                                                                   "/sleep", "/wakeup", "/pause", "/resume"):
            return target._route(req, prepared)
        if path == "/v1/completions":
            return self._completion(req, body)
        if path == "/v1/chat/completions":
            return self._chat(req, body, "chat")
        if path == "/v1/messages":
            return self._chat(req, body, "anthropic")
        if path == "/fork_master":
            return self._fork_master(req, body)
        if path == "/link_p2p":
            return self._link_p2p(req, body)
        if path == "/unlink_p2p":
            return self._unlink_p2p(req, body)
        if path == "/v1/embeddings":
            return self._embeddings(req, body)
        if path == "/v1/rerank":
            return self._rerank(req, body)
        if path == "/v1/sample":
            return self._sample(req, body)
        if path == "/v1/images/generations":
            return self._images(req, body)
        if path == "/pause":
            self.engine.pause(str(body.get("mode", "KEEP")).upper())
            return self._json(req.id, 200, {"status": "paused"})
        if path == "/resume":
            self.engine.resume()
            return self._json(req.id, 200, {"status": "running"})
        if path == "/sleep":      # releases the KV cache (level 1) and the weights too (level 2)
            level = int(body.get("level", body.get("master_status", 1)) or 1)
            self._collect_done(wait_ms=200)
            if self.calls:        # the reference's rule: a master only sleeps with no request in flight
                return self._error(req.id, 409, f"{len(self.calls)} requests in flight", "conflict")
            self.engine.sleep(level)
            return self._json(req.id, 200, {"status": "sleeping", "level": level})
        if path == "/wakeup":
            self.engine.wake_up()
            return self._json(req.id, 200, {"status": "running"})
        if path == "/start_profile":
            return self._profile(req, True, body)
        if path == "/stop_profile":
            return self._profile(req, False, body)
        return self._error(req.id, 404, f"unknown route {path}")

    # ------------------------------------------------------------------ more masters, instance links
    def _fork_master(self, req, body):
        """Serve another model from this process (the reference's `fork_master`,
        api_service.cpp:1046-1118): its own engine, scheduler and KV cache on the same device, the
        same transport; requests reach it through their `model` field.  `master_status` 1 / 2 starts
        it asleep (KV cache released / weights on the host as well) until `/wakeup`."""
        mid = str(body.get("model_id") or body.get("model") or "")
        if not mid:
            return self._error(req.id, 400, "`model_id` is required")
        if mid == self.model_name or mid in self.forks:
            return self._json(req.id, 200, {"ok": True, "message": f"master for model {mid} already exists"})
        import dataclasses
        from ..engine.llm_engine import EngineConfig, LLMEngine
        base = self.engine.cfg
        allowed = {f.name for f in dataclasses.fields(EngineConfig)}
        kw = {k: v for k, v in body.items() if k in allowed and k not in ("model", "device")}
        cfg = dataclasses.replace(base, model=str(body.get("model_path") or body.get("model") or mid), **kw)
        try:
            eng = LLMEngine(cfg)
        except Exception as e:
            return self._error(req.id, 400, f"failed to fork master {mid}: {type(e).__name__}: {e}")
        tok = None
        if os.path.isdir(cfg.model):
            try:
                from ..utils.tokenizer import load_tokenizer
                tok = load_tokenizer(cfg.model)
            except Exception:
                tok = None
        fork = ApiServer(eng, tok, model_name=mid, max_concurrent_requests=self.max_concurrent,
                         tool_call_parser=self.tool_kind, reasoning_parser=self.reason_kind,
                         request_threads=0, response_threads=self.rp.num_threads if self.rp else 0, parent=self)
        fork.request_pool = self.request_pool
        self.forks[mid] = fork
        status = int(body.get("master_status", 0) or 0)
        if status in (1, 2):
            eng.sleep(status)
        return self._json(req.id, 200, {"ok": True, "model_id": mid, "state": "SLEEPING" if eng.asleep else "READY"})

    def _link_p2p(self, req, body):
        """Pair this instance with another one for prefill/decode disaggregation (the reference's
        `link_p2p`): role "decode" listens on `port` and adopts what the peer prefills; role "prefill"
        connects to a decode instance at `host:port` and from then on hands every request over after
        its first token.  KV travels on the same connection (`SocketCopy`) unless a peer-memory link
        was installed through `attach_pd`."""
        from ..engine.pd_service import Channel, PrefillService, SocketCopy
        role = str(body.get("role", "prefill"))
        host, port = str(body.get("host", "127.0.0.1")), int(body.get("port", 0))
        if self.pd_prefill is not None or self.pd_decode is not None or self._pd_listen is not None:
            return self._error(req.id, 409, "already linked", "conflict")
        if role == "decode":
            srv = Channel.listen(host, port)
            srv.setblocking(False)
            self._pd_listen = srv
            return self._json(req.id, 200, {"ok": True, "role": "decode", "port": srv.getsockname()[1]})
        self._collect_done(wait_ms=200)
        if self.calls:
            return self._error(req.id, 409, "requests in flight", "conflict")
        try:
            ch = Channel.connect(host, port, timeout=float(body.get("timeout", 10.0)))
            self.engine.scheduler.set_hold_finished_blocks(True)
            self.pd_prefill = PrefillService(self.engine, ch, SocketCopy(self.engine.runner),
                                             hello_timeout=float(body.get("timeout", 10.0)))
        except Exception as e:
            self.engine.scheduler.set_hold_finished_blocks(False)
            self.pd_prefill = None
            return self._error(req.id, 502, f"cannot link to {host}:{port}: {type(e).__name__}: {e}", "bad_gateway")
        return self._json(req.id, 200, {"ok": True, "role": "prefill", "peer": f"{host}:{port}"})

    def _pd_accept(self):
        from ..engine.pd_service import Channel, DecodeService, SocketCopy
        try:
            conn, _ = self._pd_listen.accept()
        except (BlockingIOError, OSError):
            return
        self._pd_listen.close()
        self._pd_listen = None
        # XLLM_PD_PULL_OFFLINE=1: while idle, this decode instance asks the prefill instance for the offline
        # requests it is decoding itself
        self.pd_decode = DecodeService(self.engine, Channel(conn), SocketCopy(self.engine.runner),
                                       pull_offline=os.environ.get("XLLM_PD_PULL_OFFLINE", "0") == "1")

    def _unlink_p2p(self, req, body):
        if self.pd_prefill is not None:
            if self.pd_prefill.has_unfinished():
                return self._error(req.id, 409, "requests in flight", "conflict")
            self.pd_prefill.close()
            self.pd_prefill.ch.close()
            self.engine.runner.meta_hook = None
            self.engine.scheduler.set_hold_finished_blocks(False)
            self.pd_prefill = None
        if self._pd_listen is not None:
            self._pd_listen.close()
            self._pd_listen = None
        if self.pd_decode is not None:
            self.pd_decode.ch.close()       # the service reclaims on its next step
        return self._json(req.id, 200, {"ok": True})

    def _profile(self, req, start, body):
        from ..utils.tracing import Profiler
        if start:
            if self.profiler is None:
                backend = str(body.get("profile_backend") or os.environ.get("XLLM_PROFILE_BACKEND", "torch"))
                try:
                    self.profiler = Profiler(backend, self.engine.ps.rank)
                except ValueError as e:
                    return self._error(req.id, 400, str(e))
                self.profiler.start()
            return self._json(req.id, 200, {"status": "profiling", "backend": self.profiler.backend})
        path = ""
        if self.profiler is not None:
            path = self.profiler.stop(str(body.get("profile_dir", ".")))
            self.profiler = None
        return self._json(req.id, 200, {"status": "stopped", "trace": path})

    # ------------------------------------------------------------------ request intake
    def _sampling(self, body, max_default=5120):
        mt = body.get("max_completion_tokens") or body.get("max_tokens") or max_default
        stop = body.get("stop")
        if isinstance(stop, str):
            stop = [stop]
        lp = body.get("logprobs")
        return dict(temperature=float(body.get("temperature", 1.0)), top_p=float(body.get("top_p", 1.0)),
                    top_k=int(body.get("top_k", -1)), max_tokens=int(mt),
                    frequency_penalty=float(body.get("frequency_penalty", 0.0)),
                    presence_penalty=float(body.get("presence_penalty", 0.0)),
                    repetition_penalty=float(body.get("repetition_penalty", 1.0)),
                    ignore_eos=bool(body.get("ignore_eos", False)), seed=body.get("seed"),
                    logprobs=bool(lp) if not isinstance(lp, int) else lp > 0,
                    stop_token_ids=body.get("stop_token_ids")), (stop or [])

    def _submit(self, req, call: _Call, prompt_ids, sampling, stops):
        """End of the request stage: straight into the engine when called by the engine loop, through
        the ready queue when called by a pool thread."""
        import threading
        if self.request_pool is not None and threading.current_thread().name.startswith("xllm-req"):
            self._ready.put((req, call, prompt_ids, sampling, stops))
        else:
            self._admit(req, call, prompt_ids, sampling, stops)

    def _admit(self, req, call: _Call, prompt_ids, sampling, stops):
        if self.max_concurrent and len(self.calls) >= self.max_concurrent:
            return self._error(req.id, 429, "too many concurrent requests", "rate_limit_error")
        if self.engine.scheduler.paused():
            return self._error(req.id, 503, "the instance is paused", "unavailable")
        n = call.n
        if "mm_raw" in sampling:
            images, videos = sampling.pop("mm_raw")
            try:
                prompt_ids, sampling["mm"] = self._vlm_prepare(prompt_ids, images, videos)
            except ValueError as e:
                return self._error(req.id, 400, str(e))
        call.prompt_tokens = len(prompt_ids)
        call.t_arrival = time.time()
        call.want_logprobs = sampling["logprobs"]
        native = (self.rp is not None and call.kind in ("completion", "chat") and not call.want_logprobs
                  and not (call.kind == "chat" and (self.reason_kind or self.tool_kind)))
        for _ in range(n):
            call.decoders.append(self.tok.incremental_decoder(stops, True) if self.tok and not native else None)
            call.texts.append("")
            call.token_ids.append([])
            call.finish.append(None)
            call.logprobs.append([])
            call.reasoning.append(_rt.ReasoningParser(self.reason_kind) if self.reason_kind and call.kind != "completion" else None)
            call.reasoning_text.append("")
            call.tools.append(_rt.ToolCallParser(self.tool_kind) if self.tool_kind and call.kind != "completion" else None)
            call.tool_calls.append([])
        if self.pd_prefill is not None and n == 1:
            ok = self.pd_prefill.add_request(call.request_id, prompt_ids, **{k: v for k, v in sampling.items()
                                                                            if k not in ("logprobs",)})
        else:
            ok = self.engine.add_request(call.request_id, prompt_ids, n=n, stream=call.stream, **sampling)
        if not ok:
            return self._error(req.id, 400, "prompt is empty or longer than the model's context window")
        self.calls[call.request_id] = call
        if native:
            spec = _rt.RespCallSpec()
            spec.http_id, spec.request_id, spec.model = call.http_id, call.request_id, call.model
            spec.kind = 0 if call.kind == "completion" else 1
            spec.stream, spec.include_usage, spec.n = call.stream, call.include_usage, n
            spec.prompt_tokens, spec.created, spec.echo_text = call.prompt_tokens, call.created, call.echo_text
            spec.stops = list(stops)
            spec.t_arrival = time.monotonic()
            call.native = self.rp.open(spec)
            self._native_by_rid[call.request_id] = call.native
        _rt.metric_counter_add("server_request_total_ok", 0)

    def _rec_completion(self, req, body):
        """Generative recommendation (`--backend rec`; xllm/api_service/rec_completion_service_impl.cpp): the
        prompt is the user's history, every choice is one item of `max_tokens` tokens, best first."""
        from ..engine.rec import ItemTrie, RecEngine
        prompt = body.get("prompt", "")
        if isinstance(prompt, list) and prompt and isinstance(prompt[0], int):
            ids = [int(t) for t in prompt]
        elif self.tok is None:
            return self._error(req.id, 400, "this server has no tokenizer: send token ids as `prompt`")
        else:
            ids = self.tok.encode(prompt if isinstance(prompt, str) else (prompt[0] if prompt else ""))
        if not ids:
            return self._error(req.id, 400, "`prompt` must not be empty")
        try:
            if self.rec_engine is None:
                self.rec_engine = RecEngine(self.engine)
            steps = int(body.get("max_tokens") or 3)
            width = int(body.get("beam_width") or 32)
            trie = None
            if body.get("valid_items"):
                trie = ItemTrie([tuple(int(t) for t in it) for it in body["valid_items"]], self.engine.args.vocab_size)
            embeds = None
            if body.get("input_embeds"):
                e = body["input_embeds"]
                embeds = [(torch.tensor(e["rows"], dtype=torch.long), torch.tensor(e["values"], dtype=torch.float32))]
            items = self.rec_engine.generate([ids], beam_width=width, num_steps=steps, num_return=int(body.get("n") or width),
                                             trie=trie, prompt_embeds=embeds)[0]
        except (ValueError, KeyError, TypeError) as e:
            return self._error(req.id, 400, str(e))
        except RuntimeError as e:
            return self._error(req.id, 503, str(e))
        choices = [{"index": i, "text": self.tok.decode(it.token_ids) if self.tok is not None else "",
                    "token_ids": it.token_ids, "logprobs": {"cumulative_logprob": it.logprob}, "finish_reason": "length"}
                   for i, it in enumerate(items)]
        n_out = sum(len(it.token_ids) for it in items)
        self._json(req.id, 200, {"id": req.header("x-request-id") or f"rec-{uuid.uuid4().hex}", "object": "text_completion",
                                 "created": int(time.time()), "model": body.get("model") or self.model_name,
                                 "choices": choices,
                                 "usage": {"prompt_tokens": len(ids), "completion_tokens": n_out,
                                           "total_tokens": len(ids) + n_out}})

    def _completion(self, req, body):
        if self.backend == "rec":
            return self._rec_completion(req, body)
        prompt = body.get("prompt", "")
        if isinstance(prompt, list) and prompt and isinstance(prompt[0], int):
            ids = list(prompt)
            text = ""
        else:
            if isinstance(prompt, list):
                prompt = prompt[0] if prompt else ""
            if self.tok is None:
                return self._error(req.id, 400, "this server has no tokenizer: send token ids as `prompt`")
            t0 = time.perf_counter()
            ids, text = self.tok.encode(prompt), prompt
            _rt.metric_counter_add("tokenization_latency_seconds", time.perf_counter() - t0)
        sampling, stops = self._sampling(body, 16)
        rid = req.header("x-request-id") or f"cmpl-{uuid.uuid4().hex}"
        call = _Call(req.id, rid, "completion", bool(body.get("stream")), body.get("model") or self.model_name,
                     int(time.time()), n=int(body.get("n", 1)), echo_text=text if body.get("echo") else "",
                     include_usage=bool((body.get("stream_options") or {}).get("include_usage")))
        self._submit(req, call, ids, sampling, stops)

    def _chat(self, req, body, kind):
        if self.tok is None:
            return self._error(req.id, 400, "chat needs a tokenizer with a chat template")
        messages = list(body.get("messages") or [])
        if kind == "anthropic" and body.get("system"):
            sys_text = body["system"] if isinstance(body["system"], str) else "".join(p.get("text", "") for p in body["system"])
            messages = [{"role": "system", "content": sys_text}] + messages
        if not messages:
            return self._error(req.id, 400, "`messages` must not be empty")
        try:
            messages, images, videos = self._media_from_messages(messages)
        except ValueError as e:
            return self._error(req.id, 400, str(e))
        kwargs = dict(body.get("chat_template_kwargs") or {})
        t0 = time.perf_counter()
        prompt = self.tok.apply_chat_template(messages, tools=body.get("tools"), add_generation_prompt=True,
                                              enable_thinking=bool(kwargs.get("enable_thinking", True)))
        t1 = time.perf_counter()
        ids = self.tok.encode(prompt)
        _rt.metric_counter_add("chat_template_latency_seconds", t1 - t0)
        _rt.metric_counter_add("tokenization_latency_seconds", time.perf_counter() - t1)
        sampling, stops = self._sampling(body)
        if images or videos:
            sampling["mm_raw"] = (images, videos)          # the vision tower runs on the engine thread (_admit)
        rid = req.header("x-request-id") or (f"msg_{uuid.uuid4().hex}" if kind == "anthropic" else f"chatcmpl-{uuid.uuid4().hex}")
        call = _Call(req.id, rid, kind, bool(body.get("stream")), body.get("model") or self.model_name,
                     int(time.time()), n=int(body.get("n", 1)),
                     include_usage=bool((body.get("stream_options") or {}).get("include_usage")))
        self._submit(req, call, ids, sampling, stops)

    # ---- multimodal chat content (xllm/api_service/mm_service_utils.cpp: image_url / video_url parts)
    IMAGE_MARK = "<|vision_start|><|image_pad|><|vision_end|>"
    VIDEO_MARK = "<|vision_start|><|video_pad|><|vision_end|>"

    @staticmethod
    def _load_media(url: str, kind: str):
        import base64
        import io
        if url.startswith("data:"):
            head, _, payload = url.partition(",")
            if ";base64" not in head:
                raise ValueError("data: URLs must be base64-encoded")
            raw = base64.b64decode(payload)
        elif url.startswith("file://") or os.path.exists(url):
            with open(url[7:] if url.startswith("file://") else url, "rb") as f:
                raw = f.read()
        else:
            raise ValueError(f"cannot fetch {kind} from {url[:40]!r}: only data: URLs and local files are served here")
        if kind == "image":
            from PIL import Image
            try:
                return Image.open(io.BytesIO(raw)).convert("RGB")
            except Exception as e:
                raise ValueError(f"undecodable image: {e}")
        from ..multimodal.media import decode_video
        return decode_video(raw)[0]

    def _media_from_messages(self, messages):
        """Content lists with image_url / video_url parts become text with the model's placeholder marks;
        returns (messages with string contents, images, videos)."""
        images, videos, out = [], [], []
        for m in messages:
            c = m.get("content")
            if not isinstance(c, list):
                out.append(m)
                continue
            text = []
            for part in c:
                t = part.get("type")
                if t in ("text", "input_text"):
                    text.append(part.get("text", ""))
                elif t in ("image_url", "image"):
                    src = part.get("image_url") or part.get("image") or {}
                    images.append(self._load_media(src.get("url") if isinstance(src, dict) else src, "image"))
                    text.append(self.IMAGE_MARK)
                elif t in ("video_url", "video"):
                    src = part.get("video_url") or part.get("video") or {}
                    videos.append(self._load_media(src.get("url") if isinstance(src, dict) else src, "video"))
                    text.append(self.VIDEO_MARK)
                else:
                    raise ValueError(f"unsupported content part type {t!r}")
            out.append(dict(m, content="".join(text)))
        if (images or videos) and not hasattr(self.engine.model, "visual"):
            raise ValueError("this model takes text only")
        return out, images, videos

    def _vlm_prepare(self, ids, images, videos):
        if getattr(self, "_vlm", None) is None:
            from ..multimodal.image import Qwen2VLImageProcessor
            from .vlm import VLM
            v = VLM.__new__(VLM)
            v.engine, v.tokenizer = self.engine, self.tok
            vis = self.engine.model.visual
            v.processor = Qwen2VLImageProcessor(vis.patch, vis.merge, vis.tp)
            v.image_token_id = self.engine.args.image_token_id
            self._vlm = v
        return self._vlm.prepare(ids, images, videos)

    def _embeddings(self, req, body):
        inp = body.get("input", "")
        items = inp if isinstance(inp, list) and not (inp and isinstance(inp[0], int)) else [inp]
        from .embedding import embed_token_lists
        ids = [self.tok.encode(x) if isinstance(x, str) else list(x) for x in items]
        vecs = embed_token_lists(self.engine, ids)
        data = [{"object": "embedding", "index": i, "embedding": v} for i, v in enumerate(vecs)]
        n_tok = sum(len(x) for x in ids)
        self._json(req.id, 200, {"object": "list", "data": data, "model": self.model_name,
                                 "usage": {"prompt_tokens": n_tok, "total_tokens": n_tok}})

    def _images(self, req, body):
        """Text-to-image through the diffusion pipeline (`dit/pipeline.py`), created on first use."""
        if getattr(self, "image_pipeline", None) is None:
            from ..dit.pipeline import ImagePipeline
            self.image_pipeline = ImagePipeline()
        try:
            out = self.image_pipeline.openai_response(body)
        except ValueError as e:
            return self._error(req.id, 400, str(e))
        self._json(req.id, 200, out)

    def _rerank(self, req, body):
        from .embedding import rerank_scores
        docs = [d if isinstance(d, str) else d.get("text", "") for d in body.get("documents", [])]
        if not docs or "query" not in body:
            return self._error(req.id, 400, "rerank needs `query` and `documents`")
        trunc = int(body.get("truncate_prompt_tokens") or 0)
        enc = lambda t: self.tok.encode(t)[-trunc:] if trunc > 0 else self.tok.encode(t)
        q, ds = enc(body["query"]), [enc(d) for d in docs]
        scores = rerank_scores(self.engine, q, ds)
        order = sorted(range(len(docs)), key=lambda i: -scores[i])
        top_n = int(body.get("top_n") or len(docs))
        results = [{"index": i, "relevance_score": scores[i], "document": {"text": docs[i]}} for i in order[:top_n]]
        n_tok = len(q) + sum(len(d) for d in ds)
        self._json(req.id, 200, {"id": "rerank-" + str(req.id), "model": self.model_name, "results": results,
                                 "usage": {"prompt_tokens": n_tok, "total_tokens": n_tok}})

    def _sample(self, req, body):
        """Next-token distributions at every place of the prompt where the selector's literal ends."""
        from .embedding import next_token_logprobs
        prompt = body.get("prompt", "")
        sel = body.get("selector") or {}
        if sel.get("type", "literal") != "literal" or not sel.get("value"):
            return self._error(req.id, 400, "selector must be {\"type\": \"literal\", \"value\": ...}")
        n_lp = max(1, min(5, int(body.get("logprobs") or 1)))
        ids = self.tok.encode(prompt)
        ends, start = [], 0
        while True:
            k = prompt.find(sel["value"], start)
            if k < 0:
                break
            ends.append(k + len(sel["value"]))
            start = k + 1
        positions = [max(len(self.tok.encode(prompt[:e])), 1) - 1 for e in ends]
        tops = next_token_logprobs(self.engine, ids, positions, n_lp) if positions else []
        choices = []
        for i, (pos, top) in enumerate(zip(positions, tops)):
            choices.append({"index": i, "text": self.tok.decode([top[0][0]]), "token_position": pos,
                            "logprobs": {"tokens": [self.tok.decode([t]) for t, _ in top], "token_ids": [t for t, _ in top],
                                         "token_logprobs": [v for _, v in top]}})
        self._json(req.id, 200, {"id": body.get("request_id") or "sample-" + str(req.id), "object": "sample_completion",
                                 "created": int(time.time()), "model": self.model_name, "choices": choices,
                                 "usage": {"prompt_tokens": len(ids), "total_tokens": len(ids)}})

    # ------------------------------------------------------------------ output events
    def _sse(self, call, obj):
        self.http.stream_send(call.http_id, "data: " + json.dumps(obj, ensure_ascii=False) + "\n\n")

    def _chunk(self, call, i, delta=None, text=None, finish=None):
        if call.kind == "completion":
            return {"id": call.request_id, "object": "text_completion", "created": call.created, "model": call.model,
                    "choices": [{"index": i, "text": text or "", "finish_reason": finish}]}
        return {"id": call.request_id, "object": "chat.completion.chunk", "created": call.created, "model": call.model,
                "choices": [{"index": i, "delta": delta or {}, "finish_reason": finish}]}

    def _emit_text(self, call, i, piece):
        """Route a piece of decoded text through the reasoning / tool-call parsers; stream it."""
        if not piece:
            return
        reasoning_piece, content_piece = "", piece
        if call.reasoning[i] is not None:
            reasoning_piece, content_piece = call.reasoning[i].push(piece)
        new_calls = []
        if call.tools[i] is not None and content_piece:
            content_piece, new_calls = call.tools[i].push(content_piece)
        call.reasoning_text[i] += reasoning_piece
        call.texts[i] += content_piece
        for idx, name, args in new_calls:
            while len(call.tool_calls[i]) <= idx:
                call.tool_calls[i].append({"id": f"call_{uuid.uuid4().hex[:24]}", "type": "function",
                                           "function": {"name": "", "arguments": ""}})
            tc = call.tool_calls[i][idx]
            if name:
                tc["function"]["name"] = name
            tc["function"]["arguments"] += args
        if not call.stream:
            return
        if call.kind == "completion":
            if content_piece:
                self._sse(call, self._chunk(call, i, text=content_piece))
        elif call.kind == "chat":
            if reasoning_piece:
                self._sse(call, self._chunk(call, i, delta={"reasoning_content": reasoning_piece}))
            if content_piece:
                self._sse(call, self._chunk(call, i, delta={"content": content_piece}))
            for idx, name, args in new_calls:
                d = {"index": idx, "function": {"arguments": args}}
                if name:
                    d.update(id=call.tool_calls[i][idx]["id"], type="function")
                    d["function"]["name"] = name
                self._sse(call, self._chunk(call, i, delta={"tool_calls": [d]}))
        else:  # anthropic
            if content_piece:
                self.http.stream_send(call.http_id, "event: content_block_delta\ndata: " + json.dumps(
                    {"type": "content_block_delta", "index": 0, "delta": {"type": "text_delta", "text": content_piece}}) + "\n\n")

    def _start_stream(self, call):
        call.started = True
        self.http.stream_begin(call.http_id, 200, "text/event-stream")
        if call.kind == "chat":
            for i in range(call.n):
                self._sse(call, self._chunk(call, i, delta={"role": "assistant", "content": ""}))
        elif call.kind == "anthropic":
            self.http.stream_send(call.http_id, "event: message_start\ndata: " + json.dumps(
                {"type": "message_start", "message": {"id": call.request_id, "type": "message", "role": "assistant",
                                                      "model": call.model, "content": [],
                                                      "usage": {"input_tokens": call.prompt_tokens, "output_tokens": 0}}}) + "\n\n")
            self.http.stream_send(call.http_id, "event: content_block_start\ndata: " + json.dumps(
                {"type": "content_block_start", "index": 0, "content_block": {"type": "text", "text": ""}}) + "\n\n")
        elif call.echo_text:
            self._sse(call, self._chunk(call, 0, text=call.echo_text))

    def _on_event(self, ev):
        call = self.calls.get(ev.request_id)
        if call is None:
            return
        i = ev.seq_index
        now = time.time()
        if call.stream and not call.started:
            self._start_stream(call)
        if ev.token >= 0:
            if call.t_first == 0.0:
                call.t_first = now
                _rt.metric_histogram_observe("time_to_first_token_latency_milliseconds", (now - call.t_arrival) * 1e3)
                self.trace.event(ev.request_id, "first_token", ttft_ms=round((now - call.t_arrival) * 1e3, 3))
            call.token_ids[i].append(ev.token)
            if ev.has_logprob:
                call.logprobs[i].append(ev.logprob)
            dec = call.decoders[i]
            if dec is not None and call.finish[i] is None:
                piece, stopped = dec.push(ev.token)
                self._emit_text(call, i, piece)
                if stopped:
                    call.finish[i] = "stop"
        if ev.finished and ev.finish_reason != "abort":
            if call.decoders[i] is not None and call.finish[i] is None:
                self._emit_text(call, i, call.decoders[i].flush())
            for parser, is_reason in ((call.reasoning[i], True), (call.tools[i], False)):
                if parser is not None and is_reason:
                    r, c = parser.flush()
                    call.reasoning_text[i] += r
                    if c:
                        if call.tools[i] is not None:
                            c, _ = call.tools[i].push(c)
                        call.texts[i] += c
                        if call.stream and call.kind == "chat" and c:
                            self._sse(call, self._chunk(call, i, delta={"content": c}))
            if call.finish[i] is None:
                call.finish[i] = ev.finish_reason or "stop"
            if call.tool_calls[i] and call.finish[i] == "stop":
                call.finish[i] = "tool_calls"
            if call.stream and call.kind != "anthropic":
                self._sse(call, self._chunk(call, i, delta={}, text="", finish=call.finish[i]))
        if ev.request_finished:
            self._finish_call(call, aborted=ev.finish_reason == "abort")

    def _usage(self, call):
        gen = sum(len(t) for t in call.token_ids)
        return {"prompt_tokens": call.prompt_tokens, "completion_tokens": gen, "total_tokens": call.prompt_tokens + gen}

    def _finish_call(self, call, aborted=False):
        self.calls.pop(call.request_id, None)
        now = time.time()
        gen = sum(len(t) for t in call.token_ids)
        _rt.metric_counter_add("server_request_total_ok" if not aborted else "server_request_total_fail")
        _rt.metric_counter_add("num_generated_tokens_total", gen)
        _rt.metric_counter_add("num_prompt_tokens_total", call.prompt_tokens)
        _rt.metric_histogram_observe("end_2_end_latency_milliseconds", (now - call.t_arrival) * 1e3)
        if gen > 1 and call.t_first:
            _rt.metric_histogram_observe("inter_token_latency_milliseconds", (now - call.t_first) * 1e3 / (gen - 1))
        usage = self._usage(call)
        if call.stream:
            if not call.started:
                self._start_stream(call)
            if call.kind == "anthropic":
                s = self.http.stream_send
                s(call.http_id, "event: content_block_stop\ndata: " + json.dumps({"type": "content_block_stop", "index": 0}) + "\n\n")
                s(call.http_id, "event: message_delta\ndata: " + json.dumps(
                    {"type": "message_delta", "delta": {"stop_reason": _anthropic_reason(call.finish[0])},
                     "usage": {"output_tokens": usage["completion_tokens"]}}) + "\n\n")
                s(call.http_id, "event: message_stop\ndata: " + json.dumps({"type": "message_stop"}) + "\n\n")
            else:
                if call.include_usage:
                    obj = self._chunk(call, 0)
                    obj["choices"] = []
                    obj["usage"] = usage
                    self._sse(call, obj)
                self.http.stream_send(call.http_id, "data: [DONE]\n\n")
            self.http.stream_end(call.http_id)
            return
        if call.kind == "completion":
            choices = []
            for i in range(call.n):
                c = {"index": i, "text": call.echo_text + call.texts[i], "finish_reason": call.finish[i] or "stop"}
                if call.want_logprobs:
                    c["logprobs"] = {"token_logprobs": call.logprobs[i], "tokens": call.token_ids[i]}
                if self.tok is None:
                    c["token_ids"] = call.token_ids[i]
                choices.append(c)
            return self._json(call.http_id, 200, {"id": call.request_id, "object": "text_completion",
                                                  "created": call.created, "model": call.model, "choices": choices,
                                                  "usage": usage})
        if call.kind == "anthropic":
            return self._json(call.http_id, 200, {
                "id": call.request_id, "type": "message", "role": "assistant", "model": call.model,
                "content": [{"type": "text", "text": call.texts[0]}], "stop_reason": _anthropic_reason(call.finish[0]),
                "usage": {"input_tokens": call.prompt_tokens, "output_tokens": usage["completion_tokens"]}})
        choices = []
        for i in range(call.n):
            msg = {"role": "assistant", "content": call.texts[i]}
            if call.reasoning_text[i]:
                msg["reasoning_content"] = call.reasoning_text[i]
            if call.tool_calls[i]:
                msg["tool_calls"] = call.tool_calls[i]
            c = {"index": i, "message": msg, "finish_reason": call.finish[i] or "stop"}
            if call.want_logprobs:
                c["logprobs"] = {"content": [{"token": self.tok.decode([t], False), "logprob": lp}
                                             for t, lp in zip(call.token_ids[i], call.logprobs[i])]}
            choices.append(c)
        self._json(call.http_id, 200, {"id": call.request_id, "object": "chat.completion", "created": call.created,
                                       "model": call.model, "choices": choices, "usage": usage})


def _anthropic_reason(finish):
    return {"length": "max_tokens", "tool_calls": "tool_use"}.get(finish or "stop", "end_turn")
