"""Prefill/decode disaggregation between PROCESSES: a prefill instance and a decode instance, each
with its own engine, scheduler and KV cache, talk over a socket (control plane) while the prompt's
KV is pushed layer by layer into the decode instance's cache (data plane).

Parity: `DisaggPDScheduler` + the `DisaggPDService` RPCs (xllm/core/scheduler/disagg_pd_scheduler.cpp:326-817,
xllm/proto/disagg_pd.proto:281-287) and the layer-wise push of the worker
(xllm/core/runtime/llm_worker_impl.cpp:280-305).  The protocol, prefill side -> decode side unless
marked:

  hello      {block_size, n_layers, n_kv_heads, head_dim, dtype, tp}       topology check, once
  <- hello_ack {ok, reason, num_blocks}
  reserve    {rid, n_tokens}                      blocks for the prompt + first decode steps
  <- reserved {rid, blocks}                       empty list: the decode side is full, ask again later
  kv         {layer, blocks, k, v}                socket data plane only (no peer-addressable memory)
  first      {rid, tokens, num_prompt, sampling, epoch}   prompt + first generated token
  <- adopted {rid, ok, reason}                    ok: the sequence now decodes over there
  <- gen     {rid, token, logprob, finished, reason}      generated tokens, streamed back
  cancel     {rid}                                request aborted / finished after one token
  bye        {}

Data plane: with `PeerPush` the decode instance's cache lives in peer-mapped memory
(`PDLink`, a symmetric allocation of both processes); the prefill forward calls
`KVPusher.push_layer` for every layer right after the layer wrote its KV rows (the hook
`AttentionMetadata.kv_hook`), the last CTA of a push publishes a per-layer flag in the decode
instance's memory, and the decode instance checks all layer flags with ONE bounded device-side wait
(`xllm_kv_wait_many`) before it adopts the sequence.  With `SocketCopy` (CPU instances, or GPUs that
cannot address each other) the blocks travel as `kv` messages on the control connection.

Failure handling uses host-visible events only: a connection that closes between steps makes the
decode side give back every reservation and abort the sequences of that peer, and makes the
prefill side fail the requests it had not handed over; a flag wait that runs out makes `adopted`
come back with ok=False and the request fail.
"""
from __future__ import annotations

import select
import socket
import struct
import time
from typing import Callable, Dict, List, Optional

import msgpack
import numpy as np
import torch

from .disagg import _FirstToken


# ------------------------------------------------------------------------------------------ framing
class Channel:
    """Length-prefixed frames over a connected TCP socket; `poll` never blocks.  A frame body is a
    protobuf message behind a type byte (`xllm_b200.proto.encode`; codec "protobuf", the default) or a
    msgpack map (codec "msgpack"); both ends must use the same codec."""

    def __init__(self, sock: socket.socket, codec: str = "protobuf"):
        self.sock = sock
        self.codec = codec
        sock.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
        sock.setblocking(True)
        self._rx = bytearray()
        self.closed = False
        self.sent = 0
        self.received = 0

    @staticmethod
    def listen(host="127.0.0.1", port=0):
        srv = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
        srv.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        srv.bind((host, port))
        srv.listen(8)
        return srv

    @staticmethod
    def accept(srv, timeout=60.0) -> "Channel":
        srv.settimeout(timeout)
        conn, _ = srv.accept()
        return Channel(conn)

    @staticmethod
    def connect(host, port, timeout=60.0) -> "Channel":
        deadline = time.time() + timeout
        while True:
            try:
                return Channel(socket.create_connection((host, port), timeout=5.0))
            except OSError:
                if time.time() > deadline:
                    raise
                time.sleep(0.05)

    def send(self, msg: dict) -> bool:
        if self.closed:
            return False
        if self.codec == "protobuf":
            from .. import proto
            body = proto.encode(msg)
        else:
            body = msgpack.packb(msg, use_bin_type=True)
        try:
            self.sock.sendall(struct.pack("<I", len(body)) + body)
            self.sent += 1
            return True
        except OSError:
            self.closed = True
            return False

    def poll(self, timeout: float = 0.0) -> List[dict]:
        out: List[dict] = []
        while not self.closed:
            try:
                r, _, _ = select.select([self.sock], [], [], timeout)
            except (OSError, ValueError):
                self.closed = True
                break
            if not r:
                break
            try:
                chunk = self.sock.recv(1 << 20)
            except OSError:
                chunk = b""
            if not chunk:
                self.closed = True
                break
            self._rx += chunk
            timeout = 0.0
            while len(self._rx) >= 4:
                (n,) = struct.unpack_from("<I", self._rx, 0)
                if len(self._rx) < 4 + n:
                    break
                frame = bytes(self._rx[4:4 + n])
                if self.codec == "protobuf":
                    from .. import proto
                    out.append(proto.decode(frame))
                else:
                    out.append(msgpack.unpackb(frame, raw=False))
                del self._rx[:4 + n]
                self.received += 1
        return out

    def close(self):
        self.closed = True
        try:
            self.sock.close()
        except OSError:
            pass


# ------------------------------------------------------------------------------------------ data plane
class PDLink:
    """Peer-mapped memory shared by the processes of a prefill/decode pair: every process allocates
    one symmetric buffer (KV cache + per-layer arrival flags) and learns the others' base pointers.
    The engine's KV cache is carved from it through `ModelRunner(kv_allocator=...)`."""

    FLAG_BYTES = 4096

    def __init__(self, group, device, kv_bytes: int):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem

        t = torch.tensor([int(kv_bytes)], dtype=torch.int64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)        # one size for every process
        self.kv_bytes = (int(t.item()) + 255) & ~255
        self.buf = symm_mem.empty(self.kv_bytes + self.FLAG_BYTES, dtype=torch.uint8, device=device)
        self.hdl = symm_mem.rendezvous(self.buf, group)
        self.buf.zero_()
        self.flags = self.buf[self.kv_bytes:self.kv_bytes + self.FLAG_BYTES].view(torch.int32)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self.hdl.barrier()

    def allocator(self) -> Callable[[int], torch.Tensor]:
        def alloc(n_bytes: int) -> torch.Tensor:
            assert n_bytes <= self.kv_bytes, (n_bytes, self.kv_bytes)
            return self.buf[:n_bytes]
        return alloc

    def peer_base(self, rank_in_group: int) -> int:
        return int(self.hdl.buffer_ptrs[rank_in_group])


class PeerPush:
    """GPU data plane.  Prefill side: `push_layer` (peer stores + flag); decode side: `wait`."""

    name = "peer_push"

    def __init__(self, link: PDLink, runner, peer_rank: int, wait_budget_cycles: int = 2_000_000_000):
        from .kv_transfer import KVPusher
        self.link, self.runner, self.peer = link, runner, peer_rank
        self.budget = int(wait_budget_cycles)
        self.pusher = KVPusher(runner.kv_caches, runner.block_size, runner.device)
        self.layer_of = {int(k.data_ptr()): i for i, (k, _) in enumerate(runner.kv_caches)}
        self.n_layers = len(runner.kv_caches)
        self.target = None
        self.pushed_bytes = 0

    def set_remote(self, num_blocks: int):
        """The decode instance's cache has the layout [L, planes, num_blocks, heads, page, d] at the
        start of its buffer."""
        from .kv_transfer import PushTarget
        bb = self.pusher.block_bytes
        planes = int(self.runner.kv_tensor.shape[1])
        base = self.link.peer_base(self.peer)
        ptrs = [(base + (l * planes + 0) * num_blocks * bb, base + (l * planes + planes - 1) * num_blocks * bb)
                for l in range(self.n_layers)]
        self.target = PushTarget(ptrs, bb, base + self.link.kv_bytes)

    def begin_step(self, pairs: np.ndarray, epoch: int):
        self._pairs = torch.from_numpy(np.ascontiguousarray(pairs, dtype=np.int32)).to(self.runner.device, non_blocking=True)
        self._epoch = epoch

    def push_layer(self, k_cache: torch.Tensor):
        layer = self.layer_of[int(k_cache.data_ptr())]
        self.pusher.push_layer(layer, self._pairs, self.target, self._epoch)
        self.pushed_bytes += 2 * self._pairs.shape[0] * self.pusher.block_bytes

    def end_step(self, channel):
        pass

    # decode side
    def wait(self, epoch: int) -> int:
        """0 when every layer flag reached `epoch` within the budget, else 1 + a late layer."""
        from ..ops import _lib
        from ..ops._lib import check, ptr, stream
        check(_lib.load().xllm_kv_wait_many(ptr(self.link.flags), self.n_layers, epoch, ptr(self.link.status), self.budget,
                                            stream()), "kv_wait_many")
        return int(self.link.status.item())

    def receive(self, msg):
        raise RuntimeError("peer-push instances exchange no kv messages")


class SocketCopy:
    """Data plane over the control connection: blocks are read back after each layer wrote them and
    sent as `kv` messages at the end of the step (CPU instances; GPUs without peer access)."""

    name = "socket_copy"

    def __init__(self, runner):
        self.runner = runner
        self.layer_of = {int(k.data_ptr()): i for i, (k, _) in enumerate(runner.kv_caches)}
        self._out: List[dict] = []
        self.pushed_bytes = 0

    def set_remote(self, num_blocks: int):
        pass

    def begin_step(self, pairs: np.ndarray, epoch: int):
        self._src = torch.as_tensor(pairs[:, 0].astype(np.int64), device=self.runner.device)
        self._dst = [int(b) for b in pairs[:, 1]]
        self._out = []

    def push_layer(self, k_cache: torch.Tensor):
        layer = self.layer_of[int(k_cache.data_ptr())]
        k, v = self.runner.kv_caches[layer]
        kb = k[self._src].contiguous().cpu().view(torch.uint8).numpy().tobytes()
        vb = v[self._src].contiguous().cpu().view(torch.uint8).numpy().tobytes()
        self._out.append({"op": "kv", "layer": layer, "blocks": self._dst, "k": kb, "v": vb})
        self.pushed_bytes += len(kb) + len(vb)

    def end_step(self, channel):
        for m in self._out:
            channel.send(m)
        self._out = []

    def wait(self, epoch: int) -> int:
        return 0                       # kv messages precede `first` on the same ordered connection

    def receive(self, msg):
        k, v = self.runner.kv_caches[int(msg["layer"])]
        idx = torch.as_tensor(msg["blocks"], dtype=torch.long, device=k.device)
        shape = (len(msg["blocks"]),) + tuple(k.shape[1:])
        kb = torch.frombuffer(bytearray(msg["k"]), dtype=torch.uint8).view(k.dtype).view(shape)
        vb = torch.frombuffer(bytearray(msg["v"]), dtype=torch.uint8).view(v.dtype).view(shape)
        k[idx] = kb.to(k.device)
        v[idx] = vb.to(v.device)


# ------------------------------------------------------------------------------------------ helpers
def _topology(engine) -> dict:
    r = engine.runner
    k0 = r.kv_caches[0][0]
    return {"block_size": int(r.block_size), "n_layers": len(r.kv_caches), "n_kv_heads": int(k0.shape[1]),
            "head_dim": int(k0.shape[3]), "dtype": str(k0.dtype), "tp": int(engine.ps.tp_size),
            "planes": int(r.kv_tensor.shape[1])}


def _params_of(engine, par: dict):
    """(SamplingParams, StoppingParams) of the runtime from a plain dict."""
    rt = engine.rt
    sp = rt.SamplingParams()
    sp.temperature = float(par.get("temperature", 0.0))
    sp.top_p = float(par.get("top_p", 1.0))
    sp.top_k = int(par.get("top_k", -1))
    sp.seed = int(par.get("seed", engine.cfg.seed) or 0)
    st = rt.StoppingParams()
    st.max_tokens = int(par.get("max_tokens", 16))
    st.max_context_len = int(engine.max_model_len)
    eos = par.get("eos_token_id")
    st.eos_token_id = int(engine.args.eos_token_id if eos is None else eos)
    st.ignore_eos = bool(par.get("ignore_eos", False))
    st.stop_token_ids = list(par.get("stop_token_ids") or [])
    st.stop_sequences = [list(s) for s in (par.get("stop_sequences") or [])]
    return sp, st


class RemoteEvent:
    """A token generated by the decode instance, as the prefill side's client sees it."""

    def __init__(self, m: dict):
        self.request_id = m["rid"]
        self.token = int(m["token"])
        self.logprob = float(m.get("logprob", 0.0))
        self.finished = bool(m.get("finished", False))
        self.request_finished = self.finished
        self.finish_reason = m.get("reason", "")
        self.index = 0
        self.seq_index = 0
        self.has_logprob = False
        self.num_prompt_tokens = 0
        self.seq_id = -1


# ------------------------------------------------------------------------------------------ decode side
class DecodeService:
    """Serves one prefill peer: reserves blocks, receives KV, adopts sequences, streams tokens back."""

    def __init__(self, engine, channel: Channel, transport, pull_offline: bool = False, pull_below: int = 1,
                 pull_interval: float = 0.02):
        """`pull_offline`: while fewer than `pull_below` requests run or are reserved here, ask the prefill
        instance (at most every `pull_interval` seconds) to move one of its local offline requests over."""
        self.e, self.ch, self.t = engine, channel, transport
        self.peer_requests: set = set()
        self.stopped = False
        self.adopted = 0
        self.pull_offline, self.pull_below, self.pull_interval = bool(pull_offline), int(pull_below), float(pull_interval)
        self._last_pull = 0.0
        self.pulls_sent = 0
        self.failed_waits = 0
        self.reclaimed_blocks = 0

    def _on_message(self, m: dict):
        op = m.get("op")
        sch = self.e.scheduler
        if op == "hello":
            mine = _topology(self.e)
            bad = [k for k in ("block_size", "n_layers", "n_kv_heads", "head_dim", "dtype", "tp", "planes")
                   if m.get(k) != mine[k]]
            self.ch.send({"op": "hello_ack", "ok": not bad, "reason": "mismatch: " + ",".join(bad) if bad else "",
                          "num_blocks": int(self.e.runner.num_blocks), "transport": self.t.name})
        elif op == "reserve":
            blocks = sch.reserve_blocks(m["rid"], int(m["n_tokens"]))
            self.ch.send({"op": "reserved", "rid": m["rid"], "blocks": [int(b) for b in blocks]})
        elif op == "kv":
            self.t.receive(m)
        elif op == "first":
            rid = m["rid"]
            status = self.t.wait(int(m.get("epoch", 0)))
            ok, reason = False, ""
            if status != 0:
                self.failed_waits += 1
                reason = f"kv of layer {status - 1} did not arrive"
            else:
                sp, st = _params_of(self.e, m.get("sampling") or {})
                ok = bool(sch.adopt_reserved(rid, [int(t) for t in m["tokens"]], int(m["num_prompt"]), sp, st))
                reason = "" if ok else "no reservation"
            if ok:
                self.adopted += 1
                self.peer_requests.add(rid)
            else:
                sch.cancel_reserved(rid)
            self.ch.send({"op": "adopted", "rid": rid, "ok": ok, "reason": reason})
        elif op == "cancel":
            rid = m["rid"]
            if not sch.cancel_reserved(rid) and rid in self.peer_requests:
                self.e.abort(rid)
                self.peer_requests.discard(rid)
        elif op == "bye":
            self.stopped = True

    def _peer_gone(self):
        """The prefill side closed the connection: give everything it held here back."""
        sch = self.e.scheduler
        before = int(sch.block_stats().num_free)
        for rid in list(sch.reserved_ids()):
            sch.cancel_reserved(rid)
        for rid in list(self.peer_requests):
            self.e.abort(rid)
        self.peer_requests.clear()
        self.reclaimed_blocks += int(sch.block_stats().num_free) - before
        self.stopped = True

    def _maybe_pull(self):
        """Spare capacity here: ask the prefill instance for one of the offline requests it is decoding
        itself (the pull signal of the reference's PD-OOC scheduler, xllm/core/scheduler/pd_ooc_scheduler.cpp)."""
        if not self.pull_offline or self.stopped or self.ch.closed:
            return
        sch = self.e.scheduler
        now = time.time()
        if len(self.peer_requests) + int(sch.num_reserved()) >= self.pull_below or now - self._last_pull < self.pull_interval:
            return
        self._last_pull = now
        self.pulls_sent += 1
        self.ch.send({"op": "pull", "free_blocks": int(sch.block_stats().num_free), "max_requests": 1})

    def step(self, idle_wait: float = 0.0):
        for m in self.ch.poll(idle_wait):
            self._on_message(m)
        if self.ch.closed and not self.stopped:
            self._peer_gone()
        self._maybe_pull()
        if self.e.has_unfinished():
            events = self.e.step()
        else:
            events = self.e.drain()
        for ev in events:
            rid = ev.request_id
            if rid not in self.peer_requests:
                continue
            if ev.token >= 0 or ev.finished:
                self.ch.send({"op": "gen", "rid": rid, "token": int(ev.token), "logprob": float(getattr(ev, "logprob", 0.0)),
                              "finished": bool(ev.request_finished), "reason": str(getattr(ev, "finish_reason", ""))})
            if ev.request_finished:
                self.peer_requests.discard(rid)
        return events

    def serve(self, max_seconds: float = 600.0):
        """Until the peer says bye (or goes away) and nothing is left to decode."""
        deadline = time.time() + max_seconds
        while time.time() < deadline:
            busy = self.e.has_unfinished()
            self.step(0.0 if busy else 0.002)
            if self.stopped and not self.e.has_unfinished():
                for ev in self.e.drain():
                    pass
                return True
        return False


# ------------------------------------------------------------------------------------------ prefill side
class PrefillService:
    """Fronts the clients: prefills prompts, pushes their KV to the decode peer while the forward
    runs, hands the first token over, relays the tokens that come back."""

    RETRY_SECONDS = 0.01

    def __init__(self, engine, channel: Channel, transport, hello_timeout: float = 60.0):
        self.e, self.ch, self.t = engine, channel, transport
        self.params: Dict[str, dict] = {}
        self.prompts: Dict[str, List[int]] = {}
        self.dst_blocks: Dict[str, List[int]] = {}
        self.pushed_upto: Dict[str, int] = {}        # first block index not yet pushed completely
        self.local: set = set()                       # offline requests that decode on this instance
        self.kept_local = 0
        self.local_state: Dict[str, dict] = {}        # their prompt, parameters and the tokens produced so far
        self.migrating: set = set()                   # offline requests on their way to the decode instance
        self.migrated = 0
        self._deferred: List[dict] = []
        self.retry_at: Dict[str, float] = {}
        self.awaiting_adopt: set = set()
        self.remote: set = set()                     # decoding on the peer
        self.failed: Dict[str, str] = {}
        self.epoch = 0
        self.handed_over = 0
        self.bs = int(engine.runner.block_size)
        engine.runner.meta_hook = self._chain_hook(engine.runner.meta_hook)
        self.ch.send(dict(_topology(engine), op="hello"))
        deadline = time.time() + hello_timeout
        ack = None
        while ack is None and time.time() < deadline and not self.ch.closed:
            for m in self.ch.poll(0.05):
                if m.get("op") == "hello_ack":
                    ack = m
        if ack is None or not ack.get("ok"):
            raise RuntimeError("decode instance refused the pairing: " + (ack or {}).get("reason", "no answer"))
        self.t.set_remote(int(ack["num_blocks"]))

    # ---- the per-layer push, installed on every step that computes prompt KV
    def _chain_hook(self, prev):
        def hook(batch, meta):
            if prev is not None:
                prev(batch, meta)
            pairs = self._pairs_of(batch)
            if pairs is not None:
                self.epoch += 1
                self.t.begin_step(pairs, self.epoch)
                meta.kv_hook = self.t.push_layer
        return hook

    def _pairs_of(self, batch) -> Optional[np.ndarray]:
        """(source block, destination block) of every block whose KV this step completes or extends.
        Blocks a prefix-cache hit supplied are pushed with the first chunk that follows them."""
        nd, npf = int(batch.n_decode), int(batch.n_prefill)
        if npf == 0:
            return None
        bt = np.asarray(batch.block_tables)
        kv = np.asarray(batch.kv_lens)
        out = []
        for i in range(nd, nd + npf):
            rid = batch.request_id(i)
            dst = self.dst_blocks.get(rid)
            if dst is None:
                continue
            last = (int(kv[i]) - 1) // self.bs
            first = self.pushed_upto.get(rid, 0)
            for b in range(first, min(last, len(dst) - 1) + 1):
                out.append((int(bt[i, b]), int(dst[b])))
            self.pushed_upto[rid] = last if int(kv[i]) % self.bs else last + 1
        if not out:
            return None
        return np.asarray(out, dtype=np.int32).reshape(-1, 2)

    # ---- intake
    def add_request(self, request_id: str, prompt_token_ids, max_tokens=16, **kw) -> bool:
        """`offline=True`: the request is throughput work without a latency target (online / offline
        co-location, xllm/core/scheduler/pd_ooc_scheduler.cpp): it is not handed to the decode instance but
        decodes HERE, in the steps the scheduler has left after the online prompts, which preempt it
        (`enable_online_preempt_offline`); the decode instance's capacity stays with the online requests."""
        toks = [int(t) for t in prompt_token_ids]
        if len(toks) + 1 >= self.e.max_model_len or request_id in self.params:
            return False
        if kw.get("offline"):
            pkw = {k: v for k, v in kw.items() if k != "stop_sequences"}
            if not self.e.add_request(request_id, toks, max_tokens=int(max_tokens), **pkw):
                return False
            self.local.add(request_id)
            self.kept_local += 1
            self.local_state[request_id] = dict(prompt=toks, max_tokens=int(max_tokens), gen=[],
                                                params={k: v for k, v in kw.items() if k != "offline"})
            return True
        self.params[request_id] = dict(kw, max_tokens=int(max_tokens))
        self.prompts[request_id] = toks
        if max_tokens <= 1:
            pkw = {k: v for k, v in kw.items() if k != "stop_sequences"}
            return self.e.add_request(request_id, toks, max_tokens=1, **pkw)
        self.ch.send({"op": "reserve", "rid": request_id, "n_tokens": len(toks) + 1})
        return True

    def abort(self, request_id: str):
        if request_id in self.local:
            self.local.discard(request_id)
            self.local_state.pop(request_id, None)
            self.e.abort(request_id)
            self.e.scheduler.release_held(request_id)
            return
        self.ch.send({"op": "cancel", "rid": request_id})
        self.e.abort(request_id)
        self._forget(request_id)

    def _forget(self, rid):
        for d in (self.params, self.prompts, self.dst_blocks, self.pushed_upto, self.retry_at):
            d.pop(rid, None)
        self.awaiting_adopt.discard(rid)
        self.remote.discard(rid)
        self.migrating.discard(rid)

    def _migrate_one(self, free_blocks: int) -> Optional[str]:
        """The decode instance has spare capacity: hand it the local offline request with the most tokens
        still to produce that fits into `free_blocks`.  The request is taken out of this engine and goes
        through the ordinary handover with (prompt + tokens so far) as its prompt: with the prefix cache on,
        its blocks are found again and only the push remains; without, the KV is recomputed once."""
        best, best_left = None, 1
        for rid in self.local:
            st = self.local_state.get(rid)
            if st is None or not st["gen"]:
                continue                                   # still in its prompt: nothing to gain
            left = st["max_tokens"] - len(st["gen"])
            n_tok = len(st["prompt"]) + len(st["gen"]) + 1
            if left > best_left and (n_tok + self.bs - 1) // self.bs <= free_blocks and n_tok + left < self.e.max_model_len:
                best, best_left = rid, left
        if best is None:
            return None
        st = self.local_state.pop(best)
        self.local.discard(best)
        self.e.abort(best)
        self.e.scheduler.release_held(best)
        self.params[best] = dict(st["params"], max_tokens=best_left)
        self.prompts[best] = st["prompt"] + st["gen"]
        self.migrating.add(best)
        self.ch.send({"op": "reserve", "rid": best, "n_tokens": len(self.prompts[best]) + 1})
        return best

    def has_unfinished(self) -> bool:
        return bool(self.params) or bool(self.remote) or self.e.has_unfinished()

    # ---- one iteration
    def step(self, idle_wait: float = 0.0):
        out = []
        now = time.time()
        for rid, t in list(self.retry_at.items()):
            if now >= t:
                del self.retry_at[rid]
                self.ch.send({"op": "reserve", "rid": rid, "n_tokens": len(self.prompts[rid]) + 1})
        msgs, self._deferred = self._deferred + self.ch.poll(idle_wait if not self.e.has_unfinished() else 0.0), []
        for m in msgs:
            op = m.get("op")
            rid = m.get("rid")
            if op == "pull":
                self._migrate_one(int(m.get("free_blocks", 0)))
            elif op == "reserved":
                if rid not in self.params:
                    if m["blocks"]:
                        self.ch.send({"op": "cancel", "rid": rid})
                elif m["blocks"]:
                    self.dst_blocks[rid] = list(m["blocks"])
                    par = self.params[rid]
                    pkw = {k: v for k, v in par.items() if k not in ("stop_sequences", "max_tokens")}
                    if not self.e.add_request(rid, self.prompts[rid], max_tokens=1, **pkw):
                        if rid in self.migrating and m.get("_tries", 0) < 100:
                            # its aborted incarnation is still part of a step in flight: try again next step
                            self._deferred.append(dict(m, _tries=m.get("_tries", 0) + 1))
                            continue
                        self.ch.send({"op": "cancel", "rid": rid})
                        self.failed[rid] = "rejected by the prefill engine"
                        out.append(_failure(rid, self.failed[rid]))
                        self._forget(rid)
                else:
                    self.retry_at[rid] = now + self.RETRY_SECONDS
            elif op == "adopted":
                self.awaiting_adopt.discard(rid)
                self.e.scheduler.release_held(rid)
                if m.get("ok"):
                    self.handed_over += 1
                    if rid in self.migrating:
                        self.migrating.discard(rid)
                        self.migrated += 1
                    self.remote.add(rid)
                    for d in (self.params, self.prompts, self.dst_blocks, self.pushed_upto):
                        d.pop(rid, None)
                else:
                    self.failed[rid] = m.get("reason", "refused")
                    out.append(_failure(rid, self.failed[rid]))
                    self._forget(rid)
            elif op == "gen":
                if rid in self.remote:
                    ev = RemoteEvent(m)
                    out.append(ev)
                    if ev.finished:
                        self.remote.discard(rid)
        if self.ch.closed:
            # the decode side is gone: everything that was not finished fails here
            for rid in list(self.remote) + list(self.params):        # (offline requests run here and go on)
                self.failed[rid] = "decode instance went away"
                out.append(_failure(rid, self.failed[rid]))
                self.e.abort(rid)
                self.e.scheduler.release_held(rid)
                self._forget(rid)
            if not self.local:
                return out
        if self.e.has_unfinished():
            events = self.e.step()
            if not self.e.scheduler.has_unfinished():
                events = events + self.e.drain()
            if not self.ch.closed:
                self.t.end_step(self.ch)
            for ev in events:
                if ev.request_id in self.local:          # an offline request: its whole stream is produced here
                    out.append(ev)
                    st = self.local_state.get(ev.request_id)
                    if st is not None and ev.token >= 0:
                        st["gen"].append(int(ev.token))
                    if ev.request_finished:
                        self.local.discard(ev.request_id)
                        self.local_state.pop(ev.request_id, None)
                        self.e.scheduler.release_held(ev.request_id)
                    continue
                if ev.token < 0:
                    continue
                rid = ev.request_id
                par = self.params.get(rid)
                if par is None:
                    continue
                if par.get("max_tokens", 16) <= 1:
                    self.e.scheduler.release_held(rid)
                    self._forget(rid)
                    out.append(ev)
                    continue
                hist = self.prompts[rid] + [int(ev.token)]
                samp = {k: v for k, v in par.items() if isinstance(v, (int, float, bool, list, type(None)))}
                self.ch.send({"op": "first", "rid": rid, "tokens": hist, "num_prompt": len(hist) - 1,
                              "sampling": samp, "epoch": self.epoch})
                self.awaiting_adopt.add(rid)
                out.append(_FirstToken(ev))
        return out

    def run_until_done(self, on_event=None, max_seconds: float = 600.0):
        deadline = time.time() + max_seconds
        while self.has_unfinished() and time.time() < deadline:
            for ev in self.step(0.002):
                if on_event is not None:
                    on_event(ev)
        return not self.has_unfinished()

    def close(self):
        self.ch.send({"op": "bye"})


def _failure(rid: str, reason: str):
    return RemoteEvent({"rid": rid, "token": -1, "finished": True, "reason": "error: " + reason})
