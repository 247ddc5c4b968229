"""Prefill/decode disaggregation: one engine only prefills, another only decodes, KV blocks move
between their caches.

Parity: `DisaggPDScheduler` and the `DisaggPDService` protocol
(xllm/core/scheduler/disagg_pd_scheduler.h:50-209, proto/disagg_pd.proto:281-287):
  1. the request goes to a PREFILL instance, which asks a DECODE instance to reserve KV blocks
     (`decode_schedule`),
  2. the prefill instance runs the prompt and produces the first token,
  3. the KV blocks are pushed to the reserved blocks of the decode instance (layer by layer) and the
     first token is handed over (`prefill_send_first_generation`),
  4. the decode instance continues the sequence from its own scheduler.
The reference moves KV with Mooncake on non-CUDA back ends only; here the data plane is
`KVPusher` (csrc/kernels/spec_kv.cu `xllm_kv_push`, peer stores over NVLink, bounded flag waits) when
both caches are on GPUs that can address each other, and a plain tensor copy otherwise (CPU tests,
same-device instances).

`PDCoordinator` drives both instances in one process (the in-process form of the reference's
prefill/decode pair; tests and single-node serving).  `PrefillHandoff` is the message of step 3 for
instances in different processes: it is what a transport has to carry besides the KV itself.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch


@dataclass
class PrefillHandoff:
    request_id: str
    tokens: List[int]            # prompt + first generated token
    num_prompt_tokens: int
    src_blocks: List[int]        # blocks of the prefill instance holding the prompt's KV
    sampling: dict = field(default_factory=dict)


def copy_kv_blocks(src_caches, dst_caches, src_blocks, dst_blocks):
    """Layer-by-layer block copy between two paged caches of the same layout
    ([n_blocks, n_kv_heads, block_size, head_dim] per K and V)."""
    n = min(len(src_blocks), len(dst_blocks))
    if n == 0:
        return
    si = torch.as_tensor(src_blocks[:n], dtype=torch.long, device=src_caches[0][0].device)
    di = torch.as_tensor(dst_blocks[:n], dtype=torch.long, device=dst_caches[0][0].device)
    for (sk, sv), (dk, dv) in zip(src_caches, dst_caches):
        dk[di] = sk[si].to(dk.device, non_blocking=True)
        dv[di] = sv[si].to(dv.device, non_blocking=True)


class PDCoordinator:
    """Routes requests through a prefill engine and a decode engine.

    Both are `LLMEngine`s over the same model; the prefill engine's scheduler is created with
    `hold_finished_blocks` so that the prompt's blocks outlive the (one-token) prefill request until
    they have been transferred."""

    def __init__(self, prefill_engine, decode_engine, transfer=None):
        self.p, self.d = prefill_engine, decode_engine
        assert self.p.cfg.block_size == self.d.cfg.block_size, "P and D must use the same KV block size"
        self.transfer = transfer or copy_kv_blocks
        self.params: Dict[str, dict] = {}
        self._prompts: Dict[str, List[int]] = {}
        self.waiting_handoff: List[PrefillHandoff] = []   # prefilled, decode side had no blocks yet
        self.first_tokens: Dict[str, int] = {}
        self.transferred_blocks = 0

    # ------------------------------------------------------------------ intake
    def add_request(self, request_id: str, prompt_token_ids, max_tokens=16, **kw) -> bool:
        self.params[request_id] = dict(kw, max_tokens=max_tokens)
        self._prompts[request_id] = [int(t) for t in prompt_token_ids]
        pkw = {k: v for k, v in kw.items() if k not in ("stop_sequences",)}
        # the prefill instance produces exactly one token
        return self.p.add_request(request_id, prompt_token_ids, max_tokens=1, **pkw)

    def has_unfinished(self) -> bool:
        return self.p.has_unfinished() or self.d.has_unfinished() or bool(self.waiting_handoff)

    # ------------------------------------------------------------------ one iteration of both sides
    def step(self):
        """Returns the OutputEvents visible to the client (first tokens come from the prefill side)."""
        out = []
        if self.p.has_unfinished():
            for ev in self.p.step() + (self.p.drain() if not self.p.scheduler.has_unfinished() else []):
                if ev.token < 0:
                    continue
                rid = ev.request_id
                par = self.params.get(rid, {})
                if par.get("max_tokens", 16) <= 1:
                    self.p.scheduler.release_held(rid)
                    self.params.pop(rid, None)
                    out.append(ev)
                    continue
                hist = list(self._prompt_of(rid)) + [int(ev.token)]
                self.waiting_handoff.append(PrefillHandoff(rid, hist, len(hist) - 1,
                                                           list(self.p.scheduler.held_blocks(rid)), par))
                self.first_tokens[rid] = int(ev.token)
                out.append(_FirstToken(ev))
        still = []
        for h in self.waiting_handoff:
            if not self._handoff(h):
                still.append(h)
        self.waiting_handoff = still
        if self.d.has_unfinished():
            out.extend(self.d.step())
        return out

    def run_until_done(self, on_event=None):
        while self.has_unfinished():
            for ev in self.step():
                if on_event is not None:
                    on_event(ev)
        for ev in self.d.drain():
            if on_event is not None:
                on_event(ev)

    # ------------------------------------------------------------------ internals
    def _prompt_of(self, rid):
        return self._prompts[rid]

    def _handoff(self, h: PrefillHandoff) -> bool:
        d = self.d
        rt = d.rt
        par = h.sampling
        sp = rt.SamplingParams()
        sp.temperature = float(par.get("temperature", 0.0))
        sp.top_p = float(par.get("top_p", 1.0))
        sp.top_k = int(par.get("top_k", -1))
        sp.seed = int(par.get("seed", d.cfg.seed) or 0)
        st = rt.StoppingParams()
        st.max_tokens = int(par.get("max_tokens", 16))
        st.max_context_len = int(d.max_model_len)
        eos = par.get("eos_token_id")
        st.eos_token_id = int(d.args.eos_token_id if eos is None else eos)
        st.ignore_eos = bool(par.get("ignore_eos", False))
        st.stop_token_ids = list(par.get("stop_token_ids") or [])
        st.stop_sequences = [list(s) for s in (par.get("stop_sequences") or [])]
        blocks = d.scheduler.adopt_prefilled(h.request_id, h.tokens, h.num_prompt_tokens, sp, st)
        if len(blocks) == 0:
            return False                      # decode side is full: retry on a later step
        n_kv_blocks = (h.num_prompt_tokens + d.cfg.block_size - 1) // d.cfg.block_size
        self.transfer(self.p.runner.kv_caches, d.runner.kv_caches, h.src_blocks[:n_kv_blocks], list(blocks)[:n_kv_blocks])
        self.transferred_blocks += n_kv_blocks
        self.p.scheduler.release_held(h.request_id)
        self.params.pop(h.request_id, None)
        self._prompts.pop(h.request_id, None)
        return True


class _FirstToken:
    """The prefill side's event for the first token, re-labelled as unfinished: the decode side
    carries the request on."""

    def __init__(self, ev):
        self._ev = ev
        self.finished = False
        self.request_finished = False
        self.finish_reason = ""

    def __getattr__(self, name):
        # private and protocol names stay with the wrapper: forwarding them lets a binding layer that
        # probes objects by attribute mistake the wrapper for the event it wraps
        if name.startswith("_"):
            raise AttributeError(name)
        return getattr(self._ev, name)


def make_pd_pair(model: str, prefill_kw: Optional[dict] = None, decode_kw: Optional[dict] = None, share_model=True,
                 **common):
    """Two engines over one model (weights shared when both live on the same device)."""
    from .llm_engine import EngineConfig, LLMEngine

    pk = dict(common, **(prefill_kw or {}))
    dk = dict(common, **(decode_kw or {}))
    p = LLMEngine(EngineConfig(model=model, **pk), hold_finished_blocks=True)
    d = LLMEngine(EngineConfig(model=model, **dk), model=p.model if share_model else None,
                  model_args=p.args if share_model else None)
    return p, d
