"""Offline Python entry points: LLM.generate / beam_search / embed, SamplingParams, RequestOutput.

API parity with the reference's pybind front end (xllm/pybind/llm.py:82-519, params.py): same class
and argument names where they carry over.  Prompts may be strings (tokenised by the C++ tokenizer of
the model directory) or lists of token ids.
"""
from __future__ import annotations

import itertools
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Union

import torch

from ..engine.llm_engine import EngineConfig, LLMEngine


@dataclass
class SamplingParams:
    """Mirrors xllm.SamplingParams (xllm/pybind/params.py)."""
    n: int = 1
    best_of: Optional[int] = None
    max_tokens: int = 16
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = -1
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    repetition_penalty: float = 1.0
    logprobs: bool = False
    top_logprobs: int = 0
    skip_special_tokens: bool = True
    ignore_eos: bool = False
    stop: Optional[List[str]] = None
    stop_token_ids: Optional[List[int]] = None
    seed: Optional[int] = None
    echo: bool = False


RequestParams = SamplingParams       # the reference's name for the per-request parameter bag (xllm_export.RequestParams)


@dataclass
class PoolingParams:
    """Parameters of an embedding request (xllm/pybind/params.py PoolingParams)."""
    normalize: bool = True
    is_embeddings: bool = True


@dataclass
class BeamSearchParams:
    beam_width: int = 4
    max_tokens: int = 16
    length_penalty: float = 1.0
    ignore_eos: bool = False


@dataclass
class SequenceOutput:
    index: int
    text: str = ""
    token_ids: List[int] = field(default_factory=list)
    finish_reason: Optional[str] = None
    logprobs: Optional[List[float]] = None
    # per generated token, when the request asked for top_logprobs: [(token id, logprob), ...] best first
    top_logprobs: Optional[List[List[tuple]]] = None


@dataclass
class Usage:
    num_prompt_tokens: int = 0
    num_generated_tokens: int = 0
    num_total_tokens: int = 0
    num_cached_tokens: int = 0


@dataclass
class RequestOutput:
    request_id: str
    prompt: Optional[str] = None
    prompt_token_ids: List[int] = field(default_factory=list)
    outputs: List[SequenceOutput] = field(default_factory=list)
    finished: bool = False
    cancelled: bool = False
    usage: Usage = field(default_factory=Usage)
    # host-clock timing of the request: ttft_ms (submission -> first token), tpot_ms (mean gap between
    # tokens), e2e_ms; filled by generate()
    metrics: Dict[str, float] = field(default_factory=dict)


@dataclass
class EmbeddingOutputs:
    embedding: List[float] = field(default_factory=list)

    @property
    def embeddings(self):
        return self.embedding


@dataclass
class EmbeddingOutput:
    """Result of `LLM.embed` for one prompt (xllm/pybind/llm.py:64-80)."""
    prompt: Optional[str]
    outputs: EmbeddingOutputs
    usage: Usage
    request_output: Optional[RequestOutput] = None
    status: Optional[object] = None


class LLM:
    """Offline batch inference over one engine (single GPU, or one rank of a TP job)."""

    _ids = itertools.count()

    def __init__(self, model: str = "tiny", devices: Optional[str] = None, dtype: str = "auto",
                 block_size: int = 16, max_cache_size: int = 0, max_memory_utilization: float = 0.9,
                 enable_prefix_cache: bool = True, max_tokens_per_batch: int = 8192,
                 max_seqs_per_batch: int = 256, max_tokens_per_chunk_for_prefill: int = -1,
                 enable_chunked_prefill: bool = True, enable_schedule_overlap: bool = False,
                 enable_graph: bool = True, max_model_len: int = 0, num_blocks: int = 0,
                 policy: str = "prefill_first", seed: int = 0, random_weights: bool = False,
                 parallel_state=None, tokenizer=None, **kwargs):
        device = "auto"
        if devices:
            device = devices.split(",")[0].strip()
            if device == "cuda":
                device = "cuda:0"
        cfg = EngineConfig(model=model, dtype=dtype, device=device, block_size=block_size,
                           num_blocks=num_blocks, max_memory_utilization=max_memory_utilization,
                           max_cache_size=max_cache_size, max_seqs_per_batch=max_seqs_per_batch,
                           max_tokens_per_batch=max_tokens_per_batch, max_model_len=max_model_len,
                           enable_prefix_cache=enable_prefix_cache,
                           enable_chunked_prefill=enable_chunked_prefill,
                           max_tokens_per_chunk_for_prefill=max_tokens_per_chunk_for_prefill,
                           policy=policy, enable_schedule_overlap=enable_schedule_overlap,
                           enable_graph=enable_graph, seed=seed, random_weights=random_weights)
        for k, v in kwargs.items():
            if hasattr(cfg, k):
                setattr(cfg, k, v)
        self._workers = None
        import os as _os
        from ..engine.offline_worker import WorkerGroup, _Shim, parse_devices
        devs = parse_devices(devices)
        if len(devs) > 1 and parallel_state is None and "RANK" not in _os.environ:
            # several devices and no launcher: this process becomes rank 0 and starts the other ranks itself
            from ..engine.replica import lead_ranks
            from ..parallel.state import init_parallel
            self._workers = WorkerGroup(cfg, devs, int(kwargs.get("dp_size", 1)), int(kwargs.get("ep_size", 1)))
            _os.environ.update(self._workers.env0)
            if self._workers.visible is not None:
                _os.environ["CUDA_VISIBLE_DEVICES"] = self._workers.visible
            cfg.device = "auto"
            parallel_state = init_parallel(dp_size=int(kwargs.get("dp_size", 1)), ep_size=int(kwargs.get("ep_size", 1)))
            self.engine = LLMEngine(cfg, ps=parallel_state)
            self._lead = _Shim(self.engine)
            lead_ranks(self._lead, parallel_state)
            import atexit
            atexit.register(self.close)
        else:
            self.engine = LLMEngine(cfg, ps=parallel_state)
        self.tokenizer = tokenizer
        if tokenizer is None:
            import os
            if os.path.isdir(model):
                from ..utils.tokenizer import load_tokenizer
                self.tokenizer = load_tokenizer(model)

    def close(self):
        """Stops the worker ranks this object started (no-op otherwise)."""
        if self._workers is not None:
            w, self._workers = self._workers, None
            try:
                if w.alive():
                    self._lead.shutdown()          # broadcasts "stop" to the followers
            finally:
                w.wait()

    # ------------------------------------------------------------------ helpers
    def _encode(self, p) -> List[int]:
        if isinstance(p, str):
            if self.tokenizer is None:
                raise ValueError("string prompts need a tokenizer; pass token ids instead")
            return list(self.tokenizer.encode(p))
        if isinstance(p, torch.Tensor):
            return p.tolist()
        return list(p)

    def _decode(self, ids: Sequence[int], skip_special=True) -> str:
        if self.tokenizer is None:
            return ""
        return self.tokenizer.decode(list(ids), skip_special)

    # ------------------------------------------------------------------ generate
    def generate(self, prompts, sampling_params: Union[SamplingParams, List[SamplingParams], None] = None,
                 max_concurrency: int = 0, on_token=None) -> List[RequestOutput]:
        """Run every prompt to completion.  `max_concurrency` > 0 keeps at most that many requests in
        flight (a closed loop: a finished request admits the next one), 0 submits everything."""
        if isinstance(prompts, (str, torch.Tensor)) or (prompts and isinstance(prompts[0], int)):
            prompts = [prompts]
        n = len(prompts)
        sps = sampling_params if isinstance(sampling_params, list) else [sampling_params or SamplingParams()] * n
        outs: List[RequestOutput] = []
        by_id: Dict[str, RequestOutput] = {}
        todo = []
        for i, (p, sp) in enumerate(zip(prompts, sps)):
            ids = self._encode(p)
            rid = f"req-{next(LLM._ids)}"
            ro = RequestOutput(rid, p if isinstance(p, str) else None, ids,
                               [SequenceOutput(j) for j in range(sp.n)])
            ro.usage.num_prompt_tokens = len(ids)
            outs.append(ro)
            by_id[rid] = ro
            todo.append((rid, ids, sp))
        eng = self.engine
        in_flight = 0
        cursor = 0
        import time as _time
        t_sub: Dict[str, float] = {}
        t_first: Dict[str, float] = {}
        t_last: Dict[str, float] = {}

        def submit_some():
            nonlocal cursor, in_flight
            while cursor < n and (max_concurrency <= 0 or in_flight < max_concurrency):
                rid, ids, sp = todo[cursor]
                cursor += 1
                stop_seqs = None
                if sp.stop and self.tokenizer is not None:
                    stop_seqs = [list(self.tokenizer.encode(s)) for s in sp.stop]
                ok = eng.add_request(rid, ids, temperature=sp.temperature, top_p=sp.top_p, top_k=sp.top_k,
                                     max_tokens=sp.max_tokens, ignore_eos=sp.ignore_eos,
                                     stop_token_ids=sp.stop_token_ids, stop_sequences=stop_seqs,
                                     frequency_penalty=sp.frequency_penalty,
                                     presence_penalty=sp.presence_penalty,
                                     repetition_penalty=sp.repetition_penalty, logprobs=sp.logprobs,
                                     top_logprobs=sp.top_logprobs, seed=sp.seed, n=sp.n, offline=True)
                if not ok:
                    by_id[rid].finished = True
                    by_id[rid].cancelled = True
                else:
                    in_flight += 1
                    t_sub[rid] = _time.perf_counter()

        submit_some()
        while eng.has_unfinished() or cursor < n:
            evs = eng.step()
            now = _time.perf_counter()
            for e in evs:
                ro = by_id.get(e.request_id)
                if ro is None:
                    continue
                so = ro.outputs[e.seq_index]
                if e.token >= 0:
                    t_first.setdefault(e.request_id, now)
                    t_last[e.request_id] = now
                    so.token_ids.append(e.token)
                    if e.top_ids:
                        if so.top_logprobs is None:
                            so.top_logprobs = []
                        so.top_logprobs.append(list(zip(e.top_ids, e.top_logprobs)))
                    if e.has_logprob:
                        if so.logprobs is None:
                            so.logprobs = []
                        so.logprobs.append(e.logprob)
                    if on_token is not None:
                        on_token(ro, so, e.token)
                if e.finished:
                    so.finish_reason = e.finish_reason
                    ro.usage.num_cached_tokens = max(ro.usage.num_cached_tokens, e.prefix_hit_tokens)
                if e.request_finished and not ro.finished:
                    ro.finished = True
                    ro.cancelled = e.finish_reason == "abort"
                    in_flight -= 1
            submit_some()
        for ro, (_, _, sp) in zip(outs, todo):
            gen = 0
            for so in ro.outputs:
                gen += len(so.token_ids)
                so.text = self._decode(so.token_ids, sp.skip_special_tokens)
            ro.usage.num_generated_tokens = gen
            ro.usage.num_total_tokens = gen + ro.usage.num_prompt_tokens
            rid = ro.request_id
            if rid in t_first:
                ro.metrics = {"ttft_ms": (t_first[rid] - t_sub[rid]) * 1e3,
                              "e2e_ms": (t_last[rid] - t_sub[rid]) * 1e3,
                              "tpot_ms": (t_last[rid] - t_first[rid]) * 1e3 / (gen - 1) if gen > 1 else None}
        return outs

    # ------------------------------------------------------------------ control
    def beam_search(self, prompts, beam_width: int = 4, max_tokens: int = 16, length_penalty: float = 1.0,
                    ignore_eos: bool = False):
        """Beam search for every prompt (token-id lists or strings); returns, per prompt, the
        `beam_width` best continuations as `BeamOutput`s (xllm/pybind/llm.py beam_search)."""
        from ..engine.beam import beam_search
        outs = []
        for p in (prompts if isinstance(prompts, (list, tuple)) and not (prompts and isinstance(prompts[0], int)) else [prompts]):
            ids = self._encode(p) if isinstance(p, str) else [int(t) for t in p]
            res = beam_search(self.engine, ids, beam_width, max_tokens, length_penalty, ignore_eos=ignore_eos)
            if self.tokenizer is not None:
                for r in res:
                    r.text = self.tokenizer.decode(r.token_ids)
            outs.append(res)
        return outs

    def recommend(self, prompts, beam_width: int = 32, num_steps: int = 3, num_return: Optional[int] = None,
                  valid_items=None, prompt_embeds=None):
        """Generative recommendation: for every prompt (token-id list or string) the `beam_width` most likely
        items of `num_steps` tokens, best first, optionally restricted to `valid_items` (token tuples, or an
        `ItemTrie` built once from them and passed to every call).  All
        prompts run as one batch (engine/rec.py; the reference's rec backend)."""
        from ..engine.rec import ItemTrie, RecEngine
        if isinstance(prompts, str) or (prompts and isinstance(prompts[0], int)):
            prompts = [prompts]
        ids = [self._encode(p) if isinstance(p, str) else [int(t) for t in p] for p in prompts]
        if getattr(self, "_rec", None) is None:
            self._rec = RecEngine(self.engine)
        if isinstance(valid_items, ItemTrie):
            trie = valid_items
        else:
            trie = ItemTrie([tuple(i) for i in valid_items], self.engine.args.vocab_size) if valid_items else None
        return self._rec.generate(ids, beam_width=beam_width, num_steps=num_steps, num_return=num_return, trie=trie,
                                  prompt_embeds=prompt_embeds)

    def embed(self, prompts, pooling_params: Union[PoolingParams, List[PoolingParams], None] = None) -> List[EmbeddingOutput]:
        """Pooled embedding (final-norm hidden state of the last token, L2-normalised unless the
        pooling parameters say otherwise) of every prompt: xllm/pybind/llm.py:386-406."""
        from .embedding import embed_token_lists
        if isinstance(prompts, (str, torch.Tensor)) or (prompts and isinstance(prompts[0], int)):
            prompts = [prompts]
        pps = pooling_params if isinstance(pooling_params, list) else [pooling_params or PoolingParams()] * len(prompts)
        outs = []
        for p, pp in zip(prompts, pps):
            ids = self._encode(p)
            vec = embed_token_lists(self.engine, [ids], normalize=pp.normalize)[0]
            ro = RequestOutput(f"embed-{next(LLM._ids)}", p if isinstance(p, str) else None, ids, finished=True)
            ro.usage = Usage(len(ids), 0, len(ids), 0)
            outs.append(EmbeddingOutput(ro.prompt, EmbeddingOutputs(vec), ro.usage, ro))
        return outs

    def sample(self, prompts, selector, logprobs: int = 5) -> List[RequestOutput]:
        """For every occurrence of the `selector` token in a prompt, the `logprobs` most likely tokens
        to follow it (one forward pass per prompt, nothing is generated): xllm/pybind/llm.py:452-519.
        `selector` is a special-token string (needs a tokenizer), a {"type": "literal", "value": ...}
        dict, a token id, or one of those per prompt.  Each occurrence becomes one SequenceOutput
        whose `top_logprobs[0]` lists (token id, logprob) pairs, most likely first."""
        from .embedding import next_token_logprobs
        if isinstance(prompts, (str, torch.Tensor)) or (prompts and isinstance(prompts[0], int)):
            prompts = [prompts]
        sels = selector if isinstance(selector, (list, tuple)) else [selector] * len(prompts)
        if len(sels) != len(prompts):
            raise ValueError("selector count must match prompts count")
        outs = []
        for p, sel in zip(prompts, sels):
            ids = self._encode(p)
            if isinstance(sel, dict):
                if sel.get("type", "literal") != "literal" or not sel.get("value"):
                    raise ValueError("selector must be {'type': 'literal', 'value': <token>}")
                sel = sel["value"]
            if isinstance(sel, str):
                sid = self._encode(sel)
                if len(sid) != 1:
                    raise ValueError("selector.value must be a stable single special token")
                sel = sid[0]
            slots = [i for i, t in enumerate(ids) if t == int(sel)]
            ro = RequestOutput(f"sample-{next(LLM._ids)}", p if isinstance(p, str) else None, ids, finished=True)
            ro.usage = Usage(len(ids), 0, len(ids), 0)
            if slots:
                for j, alts in enumerate(next_token_logprobs(self.engine, ids, slots, logprobs)):
                    so = SequenceOutput(j, token_ids=[alts[0][0]], finish_reason="length", logprobs=[alts[0][1]],
                                        top_logprobs=[alts])
                    so.text = self._decode(so.token_ids)
                    ro.outputs.append(so)
            outs.append(ro)
        return outs

    def sleep(self, level: int = 1):
        """Release the KV cache (level 1) and also move the weights to host memory (level 2)."""
        self.engine.sleep(level)

    def wake_up(self):
        self.engine.wake_up()

    def update_weights(self, weights):
        self.engine.update_weights(weights)

    def stats(self):
        return self.engine.stats()
