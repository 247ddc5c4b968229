"""LLM engine: owns the model, the KV cache, the C++ scheduler and the step loop.

Capability parity with the reference's LLMEngine + the scheduler loop of LLMMaster
(xllm/core/distributed_runtime/llm_engine.cpp:188-222 init, 447-763 KV capacity + allocation,
1081-1232 step / overlap result fetch; llm_master.cpp:305-334).  One engine per process; with
tensor parallelism every rank runs the same deterministic scheduler on the same request stream,
so no per-step control traffic is needed — the only cross-rank traffic is the model's collectives.
"""
from __future__ import annotations

import os
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional

import numpy as np
import torch

from .. import _build  # noqa: F401  (keeps the build helper importable from the package)
from ..models import ModelArgs, create_model, load_model_args, preset
from ..parallel.state import ParallelState, single
from .model_runner import ModelRunner, StepOutput


def _rt():
    try:
        from .. import _rt as rt
    except ImportError:
        _build.build_runtime()
        from .. import _rt as rt
    return rt


@dataclass
class EngineConfig:
    model: str = "tiny"                 # preset name or a HuggingFace model directory
    dtype: str = "auto"
    device: str = "auto"
    block_size: int = 16
    num_blocks: int = 0                 # 0: derive from free memory
    max_memory_utilization: float = 0.9
    max_cache_size: int = 0             # bytes; 0: no explicit cap
    max_seqs_per_batch: int = 256
    max_tokens_per_batch: int = 8192
    max_model_len: int = 0              # 0: model's max_position_embeddings (capped at 32768)
    enable_prefix_cache: bool = True
    enable_chunked_prefill: bool = True
    max_tokens_per_chunk_for_prefill: int = -1
    policy: str = "prefill_first"
    priority_strategy: str = "fcfs"
    enable_schedule_overlap: bool = False
    enable_graph: bool = True
    graph_buckets: Optional[List[int]] = None
    seed: int = 0
    random_weights: bool = False
    load_format: str = "auto"
    dp_size: int = 1
    ep_size: int = 1
    num_speculative_tokens: int = 0
    host_kv_blocks: int = 0             # > 0: keep evicted prefix-cache blocks in host memory (second tier)
    host_blocks_factor: float = 0.0     # the same as a fraction of the device's block count (the reference's flag)
    enable_kvcache_store: bool = False  # third tier: blocks the host tier drops go to a store under kvcache_store_path
    kvcache_store_path: str = ""
    kvcache_store_bytes: int = 0        # 0: unbounded
    speculative_method: str = "ngram"   # drafter: "ngram" (suffix / prompt lookup, no draft model)
    draft_model: str = ""
    mla_latent_cache: bool = False      # MLA models: cache [c_kv | k_pe] rows (576 values per token) instead of per-head K/V
    activation_reserve_bytes: int = 0   # 0: estimated from max_tokens_per_batch
    fp8_execution: Optional[bool] = None  # block-scaled fp8 checkpoints: None / True = run the fp8 GEMMs, False = dequantise at load
    min_prefill_tokens: int = 0         # mixing policies: hold prompt chunks back until this many prompt tokens are pending
    max_prefill_wait_steps: int = 8     # ... or this many steps have passed
    max_running_seqs: int = 0           # cap on sequences holding KV / state at once; 0: no cap (state models: max_seqs_per_batch + 1)
    scheduler_type: str = "continuous"  # "continuous" | "zero_eviction" (never preempts: admits by simulation) | "fixed_steps" (waves)
    # latency-aware budgets: profile the model at start-up and cap the tokens of a step so that a step
    # stays under `max_global_ttft_ms` (prompt work) and the decode batch so that it stays under `max_global_tpot_ms`
    enable_xtensor: bool = False        # KV cache on the device's shared page pool: sleep gives the pages back, addresses (and CUDA graphs) survive
    enable_profile_token_budget: bool = False
    max_global_ttft_ms: float = 0.0
    max_global_tpot_ms: float = 0.0
    profile_max_prompt_length: int = 2048


_U64 = (1 << 64) - 1


def _mix64(a: int, b: int) -> int:
    """splitmix64 of (a, b): a well-spread 64-bit value for per-request random streams."""
    z = (a * 0x9E3779B97F4A7C15 + b * 0xBF58476D1CE4E5B9 + 0x94D049BB133111EB) & _U64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _U64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _U64
    return z ^ (z >> 31)


_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float16": torch.float16,
           "fp16": torch.float16, "float32": torch.float32, "fp32": torch.float32}


class LLMEngine:
    def __init__(self, cfg: EngineConfig, ps: Optional[ParallelState] = None, model=None,
                 model_args: Optional[ModelArgs] = None, hold_finished_blocks: bool = False, kv_allocator=None):
        self.cfg = cfg
        self.ps = ps or single()
        rt = _rt()
        self.rt = rt
        # ---- device / dtype
        if cfg.device == "auto":
            self.device = self.ps.device if self.ps.world_size > 1 else \
                torch.device("cuda", 0) if torch.cuda.is_available() else torch.device("cpu")
        else:
            self.device = torch.device(cfg.device)
        if self.device.type == "cuda":
            from ..utils.platform import bind_rank_to_device
            self.numa_cpus = bind_rank_to_device(self.device.index or 0)   # [] on one-node hosts or XLLM_NUMA_BIND=0
        if model_args is not None:
            self.args = model_args
        elif os.path.isdir(cfg.model):
            self.args = load_model_args(cfg.model)
        else:
            self.args = preset(cfg.model)
        if cfg.mla_latent_cache and self.args.kv_lora_rank:
            import dataclasses
            self.args = dataclasses.replace(self.args, mla_latent_cache=True)
        if self.args.quant_method == "fp8" and list(self.args.quant_block or [128, 128]) == [128, 128] \
                and cfg.fp8_execution is not False:
            import dataclasses
            self.args = dataclasses.replace(self.args, fp8_execution=True)
        if cfg.dtype == "auto":
            self.dtype = torch.bfloat16 if self.device.type == "cuda" else _DTYPES.get(self.args.dtype, torch.float32)
            if self.device.type == "cpu" and self.dtype == torch.bfloat16:
                self.dtype = torch.float32
        else:
            self.dtype = _DTYPES[cfg.dtype]
        # ---- fused tensor-parallel communicator (symmetric memory), before the model is built
        # An EAGLE-3 head reads whole hidden states of three target layers on every rank; the fused reductions
        # keep the residual stream sharded by rows between layers, so the target then reduces through the
        # process group instead (replicated activations) and the head itself runs replicated.
        eagle_tp = cfg.num_speculative_tokens > 0 and cfg.speculative_method == "eagle3" and self.ps.tp_size > 1
        if self.ps.tp_size > 1 and self.device.type == "cuda" and self.ps.comm is None and not eagle_tp:
            from ..parallel import symm
            tp = self.ps.tp_size
            shard = (self.args.vocab_size + tp - 1) // tp
            symm.attach(self.ps, max(cfg.max_tokens_per_batch, cfg.max_seqs_per_batch), self.args.hidden_size,
                        vocab_shard=shard if shard % 8 == 0 else 0, max_sample_rows=min(cfg.max_seqs_per_batch, 1024))
        # ---- model
        t0 = time.time()
        if model is not None:
            self.model = model
        else:
            self.model = create_model(self.args, self.dtype, self.device, self.ps)
            if os.path.isdir(cfg.model) and not cfg.random_weights:
                from ..utils.loader import dequant_fp8_stream, iterate_weights
                weights = iterate_weights(cfg.model)
                if self.args.quant_method == "fp8":
                    # layers that execute in fp8 take the e4m3 tensors and their block scales as they are;
                    # everything else (embeddings, router, kv_b_proj, ...) is dequantised while streaming
                    keep = {n[: -len("_scale_inv")] for n, _ in self.model.named_loaders() if n.endswith("weight_scale_inv")}
                    weights = dequant_fp8_stream(weights, keep, self.dtype)
                missing = self.model.load_weights(weights, strict=False)
                # a checkpoint that lacks tensors the model needs would otherwise run on zeros
                missing = [n for n in missing if not n.endswith("e_score_correction_bias")]
                # a weight that arrived in a wide type was quantised by its loader, which also set the scales
                gone = set(missing)
                missing = [n for n in missing if not (n.endswith("weight_scale_inv") and n[: -len("_scale_inv")] not in gone)]
                if missing and os.environ.get("XLLM_ALLOW_MISSING_WEIGHTS", "0") != "1":
                    raise KeyError(f"checkpoint {cfg.model} lacks {len(missing)} tensors the model needs, e.g. "
                                   f"{missing[:6]} (set XLLM_ALLOW_MISSING_WEIGHTS=1 to load anyway)")
            else:
                self.model.init_random(seed=cfg.seed)
        self.load_seconds = time.time() - t0
        # ---- KV capacity
        max_len = cfg.max_model_len or min(self.args.max_position_embeddings, 32768)
        self.max_model_len = max_len
        nkv = self.model.num_kv_heads_local
        per_block = ModelRunner.kv_bytes_per_block(self.args, nkv, cfg.block_size, self.dtype,
                                                   head_dim=getattr(self.model, "head_dim", None),
                                                   planes=int(getattr(self.model, "kv_planes", 2)))
        num_blocks = cfg.num_blocks or self._estimate_blocks(per_block)
        if self.ps.world_size > 1 and self.ps.tp_size > 1:
            # every tensor-parallel rank runs the same scheduler: they must agree on the size of the
            # cache, so the smallest estimate wins (free memory differs by a few MB between GPUs)
            import torch.distributed as dist
            t = torch.tensor([num_blocks], dtype=torch.int64, device=self.device if self.device.type == "cuda" else "cpu")
            dist.all_reduce(t, op=dist.ReduceOp.MIN, group=self.ps.tp_group)
            num_blocks = int(t.item())
        self.num_blocks = num_blocks
        self._kv_range = None
        if cfg.enable_xtensor and kv_allocator is None:
            from ..utils.xtensor import shared_pool
            pool = shared_pool(self.device)

            def kv_allocator(n_bytes, pool=pool):
                page = pool.page_bytes
                self._kv_range = pool.range((n_bytes + page - 1) // page * page)
                self._kv_range.ensure(n_bytes)
                self._kv_bytes = n_bytes
                return self._kv_range.tensor((n_bytes,), torch.uint8)
        self.runner = ModelRunner(self.model, cfg.block_size, num_blocks, cfg.max_seqs_per_batch,
                                  cfg.max_tokens_per_batch, max_len, self.device, self.dtype,
                                  enable_graph=cfg.enable_graph and bool(getattr(self.model, "supports_graph", True)),
                                  graph_buckets=cfg.graph_buckets, kv_allocator=kv_allocator)
        self.runner.overlap = cfg.enable_schedule_overlap
        if getattr(self.model, "needs_index_cache", False):
            self.model.alloc_index_cache(num_blocks, cfg.block_size)
        if getattr(self.model, "needs_state", False):
            # one state slot per sequence that can hold KV at the same time; the scheduler admits no
            # more than that (max_running_seqs below), so a slot is always free when one is needed
            self.state_slots = cfg.max_running_seqs or (cfg.max_seqs_per_batch + 1)
            self.model.alloc_state(self.state_slots)
            self.runner.meta_hook = self._state_hook
        # ---- scheduler
        sc = rt.SchedulerConfig()
        sc.max_tokens_per_batch = cfg.max_tokens_per_batch
        if self.ps is not single():
            self.ps.max_tokens_per_batch = cfg.max_tokens_per_batch   # sizes the expert-parallel receive buffers
        sc.max_seqs_per_batch = cfg.max_seqs_per_batch
        sc.enable_chunked_prefill = cfg.enable_chunked_prefill
        sc.max_tokens_per_chunk_for_prefill = cfg.max_tokens_per_chunk_for_prefill
        # linear-attention models carry per-sequence state that cached prompt tokens would not update
        sc.enable_prefix_cache = cfg.enable_prefix_cache and not getattr(self.model, "needs_state", False)
        sc.block_size = cfg.block_size
        sc.num_blocks = num_blocks
        sc.policy = cfg.policy
        if cfg.scheduler_type not in ("continuous", "zero_eviction", "fixed_steps"):
            raise ValueError(f"unknown scheduler_type {cfg.scheduler_type!r}")
        sc.admission = "" if cfg.scheduler_type == "continuous" else cfg.scheduler_type
        # sliding-window models (the window in every layer) give dead blocks back while they run
        if int(getattr(self.args, "sliding_window", 0) or 0) > 0 and not getattr(self.model, "mixed_window_layers", False):
            sc.sliding_window = int(self.args.sliding_window)
        sc.priority_strategy = cfg.priority_strategy
        sc.enable_schedule_overlap = cfg.enable_schedule_overlap
        sc.dp_size = 1  # one scheduler instance per DP replica
        sc.num_speculative_tokens = cfg.num_speculative_tokens
        sc.min_prefill_tokens = cfg.min_prefill_tokens
        sc.max_prefill_wait_steps = cfg.max_prefill_wait_steps
        sc.max_running_seqs = getattr(self, "state_slots", 0) or cfg.max_running_seqs
        sc.hold_finished_blocks = hold_finished_blocks   # PD disaggregation, prefill side
        self.scheduler = rt.Scheduler(sc)
        self._pending: Optional[StepOutput] = None
        self._req_counter = 0
        self.grammar = None
        self.asleep = 0
        self._host_weights = None
        self.dp_steps = self.fake_steps = 0
        self.mm = {}                 # request id -> MMInput of multimodal requests
        self.host_tier = None
        if cfg.host_kv_blocks <= 0 and cfg.host_blocks_factor > 0:
            cfg.host_kv_blocks = max(1, int(cfg.host_blocks_factor * self.runner.kv_caches[0][0].shape[0]))
        if cfg.host_kv_blocks > 0 and cfg.enable_prefix_cache:
            from .host_tier import HostKVTier
            store = None
            if cfg.enable_kvcache_store and cfg.kvcache_store_path:
                from .host_tier import DirectoryKVStore
                k0 = self.runner.kv_caches[0][0]
                # blocks are only interchangeable between engines with the same model, cache geometry and sharding
                geometry = (f"{self.args.model_type}-L{len(self.runner.kv_caches)}-{'x'.join(str(d) for d in k0.shape[1:])}-"
                            f"{str(k0.dtype).split('.')[-1]}-tp{self.ps.tp_size}r{self.ps.tp_rank}")
                store = DirectoryKVStore(cfg.kvcache_store_path, geometry, cfg.kvcache_store_bytes)
            self.host_tier = HostKVTier(self.runner.kv_caches, cfg.host_kv_blocks, self.scheduler.block_manager(0), rt,
                                        cfg.block_size, store=store)
        self.spec = None
        if cfg.num_speculative_tokens > 0:
            if cfg.enable_schedule_overlap:
                raise ValueError("speculative decoding needs enable_schedule_overlap=False: the number of tokens "
                                 "a step appends is only known after verification")
            from .speculative import SpecDecoder, make_drafter
            if getattr(self.model, "needs_state", False):
                raise ValueError("speculative decoding on a model with recurrent state needs a state rollback for "
                                 "rejected drafts, which is not implemented; run this model without it")
            if cfg.speculative_method == "mtp":
                from ..models.deepseek import MTPDraft
                self.mtp = MTPDraft(self.args, self.model, self.dtype, self.device, self.ps)
                self.mtp.init_random(seed=cfg.seed + 17)
                src = cfg.draft_model if (cfg.draft_model and os.path.isdir(cfg.draft_model)) else cfg.model
                if os.path.isdir(src) and not cfg.random_weights:
                    # the MTP layer ships inside the target's checkpoint (or in a directory exported from it)
                    from ..utils.loader import iterate_weights
                    self.mtp_tensors_loaded = self.mtp.load_from_checkpoint(iterate_weights(src), strict=False)
            elif cfg.speculative_method == "eagle3":
                from ..models.eagle3 import Eagle3Draft, aux_layer_ids
                self.model.aux_layers = aux_layer_ids(self.args.num_hidden_layers)
                self.eagle3 = Eagle3Draft(self.args, self.model, self.dtype, self.device, self.ps)
                self.eagle3.init_random(seed=cfg.seed + 19)
                if cfg.draft_model and os.path.isdir(cfg.draft_model):
                    from ..utils.loader import iterate_weights
                    self.eagle3.load_weights(iterate_weights(cfg.draft_model), strict=False)
            self.spec = SpecDecoder(self, make_drafter(cfg.speculative_method, cfg.num_speculative_tokens, self),
                                    cfg.num_speculative_tokens)
        self.profile_manager = None
        self.profiled_budget = None
        if cfg.enable_profile_token_budget and (cfg.max_global_ttft_ms > 0 or cfg.max_global_tpot_ms > 0):
            self._apply_profiled_budgets()
        from .fault import FaultPlan
        self.fault = FaultPlan.from_env(self.ps.rank)      # host-side fault hooks (XLLM_FAULT), None when unset
        self.steps = 0
        self.step_log: List[tuple] = []
        self.record_steps = False

    # ------------------------------------------------------------------ latency-aware budgets
    def _apply_profiled_budgets(self):
        """Times prompt and decode steps of this engine (ProfileManager), fits the step-time predictors
        and reconfigures the scheduler: tokens per step from the TTFT target, sequences per step from
        the TPOT target (xllm/core/scheduler/profile/profile_manager.cpp, the flags
        enable_profile_token_budget / max_global_ttft_ms / max_global_tpot_ms)."""
        from .profile_manager import ProfileManager
        cfg = self.cfg
        pm = ProfileManager.for_engine(self, repeats=2)
        top = max(128, min(cfg.profile_max_prompt_length, cfg.max_tokens_per_batch))
        sizes = sorted({max(16, top // 8), max(32, top // 4), max(64, top // 2), top})
        batches = sorted({1, max(2, cfg.max_seqs_per_batch // 8), max(4, cfg.max_seqs_per_batch // 2), cfg.max_seqs_per_batch})
        ctx = max(64, min(self.max_model_len // 2, 2048))
        pm.profile(prefill_tokens=sizes, decode_batches=batches, contexts=(ctx // 4, ctx))
        tokens = seqs = 0
        if cfg.max_global_ttft_ms > 0:
            tokens = pm.token_budget(cfg.max_global_ttft_ms / 1e3, hi=cfg.max_tokens_per_batch)
            tokens = max(tokens, cfg.block_size)                  # a step must be able to make progress
        if cfg.max_global_tpot_ms > 0:
            seqs = max(1, min(cfg.max_seqs_per_batch, pm.max_decode_batch(cfg.max_global_tpot_ms / 1e3, ctx,
                                                                         hi=cfg.max_seqs_per_batch)))
        self.scheduler.reconfigure("", int(tokens), int(seqs), 0)
        self.profile_manager = pm
        self.profiled_budget = {"max_tokens_per_batch": int(tokens) or cfg.max_tokens_per_batch,
                                "max_seqs_per_batch": int(seqs) or cfg.max_seqs_per_batch}

    # ------------------------------------------------------------------ capacity
    def _estimate_blocks(self, per_block: int) -> int:
        """KV blocks that fit next to the weights: (free memory x utilisation - activation reserve)
        / bytes per block (the reference profiles the same quantity: kv_cache_estimation.cpp)."""
        cfg = self.cfg
        if self.device.type != "cuda":
            return 4096
        free, total = torch.cuda.mem_get_info(self.device)
        used_other = total - free
        budget = int(total * cfg.max_memory_utilization) - used_other
        a = self.args
        tp = self.ps.tp_size
        T = cfg.max_tokens_per_batch
        # widest live activations of one step: qkv + gate_up + a few hidden-size buffers + logits
        inter = max(a.intermediate_size, a.moe_intermediate_size * max(a.num_experts_per_tok, 1)) // tp
        act = T * (2 * inter + 6 * a.hidden_size + (a.num_attention_heads + 2 * a.num_key_value_heads) * a.head_dim // tp) * 2 * 2
        act += cfg.max_seqs_per_batch * a.vocab_size * 4 * 2
        reserve = cfg.activation_reserve_bytes or (act + (2 << 30))
        budget -= reserve
        if cfg.max_cache_size > 0:
            budget = min(budget, cfg.max_cache_size)
        n = budget // per_block
        if n < 8:
            raise RuntimeError(f"not enough device memory for a KV cache ({budget} bytes left)")
        return int(n)

    # ------------------------------------------------------------------ intake
    def add_request(self, request_id: str, prompt_token_ids, temperature=0.0, top_p=1.0, top_k=-1,
                    max_tokens=16, ignore_eos=False, stop_token_ids=None, stop_sequences=None,
                    frequency_penalty=0.0, presence_penalty=0.0, repetition_penalty=1.0,
                    logprobs=False, top_logprobs=0, seed=None, n=1, priority=0, deadline=0.0,
                    offline=False, stream=False, eos_token_id=None, json_object=False, mm=None) -> bool:
        rt = self.rt
        sp = rt.SamplingParams()
        sp.temperature = float(temperature)
        sp.top_p = float(top_p)
        sp.top_k = int(top_k)
        sp.frequency_penalty = float(frequency_penalty)
        sp.presence_penalty = float(presence_penalty)
        sp.repetition_penalty = float(repetition_penalty)
        sp.logprobs = bool(logprobs)
        sp.top_logprobs = int(top_logprobs)
        # without an explicit seed every request gets its own random stream, derived from the
        # engine seed and the arrival order (the same on every tensor-parallel rank)
        self._req_counter += 1
        sp.seed = int(seed) & _U64 if seed is not None else _mix64(self.cfg.seed, self._req_counter)
        st = rt.StoppingParams()
        st.max_tokens = int(max_tokens)
        st.max_context_len = int(self.max_model_len)
        st.eos_token_id = int(self.args.eos_token_id if eos_token_id is None else eos_token_id)
        st.ignore_eos = bool(ignore_eos)
        extra = [t for t in self.args.stop_token_ids if t != st.eos_token_id]
        st.stop_token_ids = list(stop_token_ids or []) + extra
        st.stop_sequences = [list(s) for s in (stop_sequences or [])]
        toks = [int(t) for t in prompt_token_ids]
        if len(toks) >= self.max_model_len:
            return False
        if self.host_tier is not None:
            self.host_tier.prefetch(toks)
        if json_object:
            if self.grammar is None:
                raise ValueError("json_object needs set_grammar_vocab() (the token strings of the tokenizer)")
            if self.cfg.enable_schedule_overlap:
                raise ValueError("constrained decoding needs enable_schedule_overlap=False")
            self.grammar.start(request_id)
        if mm is not None:
            if not hasattr(self.model, "mrope_section"):
                raise ValueError("this model takes no multimodal input")
            self.mm[request_id] = mm
            self.runner.mm_hook = self._mm_hook
            return self.scheduler.add_request(request_id, toks, sp, st, n, priority, deadline, offline, stream,
                                              int(mm.hash_key) & ((1 << 63) - 1))
        return self.scheduler.add_request(request_id, toks, sp, st, n, priority, deadline, offline, stream)

    def set_grammar_vocab(self, token_text, eos_token_id=None, top_n: int = 64):
        """Enable `json_object=True` requests: `token_text[i]` is the text of token i."""
        from .grammar import GrammarFilter
        self.grammar = GrammarFilter(token_text, top_n, self.args.eos_token_id if eos_token_id is None else eos_token_id)
        self.runner.logits_hook = self._grammar_hook

    # ------------------------------------------------------------------ linear-attention state slots
    def _state_hook(self, batch, meta):
        """Gives every sequence of the batch its state slot and marks the ones that start at
        position 0 (new, or recomputed after a preemption) so that their state is reset."""
        st = self.model.state
        n = batch.n_decode + batch.n_prefill
        cu, pos = np.asarray(batch.cu_q), np.asarray(batch.positions)
        seq_ids = np.asarray(batch.seq_ids)
        slots, fresh, bounds = [], [], []
        for i in range(n):
            a, b = int(cu[i]), int(cu[i + 1])
            slots.append(st.slot_of(int(seq_ids[i])))
            fresh.append(int(pos[a]) == 0)
            bounds.append((a, b))
        meta.state_slots = torch.tensor(slots, dtype=torch.long, device=self.device)
        meta.state_fresh, meta.seq_bounds = fresh, bounds

    # ------------------------------------------------------------------ multimodal inputs
    def _mm_hook(self, batch):
        """Per-step inputs of multimodal requests: the image embeddings of the placeholder rows in
        this step's prompt chunks and the 3-axis rotary table of all rows.  None when no sequence of
        the batch is multimodal."""
        if not self.mm:
            return None
        import bisect

        import numpy as np

        from ..multimodal.image import mrope_table
        nseq = batch.n_decode + batch.n_prefill
        rids = [batch.request_id(i) for i in range(nseq)]
        if not any(r in self.mm for r in rids):
            return None
        cu = np.asarray(batch.cu_q)
        pos_h = np.asarray(batch.positions).astype(np.int64)
        T = int(cu[nseq])
        pos3 = torch.from_numpy(pos_h[:T]).repeat(3, 1)
        rows, vals = [], []
        for i, rid in enumerate(rids):
            m = self.mm.get(rid)
            if m is None:
                continue
            a, b = int(cu[i]), int(cu[i + 1])
            p0 = int(pos_h[a])
            L = m.mrope.shape[1]
            for r in range(a, b):
                p = p0 + (r - a)
                pos3[:, r] = m.mrope[:, p] if p < L else p + m.delta
            lo = bisect.bisect_left(m.positions, p0)
            hi = bisect.bisect_left(m.positions, p0 + (b - a))
            if hi > lo:
                rows.extend(a + (m.positions[j] - p0) for j in range(lo, hi))
                vals.append(m.embeds[lo:hi])
        dev = self.runner.device
        table = mrope_table(pos3.to(dev), self.args.rotary_dim, self.args.rope_theta, self.model.mrope_section,
                            interleaved=bool(getattr(self.model, "mrope_interleaved", False)))
        embeds = None
        if rows:
            embeds = (torch.tensor(rows, dtype=torch.long, device=dev), torch.cat(vals).to(dev))
        return embeds, table, torch.arange(T, dtype=torch.int64, device=dev)

    def _grammar_hook(self, batch, logits):
        if not self.grammar.state:
            return
        seq_of_row = batch.sample_seq
        for r in range(int(batch.n_samples)):
            rid = batch.request_id(int(seq_of_row[r]))
            if rid in self.grammar.state:
                self.grammar.filter_row(rid, logits[r])

    def _grammar_advance(self, events):
        if self.grammar is None or not self.grammar.state:
            return
        for ev in events:
            if ev.request_id in self.grammar.state:
                if ev.token >= 0:
                    self.grammar.advance(ev.request_id, int(ev.token))
                if ev.request_finished:
                    self.grammar.forget(ev.request_id)

    def abort(self, request_id: str) -> bool:
        return self.scheduler.abort_request(request_id)

    def has_unfinished(self) -> bool:
        return self.scheduler.has_unfinished() or self._pending is not None

    # ------------------------------------------------------------------ stepping
    def _finish(self, out: StepOutput):
        ids, lp = out.wait()
        top = out.top_host()
        if top is not None:
            self.scheduler.set_top_logprobs(out.batch_id, top[0], top[1])
        return self.scheduler.process_output(out.batch_id, ids, lp)

    def step(self):
        """One scheduler iteration. Returns the list of OutputEvent produced by it."""
        events = []
        if self.fault is not None:
            comm = getattr(self.ps, "comm", None)
            nvls = self.ps.world_size > 1 and self.device.type == "cuda" and os.environ.get("NCCL_NVLS_ENABLE", "1") != "0"
            self.fault.before_step(self.steps, multicast_bound=bool(getattr(comm, "mc_base", 0)) or nvls)
        batches = self.scheduler.schedule()
        batch = batches[0] if batches else None
        if self.ps.dp_size > 1 and self.ps.ep_size > 1:
            self._dp_lockstep(batch)
        if self.host_tier is not None:
            self.host_tier.save_evicted()   # before this step's kernels overwrite the evicted blocks
        if self.cfg.enable_schedule_overlap:
            new = self.runner.execute(batch) if batch is not None else None
            if self._pending is not None:
                events = self._finish(self._pending)
            self._pending = new
        else:
            if batch is not None and self.spec is not None and batch.n_prefill == 0 and batch.n_decode > 0 \
                    and self.spec.can_verify(batch, self.runner):
                flat, counts, lp = self.spec.step(batch)
                events = self.scheduler.process_output_multi(batch.batch_id, flat, counts, lp)
            elif batch is not None:
                out = self.runner.execute(batch)
                if self.spec is not None:
                    ids, lp = out.wait()
                    self.spec.drafter.after_execute(batch, ids)
                    events = self.scheduler.process_output(out.batch_id, ids, lp)
                else:
                    events = self._finish(out)
            else:
                events = self.scheduler.take_pending_events()
        self._grammar_advance(events)
        if getattr(self.model, "needs_state", False):
            for ev in events:
                if ev.finished and ev.seq_id >= 0:
                    self.model.state.release(int(ev.seq_id))
            for sid in self.scheduler.take_preempted():
                self.model.state.release(int(sid))     # the state is rebuilt from position 0 anyway
        if self.mm:
            for ev in events:
                if ev.request_finished:
                    self.mm.pop(ev.request_id, None)
        if batch is not None:
            self.steps += 1
            if self.record_steps:
                self.step_log.append((batch.n_decode, batch.n_prefill, batch.n_tokens))
        return events

    def drain(self):
        events = []
        if self._pending is not None:
            events = self._finish(self._pending)
            self._pending = None
        return events

    def run_until_done(self, on_event: Optional[Callable] = None, max_steps: int = 0):
        n = 0
        while self.has_unfinished():
            evs = self.step()
            if on_event is not None:
                for e in evs:
                    on_event(e)
            n += 1
            if max_steps and n >= max_steps:
                break
        return n

    # ------------------------------------------------------------------ control (RL-style)
    # ------------------------------------------------------------------ data-parallel attention
    def _dp_lockstep(self, batch):
        """With data-parallel attention and expert parallelism every rank has its own requests but the
        MoE layers are collective: a rank without a batch this step runs a one-token dummy forward
        whenever any other rank runs a real one, so that the collectives pair up (the reference's
        fake inputs for empty DP ranks, llm_engine.cpp prepare_inputs + dp_global_token_nums)."""
        import torch.distributed as dist
        flag = torch.tensor([1 if batch is not None else 0], dtype=torch.int32,
                            device=self.device if self.device.type == "cuda" else "cpu")
        dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=self.ps.world_group)
        self.dp_steps += int(flag.item())
        if batch is None and int(flag.item()) > 0:
            self._fake_forward()

    def dp_has_unfinished(self) -> bool:
        """True while ANY data-parallel rank still has work (ranks leave the serving loop together)."""
        import torch.distributed as dist
        flag = torch.tensor([1 if self.has_unfinished() else 0], dtype=torch.int32,
                            device=self.device if self.device.type == "cuda" else "cpu")
        dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=self.ps.world_group)
        return bool(flag.item())

    @torch.no_grad()
    def _fake_forward(self):
        from ..models.layers import AttentionMetadata
        dev = self.device
        meta = AttentionMetadata(
            n_decode=1, n_prefill=0, slots=torch.full((1,), -1, dtype=torch.int32, device=dev),
            block_table=torch.zeros((1, 8), dtype=torch.int32, device=dev),
            kv_lens=torch.zeros(1, dtype=torch.int32, device=dev), cu_q=torch.tensor([0, 1], dtype=torch.int32, device=dev),
            max_q_len=1, max_kv_len=0)
        self.model.forward(torch.zeros(1, dtype=torch.int64, device=dev), torch.zeros(1, dtype=torch.int64, device=dev),
                           meta, self.runner.kv_caches)
        self.fake_steps += 1

    def pause(self, mode="KEEP"):
        self.drain()
        self.scheduler.pause(getattr(self.rt.PauseMode, mode))

    def resume(self):
        self.scheduler.resume()

    # ------------------------------------------------------------------ sleep / wake-up
    def sleep(self, level: int = 1):
        """Give the device memory back while the instance is idle (the reference's sleep / wakeup /
        fork_master on its VMM page pool, llm_master.cpp:640-700, framework/xtensor/*).

        level 1: running sequences are preempted (they re-prefill after wake-up), the KV cache
        tensors are released; level 2: the weights move to pinned host memory as well.  The cached
        CUDA graphs reference the old cache tensors and are dropped."""
        if self.asleep:
            return
        self.pause("KEEP")
        self.reset_prefix_cache()
        r = self.runner
        if self._kv_range is not None:
            # page-pool cache: the physical pages go back to the pool, the tensors keep their addresses,
            # so the captured graphs stay valid and wake-up only maps pages again
            if self.device.type == "cuda":
                torch.cuda.synchronize()
            self._kv_range.release_all()
            self._kv_shapes = None
            self._host_weights = None
            if level >= 2:
                self._host_weights = []
                for name, t in self.model.named_params():
                    h = torch.empty(t.shape, dtype=t.dtype, pin_memory=t.is_cuda)
                    h.copy_(t)
                    self._host_weights.append((t, h, t.shape))
                    t.set_(torch.empty(0, dtype=t.dtype, device=t.device))
                if self.device.type == "cuda":
                    torch.cuda.synchronize()
                    torch.cuda.empty_cache()
            self.asleep = level
            return
        self._kv_shapes = [(k.shape, v.shape, k.dtype, k.device) for k, v in r.kv_caches]
        r.graphs.clear()
        r.graph_in.clear()
        r.graph_out.clear()
        r.graph_off.clear()
        r.graph_pool = None
        for i in range(len(r.kv_caches)):
            r.kv_caches[i] = None
        if getattr(self.spec, "drafter", None) is not None and hasattr(self.spec.drafter, "kv"):
            self.spec.drafter.kv = None
        self._host_weights = None
        if level >= 2:
            self._host_weights = []
            for name, t in self.model.named_params():
                h = torch.empty(t.shape, dtype=t.dtype, pin_memory=t.is_cuda)
                h.copy_(t)
                self._host_weights.append((t, h, t.shape))
                t.set_(torch.empty(0, dtype=t.dtype, device=t.device))
        if self.device.type == "cuda":
            torch.cuda.synchronize()
            torch.cuda.empty_cache()
        self.asleep = level

    def wake_up(self):
        if not self.asleep:
            return
        if self._host_weights is not None:
            for t, h, shape in self._host_weights:
                t.set_(torch.empty(shape, dtype=t.dtype, device=self.device))
                t.copy_(h, non_blocking=True)
            self._host_weights = None
        r = self.runner
        if self._kv_range is not None:
            self._kv_range.ensure(self._kv_bytes)
            r.kv_tensor.zero_()
            self.asleep = 0
            self.resume()
            return
        for i, (ks, vs, dt, dev) in enumerate(self._kv_shapes):
            r.kv_caches[i] = (torch.zeros(ks, dtype=dt, device=dev), torch.zeros(vs, dtype=dt, device=dev))
        if getattr(self.spec, "drafter", None) is not None and hasattr(self.spec.drafter, "kv"):
            k0, v0 = r.kv_caches[0]
            self.spec.drafter.kv = (torch.zeros_like(k0), torch.zeros_like(v0))
        if self.host_tier is not None:
            self.host_tier.kv = r.kv_caches
        self.asleep = 0
        self.resume()

    def reset_prefix_cache(self):
        self.scheduler.reset_prefix_cache()

    def update_weights(self, weights):
        """Hot-swap weights from an iterable of (name, tensor); the prefix cache is dropped because
        cached KV was computed with the old weights (the reference resets it on wake-up,
        llm_master.cpp:660-671)."""
        self.drain()
        self.model.load_weights(weights, strict=False)
        self.reset_prefix_cache()

    def stats(self) -> Dict[str, float]:
        bs = self.scheduler.block_stats(0)
        return {
            "steps": self.steps,
            "num_waiting": self.scheduler.num_waiting,
            "num_running": self.scheduler.num_running,
            "kv_utilization": self.scheduler.kv_utilization(0),
            "num_blocks": bs.num_blocks,
            "prefix_hit_blocks": bs.match_hits_blocks,
            "prefix_query_blocks": bs.match_query_blocks,
            "preemptions": self.scheduler.num_preemptions,
            "graph_replays": self.runner.graph_replays,
            "h2d_bytes": self.runner.h2d_bytes,
            "d2h_bytes": self.runner.d2h_bytes,
            "spec_acceptance_rate": self.spec.acceptance_rate if self.spec is not None else 0.0,
        }
