"""`python -m xllm_b200.serve --model <dir> [flags]` — start the OpenAI-compatible server.

Counterpart of the reference's `xllm` binary entry (xllm/xllm.cpp:585-625: parse flags, load the
optional JSON config, validate, build options, create the master and the HTTP server) and of its
`xllm serve` launcher (xllm/launch_server.py).  Flag names and defaults are the reference's; with
`--nnodes N` the process joins an N-rank tensor-parallel job (one process per GPU; rank 0 hosts the
HTTP server and broadcasts each step's new requests to the other ranks).
"""
from __future__ import annotations

import os
import sys


def build_engine_config(flags):
    """The reference's flag names -> `EngineConfig` (xllm/xllm.cpp builds its `Options` the same way)."""
    from .engine.llm_engine import EngineConfig
    algo = (flags.get("speculative_algorithm") or "").lower()
    n_spec = flags.get_int("num_speculative_tokens")
    method = {"mtp": "mtp", "eagle3": "eagle3", "suffix": "ngram", "ngram": "ngram", "draft": "draft"}.get(algo, "ngram")
    if n_spec > 0 and flags.get("draft_model") and algo in ("", "mtp") and not flags.is_set("speculative_algorithm"):
        method = "draft"
    scheduler = "continuous"
    if flags.get_bool("use_zero_evict"):
        scheduler = "zero_eviction"
    elif flags.get("backend") == "rec":
        scheduler = "fixed_steps"
    cfg = EngineConfig(
        model=flags.get("model") or "tiny", dtype="auto", device=("auto" if flags.get("devices") == "auto" else flags.get("devices")),
        block_size=flags.get_int("block_size"), max_memory_utilization=flags.get_double("max_memory_utilization"),
        max_cache_size=flags.get_int("max_cache_size"), max_seqs_per_batch=flags.get_int("max_seqs_per_batch"),
        max_tokens_per_batch=flags.get_int("max_tokens_per_batch"), max_model_len=flags.get_int("max_model_len"),
        enable_prefix_cache=flags.get_bool("enable_prefix_cache"),
        enable_chunked_prefill=flags.get_bool("enable_chunked_prefill"),
        max_tokens_per_chunk_for_prefill=flags.get_int("max_tokens_per_chunk_for_prefill"),
        policy=flags.get("scheduler_policy"), priority_strategy=flags.get("priority_strategy"),
        enable_schedule_overlap=flags.get_bool("enable_schedule_overlap"),
        enable_graph=flags.get_bool("enable_cuda_graph") or flags.get_bool("enable_graph"),
        random_weights=flags.get_bool("random_weights"),
        dp_size=flags.get_int("dp_size"), ep_size=flags.get_int("ep_size"),
        num_speculative_tokens=n_spec, speculative_method=method, draft_model=flags.get("draft_model"),
        scheduler_type=scheduler, enable_xtensor=flags.get_bool("enable_xtensor"),
        enable_profile_token_budget=flags.get_bool("enable_profile_token_budget") or flags.get_bool("enable_latency_aware_schedule"),
        max_global_ttft_ms=float(flags.get_int("max_global_ttft_ms")), max_global_tpot_ms=float(flags.get_int("max_global_tpot_ms")),
        host_blocks_factor=flags.get_double("host_blocks_factor"),
        enable_kvcache_store=flags.get_bool("enable_kvcache_store"),
        # the store of this build is a directory shared by the instances of a node (a tmpfs or NVMe mount)
        kvcache_store_path=os.environ.get("XLLM_KVCACHE_STORE_PATH", "") or
        (flags.get("store_master_server_address") if os.path.isabs(flags.get("store_master_server_address") or "") else ""))
    if cfg.enable_schedule_overlap and n_spec > 0:
        cfg.enable_schedule_overlap = False          # as the reference: speculation turns the overlap off
    return cfg


def main(argv=None):
    from . import _rt
    flags = _rt.FlagRegistry()
    try:
        flags.parse_args(list(sys.argv[1:] if argv is None else argv))
    except ValueError as e:
        print(f"error: {e}", file=sys.stderr)
        return 2
    if flags.help_requested():
        print(flags.help())
        return 0
    problems = flags.validate()
    if problems:
        for p in problems:
            print(f"error: {p}", file=sys.stderr)
        return 2
    if flags.get_bool("enable_dump_config_json"):
        with open(flags.get("dump_config_json_file"), "w") as f:
            f.write(flags.to_json())
    os.environ.setdefault("XLLM_GEMM", "auto" if flags.get("gemm_backend") == "tcgen05" else flags.get("gemm_backend"))
    os.environ.setdefault("XLLM_TP_COMM", flags.get("tp_comm"))
    from .api.server import ApiServer
    from .engine.llm_engine import LLMEngine
    from .parallel.state import init_parallel
    from .utils.tokenizer import load_tokenizer

    nnodes = flags.get_int("nnodes")
    ps = None
    if nnodes > 1:
        addr = flags.get("master_node_addr")
        host, _, port = addr.partition(":")
        os.environ.setdefault("MASTER_ADDR", host or "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", port or "19888")
        os.environ.setdefault("WORLD_SIZE", str(nnodes))
        os.environ.setdefault("RANK", str(flags.get_int("node_rank")))
        os.environ.setdefault("LOCAL_RANK", str(flags.get_int("node_rank")))
        ps = init_parallel(dp_size=flags.get_int("dp_size"), ep_size=flags.get_int("ep_size"))
    ecfg = build_engine_config(flags)
    model = flags.get("model")
    if (flags.get("backend") or "") == "dit" and model and os.path.exists(os.path.join(model, "model_index.json")):
        # the text engine is not what a diffusion instance serves: a placeholder keeps the server's plumbing uniform
        ecfg.model, ecfg.device, ecfg.num_blocks, ecfg.enable_graph = "tiny", "cpu", 16, False
    engine = LLMEngine(ecfg, ps=ps)
    tok = load_tokenizer(model) if model and os.path.isdir(model) else None
    name = flags.get("model_id") or (os.path.basename(model.rstrip("/")) if model else "xllm_b200")
    if ps is not None and ps.rank != 0:
        from .engine.replica import follow_rank0
        return follow_rank0(engine, ps)
    srv = ApiServer(engine, tok, model_name=name, host=flags.get("host"), port=flags.get_int("port"),
                    max_concurrent_requests=flags.get_int("max_concurrent_requests"),
                    tool_call_parser=flags.get("tool_call_parser"), reasoning_parser=flags.get("reasoning_parser"),
                    backend=flags.get("backend") or "llm")
    if ps is not None:
        from .engine.replica import lead_ranks
        lead_ranks(srv, ps)
    if (flags.get("backend") or "") == "dit" and model and os.path.exists(os.path.join(model, "model_index.json")):
        # a diffusion checkpoint directory: /v1/images/generations runs its pipeline (the DiT master of the reference)
        from .dit.pipeline import FluxImagePipeline
        import torch
        on_gpu = torch.cuda.is_available()
        srv.image_pipeline = FluxImagePipeline.from_pretrained(model, torch.bfloat16 if on_gpu else torch.float32,
                                                               "cuda:0" if on_gpu else "cpu")
    etcd = None
    if flags.get("etcd_addr"):
        # discovery as in the reference: the instance writes itself under a leased key that a keepalive
        # thread renews; when the process dies the key expires and the routing layer drops the instance
        import json as _json
        from .engine.service_client import EtcdKV
        role = flags.get("instance_role") or "DEFAULT"
        ns = flags.get("etcd_namespace").strip("/")
        key = "/".join(x for x in (ns, "XLLM", role, f"{flags.get('host') or '127.0.0.1'}:{srv.port}") if x)
        record = _json.dumps({"name": key.rsplit("/", 1)[-1], "type": role, "dp_size": flags.get_int("dp_size"),
                              "model": name})
        etcd = EtcdKV(flags.get("etcd_addr").split(",")[0], lease_s=float(flags.get_int("etcd_ttl")))
        etcd.set(key, record)
        etcd.start_keepalive(on_lost=lambda: etcd.set(key, record))
    print(f"xllm_b200 serving {name} on port {srv.port}", flush=True)
    try:
        srv.serve_forever()
    except KeyboardInterrupt:
        srv.shutdown()
    if etcd is not None:
        etcd.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
