"""Pooled sentence embeddings from the decoder's final hidden states.

Parity: the `embed` task of the reference (LLM.embed in xllm/pybind/llm.py:347-420,
EmbedWorkerImpl, CausalLM::pooler): run the prompt once, take the last token's final-norm hidden
state, L2-normalise.
"""
from __future__ import annotations

from typing import List

import torch

from ..models.layers import AttentionMetadata


@torch.no_grad()
def hidden_states(engine, ids: List[int]) -> torch.Tensor:
    """Final-norm hidden states [T, H] of one prompt, computed on a private scratch cache."""
    model, dev = engine.model, engine.device
    bs = engine.cfg.block_size
    T = len(ids)
    n_blocks = (T + bs - 1) // bs
    nkv, d = model.num_kv_heads_local, model.head_dim
    kv = [(torch.zeros(n_blocks + 1, nkv, bs, d, dtype=engine.dtype, device=dev),
           torch.zeros(n_blocks + 1, nkv, bs, d, dtype=engine.dtype, device=dev))
          for _ in range(engine.args.num_hidden_layers)]
    meta = AttentionMetadata(
        n_decode=0, n_prefill=1, slots=torch.arange(bs, bs + T, dtype=torch.int32, device=dev),
        block_table=torch.arange(1, n_blocks + 1, dtype=torch.int32, device=dev)[None],
        kv_lens=torch.tensor([T], dtype=torch.int32, device=dev),
        cu_q=torch.tensor([0, T], dtype=torch.int32, device=dev), max_q_len=T, max_kv_len=T)
    if getattr(model, "needs_state", False):        # linear-attention layers: a scratch state slot, reset for this pass
        meta.state_slots = torch.tensor([model.state.n_slots - 1], dtype=torch.long, device=dev)
        meta.state_fresh, meta.seq_bounds = [True], [(0, T)]
    return model.forward(torch.tensor(ids, dtype=torch.int64, device=dev), torch.arange(T, device=dev), meta, kv)


@torch.no_grad()
def next_token_logprobs(engine, ids: List[int], positions: List[int], top_n: int = 5):
    """For each prompt position p: the top-n (token, logprob) pairs of the token FOLLOWING position p
    (the `/v1/sample` task of the reference, api_service sample service + proto/sample.proto)."""
    h = hidden_states(engine, ids)
    rows = torch.tensor(positions, dtype=torch.long, device=h.device)
    lp = torch.log_softmax(engine.model.logits(h[rows]).float(), dim=-1)
    top = torch.topk(lp, min(top_n, lp.shape[-1]), dim=-1)
    return [[(int(t), float(v)) for t, v in zip(ti, vi)] for ti, vi in zip(top.indices.tolist(), top.values.tolist())]


def rerank_scores(engine, query_ids: List[int], doc_ids: List[List[int]]) -> List[float]:
    """Cosine similarity of pooled embeddings (the `/v1/rerank` task, proto/rerank.proto)."""
    vecs = torch.tensor(embed_token_lists(engine, [query_ids] + doc_ids))
    return (vecs[1:] @ vecs[0]).tolist()


@torch.no_grad()
def embed_token_lists(engine, token_lists: List[List[int]], normalize: bool = True) -> List[List[float]]:
    model, dev = engine.model, engine.device
    bs = engine.cfg.block_size
    out = []
    for ids in token_lists:
        T = len(ids)
        n_blocks = (T + bs - 1) // bs
        nkv, d = model.num_kv_heads_local, model.head_dim
        # a private scratch cache: embedding requests never touch the serving KV pool
        kv = [(torch.zeros(n_blocks + 1, nkv, bs, d, dtype=engine.dtype, device=dev),
               torch.zeros(n_blocks + 1, nkv, bs, d, dtype=engine.dtype, device=dev))
              for _ in range(engine.args.num_hidden_layers)]
        meta = AttentionMetadata(
            n_decode=0, n_prefill=1, slots=torch.arange(bs, bs + T, dtype=torch.int32, device=dev),
            block_table=torch.arange(1, n_blocks + 1, dtype=torch.int32, device=dev)[None],
            kv_lens=torch.tensor([T], dtype=torch.int32, device=dev),
            cu_q=torch.tensor([0, T], dtype=torch.int32, device=dev), max_q_len=T, max_kv_len=T)
        h = model.forward(torch.tensor(ids, dtype=torch.int64, device=dev), torch.arange(T, device=dev), meta, kv)
        v = h[-1].float()
        if normalize:
            v = v / v.norm().clamp_min(1e-12)
        out.append(v.cpu().tolist())
    return out


class Embedding:
    """Offline embedding entry point (xllm/pybind/embedding.py:28): `Embedding(model, ...).embed(prompts)`."""

    def __init__(self, model: str = "tiny", **kw):
        from .llm import LLM
        kw.setdefault("enable_graph", False)
        self.llm = LLM(model, **kw)

    def embed(self, prompts, pooling_params=None):
        return self.llm.embed(prompts, pooling_params)
