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
