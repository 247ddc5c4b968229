"""Beam search over the paged KV cache.

Parity: `LLM.beam_search` and the beam bookkeeping of `SequencesGroup` / the beam-search kernels
(xllm/pybind/llm.py:82-519, core/framework/request/sequences_group.*, kernels/cuda/beam_search*.cu):
per step every live beam proposes its best continuations, the global top `beam_width` survive, and
the KV cache follows the surviving parents.

Here the cache does not move: a beam is a block table.  Full blocks are immutable and shared
between beams by reference count; only the partially filled tail block of a parent is copied when a
second child branches off it (copy-on-write), so a step costs at most one block copy per beam instead
of a reorder of the whole cache.  Blocks come from the engine's own block manager, so beam search
coexists with the serving scheduler on one cache.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from ..models.layers import AttentionMetadata


@dataclass
class Beam:
    tokens: List[int]
    score: float                 # sum of token log-probabilities
    blocks: List[int]
    finished: bool = False


@dataclass
class BeamOutput:
    token_ids: List[int]
    cumulative_logprob: float
    score: float                 # length-normalised
    finish_reason: str = "length"


class _Blocks:
    """Reference counts on top of the engine's block manager."""

    def __init__(self, bm):
        self.bm = bm
        self.ref: Dict[int, int] = {}

    def new(self) -> int:
        got = self.bm.allocate(1)
        if not got:
            raise RuntimeError("beam search: out of KV blocks")
        self.ref[got[0]] = 1
        return got[0]

    def share(self, b: int):
        self.ref[b] += 1

    def drop(self, blocks):
        for b in blocks:
            self.ref[b] -= 1
            if self.ref[b] == 0:
                del self.ref[b]
                self.bm.free([b])


def beam_search(engine, prompt_token_ids, beam_width: int = 4, max_tokens: int = 16, length_penalty: float = 1.0,
                eos_token_id: Optional[int] = None, ignore_eos: bool = False, num_return: Optional[int] = None
                ) -> List[BeamOutput]:
    runner = engine.runner
    model, kv, dev = runner.model, runner.kv_caches, runner.device
    bs = engine.cfg.block_size
    eos = engine.args.eos_token_id if eos_token_id is None else eos_token_id
    W = beam_width
    pool = _Blocks(engine.scheduler.block_manager(0))
    prompt = [int(t) for t in prompt_token_ids]
    L = len(prompt)

    def forward(tokens, positions, slots, tables, kv_lens, q_lens):
        B = len(tables)
        width = max(len(t) for t in tables)
        bt = torch.zeros((B, width), dtype=torch.int32)
        for i, t in enumerate(tables):
            bt[i, : len(t)] = torch.tensor(t, dtype=torch.int32)
        cu = [0]
        for q in q_lens:
            cu.append(cu[-1] + q)
        decode = all(q == 1 for q in q_lens)
        meta = AttentionMetadata(
            n_decode=B if decode else 0, n_prefill=0 if decode else B,
            slots=torch.tensor(slots, dtype=torch.int32, device=dev), block_table=bt.to(dev),
            kv_lens=torch.tensor(kv_lens, dtype=torch.int32, device=dev),
            cu_q=torch.tensor(cu, dtype=torch.int32, device=dev), max_q_len=max(q_lens), max_kv_len=max(kv_lens))
        h = model.forward(torch.tensor(tokens, dtype=torch.int64, device=dev),
                          torch.tensor(positions, dtype=torch.int64, device=dev), meta, kv)
        last = torch.tensor([c - 1 for c in cu[1:]], dtype=torch.long, device=dev)
        return model.logits(h[last])           # raw logits: the selection kernels normalise the rows they keep

    # ---- prompt once
    blocks = [pool.new() for _ in range((L + bs - 1) // bs)]
    slots = [blocks[p // bs] * bs + p % bs for p in range(L)]
    from ..ops import select
    logits = forward(prompt, list(range(L)), slots, [blocks], [L], [L])[:1]
    if logits.dtype not in (torch.bfloat16, torch.float32):
        logits = logits.float()
    V = logits.shape[1]
    n_cand = min(2 * W, V)
    tv, ti = select.topk(logits, n_cand, normalize=True)
    top_vals, top_ids = tv[0].tolist(), ti[0].tolist()
    beams: List[Beam] = []
    done: List[BeamOutput] = []

    def norm(score, n):
        return score / (max(n, 1) ** length_penalty)

    def fork(parent_blocks, n_tokens, first_child):
        """Block table for a child that will write position n_tokens (the parent holds n_tokens KV)."""
        full = n_tokens // bs
        tbl = list(parent_blocks[:full])
        for b in tbl:
            pool.share(b)
        if n_tokens % bs:
            tail = parent_blocks[full]
            if first_child:
                pool.share(tail)
                tbl.append(tail)
            else:
                nb = pool.new()
                for k, v in kv:
                    k[nb] = k[tail]
                    v[nb] = v[tail]
                tbl.append(nb)
        else:
            tbl.append(pool.new())
        return tbl

    for tok, sc in zip(top_ids, top_vals):
        if tok == eos and not ignore_eos:
            done.append(BeamOutput([tok], sc, norm(sc, 1), "stop"))
            continue
        if len(beams) < W:
            beams.append(Beam([tok], sc, fork(blocks, L, first_child=not beams)))
    pool.drop(blocks)

    # ---- decode
    for step in range(1, max_tokens):
        if not beams:
            break
        n_ctx = L + step                      # tokens whose KV exists after this step
        toks = [b.tokens[-1] for b in beams]
        pos = [n_ctx - 1] * len(beams)
        slots = [b.blocks[(n_ctx - 1) // bs] * bs + (n_ctx - 1) % bs for b in beams]
        logits = forward(toks, pos, slots, [b.blocks for b in beams], [n_ctx] * len(beams), [1] * len(beams))
        if logits.dtype not in (torch.bfloat16, torch.float32):
            logits = logits.float()
        cum = torch.tensor([b.score for b in beams], dtype=torch.float32, device=logits.device)
        # every beam's 2W best continuations, then the 2W best of all of them: one device->host read
        t_tok, t_par, t_sc = select.beam_topk(logits, cum, min(2 * W, logits.numel()))
        t_tok, t_par, t_sc = t_tok.tolist(), t_par.tolist(), t_sc.tolist()
        new: List[Beam] = []
        used_parent = set()
        for tok, p, sc in zip(t_tok, t_par, t_sc):
            seq = beams[p].tokens + [tok]
            if tok == eos and not ignore_eos:
                done.append(BeamOutput(seq, sc, norm(sc, len(seq)), "stop"))
                continue
            if len(new) < W:
                new.append(Beam(seq, sc, fork(beams[p].blocks, n_ctx, first_child=p not in used_parent)))
                used_parent.add(p)
        for b in beams:
            pool.drop(b.blocks)
        beams = new
        if len(done) >= W and (not beams or max(d.score for d in done) >= norm(beams[0].score, len(beams[0].tokens))):
            break
    for b in beams:
        done.append(BeamOutput(b.tokens, b.score, norm(b.score, len(b.tokens)), "length"))
        pool.drop(b.blocks)
    assert not pool.ref, "beam search leaked KV blocks"
    done.sort(key=lambda d: -d.score)
    return done[: (num_return or W)]
