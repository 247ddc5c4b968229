"""Generative recommendation: a fixed number of decode rounds with a wide beam per request.

Parity: the rec stack of the reference — `RecMaster` / `RecEngine` with the LLM-backbone multi-round
pipeline (xllm/core/distributed_runtime/rec_master.cpp, rec_engine.cpp: `RecMultiRoundEnginePipeline`),
the fixed-steps scheduler (core/scheduler/fixed_steps_scheduler.cpp), the rec beam-search kernels
(core/kernels/cuda/rec_beam_search.cu) and x-attention (core/layers/cuda/xattention.cpp).  A request is a
user-history prompt (token ids, optionally with input embeddings for some rows); the answer is the
`beam_width` most likely items, an item being `num_steps` tokens (a semantic id), optionally restricted to
the items of a catalogue.

How one call runs on the device
  1. all prompts are prefilled together through the engine's model runner into paged KV blocks;
  2. the first beam step takes the top `W` first tokens of every request from the prefill logits;
  3. every later round is ONE forward of R x W rows: the rows' new KV goes to a tail cache
     [R*W, nkv, num_steps, d] and attention is x-attention (ops/xattn.py: the prompt's pages are read once
     per request on the tensor cores, the tail is merged per beam);
  4. the beam step (log-softmax, per-row top-k, per-request top-W over W*k candidates) runs in the
     selection kernels (ops/select.py) for all requests at once; only the final (tokens, scores) cross to
     the host.  Surviving beams keep their place by re-gathering the small ancestor table, not the KV.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..models.layers import AttentionMetadata
from ..ops import select


@dataclass
class RecItem:
    token_ids: List[int]
    logprob: float


class ItemTrie:
    """The catalogue of valid items as a prefix tree over their token tuples, stored as one CSR table per level
    on the device: node n of level l has the children tokens `tok[l][ptr[l][n] : ptr[l][n + 1]]` (sorted), and
    child j of that range is node `ptr[l][n] + j` of level l + 1.  A beam carries its node id; the admissible
    next tokens of a batch of beams become a boolean mask with two tensor operations (`mask_of`), and after a
    beam step the survivors' node ids follow by a binary search in their parents' ranges (`advance`) — no host
    loop over rows, so catalogues of millions of items and thousands of beam rows cost the same few launches
    (the valid-path filter of the reference's rec sampler, core/framework/sampling/valid_path_filter.cpp)."""

    def __init__(self, items: Sequence[Sequence[int]], vocab_size: int, device="cpu"):
        import numpy as np
        self.vocab = int(vocab_size)
        if isinstance(items, torch.Tensor):
            items = items.cpu().numpy()
        if isinstance(items, np.ndarray):                    # [n_items, depth] already: no per-item Python work
            arr = items.astype(np.int64).reshape(items.shape[0], -1)
        else:
            arr = np.asarray([list(map(int, it)) for it in items], dtype=np.int64).reshape(len(items), -1)
        self.depth = arr.shape[1] if arr.size else 0
        self.n_items = 0
        self.ptr: List[torch.Tensor] = []
        self.tok: List[torch.Tensor] = []
        self.key: List[torch.Tensor] = []                    # parent node * vocab + token of every child: sorted
        self.device = torch.device(device)
        if arr.size == 0:
            return
        arr = np.unique(arr, axis=0)                       # sorted lexicographically, duplicates dropped
        self.n_items = arr.shape[0]
        node = np.zeros(arr.shape[0], dtype=np.int64)        # node id (within its level) of every item's prefix
        n_nodes = 1
        for l in range(self.depth):
            key = node * self.vocab + arr[:, l]
            uniq, inv = np.unique(key, return_inverse=True)   # children of all nodes of this level, in node order
            parent = uniq // self.vocab
            ptr = np.zeros(n_nodes + 1, dtype=np.int64)
            np.add.at(ptr, parent + 1, 1)
            self.ptr.append(torch.from_numpy(np.cumsum(ptr)).to(self.device))
            self.tok.append(torch.from_numpy(uniq % self.vocab).to(self.device))
            self.key.append(torch.from_numpy(uniq).to(self.device))
            node, n_nodes = inv.reshape(-1).astype(np.int64), uniq.shape[0]

    def to(self, device) -> "ItemTrie":
        if torch.device(device) != self.device:
            self.device = torch.device(device)
            self.ptr = [t.to(device) for t in self.ptr]
            self.tok = [t.to(device) for t in self.tok]
            self.key = [t.to(device) for t in self.key]
        return self

    def root(self, rows: int) -> torch.Tensor:
        return torch.zeros(rows, dtype=torch.int64, device=self.device)

    def mask_of(self, level: int, nodes: torch.Tensor) -> torch.Tensor:
        """Boolean [rows, vocab]: the tokens that continue the prefix of each row (node < 0: a dead row, none)."""
        rows = nodes.shape[0]
        mask = torch.zeros((rows, self.vocab), dtype=torch.bool, device=self.device)
        live = nodes >= 0
        n = nodes.clamp(min=0)
        lo, hi = self.ptr[level][n], self.ptr[level][n + 1]
        cnt = torch.where(live, hi - lo, torch.zeros_like(lo))
        total = int(cnt.sum())
        if total == 0:
            return mask
        row_of = torch.repeat_interleave(torch.arange(rows, device=self.device), cnt)
        start = torch.repeat_interleave(lo, cnt)
        within = torch.arange(total, device=self.device) - torch.repeat_interleave(torch.cumsum(cnt, 0) - cnt, cnt)
        mask[row_of, self.tok[level][start + within]] = True
        return mask

    def advance(self, level: int, nodes: torch.Tensor, tokens: torch.Tensor) -> torch.Tensor:
        """Node ids (level + 1) of the rows after appending `tokens`; -1 where the token does not continue the row."""
        live = nodes >= 0
        n = nodes.clamp(min=0)
        # (parent, token) keys of a level are sorted as a whole: one binary search finds the child
        key = n * self.vocab + tokens.to(torch.int64)
        run_key = self.key[level]
        pos = torch.searchsorted(run_key, key)
        ok = live & (run_key[pos.clamp(max=run_key.shape[0] - 1)] == key)
        return torch.where(ok, pos, torch.full_like(pos, -1))

    # ---- prefix-tuple interface (host side; tests and small catalogues)
    def allowed(self, prefixes: Sequence[Sequence[int]], device) -> torch.Tensor:
        self.to(device)
        nodes = self.root(len(prefixes))
        level = len(prefixes[0]) if len(prefixes) else 0
        if level:
            p = torch.tensor([[int(t) for t in pre] for pre in prefixes], dtype=torch.int64, device=self.device)
            for l in range(level):
                nodes = self.advance(l, nodes, p[:, l])
        return self.mask_of(level, nodes)

    def __contains__(self, item):
        if len(item) != self.depth or self.depth == 0:
            return False
        nodes = self.root(1)
        t = torch.tensor([[int(x) for x in item]], dtype=torch.int64, device=self.device)
        for l in range(self.depth):
            nodes = self.advance(l, nodes, t[:, l])
        return bool(nodes[0] >= 0)


class _Tail:
    """Per-layer tail caches of the live beams plus the ancestor table (see ops/xattn.py)."""

    def __init__(self, kv_caches, rows: int, cap: int, max_rows: int):
        self.by_ptr = {}
        for k, _ in kv_caches:
            nkv, d = k.shape[1], k.shape[3]
            ku = torch.zeros((rows, nkv, cap, d), dtype=k.dtype, device=k.device)
            self.by_ptr[k.data_ptr()] = (ku, torch.zeros_like(ku))
        dev = kv_caches[0][0].device
        self.anc = torch.arange(rows, dtype=torch.int32, device=dev)[None].repeat(cap, 1).contiguous()
        self.n_tail = 0
        self.max_rows = max_rows
        self.cap = cap

    def tail_of(self, k_cache):
        return self.by_ptr[k_cache.data_ptr()]


class RecEngine:
    """Runs fixed-step beam generation on the model, KV cache and block manager of an `LLMEngine`."""

    def __init__(self, engine):
        self.engine = engine
        self.runner = engine.runner
        if getattr(self.runner.model, "needs_state", False):
            raise ValueError("fixed-step beam generation needs an attention-only model (no recurrent state)")

    # ------------------------------------------------------------------------------------------ public
    def generate(self, prompts: Sequence[Sequence[int]], beam_width: int = 32, num_steps: int = 3,
                 num_return: Optional[int] = None, trie: Optional[ItemTrie] = None,
                 prompt_embeds: Optional[Sequence[Optional[Tuple[torch.Tensor, torch.Tensor]]]] = None
                 ) -> List[List[RecItem]]:
        """`prompt_embeds[i]` = (row indices inside prompt i, values [n, hidden]) replaces the token
        embedding of those rows (the request's `input_tensors` in the reference)."""
        if trie is not None and trie.depth != num_steps:
            raise ValueError(f"catalogue items have {trie.depth} tokens, the request asks for {num_steps}")
        if not 1 <= num_steps <= 8:
            raise ValueError("num_steps must be in 1..8")
        eng, runner = self.engine, self.runner
        model, kv, dev = runner.model, runner.kv_caches, runner.device
        bs = eng.cfg.block_size
        bm = eng.scheduler.block_manager(0)
        R, W = len(prompts), int(beam_width)
        if R == 0:
            return []
        V = eng.args.vocab_size
        W = min(W, V)
        lens = [len(p) for p in prompts]
        owned: List[List[int]] = []
        try:
            for L in lens:
                got = bm.allocate((L + bs - 1) // bs)
                if len(got) < (L + bs - 1) // bs:
                    bm.free(got)
                    raise RuntimeError("rec generation: out of KV blocks")
                owned.append(list(got))
            return self._run(prompts, lens, owned, R, W, num_steps, num_return or W, trie, prompt_embeds, model, kv,
                             dev, bs, V)
        finally:
            for blocks in owned:
                bm.free(blocks)

    # ----------------------------------------------------------------------------------------- rounds
    def _run(self, prompts, lens, owned, R, W, S, n_ret, trie, prompt_embeds, model, kv, dev, bs, V):
        width = max(len(b) for b in owned)
        bt = torch.zeros((R, width), dtype=torch.int32)
        for i, b in enumerate(owned):
            bt[i, : len(b)] = torch.tensor(b, dtype=torch.int32)
        bt = bt.to(dev)
        kv_lens = torch.tensor(lens, dtype=torch.int32, device=dev)
        # ---- prompts, one batched prefill
        toks, pos, slots, cu, emb_rows, emb_vals = [], [], [], [0], [], []
        for i, p in enumerate(prompts):
            base = len(toks)
            toks.extend(int(t) for t in p)
            pos.extend(range(lens[i]))
            slots.extend(owned[i][q // bs] * bs + q % bs for q in range(lens[i]))
            cu.append(len(toks))
            if prompt_embeds is not None and prompt_embeds[i] is not None:
                rows, vals = prompt_embeds[i]
                emb_rows.append(torch.as_tensor(rows, dtype=torch.long) + base)
                emb_vals.append(vals)
        meta = AttentionMetadata(n_decode=0, n_prefill=R, slots=torch.tensor(slots, dtype=torch.int32, device=dev),
                                 block_table=bt, kv_lens=kv_lens, cu_q=torch.tensor(cu, dtype=torch.int32, device=dev),
                                 max_q_len=max(lens), max_kv_len=max(lens))
        embeds = None
        if emb_rows:
            embeds = (torch.cat(emb_rows).to(dev), torch.cat(emb_vals).to(dev))
        h = model.forward(torch.tensor(toks, dtype=torch.int64, device=dev), torch.tensor(pos, dtype=torch.int64, device=dev),
                          meta, kv, embeds=embeds) if embeds is not None else \
            model.forward(torch.tensor(toks, dtype=torch.int64, device=dev), torch.tensor(pos, dtype=torch.int64, device=dev),
                          meta, kv)
        last = torch.tensor([c - 1 for c in cu[1:]], dtype=torch.long, device=dev)
        logits = self._logits(model, h[last])                              # [R, V]
        # ---- first beam step: the W best first tokens of every request
        nodes = None
        if trie is not None:
            trie.to(dev)
            nodes = trie.root(R)
        lp, ids = self._candidates(logits, W, None if trie is None else trie.mask_of(0, nodes))      # [R, W]
        if trie is not None:
            nodes = trie.advance(0, nodes.repeat_interleave(W), ids.reshape(-1).to(torch.int64))
        cum = lp
        seqs = ids.to(torch.int64)[:, :, None]                             # [R, W, 1] tokens so far
        rows = R * W
        tail = _Tail(kv, rows, max(S - 1, 1), W)
        cu_b = torch.arange(R + 1, dtype=torch.int32, device=dev) * W
        row_pos = kv_lens.to(torch.int64).repeat_interleave(W)              # position of a beam's first own token
        row_ids = torch.arange(rows, dtype=torch.int32, device=dev)
        k_cand = min(W, V)
        for s in range(1, S):
            # forward of all beams: the token chosen in round s-1 is input, its KV becomes tail token s-1
            tail.n_tail = s
            meta = AttentionMetadata(n_decode=0, n_prefill=R, slots=row_ids * tail.cap + (s - 1), block_table=bt,
                                     kv_lens=kv_lens, cu_q=cu_b, max_q_len=W, max_kv_len=max(lens) + s, xattn=tail)
            h = model.forward(seqs[:, :, -1].reshape(rows).contiguous(), row_pos + (s - 1), meta, kv)
            logits = self._logits(model, h)                                # [R*W, V]
            lp, ids = self._candidates(logits, k_cand, None if trie is None else trie.mask_of(s, nodes))    # [R*W, k]
            tok, par, cum = select.beam_step(lp.view(R, W, k_cand), ids.view(R, W, k_cand), cum, W)
            par64 = par.to(torch.int64)
            seqs = torch.cat([seqs.gather(1, par64[:, :, None].expand(R, W, seqs.shape[2])),
                              tok.to(torch.int64)[:, :, None]], dim=2)
            if trie is not None and s + 1 < S:
                nodes = trie.advance(s, nodes.view(R, W).gather(1, par64).reshape(-1), tok.reshape(-1).to(torch.int64))
            if s + 1 < S:                                                  # survivors inherit their parents' tails
                gpar = (par64 + torch.arange(R, device=dev)[:, None] * W).reshape(rows)
                tail.anc = tail.anc[:, gpar].contiguous()
                tail.anc[s] = row_ids
        cum_h, seq_h = cum.tolist(), seqs.tolist()
        out: List[List[RecItem]] = []
        for r in range(R):
            items = [RecItem(seq_h[r][w], cum_h[r][w]) for w in range(W) if cum_h[r][w] != float("-inf")]
            items.sort(key=lambda it: -it.logprob)
            out.append(items[:n_ret])
        return out

    @staticmethod
    def _candidates(logits, k, mask=None):
        """The k most likely next tokens of every row with their log-probabilities under the model's full
        distribution; with a catalogue mask, tokens that leave the catalogue score -inf."""
        if mask is None:
            lp, ids = select.topk(logits, k, normalize=True)
        else:
            full = select.log_softmax(logits).masked_fill(~mask, float("-inf"))
            lp, ids = select.topk(full, k)
        lp = lp.float()
        return torch.where(torch.isfinite(lp), lp, torch.full_like(lp, float("-inf"))), ids

    @staticmethod
    def _logits(model, h):
        logits = model.logits(h)
        return logits if logits.dtype in (torch.bfloat16, torch.float32) else logits.float()


def _next_logprobs_dense(engine, tokens):
    """log-probabilities of the token after `tokens`, by one plain causal forward of the whole sequence."""
    runner = engine.runner
    model, dev = runner.model, runner.device
    bs = engine.cfg.block_size
    bm = engine.scheduler.block_manager(0)
    n = len(tokens)
    blocks = bm.allocate((n + bs - 1) // bs)
    try:
        slots = [blocks[q // bs] * bs + q % bs for q in range(n)]
        meta = AttentionMetadata(n_decode=0, n_prefill=1, slots=torch.tensor(slots, dtype=torch.int32, device=dev),
                                 block_table=torch.tensor([list(blocks)], dtype=torch.int32, device=dev),
                                 kv_lens=torch.tensor([n], dtype=torch.int32, device=dev),
                                 cu_q=torch.tensor([0, n], dtype=torch.int32, device=dev), max_q_len=n, max_kv_len=n)
        h = model.forward(torch.tensor(tokens, dtype=torch.int64, device=dev),
                          torch.arange(n, dtype=torch.int64, device=dev), meta, runner.kv_caches)
        return torch.log_softmax(model.logits(h[-1:]).float(), -1)[0]
    finally:
        bm.free(blocks)


def item_logprob_reference(engine, prompt: Sequence[int], item: Sequence[int]) -> float:
    """Oracle for tests: the item's log-probability after the prompt, one dense forward per token."""
    toks, total = list(prompt), 0.0
    for t in item:
        total += float(_next_logprobs_dense(engine, toks)[int(t)])
        toks.append(int(t))
    return total


def recommend_reference(engine, prompt: Sequence[int], beam_width: int, num_steps: int,
                        trie: Optional[ItemTrie] = None) -> List[RecItem]:
    """Oracle for tests: exhaustive beam expansion by re-running the whole sequence for every beam
    (no KV reuse, no x-attention), through the same model."""
    dev = engine.runner.device
    beams = [([], 0.0)]
    for s in range(num_steps):
        cand = []
        for toks, sc in beams:
            lp = _next_logprobs_dense(engine, list(prompt) + toks)
            if trie is not None:
                lp = lp.masked_fill(~trie.allowed([toks], dev)[0], float("-inf"))
            k = min(beam_width, lp.numel())
            v, i = torch.topk(lp, k)
            cand.extend((toks + [int(t)], sc + float(x)) for x, t in zip(v.tolist(), i.tolist()) if x != float("-inf"))
        cand.sort(key=lambda c: -c[1])
        beams = cand[:beam_width]
    return [RecItem(t, s) for t, s in beams]
