"""Speculative decoding: draft k tokens per sequence, verify them with ONE target forward.

Parity: `SpeculativeEngine` / `SpeculativeWorkerImpl` with its MTP, Eagle3 and suffix drafters
(xllm/core/distributed_runtime/speculative_engine.h:96-120, runtime/mtp_worker_impl.cpp:1245-1850,
runtime/suffix_worker_impl.*) and `RejectionSampler` (framework/sampling/rejection_sampler.cpp:65-360).

Flow of a decode step for B sequences and k draft tokens:
  1. the drafter proposes d_1..d_k for every sequence,
  2. the target model runs once over [last token, d_1..d_k] of every sequence: these are k+1-token
     "prompt chunks" against the paged cache, so the prefill attention kernel handles them and the
     KV of every position is written as a side effect,
  3. verification keeps the longest prefix of drafts the target agrees with (greedy: equality
     with the argmax; sampling: the rejection rule of the device kernel `xllm_spec_verify`) and adds
     the target's own next token, so every step yields between 1 and k+1 tokens,
  4. the scheduler appends the accepted tokens; KV written for rejected drafts is simply
     overwritten by later steps (the sequence's kv length never counted it).
Steps that contain prompt chunks run unspeculated.

Drafters:
  * `NgramDrafter` — prompt-lookup / suffix matching on the sequence's own tokens, no model,
  * `MTPDrafter` — the multi-token-prediction layer of DeepSeek-V3-style checkpoints with its own
    paged KV cache, fed with the target's hidden states,
  * `DraftModelDrafter` — any small causal LM sharing the tokenizer (run without a KV cache of its
    own over a short window; enough for Eagle-style single-layer drafts).
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from ..ops import reference

from .. import ops
from ..models.layers import AttentionMetadata
from ..ops import spec as spec_ops


class NgramDrafter:
    """Propose the continuation of the most recent earlier occurrence of the longest suffix
    (up to `max_ngram` tokens) of the sequence.  Without a match the last token is repeated, which
    costs nothing but a rejected draft."""

    name = "ngram"

    def __init__(self, k: int, max_ngram: int = 4, min_ngram: int = 1, window: int = 2048):
        self.k, self.max_ngram, self.min_ngram, self.window = k, max_ngram, min_ngram, window

    def propose_one(self, toks: np.ndarray) -> np.ndarray:
        k = self.k
        n = len(toks)
        out = np.full(k, toks[-1] if n else 0, dtype=np.int64)
        for g in range(min(self.max_ngram, n - 1), self.min_ngram - 1, -1):
            suffix = toks[n - g:]
            # candidate starts i with toks[i:i+g] == suffix and i + g < n, latest first
            first = np.nonzero(toks[: n - g] == suffix[0])[0]
            for i in first[::-1]:
                if i + g <= n - 1 and np.array_equal(toks[i:i + g], suffix):
                    cont = toks[i + g:i + g + k]
                    if len(cont) > 0:
                        out[: len(cont)] = cont
                        if len(cont) < k:
                            out[len(cont):] = cont[-1]
                        return out
        return out

    def propose(self, batch, n_rows: int, **_) -> np.ndarray:
        return np.stack([self.propose_one(batch.history(i, self.window)) for i in range(n_rows)])

    def observe(self, *a, **kw):
        pass

    def after_execute(self, *a, **kw):
        pass


class MTPDrafter:
    """One-token drafts from a multi-token-prediction layer (`models.deepseek.MTPDraft`,
    DeepSeek-V3 `num_nextn_predict_layers`; reference: runtime/mtp_worker_impl.cpp:1245-1850).

    The layer at position p consumes the target's hidden state h_p and the embedding of token
    x_{p+1} and predicts x_{p+2}.  It has a paged KV cache of its own with the geometry of one
    target layer, addressed through the same block tables, and is run over exactly the rows the
    target has verified: every prompt chunk and unspeculated decode row (`after_execute`), and the
    accepted rows of a verification pass (`observe`).  The prediction made at the last verified
    position of a sequence is its draft for the next step.

    More than one draft token per step (k > 1) chains the layer on itself: draft j + 1 comes from the
    layer's own output at draft j and the embedding of draft j, one single-token pass per extra draft
    over all sequences at once (the reference chains its MTP / EAGLE-3 draft passes the same way).
    Draft KV written past a sequence's last allocated block lands in the padding block, which costs
    acceptance at block boundaries, never correctness: the target verifies every draft.

    The same driver serves an EAGLE-3 head (`models.eagle3.Eagle3Draft`): it reads the three
    auxiliary hidden states the target keeps (`model.last_aux`) instead of the final one and maps its
    draft-vocabulary ids to target ids."""

    name = "mtp"

    def __init__(self, engine, k: int = 1, head=None):
        self.k = int(k)
        self.engine = engine
        self.mtp = head if head is not None else engine.mtp
        self.takes_aux = bool(getattr(self.mtp, "takes_aux", False))
        k0, v0 = engine.runner.kv_caches[0]
        heads = int(getattr(self.mtp, "kv_heads_full", 0) or k0.shape[1])
        if heads != k0.shape[1]:                     # a replicated head under tensor parallelism: all KV heads here
            shape = (k0.shape[0], heads) + tuple(k0.shape[2:])
            self.kv = (torch.zeros(shape, dtype=k0.dtype, device=k0.device), torch.zeros(shape, dtype=v0.dtype, device=v0.device))
        else:
            self.kv = (torch.zeros_like(k0), torch.zeros_like(v0))
        self.draft = {}
        engine.runner.keep_hidden = True

    def propose(self, batch, n_rows: int, **_) -> np.ndarray:
        out = np.zeros((n_rows, self.k), dtype=np.int64)
        for i in range(n_rows):
            d = self.draft.get(batch.request_id(i))
            out[i, :] = int(batch.history(i, 1)[0]) if d is None else d
        return out

    def _ids(self, hidden_rows):
        ids = self.mtp.logits(hidden_rows).argmax(-1)
        return self.mtp.to_target_ids(ids) if hasattr(self.mtp, "to_target_ids") else ids

    def _run(self, next_tokens, hidden, positions, meta, last_rows, request_ids, pos_last=None, block_tables=None):
        h = self.mtp.forward(next_tokens, hidden, positions, meta, self.kv[0], self.kv[1])
        if len(last_rows) == 0:
            return
        dev = h.device
        rows = torch.as_tensor(last_rows, dtype=torch.long, device=dev)
        hr = h[rows]
        ids = self._ids(hr)
        drafts = [ids]
        if self.k > 1:
            bs = self.engine.cfg.block_size
            n = len(last_rows)
            bt = np.ascontiguousarray(np.asarray(block_tables)[:, :]).astype(np.int32)
            bt_dev = torch.from_numpy(bt).to(dev)
            p0 = np.asarray(pos_last, dtype=np.int64)
            cu = torch.arange(0, n + 1, dtype=torch.int32, device=dev)
            for j in range(1, self.k):
                pj = p0 + j
                blk = np.where(pj // bs < bt.shape[1], bt[np.arange(n), np.minimum(pj // bs, bt.shape[1] - 1)], 0)
                slots = (blk.astype(np.int64) * bs + pj % bs).astype(np.int32)
                m = AttentionMetadata(
                    n_decode=0, n_prefill=n, slots=torch.from_numpy(slots).to(dev), block_table=bt_dev,
                    kv_lens=torch.from_numpy((pj + 1).astype(np.int32)).to(dev), cu_q=cu, max_q_len=1,
                    max_kv_len=int(pj.max()) + 1)
                hr = self.mtp.forward(ids, hr, torch.from_numpy(pj).to(dev), m, self.kv[0], self.kv[1])
                ids = self._ids(hr)
                drafts.append(ids)
        table = torch.stack(drafts, dim=1).cpu().tolist()
        for rid, t in zip(request_ids, table):
            self.draft[rid] = [int(v) for v in t]

    def after_execute(self, batch, sampled_ids):
        """After a normal (unspeculated) step: run the layer over all of its rows."""
        runner = self.engine.runner
        hidden, meta, positions = runner.last_hidden, runner.last_meta, runner.last_positions
        if hidden is None:
            return
        if self.takes_aux:
            hidden = runner.model.last_aux
        cu = np.asarray(batch.cu_q)
        pos_h = np.asarray(batch.positions)
        nseq = batch.n_decode + batch.n_prefill
        sample_seq = np.asarray(batch.sample_seq)
        sampled = {int(sample_seq[r]): int(sampled_ids[r]) for r in range(len(sample_seq))}
        nxt = np.zeros(int(cu[nseq]), dtype=np.int64)
        last_rows, rids, seqs = [], [], []
        for i in range(nseq):
            a, b = int(cu[i]), int(cu[i + 1])
            hist = batch.history(i, 0)
            p0 = int(pos_h[a])
            want = hist[p0 + 1:p0 + 1 + (b - a)]
            nxt[a:a + len(want)] = want
            if i in sampled:                       # the row of the last position takes the new token
                nxt[b - 1] = sampled[i]
                last_rows.append(b - 1)
                rids.append(batch.request_id(i))
                seqs.append(i)
        self._run(torch.from_numpy(nxt).to(hidden.device), hidden[: len(nxt)], positions[: len(nxt)], meta, last_rows, rids,
                  pos_last=[int(pos_h[r]) for r in last_rows],
                  block_tables=np.asarray(batch.block_tables)[seqs] if seqs else None)

    def observe(self, batch, n_rows, hidden_rows, counts, tokens=None, kv0=None, block_tables=None):
        """After a verification pass: hidden_rows [B, 2, H]; row j < counts[i] of sequence i is
        verified and its next token is tokens[i, j]."""
        dev = hidden_rows.device
        bs = self.engine.cfg.block_size
        sel, nxt, pos, slots, cu, last_rows, rids = [], [], [], [], [0], [], []
        for i in range(n_rows):
            c = int(counts[i])
            for j in range(c):
                p = int(kv0[i]) - 1 + j
                sel.append(i * hidden_rows.shape[1] + j)
                nxt.append(int(tokens[i, j]))
                pos.append(p)
                slots.append(int(block_tables[i, p // bs]) * bs + p % bs)
            cu.append(cu[-1] + c)
            last_rows.append(cu[-1] - 1)
            rids.append(batch.request_id(i))
        H = hidden_rows.shape[-1]
        hid = hidden_rows.reshape(-1, H)[torch.as_tensor(sel, dtype=torch.long, device=dev)]
        meta = AttentionMetadata(
            n_decode=0, n_prefill=n_rows, slots=torch.tensor(slots, dtype=torch.int32, device=dev),
            block_table=torch.from_numpy(np.ascontiguousarray(block_tables)).to(dev),
            kv_lens=torch.tensor([int(kv0[i]) - 1 + int(counts[i]) for i in range(n_rows)], dtype=torch.int32, device=dev),
            cu_q=torch.tensor(cu, dtype=torch.int32, device=dev), max_q_len=int(max(counts)),
            max_kv_len=int(max(kv0)) + 1)
        self._run(torch.tensor(nxt, dtype=torch.int64, device=dev), hid, torch.tensor(pos, dtype=torch.int64, device=dev),
                  meta, last_rows, rids, pos_last=[pos[r] for r in last_rows], block_tables=block_tables[:n_rows])

    def forget(self, request_id):
        self.draft.pop(request_id, None)


class DraftModelDrafter:
    """Greedy k-token drafts from a small causal LM run over the last `window` tokens of every
    sequence without a persistent cache (callable: tokens [B, W] -> logits [B, W, V])."""

    name = "draft_model"

    def __init__(self, fn, k: int, window: int = 64):
        self.fn, self.k, self.window = fn, k, window

    def propose(self, batch, n_rows: int, **_) -> np.ndarray:
        out = np.zeros((n_rows, self.k), dtype=np.int64)
        for i in range(n_rows):
            ctx = list(batch.history(i, self.window))
            for j in range(self.k):
                logits = self.fn(torch.tensor([ctx[-self.window:]], dtype=torch.int64))
                t = int(logits[0, -1].argmax())
                out[i, j] = t
                ctx.append(t)
        return out

    def observe(self, *a, **kw):
        pass

    def after_execute(self, *a, **kw):
        pass


class SpecDecoder:
    """Runs the verification pass on the engine's model runner."""

    def __init__(self, engine, drafter, k: int):
        self.engine, self.runner, self.drafter, self.k = engine, engine.runner, drafter, k
        self.block_size = engine.cfg.block_size
        self.proposed = 0
        self.accepted = 0
        self.steps = 0

    @property
    def acceptance_rate(self) -> float:
        return self.accepted / self.proposed if self.proposed else 0.0

    def step(self, batch):
        """`batch` is a decode-only batch.  Returns (tokens_flat int64, counts int32, logprobs|None)."""
        k, bs = self.k, self.block_size
        B = batch.n_decode
        dev = self.runner.device
        kv0 = np.asarray(batch.kv_lens)[:B].astype(np.int64)       # context incl. the last token
        last = np.asarray(batch.tokens)[:B].astype(np.int64)
        drafts = self.drafter.propose(batch, B).astype(np.int64)    # [B, k]
        toks = np.concatenate([last[:, None], drafts], axis=1)      # [B, k+1]
        pos = (kv0 - 1)[:, None] + np.arange(k + 1)[None, :]        # position of every input token
        bt = np.asarray(batch.block_tables)[:B]
        slots = (bt[np.arange(B)[:, None], pos // bs].astype(np.int64) * bs + pos % bs).astype(np.int32)
        T = B * (k + 1)
        t_tokens = torch.from_numpy(toks.reshape(-1)).to(dev)
        t_pos = torch.from_numpy(pos.reshape(-1)).to(dev)
        meta = AttentionMetadata(
            n_decode=0, n_prefill=B,
            slots=torch.from_numpy(slots.reshape(-1)).to(dev),
            block_table=torch.from_numpy(np.ascontiguousarray(bt)).to(dev),
            kv_lens=torch.from_numpy((kv0 + k).astype(np.int32)).to(dev),
            cu_q=torch.arange(0, T + 1, k + 1, dtype=torch.int32, device=dev),
            max_q_len=k + 1, max_kv_len=int(kv0.max()) + k)
        hidden = self.runner.model.forward(t_tokens, t_pos, meta, self.runner.kv_caches)
        logits = self.runner.model.logits(hidden).float().view(B, k + 1, -1)
        temperature = np.asarray(batch.temperature)[:B]
        greedy = temperature <= 0
        d_dev = torch.from_numpy(drafts).to(dev)
        lp = None
        if greedy.all():
            tgt = logits.argmax(-1)                                           # [B, k+1]
            agree = (tgt[:, :k] == d_dev).to(torch.int32)
            n_acc = torch.cumprod(agree, dim=1).sum(1)                        # accepted drafts per row
            counts = (n_acc + 1).to(torch.int32)
            out = tgt                                                         # tokens 0..n_acc are the target's own
            if batch.any_logprobs:
                lp = torch.log_softmax(logits, dim=-1).gather(-1, out.unsqueeze(-1)).squeeze(-1)
        else:
            # the verified distribution is the one the sampler would have drawn from: temperature,
            # then the top-k / top-p filter, renormalised (the reference's rejection sampler works on
            # the filtered target distribution too: sampling/rejection_sampler.cpp:65-360)
            rep = lambda a, dt: torch.from_numpy(np.repeat(np.asarray(a)[:B], k + 1).astype(dt)).to(dev)
            probs = reference.filtered_distribution(logits.view(B * (k + 1), -1), rep(temperature, np.float32),
                                                    rep(batch.top_k, np.int32), rep(batch.top_p, np.float32))
            probs = probs.float().view(B, k + 1, -1).contiguous()
            seeds = torch.from_numpy(np.asarray(batch.seeds)[:B].astype(np.uint64).view(np.int64)).to(dev)
            offs = torch.from_numpy(np.asarray(batch.sample_offsets)[:B].astype(np.int32)).to(dev)
            out, counts = spec_ops.verify(d_dev, probs, None, torch.from_numpy(greedy).to(dev), seeds=seeds, offsets=offs)
            if batch.any_logprobs:
                lp = torch.log(probs.gather(-1, out.clamp_min(0).unsqueeze(-1)).squeeze(-1).clamp_min(1e-30))
        counts_h = counts.cpu().numpy().astype(np.int32)
        out_h = out.cpu().numpy()
        flat = np.concatenate([out_h[i, : counts_h[i]] for i in range(B)]).astype(np.int64)
        lp_flat = None
        if lp is not None:
            lp_h = lp.float().cpu().numpy()
            lp_flat = np.concatenate([lp_h[i, : counts_h[i]] for i in range(B)]).astype(np.float32)
        seen = self.runner.model.last_aux if getattr(self.drafter, "takes_aux", False) else hidden
        self.drafter.observe(batch, B, seen.view(B, k + 1, -1), counts_h, tokens=out_h, kv0=kv0, block_tables=bt)
        self.proposed += B * k
        self.accepted += int(counts_h.sum()) - B
        self.steps += 1
        return flat, counts_h, lp_flat

    @staticmethod
    def can_verify(batch, runner) -> bool:
        """Whether one verification pass can honour every request of the batch.  Penalties depend on
        the tokens drafted so far, grammar masks on the automaton state after each of them, and
        top_logprobs needs the host in the loop: such batches take the ordinary one-token step."""
        return not (batch.any_penalty or runner.logits_hook is not None or batch.max_top_logprobs > 0)


def make_drafter(kind: str, k: int, engine=None, **kw):
    if kind in ("ngram", "suffix", "prompt_lookup"):
        return NgramDrafter(k, **kw)
    if kind == "mtp":
        return MTPDrafter(engine, k)
    if kind == "eagle3":
        return MTPDrafter(engine, k, head=engine.eagle3)
    raise ValueError(f"unknown drafter {kind!r}")
