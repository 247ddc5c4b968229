"""Step-time model of the engine: measured once at start-up, used by the scheduler's budgets.

Parity: `ProfileManager` + `TimePredictor` (xllm/core/scheduler/profile/profile_manager.cpp,
time_predictor.cpp): prefill and decode steps are timed on synthetic batches, a polynomial is fitted
to each (prefill: tokens and tokens^2 for the attention term; decode: batch size and total context),
and the fit answers "how many tokens fit into a step that must finish within the TPOT / TTFT
target" (`token_budget`), which caps `max_tokens_per_batch` for SLO-aware scheduling.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple

import numpy as np


class TimePredictor:
    """Least-squares fit t = w . phi(x) over a small feature map."""

    def __init__(self, features: Callable[[np.ndarray], np.ndarray]):
        self.features = features
        self.w: Optional[np.ndarray] = None

    def fit(self, xs: Sequence[Sequence[float]], ts: Sequence[float]):
        X = np.stack([self.features(np.asarray(x, dtype=np.float64)) for x in xs])
        self.w, *_ = np.linalg.lstsq(X, np.asarray(ts, dtype=np.float64), rcond=None)
        return self

    def predict(self, x: Sequence[float]) -> float:
        assert self.w is not None, "fit() first"
        return float(self.features(np.asarray(x, dtype=np.float64)) @ self.w)


def prefill_features(x):      # x = [new tokens, context already in the cache]
    n, c = x[0], x[1] if len(x) > 1 else 0.0
    return np.array([1.0, n, n * n + 2.0 * n * c])


def decode_features(x):       # x = [batch size, total context tokens]
    return np.array([1.0, x[0], x[1]])


class ProfileManager:
    def __init__(self, time_prefill: Callable[[int, int], float], time_decode: Callable[[int, int], float]):
        """time_prefill(n_tokens, context) and time_decode(batch, context_per_seq) return seconds
        for one step; `for_engine` builds them from a live engine."""
        self.time_prefill, self.time_decode = time_prefill, time_decode
        self.prefill = TimePredictor(prefill_features)
        self.decode = TimePredictor(decode_features)
        self.samples_prefill: List[Tuple[int, int, float]] = []
        self.samples_decode: List[Tuple[int, int, float]] = []

    def profile(self, prefill_tokens=(128, 512, 1024, 2048, 4096), decode_batches=(1, 8, 32, 128, 256),
                contexts=(256, 2048)):
        for n in prefill_tokens:
            for c in (0, contexts[0]):
                self.samples_prefill.append((n, c, self.time_prefill(n, c)))
        for b in decode_batches:
            for c in contexts:
                self.samples_decode.append((b, c, self.time_decode(b, c)))
        self.prefill.fit([(n, c) for n, c, _ in self.samples_prefill], [t for *_, t in self.samples_prefill])
        self.decode.fit([(b, b * c) for b, c, _ in self.samples_decode], [t for *_, t in self.samples_decode])
        return self

    def predict_prefill(self, n_tokens: int, context: int = 0) -> float:
        return self.prefill.predict((n_tokens, context))

    def predict_decode(self, batch: int, context_per_seq: int) -> float:
        return self.decode.predict((batch, batch * context_per_seq))

    def token_budget(self, latency_s: float, decode_batch: int = 0, context_per_seq: int = 0, lo=16, hi=65536) -> int:
        """Largest number of prompt tokens that can ride along with `decode_batch` decode rows in a
        step of at most `latency_s` seconds (0 when even the decode rows do not fit)."""
        base = self.predict_decode(decode_batch, context_per_seq) if decode_batch else 0.0
        if base + self.predict_prefill(lo) > latency_s:
            return 0
        while lo < hi:
            mid = (lo + hi + 1) // 2
            if base + self.predict_prefill(mid) <= latency_s:
                lo = mid
            else:
                hi = mid - 1
        return lo

    def max_decode_batch(self, tpot_s: float, context_per_seq: int, hi: int = 4096) -> int:
        lo = 0
        while lo < hi:
            mid = (lo + hi + 1) // 2
            if self.predict_decode(mid, context_per_seq) <= tpot_s:
                lo = mid
            else:
                hi = mid - 1
        return lo

    @classmethod
    def for_engine(cls, engine, repeats: int = 3):
        """Time real steps of `engine`'s model runner on synthetic token ids (its KV cache is used as
        scratch: call before serving)."""
        import time

        import torch

        runner, bs = engine.runner, engine.cfg.block_size
        dev = runner.device
        nblk = engine.num_blocks

        def run(tokens_per_seq, ctx, nseq):
            from ..models.layers import AttentionMetadata as Meta
            q = tokens_per_seq
            per = (ctx + q + bs - 1) // bs
            if nseq * per >= nblk:
                nseq = max(1, (nblk - 1) // per)
            bt = (1 + torch.arange(nseq * per, dtype=torch.int32).view(nseq, per)).to(dev)
            pos = (ctx + torch.arange(q)).repeat(nseq)
            slots = (bt.cpu()[:, None, :].expand(nseq, q, per).reshape(nseq * q, per)
                     .gather(1, (pos // bs).view(-1, 1).long()).view(-1) * bs + (pos % bs).int()).int().to(dev)
            meta = Meta(n_decode=nseq if q == 1 else 0, n_prefill=0 if q == 1 else nseq, slots=slots, block_table=bt,
                        kv_lens=torch.full((nseq,), ctx + q, dtype=torch.int32, device=dev),
                        cu_q=torch.arange(0, nseq * q + 1, q, dtype=torch.int32, device=dev), max_q_len=q,
                        max_kv_len=ctx + q)
            toks = torch.zeros(nseq * q, dtype=torch.int64, device=dev)
            best = 1e9
            for _ in range(repeats):
                if dev.type == "cuda":
                    torch.cuda.synchronize()
                t0 = time.perf_counter()
                runner.model.logits(runner.model.forward(toks, pos.to(dev), meta, runner.kv_caches)[-1:])
                if dev.type == "cuda":
                    torch.cuda.synchronize()
                best = min(best, time.perf_counter() - t0)
            return best

        return cls(lambda n, c: run(n, c, 1), lambda b, c: run(1, c, b))
