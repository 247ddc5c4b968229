"""Step caches for diffusion transformers: skip transformer blocks on denoising steps whose output
can be predicted from earlier steps.

Parity: xllm/core/framework/dit_cache/{fbcache,taylorseer,fbcache_taylorseer,residual_cache}.cpp
(configured by `DiTCacheConfig`, dit_cache_config.h).
  * `FBCache` (first-block cache): run only the first block; if its residual moved by less than
    `threshold` (relative L1) since the previous step, reuse the cached residual of the remaining
    blocks instead of running them.
  * `TaylorSeer`: keep finite-difference derivatives of the model output over the steps where the
    model really ran and extrapolate with a Taylor series on the steps in between
    (`n_derivatives` terms, a real evaluation every `skip_interval` steps after `warmup` steps).
  * `ResidualCache`: plain reuse of the whole-stack residual every other step.
`FBCacheTaylorSeer` = FBCache's decision + TaylorSeer's extrapolation of the remaining-blocks
residual.

The caches are model-agnostic: `run(step, x, first_block, rest_blocks)` takes callables.
"""
from __future__ import annotations

import math
from typing import Callable, List, Optional

import torch


class ResidualCache:
    def __init__(self, skip_interval: int = 2, warmup: int = 1):
        self.k, self.warmup = max(1, skip_interval), warmup
        self.res: Optional[torch.Tensor] = None
        self.computed = self.skipped = 0

    def reset(self):
        self.res = None
        self.computed = self.skipped = 0

    def run(self, step: int, x, first_block: Callable, rest_blocks: Callable):
        full = lambda t: rest_blocks(first_block(t))
        if self.res is None or step < self.warmup or (step - self.warmup) % self.k == 0:
            y = full(x)
            self.res = y - x
            self.computed += 1
            return y
        self.skipped += 1
        return x + self.res


class FBCache:
    def __init__(self, threshold: float = 0.08, max_consecutive_skips: int = 3):
        self.th, self.max_skips = threshold, max_consecutive_skips
        self.prev_first: Optional[torch.Tensor] = None
        self.rest_res: Optional[torch.Tensor] = None
        self.consecutive = 0
        self.computed = self.skipped = 0

    def reset(self):
        self.__init__(self.th, self.max_skips)

    def _similar(self, first_res) -> bool:
        if self.prev_first is None or self.rest_res is None:
            return False
        num = (first_res - self.prev_first).abs().mean()
        den = self.prev_first.abs().mean().clamp_min(1e-12)
        return float(num / den) < self.th

    def _rest(self, step, h, rest_blocks):
        y = rest_blocks(h)
        self.rest_res = y - h
        return y

    def _approx(self, step, h):
        return h + self.rest_res

    def run(self, step: int, x, first_block: Callable, rest_blocks: Callable):
        h = first_block(x)
        first_res = h - x
        if self._similar(first_res) and self.consecutive < self.max_skips:
            self.consecutive += 1
            self.skipped += 1
            y = self._approx(step, h)
        else:
            self.consecutive = 0
            self.computed += 1
            y = self._rest(step, h, rest_blocks)
            self.prev_first = first_res
        return y


class TaylorSeer:
    def __init__(self, n_derivatives: int = 2, skip_interval: int = 3, warmup: int = 2):
        self.n, self.k, self.warmup = n_derivatives, max(1, skip_interval), warmup
        self.derivs: List[torch.Tensor] = []
        self.last_step: Optional[int] = None
        self.computed = self.skipped = 0

    def reset(self):
        self.derivs, self.last_step = [], None
        self.computed = self.skipped = 0

    def should_compute(self, step: int) -> bool:
        return self.last_step is None or step < self.warmup or step - self.last_step >= self.k

    def update(self, step: int, y: torch.Tensor):
        """Finite differences of increasing order against the previous real evaluation."""
        new = [y]
        if self.last_step is not None:
            dt = float(step - self.last_step)
            for i in range(min(self.n, len(self.derivs))):
                new.append((new[i] - self.derivs[i]) / dt)
        self.derivs, self.last_step = new, step

    def approximate(self, step: int) -> torch.Tensor:
        dt = float(step - self.last_step)
        out = torch.zeros_like(self.derivs[0])
        for i, d in enumerate(self.derivs):
            out = out + d * (dt ** i) / math.factorial(i)
        return out

    def run(self, step: int, x, first_block: Callable, rest_blocks: Callable):
        if self.should_compute(step):
            y = rest_blocks(first_block(x))
            self.update(step, y - x)
            self.computed += 1
            return y
        self.skipped += 1
        return x + self.approximate(step)


class FBCacheTaylorSeer(FBCache):
    """First-block decision; the remaining-blocks residual is extrapolated, not just replayed."""

    def __init__(self, threshold: float = 0.08, max_consecutive_skips: int = 3, n_derivatives: int = 1):
        super().__init__(threshold, max_consecutive_skips)
        self.ts = TaylorSeer(n_derivatives, 1, 0)

    def _rest(self, step, h, rest_blocks):
        y = rest_blocks(h)
        self.rest_res = y - h
        self.ts.update(step, self.rest_res)
        return y

    def _approx(self, step, h):
        return h + self.ts.approximate(step)


def make_cache(kind: str, **kw):
    kinds = {"none": None, "fbcache": FBCache, "taylorseer": TaylorSeer, "residual": ResidualCache,
             "fbcache_taylorseer": FBCacheTaylorSeer}
    if kind not in kinds:
        raise ValueError(f"unknown DiT cache {kind!r}")
    return kinds[kind](**kw) if kinds[kind] is not None else None
