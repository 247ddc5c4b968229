"""DiT step caches: they skip work and stay close to the uncached trajectory; TaylorSeer is exact on
outputs that are linear in the step."""
import torch

from xllm_b200.dit import FBCache, ResidualCache, TaylorSeer, make_cache
from xllm_b200.dit.model import TinyDiT


def test_taylorseer_exact_on_linear_signal():
    ts = TaylorSeer(n_derivatives=1, skip_interval=3, warmup=3)
    base = torch.randn(4, 5)
    f = lambda s: base * (2.0 - 0.25 * s)
    for step in range(12):
        x = torch.zeros(4, 5)
        y = ts.run(step, x, lambda z: z, lambda z, s=step: z + f(s))
        if step >= 3:
            assert torch.allclose(y, f(step), atol=1e-4), step
    assert ts.skipped >= 5 and ts.computed >= 4


def test_caches_on_a_tiny_dit_trajectory():
    torch.manual_seed(0)
    m = TinyDiT().eval()
    for p in m.parameters():          # adaLN-zero style small weights keep the flow smooth
        p.data.mul_(0.5)
    noise = torch.randn(2, 4, 8, 8)
    ref = m.sample(noise, steps=24)
    scale = ref.abs().mean()
    for kind, kw in (("fbcache", dict(threshold=0.15)), ("taylorseer", dict(n_derivatives=1, skip_interval=2, warmup=2)),
                     ("residual", dict(skip_interval=2)), ("fbcache_taylorseer", dict(threshold=0.15))):
        c = make_cache(kind, **kw)
        out = m.sample(noise, steps=24, cache=c)
        assert c.skipped > 0, kind
        assert (out - ref).abs().mean() < 0.1 * scale, (kind, float((out - ref).abs().mean() / scale))
    assert make_cache("none") is None
    strict = FBCache(threshold=0.0)
    assert torch.allclose(m.sample(noise, steps=6, cache=strict), m.sample(noise, steps=6), atol=1e-5)
    assert strict.skipped == 0
