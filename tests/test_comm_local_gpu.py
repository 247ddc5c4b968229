"""Communication kernels on ONE GPU: the one-shot fused all-reduce, the sharded arg-max and the
column gather with a world of one rank (the kernel's own buffer is its only peer), and flag waits
that run out.

The expiring waits follow the form allowed on shared GPUs: the kernel is told about a second rank
whose flag slot nobody ever sets, the wait gets a budget of a few hundred microseconds, and the
test checks that the kernel returned, that its error word names the missing peer, and that the
context still works afterwards.  Nothing here traps, faults or spins without a limit.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

H = 1024


def _lib():
    from xllm_b200.ops import _lib
    from xllm_b200.parallel import symm  # noqa: F401  (registers the signatures)
    from xllm_b200.parallel import ep  # noqa: F401
    return _lib.load()


class Local:
    """A 'symmetric' buffer and signal pad of a one-GPU world: pointer tables that name the local
    allocations `world` times."""

    def __init__(self, nbytes, world=1):
        dev = torch.device("cuda", 0)
        self.buf = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
        self.pad = torch.zeros(4096, dtype=torch.int32, device=dev)
        self.bufs = torch.tensor([self.buf.data_ptr()] * world, dtype=torch.int64, device=dev)
        self.pads = torch.tensor([self.pad.data_ptr()] * world, dtype=torch.int64, device=dev)
        self.state = torch.zeros(4, dtype=torch.int32, device=dev)
        self.err = torch.zeros(1, dtype=torch.int32, device=dev)


def _s():
    return torch.cuda.current_stream().cuda_stream


@pytest.mark.parametrize("T,hidden", [(1, 1024), (5, 256), (300, 4096), (64, 5120), (17, 7168)])
def test_oneshot_world_of_one_matches_reference(T, hidden):
    from xllm_b200.ops import reference as ref
    lib = _lib()
    L = Local(2 * T * hidden * 2 + 512)
    x = torch.randn(T, hidden, device="cuda", dtype=torch.bfloat16)
    res = torch.randn(T, hidden, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(hidden, device="cuda") * 0.1 + 1).to(torch.bfloat16)
    want_res = (x.float() + res.float()).to(torch.bfloat16)
    want, _ = ref.rmsnorm(want_res, w, 1e-6)
    out = torch.empty_like(x)
    for call in range(2):                     # consecutive calls use the two partial buffers in turn
        off = call * ((T * hidden * 2 + 255) & ~255)
        L.buf[off: off + T * hidden * 2].view(torch.bfloat16).view(T, hidden).copy_(x)
        r = res.clone()
        rc = lib.xllm_tp_oneshot_norm(L.bufs.data_ptr(), L.pads.data_ptr(), 0, off, 64, L.state.data_ptr(),
                                      r.data_ptr(), r.data_ptr(), w.data_ptr(), out.data_ptr(), L.err.data_ptr(),
                                      T, hidden, 0, 1, 1e-6, 296, _s())
        assert rc == 0
        torch.cuda.synchronize()
        assert int(L.err.item()) == 0
        assert torch.equal(r, want_res)
        assert torch.allclose(out.float(), want.float(), atol=0.03, rtol=0.02)
    assert int(L.state[0].item()) == 2        # the kernel advanced its own epoch twice


def test_argmax_and_gather_world_of_one():
    lib = _lib()
    B, Vs = 37, 1000
    logits = torch.randn(B, Vs + 8, device="cuda", dtype=torch.bfloat16)[:, :Vs]
    logits[2, 11] = logits[2, 900] = 40.0
    L = Local(2 * 1024 * 8 + B * 1024 * 2 + 512)
    ids = torch.empty(B, dtype=torch.int64, device="cuda")
    rc = lib.xllm_tp_argmax(logits.data_ptr(), logits.stride(0), L.bufs.data_ptr(), L.pads.data_ptr(), 0, 96,
                            L.state.data_ptr(), ids.data_ptr(), L.err.data_ptr(), B, Vs, 5000, 1024, 0, 1, _s())
    assert rc == 0
    torch.cuda.synchronize()
    want = logits.float().argmax(-1) + 5000
    want[2] = 5011
    assert torch.equal(ids, want) and int(L.err.item()) == 0
    src = torch.randn(B, 1024, device="cuda", dtype=torch.bfloat16)
    goff = 2 * 1024 * 8
    st = torch.zeros(2, dtype=torch.int32, device="cuda")
    rc = lib.xllm_tp_gather_cols(src.data_ptr(), src.stride(0), L.bufs.data_ptr(), L.pads.data_ptr(), 0, goff, 1024,
                                 128, st.data_ptr(), L.err.data_ptr(), B, 1024, 0, 1, _s())
    assert rc == 0
    torch.cuda.synchronize()
    got = L.buf[goff: goff + B * 1024 * 2].view(torch.bfloat16).view(B, 1024)
    assert torch.equal(got, src) and int(L.err.item()) == 0


def _short_budget(fn_name, cycles=600_000):
    import xllm_b200.parallel.ep  # noqa: F401 - declares the setters' signatures
    import xllm_b200.parallel.symm  # noqa: F401
    f = getattr(_lib(), fn_name)
    return f, f(cycles)


def test_oneshot_wait_runs_out_and_reports_the_missing_peer():
    lib = _lib()
    setter, old = _short_budget("xllm_comm_set_wait_budget")
    try:
        T = 8
        L = Local(1 << 17, world=2)          # rank 0 of a world of two whose rank 1 never shows up
        out = torch.empty(T, H, device="cuda", dtype=torch.bfloat16)
        rc = lib.xllm_tp_oneshot_norm(L.bufs.data_ptr(), L.pads.data_ptr(), 0, 0, 64, L.state.data_ptr(), None, None,
                                      None, out.data_ptr(), L.err.data_ptr(), T, H, 0, 2, 1e-6, 4, _s())
        assert rc == 0
        torch.cuda.synchronize()                       # the kernel returned by itself
        assert int(L.err.item()) == 301                # 300 + the peer whose flag never came
        ids = torch.empty(4, dtype=torch.int64, device="cuda")
        logits = torch.randn(4, 64, device="cuda", dtype=torch.bfloat16)
        L.err.zero_()
        rc = lib.xllm_tp_argmax(logits.data_ptr(), logits.stride(0), L.bufs.data_ptr(), L.pads.data_ptr(), 0, 96,
                                L.state.data_ptr() + 8, ids.data_ptr(), L.err.data_ptr(), 4, 64, 0, 1024, 0, 2, _s())
        assert rc == 0
        torch.cuda.synchronize()
        assert int(L.err.item()) == 401
        # the two-shot kernel: its opening flag exchange gives up the same way
        L.err.zero_()
        L2 = Local(2 * T * H * 2 + 512, world=2)
        rc = lib.xllm_tp_allreduce_norm(L2.bufs.data_ptr(), L2.pads.data_ptr(), 0, 0, T * H * 2, 0, L2.state.data_ptr(),
                                        None, None, L2.err.data_ptr(), T, H, 0, 2, 0, 0.0, 2, _s())
        assert rc == 0
        torch.cuda.synchronize()
        assert int(L2.err.item()) != 0
    finally:
        setter(old)
    # the context is intact: an ordinary kernel still runs
    assert float(torch.ones(8, device="cuda").sum().item()) == 8.0


def test_expert_parallel_barrier_wait_runs_out():
    lib = _lib()
    setter, old = _short_budget("xllm_ep_set_wait_budget")
    try:
        L = Local(1 << 16, world=2)
        rc = lib.xllm_ep_barrier(L.bufs.data_ptr(), L.pads.data_ptr(), 0, 1024, 2048, 0, L.state.data_ptr(),
                                 L.err.data_ptr(), 0, 2, 8, 64, 128, _s())
        assert rc == 0
        torch.cuda.synchronize()
        assert int(L.err.item()) == 2                  # 1 + the peer whose flag never came
    finally:
        setter(old)
    assert float(torch.ones(8, device="cuda").sum().item()) == 8.0
