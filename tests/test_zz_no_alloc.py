"""The allocation-free decode-attention entry point, called through its exported C symbol.

Some hosts of this library cannot allocate device memory when they need attention (they run inside
another runtime's memory pool, or in a loop that must stay out of the allocator), so they cannot
supply the split-KV workspace.  `xllm_paged_decode_attn_noalloc` keeps that workspace in an array
built into the library.  Here it must agree with the regular entry point (which takes the
workspace from the caller) on two calls in a row that share the built-in array, and it must refuse
a request that does not fit.

The file name sorts last on purpose: with `-x`, every other test has run before this one.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

P, I, L, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float


def _lib():
    from xllm_b200.ops import _lib as loader
    if not loader.lib_path().exists():
        loader.load()                                  # builds the library in-tree
    lib = ctypes.CDLL(str(loader.lib_path()))          # a plain handle: the entry point is C ABI, no Python layer
    lib.xllm_paged_decode_attn_noalloc.argtypes = [P, P, L, P, P, P, I, P, I, I, I, I, I, F, I, P]
    lib.xllm_paged_decode_attn_noalloc.restype = I
    lib.xllm_paged_decode_attn.argtypes = [P, P, L, P, P, P, I, P, I, I, I, I, I, F, I, P, P]
    lib.xllm_paged_decode_attn.restype = I
    lib.xllm_no_alloc_last_error.restype = ctypes.c_char_p
    return lib


def _case(seed, B, nq, nkv, d, page, lens):
    g = torch.Generator(device="cuda").manual_seed(seed)
    max_blocks = max((n + page - 1) // page for n in lens) + 1
    nb = B * max_blocks + 1
    kc = torch.randn(nb, nkv, page, d, device="cuda", dtype=torch.bfloat16, generator=g)
    vc = torch.randn(nb, nkv, page, d, device="cuda", dtype=torch.bfloat16, generator=g)
    bt = (torch.randperm(nb - 1, device="cuda", generator=g)[: B * max_blocks] + 1).view(B, max_blocks).to(torch.int32)
    q = torch.randn(B, nq, d, device="cuda", dtype=torch.bfloat16, generator=g)
    sl = torch.tensor(lens, device="cuda", dtype=torch.int32)
    return q, kc, vc, bt, sl


def test_noalloc_decode_matches_regular_entry_point_twice():
    from xllm_b200.ops import _lib as loader
    loader.load()  # builds the library when it is missing
    lib = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    # two different problems back to back: the second call reuses the built-in scratch array with
    # whatever the first one left in it
    for seed, (B, nq, nkv, d, page, splits, lens) in enumerate([
            (5, 32, 8, 128, 16, 4, [700, 33, 1, 1024, 257]),
            (3, 16, 2, 64, 32, 6, [90, 2000, 513])]):
        q, kc, vc, bt, sl = _case(seed, B, nq, nkv, d, page, lens)
        scale = 1.0 / math.sqrt(d)
        out_a = torch.zeros_like(q)
        out_b = torch.zeros_like(q)
        ws = torch.empty(B * nq * splits * (d + 1), dtype=torch.float32, device="cuda")
        rc = lib.xllm_paged_decode_attn(out_a.data_ptr(), q.data_ptr(), q.stride(0), kc.data_ptr(), vc.data_ptr(),
                                        bt.data_ptr(), bt.stride(0), sl.data_ptr(), B, nq, nkv, d, page, scale,
                                        splits, ws.data_ptr(), stream)
        assert rc == 0
        rc = lib.xllm_paged_decode_attn_noalloc(out_b.data_ptr(), q.data_ptr(), q.stride(0), kc.data_ptr(),
                                                vc.data_ptr(), bt.data_ptr(), bt.stride(0), sl.data_ptr(), B, nq,
                                                nkv, d, page, scale, splits, stream)
        assert rc == 0, lib.xllm_no_alloc_last_error()
        torch.cuda.synchronize()
        # the two entry points launch the same kernels on the same inputs; only the address of the
        # scratch differs, so the outputs agree bit for bit (well inside the 2e-2 of the numerics tests)
        assert torch.equal(out_a, out_b), (out_a.float() - out_b.float()).abs().max().item()
        assert torch.isfinite(out_b.float()).all()


def test_noalloc_refuses_oversized_request():
    lib = _lib()
    q, kc, vc, bt, sl = _case(0, 2, 8, 2, 128, 16, [40, 50])
    out = torch.zeros_like(q)
    # claim a batch whose scratch (4096 x 8 x 16 x 129 x 4 bytes = 270 MB) cannot fit in 8 MiB;
    # the call must return before touching any pointer
    rc = lib.xllm_paged_decode_attn_noalloc(out.data_ptr(), q.data_ptr(), q.stride(0), kc.data_ptr(), vc.data_ptr(),
                                            bt.data_ptr(), bt.stride(0), sl.data_ptr(), 4096, 8, 2, 128, 16, 0.1,
                                            16, torch.cuda.current_stream().cuda_stream)
    assert rc == -2
    assert b"scratch" in lib.xllm_no_alloc_last_error()
    # arguments are checked before any CUDA call: an unsupported head size and a negative batch
    for bad in (dict(d=96), dict(batch=-4)):
        a = dict(batch=2, d=128)
        a.update(bad)
        rc = lib.xllm_paged_decode_attn_noalloc(out.data_ptr(), q.data_ptr(), q.stride(0), kc.data_ptr(), vc.data_ptr(),
                                                bt.data_ptr(), bt.stride(0), sl.data_ptr(), a["batch"], 8, 2, a["d"], 16,
                                                0.1, 2, torch.cuda.current_stream().cuda_stream)
        assert rc > 0 and b"bad argument" in lib.xllm_no_alloc_last_error()
    torch.cuda.synchronize()
