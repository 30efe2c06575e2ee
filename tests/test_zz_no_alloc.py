"""The allocation-free decode attention entry point, called through its exported C symbol
(GPU).  Collected last on purpose: a run that stops at the first failure has then already
run every other test.

`ilb_attention_decode_static` serves callers that may not allocate device memory (a host
with a fixed memory budget, code between the capture and the replay of a CUDA graph, a
real-time loop, a C caller without torch): its scratch is a static array inside the
library.  The test itself is free to allocate its inputs; what it checks is that the entry
point needs no buffer from the caller, gives what `ilb_attention_decode` gives, twice in a
row with different batches (the array keeps the first call's contents), and refuses sizes
beyond its built-in limit.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _batch(seed, lens, nq, nkv, d, page):
    g = torch.Generator().manual_seed(seed)
    n_pages = sum(-(-n // page) for n in lens) + 2
    k_cache = torch.randn(n_pages, nkv, page, d, generator=g).to(torch.bfloat16).cuda()
    v_cache = torch.randn(n_pages, nkv, page, d, generator=g).to(torch.bfloat16).cuda()
    max_blocks = max(-(-n // page) for n in lens)
    table = torch.full((len(lens), max_blocks), -1, dtype=torch.int32)
    order = torch.randperm(n_pages, generator=g).tolist()
    for s, n in enumerate(lens):
        for b in range(-(-n // page)):
            table[s, b] = order.pop()
    q = torch.randn(len(lens), nq * d, generator=g).to(torch.bfloat16).cuda()
    positions = torch.tensor([n - 1 for n in lens], dtype=torch.int32).cuda()
    cu_q = torch.arange(len(lens) + 1, dtype=torch.int32).cuda()
    return q, k_cache, v_cache, table.cuda(), positions, cu_q


def _call_static(lib, q, out, k_cache, v_cache, positions, cu_q, table, nq, nkv, d, chunk, max_chunks):
    fn = lib.ilb_attention_decode_static
    fn.restype = ctypes.c_int
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    i = ctypes.c_int
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    return fn(p(q), p(out), p(k_cache), p(v_cache), p(positions), p(cu_q), p(table), i(table.shape[1]),
              i(k_cache.shape[2]), i(k_cache.shape[0]), i(0), ctypes.c_float(1.0 / math.sqrt(d)), i(q.shape[0]),
              i(nq), i(nkv), i(d), i(q.shape[1]), i(out.shape[1]), i(chunk), i(max_chunks), stream)


def test_static_entry_point_equals_the_ordinary_one_twice_in_a_row():
    from inferloop_b200.csrc import ops
    from inferloop_b200.csrc.build import load_module
    lib = load_module("attention_flash")
    nq, nkv, d, page, chunk = 8, 2, 64, 16, 256
    for seed, lens in ((1, [700, 3, 1030, 256, 257]), (2, [90, 1537, 64])):     # second call: other sizes, stale scratch
        q, k_cache, v_cache, table, positions, cu_q = _batch(seed, lens, nq, nkv, d, page)
        max_chunks = -(-table.shape[1] * page // chunk)
        want = torch.full((len(lens), nq * d), float("nan"), dtype=torch.bfloat16, device="cuda")
        scratch = torch.empty(len(lens) * nkv * max_chunks * (nq // nkv) * (d + 2), dtype=torch.float32, device="cuda")
        tickets = torch.zeros(len(lens) * nkv, dtype=torch.int32, device="cuda")
        ops.attention_decode(q, want, k_cache, v_cache, positions, cu_q, table, 0, 1.0 / math.sqrt(d), len(lens),
                             nq, nkv, d, chunk, max_chunks, scratch, tickets)
        got = torch.full_like(want, float("nan"))
        rc = _call_static(lib, q, got, k_cache, v_cache, positions, cu_q, table, nq, nkv, d, chunk, max_chunks)
        assert rc == 0, lib.ilb_last_error().decode()
        torch.cuda.synchronize()
        assert torch.isfinite(got.float()).all()
        # the kernels' own tolerance: 2^-8 * (|ref| + max|v|); the two paths run the same
        # kernel with the same cut of the keys, so in practice they agree to the bit
        err = (got.double() - want.double()).abs()
        bound = (2.0 ** -8) * (want.double().abs() + float(v_cache.float().abs().max()))
        assert (err <= bound).all(), err.max().item()


def test_static_entry_point_refuses_what_exceeds_its_array():
    from inferloop_b200.csrc.build import load_module
    lib = load_module("attention_flash")
    nq, nkv, d, page, chunk = 32, 8, 128, 16, 256
    q, k_cache, v_cache, table, positions, cu_q = _batch(3, [20] * 4, nq, nkv, d, page)
    out = torch.empty(4, nq * d, dtype=torch.bfloat16, device="cuda")
    rc = _call_static(lib, q, out, k_cache, v_cache, positions, cu_q, table, nq, nkv, d, chunk, 4096)
    assert rc != 0 and "exceed the built-in" in lib.ilb_last_error().decode()
