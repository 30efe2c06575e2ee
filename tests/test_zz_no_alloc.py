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


def _gather(cache, table, seq, n, page):
    """Keys (or values) [n, nkv, d] of one sequence, read back through its block table."""
    rows = [cache[int(table[seq, t // page]), :, t % page, :] for t in range(n)]
    return torch.stack(rows).double().cpu()


def _plain(q, k_cache, v_cache, table, lens, nq, nkv, d, page):
    """64-bit softmax attention of every sequence's one query over its keys (the formula of
    crates/testing/cpu/reference-ops/src/kernels.rs:251-297), sharing nothing with the kernel."""
    out = torch.zeros(len(lens), nq * d, dtype=torch.float64)
    tab = table.cpu()
    for s, n in enumerate(lens):
        k, v = _gather(k_cache, tab, s, n, page), _gather(v_cache, tab, s, n, page)
        for h in range(nq):
            kh = h // (nq // nkv)
            scores = (k[:, kh] @ q[s].double().cpu().view(nq, d)[h]) / math.sqrt(d)
            out[s, h * d:(h + 1) * d] = torch.softmax(scores, 0) @ v[:, kh]
    return out


def test_static_entry_point_equals_the_ordinary_one_twice_in_a_row():
    from inferloop_b200.csrc import ops
    from inferloop_b200.csrc.build import load_module
    lib = load_module("attention_flash")
    nq, nkv, d, page, chunk = 8, 2, 64, 16, 256
    # The second call uses fewer (sequence, kv head) pairs and fewer chunks than the first, so
    # records and counters of the first call lie beyond what it touches.
    for seed, lens in ((1, [700, 3, 1030, 256, 257]), (2, [90, 1537, 64])):
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
        # the kernels' own tolerance: 2^-8 * (|ref| + max|v|)
        vmax = float(v_cache.float().abs().max())
        err = (got.double() - want.double()).abs()
        assert (err <= (2.0 ** -8) * (want.double().abs() + vmax)).all(), err.max().item()
        # and against a 64-bit statement of the formula that shares no code with either path
        ref = _plain(q, k_cache, v_cache, table, lens, nq, nkv, d, page)
        err = (got.double().cpu() - ref).abs()
        assert (err <= (2.0 ** -8) * (ref.abs() + vmax)).all(), err.max().item()


def test_static_entry_point_on_a_small_batch_after_a_large_one():
    """A call over many (sequence, kv head) pairs and chunks fills the built-in array; the
    next call uses a single sequence, so most of what the first left (records, and counters
    if any were left non-zero) lies around what it touches.  Both are checked against the
    64-bit formula, not against another entry point."""
    from inferloop_b200.csrc.build import load_module
    lib = load_module("attention_flash")
    nq, nkv, d, page, chunk = 12, 4, 32, 8, 256
    for seed, lens in ((5, [300, 600, 900, 1200, 50, 513]), (6, [1100])):
        q, k_cache, v_cache, table, positions, cu_q = _batch(seed, lens, nq, nkv, d, page)
        max_chunks = -(-table.shape[1] * page // chunk)
        got = torch.full((len(lens), nq * d), float("nan"), dtype=torch.bfloat16, device="cuda")
        rc = _call_static(lib, q, got, k_cache, v_cache, positions, cu_q, table, nq, nkv, d, chunk, max_chunks)
        assert rc == 0, lib.ilb_last_error().decode()
        torch.cuda.synchronize()
        ref = _plain(q, k_cache, v_cache, table, lens, nq, nkv, d, page)
        err = (got.double().cpu() - ref).abs()
        assert (err <= (2.0 ** -8) * (ref.abs() + float(v_cache.float().abs().max()))).all(), err.max().item()


def test_both_entry_points_refuse_grids_that_would_write_outside_or_never_finish():
    """Host-side refusals, before any launch: too few chunks for the keys the block tables
    can name (the row would never be written), and more (head, chunk) weights than the
    kernel's shared memory holds."""
    from inferloop_b200.csrc.build import load_module
    lib = load_module("attention_flash")
    nq, nkv, d, page, chunk = 16, 1, 32, 16, 256
    q, k_cache, v_cache, table, positions, cu_q = _batch(7, [600], nq, nkv, d, page)
    out = torch.zeros(1, nq * d, dtype=torch.bfloat16, device="cuda")
    need = -(-table.shape[1] * page // chunk)
    rc = _call_static(lib, q, out, k_cache, v_cache, positions, cu_q, table, nq, nkv, d, chunk, need - 1)
    assert rc != 0 and "do not cover" in lib.ilb_last_error().decode()
    # 16 heads a group x 400 chunks x 4 bytes > the 20 KiB the head size 32 kernel has
    rc = _call_static(lib, q, out, k_cache, v_cache, positions, cu_q, table, nq, nkv, d, chunk, 400)
    assert rc != 0 and "merge weights" in lib.ilb_last_error().decode()
    torch.cuda.synchronize()
    assert float(out.float().abs().max()) == 0.0        # nothing was launched


def test_static_entry_point_refuses_what_exceeds_its_array():
    from inferloop_b200.csrc.build import load_module
    lib = load_module("attention_flash")
    nq, nkv, d, page, chunk = 32, 8, 128, 16, 256
    q, k_cache, v_cache, table, positions, cu_q = _batch(3, [20] * 4, nq, nkv, d, page)
    out = torch.empty(4, nq * d, dtype=torch.bfloat16, device="cuda")
    rc = _call_static(lib, q, out, k_cache, v_cache, positions, cu_q, table, nq, nkv, d, chunk, 4096)
    assert rc != 0 and "exceed the built-in" in lib.ilb_last_error().decode()
