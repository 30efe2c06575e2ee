"""Each kernel alone against a plain 64-bit statement of the same operation, at sizes
other than the engine configurations' (GPU)."""
import math
import random

import pytest
import torch

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def tol(dtype, ref, scale=1.0):
    """float32: 1e-5 + 1e-5 |ref|; bfloat16 outputs: one rounding of the result (2^-8
    relative) on top of that."""
    if dtype == "float32":
        return 1e-5 * scale + 1e-5 * ref.abs()
    return 1e-5 * scale + (2.0 ** -8) * ref.abs() + 2.0 ** -8 * scale * 0.05


def close(got, ref, dtype, scale=1.0, what=""):
    got, ref = got.double().cpu(), ref.double().cpu()
    err = (got - ref).abs()
    bad = err > tol(dtype, ref, scale)
    assert not bad.any(), f"{what}: {int(bad.sum())} bad, max err {err.max().item():.3e} at {torch.nonzero(bad)[0].tolist()}"


def ops():
    from inferloop_b200.csrc import ops as o
    return o


@pytest.mark.parametrize("table_dtype", ["float32", "bfloat16"])
def test_embed(table_dtype):
    V, H = 517, 72
    table = torch.randn(V, H).to(DT[table_dtype])
    tokens = torch.tensor([0, 516, 3, 3, 100], dtype=torch.int32)
    out = torch.empty(5, H, device="cuda")
    ops().embed(tokens.cuda(), table.cuda(), out)
    assert torch.equal(out.cpu(), table.float()[tokens.long()])


@pytest.mark.parametrize("width,rows,eps", [(72, 5, 1e-6), (100, 3, 1e-5), (4096, 2, 1e-6), (5120, 1, 1e-6), (48, 17, 3e-6)])
@pytest.mark.parametrize("out_dtype", ["float32", "bfloat16"])
def test_rmsnorm(width, rows, eps, out_dtype):
    x = torch.randn(rows, width) * 3
    w = 1 + 0.1 * torch.randn(width)
    out = torch.empty(rows, width, dtype=DT[out_dtype], device="cuda")
    ops().rmsnorm(x.cuda(), w.cuda(), eps, out)
    xd = x.double()
    ref = xd / torch.sqrt((xd * xd).mean(-1, keepdim=True) + eps) * w.double()
    close(out, ref, out_dtype, what="rmsnorm")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_silu_mul(dtype):
    rows, width = 7, 176
    gu = (torch.randn(rows, 2 * width) * 4).to(DT[dtype])
    gu[0, 0], gu[0, 1] = 80.0, -80.0          # far tails must not overflow
    out = torch.empty(rows, width, dtype=DT[dtype], device="cuda")
    ops().silu_mul(gu.cuda(), out)
    g, u = gu.double()[:, :width], gu.double()[:, width:]
    close(out, g * torch.sigmoid(g) * u, dtype, what="silu_mul")
    assert torch.isfinite(out).all()


def test_gather_rows_and_rope_table():
    x = torch.randn(9, 40)
    idx = torch.tensor([8, 0, 3, 3], dtype=torch.int32)
    out = torch.empty(4, 40, device="cuda")
    ops().gather_rows(x.cuda(), idx.cuda(), out)
    assert torch.equal(out.cpu(), x[idx.long()])
    pos = torch.tensor([0, 1, 77, 4095, 131071], dtype=torch.int32)
    for theta, rd in ((10000.0, 16), (1e6, 128), (50000.0, 24)):
        inv = torch.tensor([theta ** (-(2.0 * i) / rd) for i in range(rd // 2)], dtype=torch.float64)
        table = torch.empty(5, rd // 2, 2, device="cuda")
        ops().rope_table(pos.cuda(), inv.cuda(), table)
        angle = pos.double()[:, None] * inv[None, :]
        ref = torch.stack([torch.cos(angle), torch.sin(angle)], -1)
        assert (table.double().cpu() - ref).abs().max() < 1e-7      # one rounding to 32-bit


# (K = 70, 50: rows that are no multiple of 16 bytes take the kernel that reads element by element)
@pytest.mark.parametrize("M,N,K", [(1, 96, 64), (5, 100, 72), (16, 515, 80), (17, 64, 200), (130, 224, 96), (64, 1000, 1024),
                                   (3, 50, 70), (40, 70, 50), (8, 300, 4096), (300, 260, 1040)])
@pytest.mark.parametrize("in_dtype,out_dtype", [("float32", "float32"), ("bfloat16", "bfloat16"), ("bfloat16", "float32")])
@pytest.mark.parametrize("bias,accumulate", [(False, False), (True, True)])
def test_gemm_simt(M, N, K, in_dtype, out_dtype, bias, accumulate):
    if accumulate and out_dtype != "float32":
        pytest.skip("accumulation needs a 32-bit output")
    a = torch.randn(M, K).to(DT[in_dtype])
    w = (torch.randn(N, K) * 0.05).to(DT[in_dtype])
    b = torch.randn(N) if bias else None
    base = torch.randn(M, N)
    out = base.clone().to(DT[out_dtype]).cuda() if accumulate else torch.empty(M, N, dtype=DT[out_dtype], device="cuda")
    ops().gemm_simt(a.cuda(), w.cuda(), out, None if b is None else b.cuda(), accumulate)
    ref = a.double() @ w.double().T
    if bias:
        ref = ref + b.double()
    if accumulate:
        ref = ref + base.double()
    close(out, ref, out_dtype, scale=float(ref.abs().max()), what="gemm")


def test_gemm_simt_rows_do_not_depend_on_the_batch():
    """The same row gives the same bits alone, among 5 rows and among 100 rows."""
    K, N = 136, 200
    a = torch.randn(100, K).cuda()
    w = torch.randn(N, K).cuda()
    outs = []
    for M in (1, 5, 16, 17, 100):
        out = torch.empty(M, N, device="cuda")
        ops().gemm_simt(a[:M].contiguous(), w, out)
        outs.append(out[0].clone())
    for o in outs[1:]:
        assert torch.equal(o, outs[0])


@pytest.mark.parametrize("M", [4, 40])
def test_gemm_simt_kernels_agree_bit_for_bit(M):
    """Operands that start on a 16-byte boundary take the kernels that read four k at a time,
    others the kernel that reads element by element: the sums are the same chains in the same
    order, so the same numbers give the same bits."""
    K, N = 136, 200
    torch.manual_seed(M)
    a = torch.randn(M, K).cuda()
    w = torch.randn(N, K).cuda()
    out = torch.empty(M, N, device="cuda")
    ops().gemm_simt(a, w, out)
    shifted_a = torch.empty(M * K + 1, device="cuda")[1:].view(M, K)       # 4 bytes past a 16-byte boundary
    shifted_a.copy_(a)
    shifted_w = torch.empty(N * K + 1, device="cuda")[1:].view(N, K)
    shifted_w.copy_(w)
    assert shifted_a.data_ptr() % 16 != 0 and shifted_w.data_ptr() % 16 != 0
    out2 = torch.empty(M, N, device="cuda")
    ops().gemm_simt(shifted_a, shifted_w, out2)
    assert torch.equal(out, out2)


# ------------------------------------------------------------------ attention pieces
def build_cache(seqs_kv, nkv, d, page_size, num_pages, dtype, seed=0, page_order="shuffled"):
    """Scatter each sequence's keys/values into pages; returns cache tensors and the block
    table [S, max_blocks].  `page_order`: "shuffled", "ordered" (a sequence's pages follow
    one another in the pool, as a fresh pool hands them out) or "mixed" (ordered with every
    fifth pair of neighbours swapped, so that runs and broken runs alternate)."""
    rng = random.Random(seed)
    pages = list(range(num_pages))
    if page_order == "shuffled":
        rng.shuffle(pages)
    else:
        pages.reverse()                       # pop() hands out 0, 1, 2, ...
        if page_order == "mixed":
            for i in range(3, num_pages - 1, 5):
                pages[i], pages[i + 1] = pages[i + 1], pages[i]
    k_cache = torch.full((num_pages, nkv, page_size, d), 7.0)      # stale contents must not matter
    v_cache = torch.full((num_pages, nkv, page_size, d), -9.0)
    max_blocks = max(-(-k.shape[0] // page_size) for k, _ in seqs_kv)
    table = torch.full((len(seqs_kv), max_blocks), -1, dtype=torch.int32)
    for s, (k, v) in enumerate(seqs_kv):
        for b in range(-(-k.shape[0] // page_size)):
            page = pages.pop()
            table[s, b] = page
            n = min(page_size, k.shape[0] - b * page_size)
            k_cache[page, :, :n] = k[b * page_size:b * page_size + n].transpose(0, 1)
            v_cache[page, :, :n] = v[b * page_size:b * page_size + n].transpose(0, 1)
    return k_cache.to(dtype), v_cache.to(dtype), table


def ref_attention(q, k, v, pos, window):
    """q [nq, d] at position pos over keys k, v [n, nkv, d] (64-bit)."""
    nq, d = q.shape
    nkv = k.shape[1]
    lo = max(0, pos + 1 - window) if window else 0
    out = torch.zeros(nq, d, dtype=torch.float64)
    for h in range(nq):
        kh = h // (nq // nkv)
        s = (k[lo:pos + 1, kh] @ q[h]) / math.sqrt(d)
        out[h] = torch.softmax(s, 0) @ v[lo:pos + 1, kh]
    return out


@pytest.mark.parametrize("nq,nkv,d,page_size,window", [(4, 2, 16, 4, 0), (6, 2, 32, 8, 0), (5, 5, 48, 16, 20),
                                                         (8, 1, 80, 16, 0), (3, 3, 256, 32, 33), (32, 8, 128, 16, 0)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_paged_attention_mixed_batch(nq, nkv, d, page_size, window, dtype):
    """Three sequences: a whole prompt, a portion that starts mid-sequence, one decode
    token; pages shuffled; compared per token with the plain softmax."""
    torch.manual_seed(nq * 100 + d)
    lens = [37, 90, 131]                  # keys in the cache after the step
    q_lens = [37, 23, 1]                  # tokens of this step
    seqs = [(torch.randn(n, nkv, d).to(DT[dtype]).double(), torch.randn(n, nkv, d).to(DT[dtype]).double()) for n in lens]
    k_cache, v_cache, table = build_cache([(k.float(), v.float()) for k, v in seqs], nkv, d, page_size, 72, DT[dtype])
    T = sum(q_lens)
    q = (torch.randn(T, nq * d)).to(DT[dtype])
    positions, seq_of = [], []
    for s, (n, ql) in enumerate(zip(lens, q_lens)):
        positions += list(range(n - ql, n))
        seq_of += [s] * ql
    out = torch.empty(T, nq * d, dtype=DT[dtype], device="cuda")
    ops().paged_attention_simple(q.cuda(), out, k_cache.cuda(), v_cache.cuda(),
                                 torch.tensor(positions, dtype=torch.int32).cuda(),
                                 torch.tensor(seq_of, dtype=torch.int32).cuda(), table.cuda(),
                                 window, 1.0 / math.sqrt(d), nq, nkv, d)
    ref = torch.stack([ref_attention(q[t].double().view(nq, d), *seqs[seq_of[t]], positions[t], window).reshape(-1)
                       for t in range(T)])
    close(out, ref, dtype, scale=1.0, what="attention")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_finds_one_far_key_and_respects_the_window_edge(dtype):
    """One key among hundreds is made to dominate; the output must be its value.  With a
    window, a dominant key just outside must be ignored and one just inside found."""
    nq, nkv, d, page = 2, 1, 32, 16
    n = 700
    torch.manual_seed(1)
    k = torch.randn(n, nkv, d) * 0.1
    v = torch.arange(n, dtype=torch.float32)[:, None, None].expand(n, nkv, d).clone()   # value = its position
    qv = torch.randn(nq * d) * 0.1
    for far, window, expect in ((13, 0, 13.0), (699 - 50 + 1, 50, 650.0), (699 - 50, 50, None), (352, 0, 352.0)):
        kk = k.clone()
        direction = torch.randn(d)
        direction /= direction.norm()
        kk[far, 0] = direction * 40
        q = qv.clone().view(nq, d)
        q[:] = direction * 40                   # score 1600 / sqrt(32): everything else vanishes
        k_cache, v_cache, table = build_cache([(kk, v)], nkv, d, page, 64, DT[dtype], seed=far)
        out = torch.empty(1, nq * d, dtype=DT[dtype], device="cuda")
        ops().paged_attention_simple(q.reshape(1, -1).to(DT[dtype]).cuda(), out, k_cache.cuda(), v_cache.cuda(),
                                     torch.tensor([n - 1], dtype=torch.int32).cuda(),
                                     torch.tensor([0], dtype=torch.int32).cuda(), table.cuda(),
                                     window, 1.0 / math.sqrt(d), nq, nkv, d)
        got = out.float().cpu()
        if expect is not None:
            assert torch.allclose(got, torch.full_like(got, expect), rtol=2.0 ** -8), (far, window, got[0, :4])
        else:       # the dominant key is outside: the result is an average over the window
            assert 650.0 <= got.min().item() and got.max().item() <= 699.0


@pytest.mark.parametrize("nq,nkv,d,rd,page_size", [(4, 2, 16, 16, 4), (6, 2, 32, 32, 8), (5, 5, 48, 24, 16), (8, 2, 128, 128, 16), (2, 1, 80, 80, 32),
                                                    (3, 1, 128, 128, 32), (26, 2, 128, 128, 16), (8, 2, 128, 64, 16), (64, 8, 128, 128, 16), (40, 8, 128, 128, 16)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("use_norm", [True, False])
def test_qk_norm_rope_cache(nq, nkv, d, rd, page_size, dtype, use_norm):
    torch.manual_seed(d)
    T, S = 11, 2
    eps, theta = 1e-5, 1e6
    width = (nq + 2 * nkv) * d
    qkv = torch.randn(T, width).to(DT[dtype])
    qw, kw = 1 + 0.1 * torch.randn(d), 1 + 0.1 * torch.randn(d)
    positions = torch.tensor([5, 6, 7, 8, 9, 10, 11, 40, 41, 42, 43], dtype=torch.int32)
    seq_of = torch.tensor([0] * 7 + [1] * 4, dtype=torch.int32)
    num_pages = 24
    max_blocks = -(-44 // page_size)
    perm = torch.randperm(num_pages)[:S * max_blocks].to(torch.int32).view(S, max_blocks)
    inv = torch.tensor([theta ** (-(2.0 * i) / rd) for i in range(rd // 2)], dtype=torch.float64)
    table = torch.empty(T, rd // 2, 2, device="cuda")
    ops().rope_table(positions.cuda(), inv.cuda(), table)
    k_cache = torch.zeros(num_pages, nkv, page_size, d, dtype=DT[dtype], device="cuda")
    v_cache = torch.zeros_like(k_cache)
    q_out = torch.empty(T, nq * d, dtype=DT[dtype], device="cuda")
    ops().qk_norm_rope_cache(qkv.cuda(), q_out, qw.cuda() if use_norm else None, kw.cuda() if use_norm else None,
                             eps, table, rd, positions.cuda(), seq_of.cuda(), perm.cuda(), page_size,
                             k_cache, v_cache, nq, nkv, d)
    x = qkv.double()
    q, k, v = x[:, :nq * d].view(T, nq, d), x[:, nq * d:(nq + nkv) * d].view(T, nkv, d), x[:, (nq + nkv) * d:].view(T, nkv, d)

    def norm(t, w):
        return t / torch.sqrt((t * t).mean(-1, keepdim=True) + eps) * w.double() if use_norm else t

    def rope(t):
        half = rd // 2
        ang = positions.double()[:, None] * inv[None, :]
        c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        out = t.clone()
        a, b = t[..., :half], t[..., half:rd]
        out[..., :half] = a * c - b * s
        out[..., half:rd] = a * s + b * c
        return out

    q_ref, k_ref = rope(norm(q, qw)), rope(norm(k, kw))
    close(q_out.view(T, nq, d), q_ref, dtype, scale=float(q_ref.abs().max()), what="q")
    kc, vc = k_cache.double().cpu(), v_cache.double().cpu()
    written = torch.zeros(num_pages, page_size, dtype=torch.bool)
    for t in range(T):
        p = int(positions[t]); page = int(perm[seq_of[t], p // page_size]); slot = p % page_size
        close(kc[page, :, slot], k_ref[t], dtype, scale=float(k_ref.abs().max()), what=f"k token {t}")
        close(vc[page, :, slot], v[t], dtype, scale=float(v.abs().max()), what=f"v token {t}")
        written[page, slot] = True
    assert (kc.abs().sum((1, 3))[~written] == 0).all(), "a slot no token owns was written"


def test_kernels_refuse_what_they_cannot_do():
    from inferloop_b200.csrc.ops import KernelError
    o = ops()
    with pytest.raises(KernelError, match="CUDA only"):
        o.rmsnorm(torch.randn(2, 8), torch.ones(8), 1e-6, torch.empty(2, 8))
    q = torch.randn(1, 2 * 272, device="cuda")
    kc = torch.zeros(2, 1, 16, 272, device="cuda")
    with pytest.raises(KernelError, match="head size"):
        o.paged_attention_simple(q, torch.empty_like(q), kc, kc, torch.zeros(1, dtype=torch.int32, device="cuda"),
                                 torch.zeros(1, dtype=torch.int32, device="cuda"),
                                 torch.zeros(1, 1, dtype=torch.int32, device="cuda"), 0, 1.0, 2, 1, 272)
    with pytest.raises(KernelError, match="multiple"):
        kc = torch.zeros(2, 2, 16, 16, device="cuda")
        q = torch.randn(1, 3 * 16, device="cuda")
        o.paged_attention_simple(q, torch.empty_like(q), kc, kc, torch.zeros(1, dtype=torch.int32, device="cuda"),
                                 torch.zeros(1, dtype=torch.int32, device="cuda"),
                                 torch.zeros(1, 1, dtype=torch.int32, device="cuda"), 0, 1.0, 3, 2, 16)


# ------------------------------------------------------------------ tensor-core GEMM
# (256, 19200, 64) and (300, 9728, 128): one whole-tile round, then 2 tiles of 1-2 K blocks
# shared by far fewer CTAs than the grid holds
TC_SHAPES = [(256, 19200, 64), (300, 9728, 128), (1, 128, 64), (3, 200, 72), (8, 512, 4096), (16, 4096, 1024), (17, 300, 136), (33, 96, 512),
             (64, 1000, 1024), (65, 256, 256), (128, 384, 320), (129, 520, 264), (300, 515 * 1 + 5, 96), (512, 1024, 2048),
             # few tiles of many tokens: the K ranges of a tile run as a cluster that shares the write-out
             (200, 700, 1024), (129, 256, 1024), (256, 4096, 1024), (500, 1100, 4096), (1024, 520, 512),
             # 256 x 192 and 256 x 256 tiles in whole rounds, a last round that is not full
             (2048, 6144, 256), (1500, 4100, 192),
             # accumulating: whole rounds and 12 tiles dealt out by K blocks; fewer tiles than SMs, all
             # dealt out by K blocks; one row block per tile.  The K ranges of a tile are added in memory.
             (2048, 5120, 512), (512, 4096, 2048), (200, 1024, 4096),
             # 128 x 192 tiles: 128 of them where 256-wide ones would be 96
             (512, 6144, 320),
             # 65 to 128 tokens into a wide output: accumulating, tokens go on the MMA's rows and the K ranges meet in memory
             (100, 4096, 1024), (72, 5120, 2048)]


@pytest.mark.parametrize("M,N,K", TC_SHAPES)
@pytest.mark.parametrize("out_dtype,bias,accumulate", [("bfloat16", False, False), ("float32", True, True), ("float32", False, False)])
def test_gemm_tcgen05(M, N, K, out_dtype, bias, accumulate):
    o = ops()
    torch.manual_seed(M * 7 + N)
    a = torch.randn(M, K).to(torch.bfloat16)
    w = (torch.randn(N, K) * 0.05).to(torch.bfloat16)
    b = torch.randn(N) if bias else None
    base = torch.randn(M, N)
    out = base.clone().cuda() if accumulate else torch.full((M, N), float("nan"), dtype=DT[out_dtype], device="cuda")
    assert o.gemm_tc_eligible(a.cuda(), w.cuda(), out)
    o.gemm_tc(a.cuda(), w.cuda(), out, None if b is None else b.cuda(), accumulate)
    o.check_device_errors()
    ref = a.double() @ w.double().T
    if bias:
        ref = ref + b.double()
    if accumulate:
        ref = ref + base.double()
    close(out, ref, out_dtype, scale=float(ref.abs().max()), what=f"gemm_tc {M}x{N}x{K}")


@pytest.mark.parametrize("epilogue", ["store_bf16", "store_f32", "accumulate", "accumulate_bias", "store_bias", "swiglu"])
@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (300, 520, 264), (100, 1000, 512), (512, 768, 2048), (1100, 384, 4096),
                                   (2048, 1280, 1024), (129, 256, 8), (2048, 7168, 128)])
def test_gemm_tcgen05_on_pairs_of_ctas(M, N, K, epilogue):
    """The 256 x 256 tiles of a pair of CTAs (one MMA unit over two SMs), forced at sizes
    where the launcher would not choose them: token tiles whose second half lies partly or
    wholly beyond M, widths and depths that fill no tile, every epilogue, K long enough
    that the accumulating products cut a tile into ranges that meet in memory, and (the last
    shape: 224 tiles) four tiles per pair, so that both accumulators and every barrier are
    used a second time."""
    o = ops()
    swiglu = epilogue == "swiglu"
    if swiglu and N % 128:
        N = (N + 127) // 128 * 128
    torch.manual_seed(M + N + K)
    a = torch.randn(M, K).to(torch.bfloat16)
    w = (torch.randn(N, K) * 0.05).to(torch.bfloat16)
    b = torch.randn(N) if epilogue.endswith("bias") else None
    base = torch.randn(M, N)
    ref = a.double() @ w.double().T
    if b is not None:
        ref = ref + b.double()
    if swiglu:
        g = ref.view(M, N // 128, 2, 64)
        ref = (torch.nn.functional.silu(g[:, :, 0]) * g[:, :, 1]).reshape(M, N // 2)
        out = torch.full((M, N // 2), float("nan"), dtype=torch.bfloat16, device="cuda")
    elif epilogue.startswith("accumulate"):
        ref = ref + base.double()
        out = base.clone().cuda()
    else:
        out = torch.full((M, N), float("nan"), dtype=torch.float32 if epilogue == "store_f32" else torch.bfloat16, device="cuda")
    o.gemm_pairs(2)
    try:
        plan = o.gemm_tc_plan(M, N, K, accumulate=epilogue.startswith("accumulate"), swiglu=swiglu)
        if M > 128:
            assert plan["pairs"] >= 1 and (plan["pair_split"] == 1 or epilogue.startswith("accumulate")), plan
        o.gemm_tc(a.cuda(), w.cuda(), out, None if b is None else b.cuda(), accumulate=epilogue.startswith("accumulate"), swiglu=swiglu)
        o.check_device_errors()
    finally:
        o.gemm_pairs(1)
    close(out, ref, "float32" if out.dtype == torch.float32 else "bfloat16", scale=float(ref.abs().max()), what=f"gemm on pairs {M}x{N}x{K} {epilogue}")


@pytest.mark.parametrize("max_ctas", [0, 1, 3, 7, 50])
@pytest.mark.parametrize("M,N,K", [(8, 640, 2048), (200, 700, 1024)])
def test_gemm_tcgen05_shared_tiles_are_deterministic_and_reusable(max_ctas, M, N, K):
    """However the K blocks of a tile are shared among CTAs, the shares are added in K
    order by whichever CTA arrives last: runs give the same bits, and the tickets are back
    at zero for the next launch."""
    o = ops()
    torch.manual_seed(max_ctas + M)
    a = torch.randn(M, K).to(torch.bfloat16).cuda()
    w = (torch.randn(N, K) * 0.05).to(torch.bfloat16).cuda()
    outs = []
    for _ in range(3):
        out = torch.empty(M, N, device="cuda")
        o.gemm_tc(a, w, out, max_ctas=max_ctas)
        outs.append(out.clone())
    o.check_device_errors()
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    ref = a.double().cpu() @ w.double().cpu().T
    close(outs[0], ref, "float32", scale=float(ref.abs().max()), what="stream-k")
    from inferloop_b200.csrc.ops import _tc_state
    assert int(_tc_state(a.device).tickets.abs().sum()) == 0


def test_gemm_tcgen05_last_round_in_memory_can_be_switched_off():
    """Accumulating products of many tokens cut the tiles of their last round into K ranges
    that meet in memory; switched off, the same product runs whole tiles and gives the same
    bits every time.  Both agree with the plain product."""
    o = ops()
    M, N, K = 2048, 5120, 1024                  # 160 tiles of 256 x 256: one round and 12 tiles
    torch.manual_seed(5)
    a = torch.randn(M, K).to(torch.bfloat16).cuda()
    w = (torch.randn(N, K) * 0.05).to(torch.bfloat16).cuda()
    base = torch.randn(M, N).cuda()
    ref = base.double().cpu() + a.double().cpu() @ w.double().cpu().T
    assert o.gemm_tc_plan(M, N, K, accumulate=True)["sums_meet_in_memory"] == 1
    assert o.gemm_tc_plan(200, 256, 1024, accumulate=True)["sums_meet_in_memory"] == 0      # a handful of tiles: never
    few = o.gemm_tc_plan(100, 4096, 1024, accumulate=True)                                  # 65 to 128 tokens, a wide output
    assert few["sums_meet_in_memory"] == 1 and few["swap"] == 0 and few["row_blocks"] == 1
    assert o.gemm_tc_plan(64, 4096, 1024, accumulate=True)["swap"] == 1 and o.gemm_tc_plan(100, 4096, 1024)["swap"] == 1
    out = base.clone()
    o.gemm_tc(a, w, out, accumulate=True)
    close(out, ref, "float32", scale=float(ref.abs().max()), what="last round in memory")
    o.gemm_sums_in_memory(False)
    try:
        assert o.gemm_tc_plan(M, N, K, accumulate=True)["sums_meet_in_memory"] == 0
        outs = []
        for _ in range(3):
            out = base.clone()
            o.gemm_tc(a, w, out, accumulate=True)
            outs.append(out)
        assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
        close(outs[0], ref, "float32", scale=float(ref.abs().max()), what="whole tiles only")
    finally:
        o.gemm_sums_in_memory(True)
    o.check_device_errors()


@pytest.mark.parametrize("M", [1, 2, 4, 7, 8])
@pytest.mark.parametrize("N,K,bias", [(4096, 4096, False), (2048, 6144, True), (2560, 2048, False)])
def test_gemm_tcgen05_few_tokens_add_their_ranges_in_memory(M, N, K, bias):
    """Accumulating products of up to four tokens with a large weight: the K ranges of a tile
    are separate CTAs that add into the output.  Right against the 64-bit product; the bias is
    added once; switched off, the ranges meet inside a cluster again and runs give the same bits."""
    o = ops()
    torch.manual_seed(M + N)
    a = torch.randn(M, K).to(torch.bfloat16)
    w = (torch.randn(N, K) * 0.05).to(torch.bfloat16)
    b = torch.randn(N) if bias else None
    base = torch.randn(M, N)
    ref = base.double() + a.double() @ w.double().T + (b.double() if bias else 0)
    plan = o.gemm_tc_plan(M, N, K, accumulate=True)
    assert plan["swap"] == 1 and plan["sums_meet_in_memory"] == 1 and plan["cluster"] == 1 and plan["grid"] > plan["tiles"], plan
    assert o.gemm_tc_plan(16, N, K, accumulate=True)["sums_meet_in_memory"] == 0         # sixteen tokens keep the cluster
    assert o.gemm_tc_plan(M, 512, 512, accumulate=True)["sums_meet_in_memory"] == 0      # and so do small weights
    for _ in range(3):
        out = base.clone().cuda()
        o.gemm_tc(a.cuda(), w.cuda(), out, None if b is None else b.cuda(), accumulate=True)
        close(out, ref, "float32", scale=float(ref.abs().max()), what=f"few tokens in memory {M}x{N}x{K}")
    o.gemm_sums_in_memory(False)
    try:
        assert o.gemm_tc_plan(M, N, K, accumulate=True)["sums_meet_in_memory"] == 0
        outs = []
        for _ in range(3):
            out = base.clone().cuda()
            o.gemm_tc(a.cuda(), w.cuda(), out, None if b is None else b.cuda(), accumulate=True)
            outs.append(out)
        assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
        close(outs[0], ref, "float32", scale=float(ref.abs().max()), what="few tokens in a cluster")
    finally:
        o.gemm_sums_in_memory(True)
    o.check_device_errors()


def test_gemm_tuning_knobs_move_the_plan():
    """The knobs behind the measured defaults: how many tokens send their K ranges to memory,
    and how many ranges a tile of a pair may be cut into."""
    o = ops()
    try:
        assert o.gemm_tc_plan(2, 4096, 4096, accumulate=True)["sums_meet_in_memory"] == 1
        o.gemm_tuning(few_tokens_in_memory=0)
        few = o.gemm_tc_plan(2, 4096, 4096, accumulate=True)
        assert few["sums_meet_in_memory"] == 0 and few["cluster"] > 1
        o.gemm_tuning(few_tokens_in_memory=8)
        assert o.gemm_tc_plan(2, 4096, 4096, accumulate=True)["sums_meet_in_memory"] == 1
        assert o.gemm_tc_plan(2048, 5120, 5120, accumulate=True)["pair_split"] > 1
        o.gemm_tuning(pair_ranges=1)
        assert o.gemm_tc_plan(2048, 5120, 5120, accumulate=True)["pair_split"] <= 1
    finally:
        o.gemm_tuning(few_tokens_in_memory=8, pair_ranges=8)


def test_gemm_tcgen05_refuses_unaligned_rows():
    o = ops()
    a = torch.randn(4, 100).to(torch.bfloat16).cuda()       # 200-byte rows: not a multiple of 16
    w = torch.randn(32, 100).to(torch.bfloat16).cuda()
    out = torch.empty(4, 32, device="cuda")
    assert not o.gemm_tc_eligible(a, w, out)
    with pytest.raises(o.KernelError, match="multiples of 8"):
        o.gemm_tc(a, w, out)


def test_gemm_tcgen05_plans_cover_every_tile_once():
    """What the launcher decides for the layer shapes of a served model: few tokens put the
    weight on the MMA's rows and cut the K range of a tile over a cluster that fits the device
    at once; many tokens run whole tiles in rounds.  In every case tiles = whole + shared."""
    o = ops()
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    for M in (1, 8, 16, 33, 64, 128, 200, 384, 1024, 2048):
        for N, K, kw in ((6144, 4096, {}), (4096, 4096, {"accumulate": True}), (24576, 4096, {"swiglu": True}),
                         (4096, 12288, {"accumulate": True}), (151936, 4096, {})):
            plan = o.gemm_tc_plan(M, N, K, **kw)
            what = f"M={M} N={N} K={K}: {plan}"
            assert plan["swap"] == (1 if M <= 128 and (not plan["sums_meet_in_memory"] or M <= 8) else 0), what
            assert plan["cluster"] in (1, 2, 4, 8) and plan["grid"] % plan["cluster"] == 0, what
            assert 0 <= plan["tiles_stream_k"] <= plan["tiles"], what
            assert not plan["sums_meet_in_memory"] or (kw.get("accumulate") and (not plan["swap"] or M <= 8) and plan["cluster"] == 1), what
            assert 0 <= plan["pairs"] <= sms // 2 and (plan["pairs"] == 0 or (not plan["swap"] and 1 <= plan["pair_split"] <= 8)), what
            assert plan["pair_split"] <= 1 or kw.get("accumulate"), what             # only adding products are cut on pairs
            if plan["swap"]:
                assert plan["tile_n"] >= min(M, 128) and plan["grid"] <= 2 * sms, what
                if plan["cluster"] > 1:
                    assert plan["grid"] == plan["tiles"] * plan["cluster"], what
            else:
                assert plan["grid"] <= sms, what
                assert plan["rounds"] * plan["grid"] >= plan["tiles"] - plan["tiles_stream_k"], what
    # a prompt's worth of tokens runs on pairs of CTAs; a product with too few tiles for them does not
    assert o.gemm_tc_plan(2048, 24576, 4096, swiglu=True)["pairs"] > 0 and o.gemm_tc_plan(2048, 4096, 12288, accumulate=True)["pairs"] > 0
    assert o.gemm_tc_plan(512, 6144, 4096)["pairs"] == 0
    o.gemm_pairs(0)
    try:
        assert o.gemm_tc_plan(2048, 24576, 4096, swiglu=True)["pairs"] == 0
    finally:
        o.gemm_pairs(1)


def test_decode_attention_plan_keeps_the_launch_resident():
    o = ops()
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    last = 17
    for n_seqs in (1, 2, 4, 8, 16, 64, 256):
        split, stages, chunks = o.attention_decode_plan(n_seqs, 32, 8, 128, 16)
        assert 1 <= chunks <= 8 and (chunks == 1 or split == 16)
        assert split in (1, 2, 4, 8, 16) and stages in (3, 6, 12)
        assert split <= last                      # more sequences never widen the clusters
        assert split == 1 or split * n_seqs * 8 <= 4 * sms, (n_seqs, split, stages)
        last = split


# ------------------------------------------------------------------ tensor-core attention
def close_flash(got, ref, vmax, what):
    """The tensor-core kernels round the probabilities to bfloat16 before the value
    product (as the reference's grouped decode does), so each output carries up to
    2^-9 * sum_j p_j |v_j| <= 2^-9 * max|v| of error besides the rounding of the result:
    bound 2^-8 * (|ref| + max|v|)."""
    got, ref = got.double().cpu(), ref.double().cpu()
    assert torch.isfinite(got).all(), f"{what}: non-finite output"
    err = (got - ref).abs()
    bad = err > (2.0 ** -8) * (ref.abs() + vmax)
    assert not bad.any(), f"{what}: {int(bad.sum())} bad, max err {err.max().item():.3e} at {torch.nonzero(bad)[0].tolist()}"


class _Step:
    """The few batch facts the attention dispatcher reads."""

    def __init__(self, positions, seq_of, cu_q, q_lens):
        self.positions = torch.tensor(positions, dtype=torch.int32).cuda()
        self.seq_of_token = torch.tensor(seq_of, dtype=torch.int32).cuda()
        self.cu_q = torch.tensor(cu_q, dtype=torch.int32).cuda()
        self.h_q_len = list(q_lens)
        self.n_seqs = len(q_lens)
        self.decode_only = all(n == 1 for n in q_lens)


def run_flash(q, seqs, lens, q_lens, nq, nkv, d, page_size, window, chunk=256, seed=0, cluster=True,
              page_order="shuffled", release_passed_pages=False):
    """`cluster`: split-KV decode merges inside a thread-block cluster (the default of the
    dispatcher) or through scratch records and tickets.  `release_passed_pages`: pages that
    lie wholly below the window of the step's first token are taken out of the block table
    (-1) and overwritten, as the cache manager does once a window has passed them."""
    from inferloop_b200.parts import Workspace
    o = ops()
    n_pages = sum(-(-n // page_size) for n in lens) + 3
    k_cache, v_cache, table = build_cache([(k.float(), v.float()) for k, v in seqs], nkv, d, page_size, n_pages,
                                          torch.bfloat16, seed=seed, page_order=page_order)
    positions, seq_of, cu = [], [], [0]
    for s, (n, ql) in enumerate(zip(lens, q_lens)):
        positions += list(range(n - ql, n))
        seq_of += [s] * ql
        cu.append(cu[-1] + ql)
    step = _Step(positions, seq_of, cu, q_lens)
    if release_passed_pages:
        assert window > 0
        for s, (n, ql) in enumerate(zip(lens, q_lens)):
            for b in range(max(0, (n - ql) + 1 - window) // page_size):
                k_cache[table[s, b]] = float("nan")          # whoever follows the entry reads poison
                v_cache[table[s, b]] = float("nan")
                table[s, b] = -1
    out = torch.full((len(positions), nq * d), float("nan"), dtype=torch.bfloat16, device="cuda")
    ws = Workspace(torch.device("cuda:0"))
    was = o.DECODE_CLUSTER_ENABLED
    o.DECODE_CLUSTER_ENABLED = cluster
    try:
        for _ in range(2):      # twice: the tickets must be back at zero after the first launch
            o.attention(q.cuda(), out, k_cache.cuda(), v_cache.cuda(), step, table.cuda(), window, 1.0 / math.sqrt(d),
                        nq, nkv, d, workspace=ws, decode_chunk=chunk)
    finally:
        o.DECODE_CLUSTER_ENABLED = was
    return out, positions, seq_of


@pytest.mark.parametrize("nq,nkv,d,page_size,window", [(4, 2, 32, 4, 0), (6, 2, 64, 8, 0), (5, 5, 96, 16, 20),
                                                         (32, 8, 128, 16, 0), (8, 1, 128, 16, 0), (40, 2, 64, 32, 0),
                                                         (3, 3, 128, 16, 33)])
def test_flash_prefill_mixed_batch(nq, nkv, d, page_size, window):
    torch.manual_seed(nq + d)
    lens, q_lens = [37, 90, 131, 300], [37, 23, 1, 70]
    seqs = [(torch.randn(n, nkv, d).to(torch.bfloat16).double(), torch.randn(n, nkv, d).to(torch.bfloat16).double()) for n in lens]
    q = torch.randn(sum(q_lens), nq * d).to(torch.bfloat16)
    out, positions, seq_of = run_flash(q, seqs, lens, q_lens, nq, nkv, d, page_size, window)
    ref = torch.stack([ref_attention(q[t].double().view(nq, d), *seqs[seq_of[t]], positions[t], window).reshape(-1)
                       for t in range(len(positions))])
    close_flash(out, ref, max(float(v.abs().max()) for _, v in seqs), "flash prefill")


@pytest.mark.parametrize("nq,nkv,d,page_size,window,chunk", [(4, 2, 32, 4, 0, 256), (6, 2, 64, 8, 0, 256), (5, 5, 96, 16, 300, 256),
                                                               (32, 8, 128, 16, 0, 256), (8, 1, 128, 16, 0, 512), (40, 2, 64, 32, 0, 256),
                                                               (8, 2, 128, 16, 100, 256), (6, 3, 64, 64, 40, 256)])
@pytest.mark.parametrize("cluster", [True, False])
def test_flash_decode_split_kv(nq, nkv, d, page_size, window, chunk, cluster):
    """One token per sequence, lengths below, at and far above the chunk length (ticketed
    kernel) and with fewer tiles than the cluster has CTAs, exactly as many, and many more."""
    torch.manual_seed(nq + d + 1)
    lens = [1, 2, 31, 32, 33, 63, 64, 65, 255, 256, 257, 700, 1030, 1537]
    q_lens = [1] * len(lens)
    seqs = [(torch.randn(n, nkv, d).to(torch.bfloat16).double(), torch.randn(n, nkv, d).to(torch.bfloat16).double()) for n in lens]
    q = torch.randn(len(lens), nq * d).to(torch.bfloat16)
    out, positions, seq_of = run_flash(q, seqs, lens, q_lens, nq, nkv, d, page_size, window, chunk, cluster=cluster)
    ref = torch.stack([ref_attention(q[t].double().view(nq, d), *seqs[seq_of[t]], positions[t], window).reshape(-1)
                       for t in range(len(positions))])
    close_flash(out, ref, max(float(v.abs().max()) for _, v in seqs), "flash decode")


@pytest.mark.parametrize("nq,nkv,d,page_size,window,use_norm,use_rope", [(32, 8, 128, 16, 0, True, True), (8, 2, 64, 32, 50, True, True),
                                                                         (40, 2, 128, 16, 0, False, True), (4, 4, 128, 64, 0, True, False),
                                                                         (12, 2, 128, 16, 0, True, True), (3, 1, 64, 16, 7, True, True), (32, 2, 64, 32, 0, True, True)])
def test_decode_attention_with_the_input_stage_inside(nq, nkv, d, page_size, window, use_norm, use_rope):
    """One launch takes q, k, v of the step's token from the fused projection output: per-head
    norm, rotation, the cache write of the new key and value, and attention over old keys plus
    the new one.  Lengths put the new position at the start, the middle and the end of a
    32-key tile and of a page, and on tiles of every CTA of the cluster."""
    run_fused_decode(nq, nkv, d, page_size, window, use_norm, use_rope, [1, 2, 16, 17, 32, 33, 48, 64, 65, 100, 257, 700, 1031])


@pytest.mark.parametrize("lens,window", [([9000], 0), ([5000, 70], 0), ([3, 8200], 3000), ([4100, 4200, 300], 0)])
def test_decode_attention_of_few_long_sequences(lens, window):
    """With few sequences several clusters share one (sequence, kv head): each takes a run of
    the tiles, their records meet in a scratch buffer and the owner with the last ticket adds
    them.  Short sequences in the same launch keep to one cluster; a window moves the runs."""
    o = ops()
    split, stages, chunks = o.attention_decode_plan(len(lens), 32, 8, 128, 16, long_context=True)
    assert chunks >= 2, "this device leaves no room for a second cluster per sequence"
    run_fused_decode(32, 8, 128, 16, window, True, True, lens, long_context=True)
    from inferloop_b200.csrc.ops import _tc_state
    assert int(_tc_state(torch.device("cuda", 0)).attn_counters.abs().sum()) == 0       # tickets are back at zero


def run_fused_decode(nq, nkv, d, page_size, window, use_norm, use_rope, lens, long_context=False):
    o = ops()
    torch.manual_seed(nq + d + page_size)
    eps, theta = 1e-6, 1e4
    S = len(lens)
    G = nq // nkv
    old = [(torch.randn(n - 1, nkv, d).to(torch.bfloat16).double(), torch.randn(n - 1, nkv, d).to(torch.bfloat16).double()) for n in lens]
    qkv = torch.randn(S, (nq + 2 * nkv) * d).to(torch.bfloat16)
    qw, kw = (1 + 0.1 * torch.randn(d)).float(), (1 + 0.1 * torch.randn(d)).float()
    positions = torch.tensor([n - 1 for n in lens], dtype=torch.int32)
    inv = torch.tensor([theta ** (-(2.0 * i) / d) for i in range(d // 2)], dtype=torch.float64)
    table = torch.empty(S, d // 2, 2, device="cuda")
    o.rope_table(positions.cuda(), inv.cuda(), table)

    def norm(t, w):
        return t / torch.sqrt((t * t).mean(-1, keepdim=True) + eps) * w.double() if use_norm else t

    def rope(t, pos):
        if not use_rope:
            return t
        ang = pos.double()[:, None] * inv[None, :]
        c, s_ = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        a, b = t[..., :d // 2], t[..., d // 2:]
        return torch.cat([a * c - b * s_, a * s_ + b * c], dim=-1)

    x = qkv.double()
    q_new = rope(norm(x[:, :nq * d].view(S, nq, d), qw), positions).to(torch.bfloat16).double()
    k_new = rope(norm(x[:, nq * d:(nq + nkv) * d].view(S, nkv, d), kw), positions).to(torch.bfloat16).double()
    v_new = x[:, (nq + nkv) * d:].view(S, nkv, d)
    # the cache holds the old keys; the slot of the new position holds something else
    padded = [(torch.cat([k, torch.full((1, nkv, d), 5.0, dtype=torch.float64)]), torch.cat([v, torch.full((1, nkv, d), -3.0, dtype=torch.float64)]))
              for k, v in old]
    n_pages = sum(-(-n // page_size) for n in lens) + 3
    k_cache, v_cache, btable = build_cache(padded, nkv, d, page_size, n_pages, torch.bfloat16, seed=3, page_order="mixed")
    k_cache, v_cache = k_cache.cuda(), v_cache.cuda()
    out = torch.full((S, nq * d), float("nan"), dtype=torch.bfloat16, device="cuda")
    cu = torch.arange(S + 1, dtype=torch.int32).cuda()
    for _ in range(2):                       # the second run finds the new key already in the cache: same answer
        o.attention_decode_fused(qkv.cuda(), out, qw.cuda() if use_norm else None, kw.cuda() if use_norm else None, eps,
                                 table if use_rope else None, k_cache, v_cache, True, positions.cuda(), cu, btable.cuda(),
                                 window, 1.0 / math.sqrt(d), S, nq, nkv, d, long_context=long_context)
    o.check_device_errors()
    ref = torch.stack([ref_attention(q_new[s], torch.cat([old[s][0], k_new[s:s + 1]]), torch.cat([old[s][1], v_new[s:s + 1]]),
                                     lens[s] - 1, window).reshape(-1) for s in range(S)])
    close_flash(out, ref, max(float(v.abs().max()) for _, v in padded), "decode with input stage")
    for s, n in enumerate(lens):             # the new key and value are in the cache now, exactly as the separate kernel rounds them
        page, slot = int(btable[s, (n - 1) // page_size]), (n - 1) % page_size
        assert torch.equal(v_cache[page, :, slot].cpu().double(), v_new[s])
        close(k_cache[page, :, slot], k_new[s], "bfloat16", scale=float(k_new[s].abs().max()), what="new key")


@pytest.mark.parametrize("q_len,cluster", [(1, True), (1, False), (5, True)])
def test_flash_attention_finds_one_far_key_and_respects_the_window_edge(q_len, cluster):
    nq, nkv, d, page = 4, 1, 64, 16
    n = 900
    torch.manual_seed(2)
    k = torch.randn(n, nkv, d) * 0.1
    v = torch.arange(n, dtype=torch.float32)[:, None, None].expand(n, nkv, d).clone()
    for far, window, expect in ((13, 0, 13.0), (899 - 50 + 1, 50, 850.0), (899 - 50, 50, None), (511, 0, 511.0), (512, 0, 512.0)):
        kk = k.clone()
        direction = torch.randn(d)
        direction /= direction.norm()
        kk[far, 0] = direction * 40
        q = torch.randn(q_len, nq, d) * 0.01
        q[-1, :] = direction * 40                     # only the last token looks for the far key
        out, _, _ = run_flash(q.reshape(q_len, -1).to(torch.bfloat16), [(kk.to(torch.bfloat16).double(), v.double())],
                              [n], [q_len], nq, nkv, d, page, window, seed=far, cluster=cluster)
        got = out[-1].float().cpu()
        if expect is not None:
            assert torch.allclose(got, torch.full_like(got, expect), rtol=2.0 ** -7), (far, window, got[:4])
        else:
            assert 850.0 <= got.min().item() and got.max().item() <= 899.0


@pytest.mark.parametrize("M,I,K,max_ctas", [(1, 64, 64, 0), (8, 192, 256, 0), (8, 12288 // 8, 512, 0), (40, 128, 136, 0),
                                            (100, 320, 1024, 7), (130, 128, 64, 0), (300, 448, 512, 0), (2048, 1536, 512, 0),
                                            (300, 448, 512, 5), (8, 192, 2048, 50)])
@pytest.mark.parametrize("out_dtype", ["bfloat16", "float32"])
def test_gemm_tcgen05_swiglu_epilogue(M, I, K, max_ctas, out_dtype):
    """Weight rows in blocks of 64 gate + 64 up; out = silu(x Wg^T) * (x Wu^T)."""
    o = ops()
    torch.manual_seed(M + I)
    a = torch.randn(M, K).to(torch.bfloat16)
    wg = (torch.randn(I, K) * 0.1).to(torch.bfloat16)
    wu = (torch.randn(I, K) * 0.1).to(torch.bfloat16)
    w = torch.stack([wg.view(I // 64, 64, K), wu.view(I // 64, 64, K)], dim=1).reshape(2 * I, K).contiguous()
    out = torch.full((M, I), float("nan"), dtype=DT[out_dtype], device="cuda")
    o.gemm_tc(a.cuda(), w.cuda(), out, swiglu=True, max_ctas=max_ctas)
    o.check_device_errors()
    g = a.double() @ wg.double().T
    u = a.double() @ wu.double().T
    ref = g * torch.sigmoid(g) * u
    close(out, ref, out_dtype, scale=float(ref.abs().max()), what=f"swiglu {M}x{I}x{K}")


# ------------------------------------------------------------------ tcgen05 prefill attention
@pytest.mark.parametrize("nq,nkv,d,page_size,window", [(32, 8, 128, 16, 0), (8, 1, 128, 16, 0), (4, 2, 64, 32, 0),
                                                         (16, 16, 64, 16, 0), (32, 8, 128, 64, 100), (2, 2, 128, 128, 0),
                                                         (64, 2, 64, 16, 300), (10, 2, 128, 16, 0), (40, 8, 128, 16, 0),
                                                         (6, 2, 64, 32, 0), (7, 1, 128, 16, 90), (9, 1, 64, 16, 0)])
@pytest.mark.parametrize("row_blocks,split", [(1, True), (2, True), (0, False)])
def test_tc_prefill_mixed_batch(nq, nkv, d, page_size, window, row_blocks, split, monkeypatch):
    """Whole prompts, a portion that starts mid-sequence, single tokens, a long prompt whose
    row tiles cross many key tiles; pages shuffled.  Groups of 5, 3, 7 and 9 heads do not
    divide the 128 rows of a tile: its last rows then hold no query.  With one block of 128
    rows per CTA and with two that share the key and value tiles; the single tokens through
    the decode kernel (as the dispatcher sends them) or through the prefill kernel too."""
    o = ops()
    assert o.attention_tc_supported(nq, nkv, d, page_size)
    monkeypatch.setattr(o, "TC_ATTENTION_ROW_BLOCKS", row_blocks)
    monkeypatch.setattr(o, "MIXED_SPLIT_ENABLED", split)
    torch.manual_seed(nq * 3 + d)
    lens, q_lens = [37, 390, 131, 700, 129], [37, 123, 1, 700, 2]
    seqs = [(torch.randn(n, nkv, d).to(torch.bfloat16).double(), torch.randn(n, nkv, d).to(torch.bfloat16).double()) for n in lens]
    q = torch.randn(sum(q_lens), nq * d).to(torch.bfloat16)
    out, positions, seq_of = run_flash(q, seqs, lens, q_lens, nq, nkv, d, page_size, window)
    o.check_device_errors()
    ref = torch.stack([ref_attention(q[t].double().view(nq, d), *seqs[seq_of[t]], positions[t], window).reshape(-1)
                       for t in range(len(positions))])
    close_flash(out, ref, max(float(v.abs().max()) for _, v in seqs), "tc prefill")
    if row_blocks != 1:
        return
    # the mma.sync kernel at the same geometry, for the record that both paths are alive
    o.TC_ATTENTION_ENABLED = False
    try:
        out2, _, _ = run_flash(q, seqs, lens, q_lens, nq, nkv, d, page_size, window)
    finally:
        o.TC_ATTENTION_ENABLED = True
    close_flash(out2, ref, max(float(v.abs().max()) for _, v in seqs), "flash prefill")


@pytest.mark.parametrize("page_order", ["ordered", "mixed"])
@pytest.mark.parametrize("nq,nkv,d,page_size,window", [(32, 8, 128, 16, 0), (4, 2, 64, 32, 70)])
def test_tc_prefill_and_decode_with_pages_in_runs(nq, nkv, d, page_size, window, page_order):
    """Pages that follow one another in the pool are fetched as one box per tile; tiles whose
    run is broken, and the last tile of a sequence, take the box-per-page path."""
    torch.manual_seed(nq + d + page_size)
    for lens, q_lens in (([300, 1000, 129], [300, 260, 129]), ([513, 77, 1024, 130], [1, 1, 1, 1])):
        seqs = [(torch.randn(n, nkv, d).to(torch.bfloat16).double(), torch.randn(n, nkv, d).to(torch.bfloat16).double()) for n in lens]
        q = torch.randn(sum(q_lens), nq * d).to(torch.bfloat16)
        out, positions, seq_of = run_flash(q, seqs, lens, q_lens, nq, nkv, d, page_size, window, page_order=page_order)
        ops().check_device_errors()
        ref = torch.stack([ref_attention(q[t].double().view(nq, d), *seqs[seq_of[t]], positions[t], window).reshape(-1)
                           for t in range(len(positions))])
        close_flash(out, ref, max(float(v.abs().max()) for _, v in seqs), f"pages {page_order}")


@pytest.mark.parametrize("cluster", [True, False])
@pytest.mark.parametrize("nq,nkv,d,page_size,window", [(8, 2, 128, 16, 40), (4, 2, 64, 32, 100), (10, 2, 128, 16, 70)])
def test_attention_never_follows_a_released_page(nq, nkv, d, page_size, window, cluster):
    """Block-table rows whose leading entries are -1 (pages a window has passed, given back
    and poisoned here) through the tcgen05 prefill kernel, the TMA decode kernel and the
    ticketed decode kernel."""
    torch.manual_seed(nq + d + window)
    for lens, q_lens in (([300, 1000, 129, 40], [30, 260, 2, 40]), ([513, 77, 1024, 130], [1, 1, 1, 1])):
        seqs = [(torch.randn(n, nkv, d).to(torch.bfloat16).double(), torch.randn(n, nkv, d).to(torch.bfloat16).double()) for n in lens]
        q = torch.randn(sum(q_lens), nq * d).to(torch.bfloat16)
        out, positions, seq_of = run_flash(q, seqs, lens, q_lens, nq, nkv, d, page_size, window, cluster=cluster,
                                           release_passed_pages=True)
        ops().check_device_errors()
        ref = torch.stack([ref_attention(q[t].double().view(nq, d), *seqs[seq_of[t]], positions[t], window).reshape(-1)
                           for t in range(len(positions))])
        close_flash(out, ref, max(float(v.abs().max()) for _, v in seqs), f"released pages, lens {lens}")


def test_tc_prefill_finds_one_far_key_and_respects_the_window_edge():
    nq, nkv, d, page = 4, 1, 128, 16
    n = 900
    torch.manual_seed(4)
    k = torch.randn(n, nkv, d) * 0.1
    v = torch.arange(n, dtype=torch.float32)[:, None, None].expand(n, nkv, d).clone()
    for far, window, expect in ((13, 0, 13.0), (899 - 50 + 1, 50, 850.0), (899 - 50, 50, None), (511, 0, 511.0), (640, 0, 640.0)):
        kk = k.clone()
        direction = torch.randn(d)
        direction /= direction.norm()
        kk[far, 0] = direction * 40
        q = torch.randn(5, nq, d) * 0.01
        q[-1, :] = direction * 40
        out, _, _ = run_flash(q.reshape(5, -1).to(torch.bfloat16), [(kk.to(torch.bfloat16).double(), v.double())],
                              [n], [5], nq, nkv, d, page, window, seed=far)
        ops().check_device_errors()
        got = out[-1].float().cpu()
        if expect is not None:
            assert torch.allclose(got, torch.full_like(got, expect), rtol=2.0 ** -7), (far, window, got[:4])
        else:
            assert 850.0 <= got.min().item() and got.max().item() <= 899.0
