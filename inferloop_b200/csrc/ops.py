"""Python face of the CUDA kernels: thin, checked ctypes calls on torch tensors.

Every function launches on torch's current stream of the tensors' device and returns
without synchronising.  There is no CPU path: a tensor that is not on a CUDA device, or
a library that cannot be built or loaded, raises.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .build import load_module

F32, BF16 = 0, 1


class KernelError(RuntimeError):
    pass


def _code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"unsupported element type {t.dtype}")


def _ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _stream(t: torch.Tensor) -> ctypes.c_void_p:
    """torch's current stream on the tensor's device, as the raw handle the launchers take."""
    return ctypes.c_void_p(torch._C._cuda_getCurrentRawStream(t.device.index))


def _need(t: Optional[torch.Tensor], what: str, dtype: Optional[torch.dtype] = None,
          contiguous: bool = True) -> None:
    if t is None:
        return
    if not t.is_cuda:
        raise KernelError(f"{what}: tensor is on {t.device}; inferloop_b200 kernels run on CUDA only")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{what}: tensor must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{what}: expected {dtype}, found {t.dtype}")


LAUNCHES = 0          # kernels launched through this module since import


_FUNCTIONS: dict = {}  # launcher name -> (function, its library)


SCOPE = "other"       # the op class the next launches belong to (see `scope`)
TIMER = None          # an engine.timing.DeviceTimer in "node" mode, or None


def scope(name: str) -> None:
    """Name the op class of the launches that follow (a part calls this before its kernels);
    it costs one assignment and only the per-kernel device timer reads it."""
    global SCOPE
    SCOPE = name


def _call(module: str, fn: str, *args) -> None:
    global LAUNCHES
    LAUNCHES += 1
    entry = _FUNCTIONS.get(fn)
    if entry is None:
        lib = load_module(module)
        f = getattr(lib, fn)
        f.restype = ctypes.c_int
        entry = _FUNCTIONS[fn] = (f, lib)
    timer = TIMER
    begin = timer.node_begin() if timer is not None else None
    rc = entry[0](*args)
    if rc != 0:
        raise KernelError(entry[1].ilb_last_error().decode())
    if begin is not None:
        timer.node_end(SCOPE, fn, begin)


def _i(v) -> ctypes.c_int:
    return ctypes.c_int(int(v))


def _f(v) -> ctypes.c_float:
    return ctypes.c_float(float(v))


# --------------------------------------------------------------------------- rows
def embed(tokens: torch.Tensor, table: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, :] = table[tokens[t], :] widened to 32-bit."""
    _need(tokens, "embed tokens", torch.int32); _need(table, "embed table"); _need(out, "embed out", torch.float32)
    T, H = out.shape
    if tokens.numel() != T or table.shape[1] != H:
        raise KernelError("embed: shapes do not agree")
    _call("elementwise", "ilb_embed", _ptr(tokens), _ptr(table), _i(_code(table)), _ptr(out),
          _i(T), _i(H), _i(table.shape[0]), _stream(out))


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    """out = x / sqrt(mean(x^2) + eps) * weight over the last dimension; x is 32-bit."""
    _need(x, "rmsnorm x", torch.float32); _need(weight, "rmsnorm weight", torch.float32); _need(out, "rmsnorm out")
    width = x.shape[-1]
    if weight.numel() != width or out.shape != x.shape:
        raise KernelError("rmsnorm: shapes do not agree")
    rows = x.numel() // width
    _call("elementwise", "ilb_rmsnorm", _ptr(x), _ptr(weight), _ptr(out), _i(_code(out)),
          _i(rows), _i(width), _f(eps), _stream(x))


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out = silu(gate_up[:, :I]) * gate_up[:, I:2I]."""
    _need(gate_up, "silu_mul in"); _need(out, "silu_mul out", gate_up.dtype)
    rows, width = out.shape
    if gate_up.shape[0] != rows or gate_up.shape[1] != 2 * width:
        raise KernelError("silu_mul: shapes do not agree")
    _call("elementwise", "ilb_silu_mul", _ptr(gate_up), _ptr(out), _i(_code(out)), _i(rows),
          _i(width), _i(gate_up.shape[1]), _stream(out))


def gather_rows(x: torch.Tensor, index: torch.Tensor, out: torch.Tensor) -> None:
    _need(x, "gather x", torch.float32); _need(index, "gather index", torch.int32); _need(out, "gather out", torch.float32)
    if out.shape[0] != index.numel() or out.shape[1] != x.shape[1]:
        raise KernelError("gather_rows: shapes do not agree")
    _call("elementwise", "ilb_gather_rows", _ptr(x), _ptr(index), _ptr(out), _i(out.shape[0]),
          _i(x.shape[1]), _i(x.shape[0]), _stream(x))


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, i] = (cos, sin)(positions[t] * inv_freq[i]); inv_freq is 64-bit."""
    _need(positions, "rope positions", torch.int32); _need(inv_freq, "rope inv_freq", torch.float64)
    _need(out, "rope table", torch.float32)
    T, half = positions.numel(), inv_freq.numel()
    if tuple(out.shape) != (T, half, 2):
        raise KernelError("rope_table: out must be [T, rotary_dim/2, 2]")
    _call("elementwise", "ilb_rope_table", _ptr(positions), _ptr(inv_freq), _ptr(out), _i(T),
          _i(half), _stream(out))


def add_inplace(x: torch.Tensor, y: torch.Tensor) -> None:
    _need(x, "add x", torch.float32); _need(y, "add y", torch.float32)
    if x.numel() != y.numel():
        raise KernelError("add_inplace: sizes differ")
    _call("elementwise", "ilb_add_inplace", _ptr(x), _ptr(y), ctypes.c_longlong(x.numel()), _stream(x))


def scale_cap_inplace(x: torch.Tensor, scale: float = 1.0, cap: float = 0.0) -> None:
    """x = x * scale, then (cap > 0) x = cap * tanh(x / cap); x is 32-bit."""
    _need(x, "scale_cap x", torch.float32)
    _call("elementwise", "ilb_scale_cap_inplace", _ptr(x), _f(scale), _f(cap), ctypes.c_longlong(x.numel()), _stream(x))


def decode_advance(tokens: torch.Tensor, positions: torch.Tensor, kv_len: torch.Tensor,
                   drawn: torch.Tensor, n_live: int) -> None:
    """tokens[:n_live] = drawn[:n_live]; positions and kv_len of those advance by one."""
    for t, what in ((tokens, "tokens"), (positions, "positions"), (kv_len, "kv_len"), (drawn, "drawn")):
        _need(t, what, torch.int32)
    _call("elementwise", "ilb_decode_advance", _ptr(tokens), _ptr(positions), _ptr(kv_len), _ptr(drawn),
          _i(n_live), _i(tokens.numel()), _stream(tokens))


# --------------------------------------------------------------------------- GEMM
def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor,
              bias: Optional[torch.Tensor] = None, accumulate: bool = False) -> None:
    """out (+)= a @ w.T (+ bias) with 32-bit fused multiply-adds in a fixed order."""
    _need(a, "gemm a"); _need(w, "gemm w", a.dtype); _need(out, "gemm out")
    _need(bias, "gemm bias", torch.float32)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or tuple(out.shape) != (M, N) or (bias is not None and bias.numel() != N):
        raise KernelError(f"gemm: shapes do not agree: a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    if accumulate and out.dtype != torch.float32:
        raise KernelError("gemm: accumulation needs a 32-bit output")
    _call("gemm_simt", "ilb_gemm_simt", _ptr(a), _ptr(w), _ptr(bias), _ptr(out), _i(_code(a)),
          _i(_code(out)), _i(M), _i(N), _i(K), _i(K), _i(K), _i(N), _i(1 if accumulate else 0),
          _stream(out))


# --------------------------------------------------------------------------- attention
def qk_norm_rope_cache(qkv: torch.Tensor, q_out: torch.Tensor, q_weight: Optional[torch.Tensor],
                       k_weight: Optional[torch.Tensor], eps: float,
                       rope: Optional[torch.Tensor], rotary_dim: int, positions: torch.Tensor,
                       seq_of_token: torch.Tensor, block_table: Optional[torch.Tensor],
                       page_size: int, k_cache: Optional[torch.Tensor],
                       v_cache: Optional[torch.Tensor], nq: int, nkv: int, d: int) -> None:
    """Per-head q/k RMSNorm, rotation, q -> q_out, k/v -> cache pages (see qk_norm_rope.cu)."""
    _need(qkv, "qkv"); _need(q_out, "q_out", qkv.dtype)
    _need(q_weight, "q_norm weight", torch.float32); _need(k_weight, "k_norm weight", torch.float32)
    _need(rope, "rope table", torch.float32); _need(positions, "positions", torch.int32)
    _need(seq_of_token, "seq_of_token", torch.int32); _need(block_table, "block table", torch.int32)
    _need(k_cache, "k cache"); _need(v_cache, "v cache")
    T = qkv.shape[0]
    if k_cache is not None:
        if tuple(k_cache.shape[1:]) != (nkv, page_size, d) or v_cache.shape != k_cache.shape:
            raise KernelError(f"cache shape {tuple(k_cache.shape)} is not [pages, {nkv}, {page_size}, {d}]")
        if block_table is None:
            raise KernelError("a cache write needs a block table")
    max_blocks = 0 if block_table is None else block_table.shape[1]
    num_pages = 0 if k_cache is None else k_cache.shape[0]
    cache_code = _code(k_cache) if k_cache is not None else _code(qkv)
    _call("qk_norm_rope", "ilb_qk_norm_rope_cache", _ptr(qkv), _ptr(q_out), _i(_code(qkv)),
          _ptr(q_weight), _ptr(k_weight), _f(eps), _ptr(rope), _i(rotary_dim), _ptr(positions),
          _ptr(seq_of_token), _ptr(block_table), _i(max_blocks), _i(page_size), _i(num_pages),
          _ptr(k_cache), _ptr(v_cache), _i(cache_code), _i(T), _i(nq), _i(nkv), _i(d),
          _i(qkv.shape[1]), _i(q_out.shape[1]), _stream(qkv))


def paged_attention_simple(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor,
                           v_cache: torch.Tensor, positions: torch.Tensor,
                           seq_of_token: torch.Tensor, block_table: torch.Tensor, window: int,
                           scale: float, nq: int, nkv: int, d: int) -> None:
    _need(q, "attention q"); _need(out, "attention out", q.dtype)
    _need(k_cache, "k cache"); _need(v_cache, "v cache", k_cache.dtype)
    _need(positions, "positions", torch.int32); _need(seq_of_token, "seq_of_token", torch.int32)
    _need(block_table, "block table", torch.int32)
    num_pages, nkv_c, page_size, d_c = k_cache.shape
    if (nkv_c, d_c) != (nkv, d):
        raise KernelError("attention: cache shape does not match the heads")
    _call("attention_simple", "ilb_paged_attention_simple", _ptr(q), _ptr(out), _i(_code(q)),
          _ptr(k_cache), _ptr(v_cache), _i(_code(k_cache)), _ptr(positions), _ptr(seq_of_token),
          _ptr(block_table), _i(block_table.shape[1]), _i(page_size), _i(num_pages),
          _i(window or 0), _f(scale), _i(q.shape[0]), _i(nq), _i(nkv), _i(d), _i(q.shape[1]),
          _i(out.shape[1]), _stream(q))


# --------------------------------------------------------------------------- sampling
def argmax(logits: torch.Tensor, out: torch.Tensor, bad: Optional[torch.Tensor] = None) -> None:
    _need(logits, "argmax logits", torch.float32); _need(out, "argmax out", torch.int32)
    _need(bad, "argmax flags", torch.int32)
    rows, vocab = logits.shape
    _call("sampling", "ilb_argmax", _ptr(logits), _ptr(out), _ptr(bad), _i(rows), _i(vocab),
          _i(logits.stride(0)), _stream(logits))


def sample_filter_max_vocab() -> int:
    """Largest vocabulary whose draws can be filtered (top-k, top-p, min-p) on the device."""
    lib = load_module("sampling")
    lib.ilb_sample_filter_max_vocab.restype = ctypes.c_int
    return int(lib.ilb_sample_filter_max_vocab())


def mark_tokens(rows: torch.Tensor, tokens: torch.Tensor, is_generated: torch.Tensor, seen: torch.Tensor,
                generated: torch.Tensor, vocab: int) -> None:
    """Set bit t of row r of `seen` ([rows, ceil(vocab / 32)] int32, zeroed by the caller) for
    every entry (r, t), and of `generated` for entries flagged as generated."""
    for t, w in ((rows, "rows"), (tokens, "tokens"), (is_generated, "flags"), (seen, "seen bits"), (generated, "generated bits")):
        _need(t, "mark_tokens " + w, torch.int32)
    _call("sampling", "ilb_mark_tokens", _ptr(rows), _ptr(tokens), _ptr(is_generated), _i(tokens.numel()), _ptr(seen),
          _ptr(generated), _i(seen.shape[0]), _i(vocab), _stream(seen))


def sample_temperature(logits: torch.Tensor, temperature: torch.Tensor, uniform: torch.Tensor,
                       out: torch.Tensor, bad: Optional[torch.Tensor] = None, top_k: Optional[torch.Tensor] = None,
                       top_p: Optional[torch.Tensor] = None, min_p: Optional[torch.Tensor] = None,
                       penalties: Optional[tuple] = None) -> None:
    """One draw per row from softmax(logits / T) by the reference's sorted-walk rule, after
    its filters if given: top_k [rows] int32 (0 = none), top_p and min_p [rows] float32;
    `penalties` = (seen bits, generated bits, repetition [rows], presence [rows]) applies
    the reference's penalties to the logits first (see mark_tokens)."""
    _need(logits, "sample logits", torch.float32); _need(temperature, "temperature", torch.float32)
    _need(uniform, "uniform", torch.float64); _need(out, "sample out", torch.int32)
    _need(bad, "sample flags", torch.int32); _need(top_k, "top-k", torch.int32)
    _need(top_p, "top-p", torch.float32); _need(min_p, "min-p", torch.float32)
    rows, vocab = logits.shape
    seen = gen = rep = pres = None
    if penalties is not None:
        seen, gen, rep, pres = penalties
        _need(seen, "seen bits", torch.int32); _need(gen, "generated bits", torch.int32)
        _need(rep, "repetition penalty", torch.float32); _need(pres, "presence penalty", torch.float32)
        if tuple(seen.shape) != (rows, (vocab + 31) // 32) or tuple(gen.shape) != tuple(seen.shape):
            raise KernelError("sample: token bitmaps must be [rows, ceil(vocab / 32)]")
    _call("sampling", "ilb_sample_temperature", _ptr(logits), _ptr(temperature), _ptr(uniform), _ptr(top_k), _ptr(top_p),
          _ptr(min_p), _ptr(seen), _ptr(gen), _ptr(rep), _ptr(pres), _ptr(out), _ptr(bad), _i(rows), _i(vocab),
          _i(logits.stride(0)), _stream(logits))


# --------------------------------------------------------------------------- tensor-core GEMM
class _TcState:
    """Per-device scratch of the tensor-core kernels: the GEMM's split-K workspace and tile
    tickets (zero between launches), and the flag a kernel raises when a bounded wait runs out."""

    def __init__(self, device: torch.device) -> None:
        lib = load_module("gemm_tcgen05")
        lib.ilb_gemm_tc_workspace_floats.restype = ctypes.c_longlong
        self.floats = int(lib.ilb_gemm_tc_workspace_floats())
        self.n_tickets = int(lib.ilb_gemm_tc_max_tickets())
        self.workspace = torch.empty(self.floats, dtype=torch.float32, device=device)
        self.tickets = torch.zeros(self.n_tickets, dtype=torch.int32, device=device)
        self.error = torch.zeros(1, dtype=torch.int32, device=device)
        # decode attention of few, long sequences: records of the clusters that share a sequence, and their tickets
        self.attn_scratch = torch.empty(1 << 20, dtype=torch.float32, device=device)
        self.attn_counters = torch.zeros(1 << 14, dtype=torch.int32, device=device)


_TC: dict = {}
TC_ENABLED = True          # tests switch it off to exercise the fallback


def _tc_state(device: torch.device) -> _TcState:
    st = _TC.get(device)
    if st is None:
        st = _TC[device] = _TcState(device)
    return st


def gemm_tc_eligible(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> bool:
    """bfloat16 operands whose rows are multiples of 16 bytes (TMA's rule)."""
    if not TC_ENABLED or a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        return False
    K = a.shape[1]
    return (K % 8 == 0 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and a.shape[0] > 0)


def gemm_tc(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
            accumulate: bool = False, max_ctas: int = 0, swiglu: bool = False) -> None:
    """out (+)= a @ w.T (+ bias) on tcgen05 tensor cores (see gemm_tcgen05.cu).  With
    `swiglu`, `w` holds blocks of 64 gate rows followed by their 64 up rows and `out` is
    [M, N/2] = silu(gate) * up."""
    _need(a, "gemm a", torch.bfloat16); _need(w, "gemm w", torch.bfloat16); _need(out, "gemm out")
    _need(bias, "gemm bias", torch.float32)
    M, K = a.shape
    N = w.shape[0]
    n_out = N // 2 if swiglu else N
    if w.shape[1] != K or tuple(out.shape) != (M, n_out) or (bias is not None and bias.numel() != N):
        raise KernelError(f"gemm: shapes do not agree: a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    if accumulate and (out.dtype != torch.float32 or swiglu):
        raise KernelError("gemm: accumulation needs a 32-bit output and no SwiGLU epilogue")
    st = _tc_state(a.device)
    mode = 2 if swiglu else (1 if accumulate else 0)
    _call("gemm_tcgen05", "ilb_gemm_tc", _ptr(a), _ptr(w), _ptr(bias), _ptr(out),
          _i(1 if out.dtype == torch.float32 else 0), _i(M), _i(N), _i(K), _i(a.stride(0)), _i(w.stride(0)),
          _i(out.stride(0)), _i(mode), _ptr(st.workspace), ctypes.c_longlong(st.floats),
          _ptr(st.tickets), _i(st.n_tickets), _ptr(st.error), _i(max_ctas), _stream(out))


def gemm_sums_in_memory(on: bool) -> None:
    """Whether products that accumulate into a 32-bit output may let the K ranges of a tile meet
    in memory: the tiles of the last round of many tokens (on single CTAs or on pairs), and every
    tile of up to eight tokens when the weight is large (faster; the order of that 32-bit sum
    is not fixed, so two runs agree beyond rounding but not bit for bit).  On by default;
    off gives sums whose bits do not change from run to run."""
    load_module("gemm_tcgen05").ilb_gemm_tc_sums_in_memory(_i(1 if on else 0))


def gemm_pairs(mode: int) -> None:
    """Products of many tokens on pairs of CTAs that the tensor cores treat as one unit
    (256 x 256 tiles, `tcgen05.mma.cta_group::2`): 0 never, 1 where the sizes favour it (the
    default), 2 wherever the kernel can run (tests use it at small sizes)."""
    load_module("gemm_tcgen05").ilb_gemm_tc_pairs(_i(int(mode)))


def gemm_tuning(few_tokens_in_memory: Optional[int] = None, few_tokens_ranges: int = 8,
                pair_ranges: Optional[int] = None, pair_fill_plain: float = 0.75, pair_fill_adding: float = 0.85) -> None:
    """Knobs behind the measured defaults, for A/B runs (the defaults are what the profiles
    report).  `few_tokens_in_memory`: accumulating products of up to this many tokens (and a
    weight of at least 2,048 x 2,048) add the K ranges of a tile in memory instead of inside a
    cluster, cut into up to `few_tokens_ranges` ranges (default 8 tokens; 0: never).
    `pair_ranges`: the most K ranges a tile of a pair of CTAs is cut into (default 8), with
    the shares of busy pairs that plain and adding products ask for before they take pairs."""
    lib = load_module("gemm_tcgen05")
    if few_tokens_in_memory is not None:
        lib.ilb_gemm_tc_red_few(_i(int(few_tokens_in_memory)), _i(int(few_tokens_ranges)))
    if pair_ranges is not None:
        lib.ilb_gemm_tc_pair_tuning(_i(int(pair_ranges)), _i(int(round(pair_fill_plain * 1000))),
                                    _i(int(round(pair_fill_adding * 1000))))


def gemm_tc_plan(M: int, N: int, K: int, accumulate: bool = False, swiglu: bool = False) -> dict:
    """How `gemm_tc` deals out a product of these sizes (needs a device: the answer depends
    on how many CTAs fit it).  `pairs` > 0: the product runs on that many pairs of CTAs, each
    tile left over after the whole rounds (or every tile) cut into `pair_split` K ranges, and
    `sums_meet_in_memory` speaks of those; the other fields then describe the single-CTA deal
    that `gemm_pairs(0)` would use."""
    lib = load_module("gemm_tcgen05")
    out = (ctypes.c_int * 11)()
    lib.ilb_gemm_tc_plan.restype = ctypes.c_int
    if lib.ilb_gemm_tc_plan(_i(M), _i(N), _i(K), _i(2 if swiglu else (1 if accumulate else 0)), out) != 0:
        raise KernelError(lib.ilb_last_error().decode())
    keys = ("swap", "tile_n", "row_blocks", "grid", "cluster", "rounds", "tiles", "tiles_stream_k", "sums_meet_in_memory",
            "pairs", "pair_split")
    return dict(zip(keys, list(out)))


def device_error_tensor(device) -> Optional[torch.Tensor]:
    """The one-int flag that kernels on `device` raise when a bounded wait runs out (None
    while no tensor-core kernel has run there yet)."""
    st = _TC.get(torch.device(device))
    return None if st is None else st.error


def check_device_errors() -> None:
    """Raise if a kernel gave up a bounded wait since the last check (synchronises)."""
    for dev, st in _TC.items():
        if int(st.error.item()) != 0:
            st.error.zero_()
            st.tickets.zero_()
            raise KernelError(f"a tensor-core kernel on {dev} gave up waiting on a barrier; its output is invalid")


# --------------------------------------------------------------------------- attention dispatch
DECODE_CHUNK_MIN = 256      # keys per decode CTA; boundaries depend on the key index alone


def decode_chunk_for(max_positions: int) -> int:
    """Chunk length of split-KV decode for a model that reaches `max_positions`: 256 keys,
    or more for very long contexts so that a sequence never has more than 32 chunks."""
    chunk = DECODE_CHUNK_MIN
    while chunk * 32 < max_positions:
        chunk *= 2
    return chunk


def attention_flash_supported(d: int) -> bool:
    return d in (32, 64, 96, 128)


def attention_tc_supported(nq: int, nkv: int, d: int, page_size: int) -> bool:
    """Geometries the tcgen05 prefill attention is built for."""
    if nkv <= 0 or nq % nkv:
        return False
    g = nq // nkv
    return d in (64, 128) and g <= 128 and page_size in (16, 32, 64, 128)


def attention_prefill_tc(q, out, k_cache, v_cache, positions, cu_q, block_table, window, scale, n_seqs,
                         n_tiles, nq, nkv, d, row_blocks: int = 1, skip_single: bool = False) -> None:
    """Prefill attention on tcgen05 tensor cores (attention_tc.cu); a CTA takes `row_blocks`
    (1 or 2) blocks of 128 // (nq / nkv) tokens of one sequence, and n_tiles counts the CTAs
    over the sequences (with `skip_single`, over those that bring more than one token: the
    others' rows of `out` are left alone)."""
    for t, w in ((q, "q"), (out, "out"), (k_cache, "k cache"), (v_cache, "v cache")):
        _need(t, "attention " + w, torch.bfloat16)
    num_pages, _, page_size, _ = k_cache.shape
    st = _tc_state(q.device)
    _call("attention_tc", "ilb_attention_prefill_tc", _ptr(q), _ptr(out), _ptr(k_cache), _ptr(v_cache),
          _ptr(positions), _ptr(cu_q), _ptr(block_table), _i(block_table.shape[1]), _i(page_size),
          _i(num_pages), _i(window or 0), _f(scale), _i(q.shape[0]), _i(n_seqs), _i(n_tiles), _i(row_blocks), _i(1 if skip_single else 0), _i(nq), _i(nkv),
          _i(d), _i(q.shape[1]), _i(out.shape[1]), _ptr(st.error), _stream(q))


def attention_prefill(q, out, k_cache, v_cache, positions, cu_q, block_table, window, scale, n_seqs,
                      n_tiles, nq, nkv, d) -> None:
    for t, w in ((q, "q"), (out, "out"), (k_cache, "k cache"), (v_cache, "v cache")):
        _need(t, "attention " + w, torch.bfloat16)
    num_pages, _, page_size, _ = k_cache.shape
    _call("attention_flash", "ilb_attention_prefill", _ptr(q), _ptr(out), _ptr(k_cache), _ptr(v_cache),
          _ptr(positions), _ptr(cu_q), _ptr(block_table), _i(block_table.shape[1]), _i(page_size),
          _i(num_pages), _i(window or 0), _f(scale), _i(n_seqs), _i(n_tiles), _i(nq), _i(nkv), _i(d),
          _i(q.shape[1]), _i(out.shape[1]), _stream(q))


def attention_decode(q, out, k_cache, v_cache, positions, cu_q, block_table, window, scale, n_seqs,
                     nq, nkv, d, chunk, max_chunks, scratch, tickets) -> None:
    for t, w in ((q, "q"), (out, "out"), (k_cache, "k cache"), (v_cache, "v cache")):
        _need(t, "attention " + w, torch.bfloat16)
    _need(scratch, "attention scratch", torch.float32); _need(tickets, "attention tickets", torch.int32)
    num_pages, _, page_size, _ = k_cache.shape
    _call("attention_flash", "ilb_attention_decode", _ptr(q), _ptr(out), _ptr(k_cache), _ptr(v_cache),
          _ptr(positions), _ptr(cu_q), _ptr(block_table), _i(block_table.shape[1]), _i(page_size),
          _i(num_pages), _i(window or 0), _f(scale), _i(n_seqs), _i(nq), _i(nkv), _i(d), _i(q.shape[1]),
          _i(out.shape[1]), _i(chunk), _i(max_chunks), _ptr(scratch), ctypes.c_longlong(scratch.numel()),
          _ptr(tickets), _i(tickets.numel()), _stream(q))


def attention_decode_tma_supported(nq: int, nkv: int, d: int, page_size: int) -> bool:
    """Geometries the cluster-merged TMA decode attention is built for."""
    return nkv > 0 and nq > 0 and nq % nkv == 0 and d in (64, 128) and page_size in (16, 32, 64, 128)


# A decode step whose longest sequence holds at least this many keys is launched for the most
# CTAs at work: narrower clusters, several of them sharing a (sequence, kv head) when the
# sequences are few.  Recorded decode graphs are kept apart by this flag.
DECODE_LONG_CONTEXT = 8192


def attention_decode_plan(n_seqs: int, nq: int, nkv: int, d: int, page_size: int, long_context: bool = False) -> tuple:
    """(CTAs of a cluster, stages of the tile ring, clusters that may share a long sequence)
    that a decode step of this geometry gets."""
    lib = load_module("attention_decode")
    split, stages, chunks = ctypes.c_int(0), ctypes.c_int(0), ctypes.c_int(0)
    lib.ilb_attention_decode_plan.restype = ctypes.c_int
    if lib.ilb_attention_decode_plan(_i(n_seqs), _i(nq), _i(nkv), _i(d), _i(page_size), _i(1 if long_context else 0), ctypes.byref(split),
                                     ctypes.byref(stages), ctypes.byref(chunks)) != 0:
        raise KernelError(lib.ilb_last_error().decode())
    return split.value, stages.value, chunks.value


def attention_decode_tma(q, out, k_cache, v_cache, positions, cu_q, block_table, window, scale, n_seqs,
                         nq, nkv, d, long_context: bool = False) -> None:
    """Split-KV decode whose tiles come by TMA and whose partial results meet inside a
    thread-block cluster (no scratch)."""
    for t, w in ((q, "q"), (out, "out"), (k_cache, "k cache"), (v_cache, "v cache")):
        _need(t, "attention " + w, torch.bfloat16)
    num_pages, _, page_size, _ = k_cache.shape
    st = _tc_state(q.device)
    _call("attention_decode", "ilb_attention_decode_tma", _ptr(q), _ptr(out), _ptr(k_cache), _ptr(v_cache),
          _ptr(positions), _ptr(cu_q), _ptr(block_table), _i(block_table.shape[1]), _i(page_size),
          _i(num_pages), _i(window or 0), _f(scale), _i(n_seqs), _i(nq), _i(nkv), _i(d), _i(q.shape[1]),
          _i(out.shape[1]), _i(1 if long_context else 0), _ptr(st.attn_scratch), ctypes.c_longlong(st.attn_scratch.numel()), _ptr(st.attn_counters),
          ctypes.c_longlong(st.attn_counters.numel()), _ptr(st.error), _stream(q))


def attention_decode_fused_supported(dtype: torch.dtype, cache_dtype: torch.dtype, nq: int, nkv: int, d: int,
                                     page_size: int, rotary_dim: int, has_rope: bool) -> bool:
    """Whether a decode-only step can take q/k/v straight from the fused projection output:
    the TMA decode kernel's geometry, bfloat16 throughout, rotation over the whole head."""
    return (DECODE_CLUSTER_ENABLED and DECODE_FUSED_ENABLED and FLASH_ENABLED and dtype == torch.bfloat16
            and cache_dtype == torch.bfloat16 and attention_decode_tma_supported(nq, nkv, d, page_size)
            and (not has_rope or rotary_dim == d))


def attention_decode_fused(qkv, out, q_weight, k_weight, eps, rope_table, k_cache, v_cache, write_kv, positions, cu_q,
                           block_table, window, scale, n_seqs, nq, nkv, d, long_context: bool = False) -> None:
    """Decode attention with the per-head q/k norm, the rotation and the cache write of the
    step's own key and value inside the attention kernel (one launch instead of two)."""
    for t, w in ((qkv, "qkv"), (out, "out"), (k_cache, "k cache"), (v_cache, "v cache")):
        _need(t, "attention " + w, torch.bfloat16)
    for t, w in ((q_weight, "q norm weight"), (k_weight, "k norm weight"), (rope_table, "rope table")):
        if t is not None:
            _need(t, "attention " + w, torch.float32)
    num_pages, _, page_size, _ = k_cache.shape
    st = _tc_state(qkv.device)
    _call("attention_decode", "ilb_attention_decode_fused", _ptr(qkv), _i(qkv.shape[1]), _ptr(q_weight), _ptr(k_weight),
          _f(eps if eps and eps > 0 else 1e-6), _ptr(rope_table), _i(1 if write_kv else 0), _ptr(out), _ptr(k_cache),
          _ptr(v_cache), _ptr(positions),
          _ptr(cu_q), _ptr(block_table), _i(block_table.shape[1]), _i(page_size), _i(num_pages), _i(window or 0),
          _f(scale), _i(n_seqs), _i(nq), _i(nkv), _i(d), _i(out.shape[1]), _i(1 if long_context else 0), _ptr(st.attn_scratch),
          ctypes.c_longlong(st.attn_scratch.numel()), _ptr(st.attn_counters), ctypes.c_longlong(st.attn_counters.numel()),
          _ptr(st.error), _stream(qkv))


def attention(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
              step, block_table: torch.Tensor, window: int, scale: float, nq: int, nkv: int,
              d: int, workspace=None, decode_chunk: int = DECODE_CHUNK_MIN) -> None:
    """Causal attention of the step's tokens over the cache; picks the kernel: the
    tensor-core kernels for a bfloat16 cache and a head size they are built for (split-KV
    when every sequence brings one token), else the exact kernel."""
    fast = (q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and attention_flash_supported(d)
            and workspace is not None and FLASH_ENABLED)
    if not fast:
        paged_attention_simple(q, out, k_cache, v_cache, step.positions, step.seq_of_token,
                               block_table, window, scale, nq, nkv, d)
        return
    G = nq // nkv
    if step.decode_only and DECODE_CLUSTER_ENABLED and attention_decode_tma_supported(nq, nkv, d, k_cache.shape[2]):
        attention_decode_tma(q, out, k_cache, v_cache, step.positions, step.cu_q, block_table, window, scale,
                             step.n_seqs, nq, nkv, d, getattr(step, "max_kv_len", 0) >= DECODE_LONG_CONTEXT)
    elif step.decode_only:
        page_size = k_cache.shape[2]
        capacity = block_table.shape[1] * page_size
        max_chunks = max(1, -(-capacity // decode_chunk))
        scratch = workspace.buffer("attn.decode_scratch", (step.n_seqs * nkv * max_chunks * G * (d + 2),), torch.float32)
        tickets = workspace.zeroed("attn.decode_tickets", (max(step.n_seqs * nkv, 4096),), torch.int32)
        attention_decode(q, out, k_cache, v_cache, step.positions, step.cu_q, block_table, window, scale,
                         step.n_seqs, nq, nkv, d, decode_chunk, max_chunks, scratch, tickets)
    elif TC_ATTENTION_ENABLED and attention_tc_supported(nq, nkv, d, k_cache.shape[2]):
        # A mixed step: the sequences that bring one token go to the split-KV decode kernel
        # (it leaves the others alone), the portions to the prefill kernel (which leaves those).
        lens = step.h_q_len
        kv_lens = getattr(step, "h_kv_len", None) or lens
        split = (MIXED_SPLIT_ENABLED and DECODE_CLUSTER_ENABLED and 1 in lens and max(lens) > 1
                 and attention_decode_tma_supported(nq, nkv, d, k_cache.shape[2]))
        if split:
            attention_decode_tma(q, out, k_cache, v_cache, step.positions, step.cu_q, block_table, window, scale,
                                 step.n_seqs, nq, nkv, d, False)
            kv_lens = [k for n, k in zip(lens, kv_lens) if n > 1]
            lens = [n for n in lens if n > 1]
        per_block = 128 // G
        n_one = sum(-(-n // per_block) for n in lens)
        n_two = sum(-(-n // (2 * per_block)) for n in lens)
        blocks = TC_ATTENTION_ROW_BLOCKS or tc_row_blocks(n_one * nkv, n_two * nkv, _sm_count(q.device),
                                                          all(k >= 2 * n for n, k in zip(lens, kv_lens)))
        n_tiles = n_two if blocks == 2 else n_one
        attention_prefill_tc(q, out, k_cache, v_cache, step.positions, step.cu_q, block_table, window, scale,
                             step.n_seqs, n_tiles, nq, nkv, d, blocks, skip_single=split)
    else:
        n_tiles = sum(-(-n * G // 64) for n in step.h_q_len)
        attention_prefill(q, out, k_cache, v_cache, step.positions, step.cu_q, block_table, window, scale,
                          step.n_seqs, n_tiles, nq, nkv, d)


def tc_row_blocks(ctas_one: int, ctas_two: int, sms: int, behind_cache: bool) -> int:
    """Row blocks per CTA of the tcgen05 prefill kernel.  Two blocks share the K and V tiles
    and keep the tensor core busier, but a tile then takes 4,150 clocks for the pair against
    2,400 for one block (measured), and there are half as many CTAs.
    Portions behind a long cached prefix: every CTA walks about as many keys, the launch runs
    in rounds of one CTA per SM, and the cheaper of rounds x tile time wins (512 tokens of 40 / 8
    heads behind 3,584: 168 CTAs in two rounds, or 88 in one).  Prompts from their start: the
    CTAs' runs differ and pack well, and two blocks pay once there is a CTA for every SM."""
    if behind_cache:
        return 2 if -(-ctas_two // sms) * 1.7 < -(-ctas_one // sms) else 1
    return 2 if ctas_two >= sms else 1


DECODE_FUSED_ENABLED = True     # tests switch it off to run q/k norm + rotation + cache write as a launch of its own
DECODE_CLUSTER_ENABLED = True   # tests switch it off to reach the ticketed split-KV decode kernel
FLASH_ENABLED = True       # tests switch it off to exercise the exact kernel in bfloat16
TC_ATTENTION_ENABLED = True   # tests switch it off to reach the mma.sync prefill kernel at its geometries
TC_ATTENTION_ROW_BLOCKS = 0   # tests set 1 or 2 to force the row blocks per CTA of the tcgen05 prefill kernel
MIXED_SPLIT_ENABLED = True    # tests switch it off to send a mixed step's single tokens through the prefill kernel

_SM_COUNT: dict = {}


def _sm_count(device) -> int:
    n = _SM_COUNT.get(device)
    if n is None:
        n = _SM_COUNT[device] = torch.cuda.get_device_properties(device).multi_processor_count
    return n
