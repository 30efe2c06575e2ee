"""Each part alone (GPU): built from a spec with sizes of its own, given random
tensors, run on a small mixed batch and compared with the plain functions."""
import math

import pytest
import torch

import plain_qwen3 as plain
from inferloop_b200.config.spec import LayerSpec, PartSpec, RunEntry

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def env(dtype):
    from inferloop_b200.parts import BuildContext, Workspace
    dev = torch.device("cuda:0")
    return BuildContext(DT[dtype], dev, Workspace(dev))


def give(part, dtype, seed=0):
    """Random tensors for everything the part declares; returns {name: float64 copy}."""
    from inferloop_b200.weights import random_tensor, target_dtype
    tensors = {d.name: random_tensor(d, seed, target_dtype(d.role, DT[dtype]), "cuda") for d in part.declare_weights()}
    part.bind(tensors)
    return {k: v.double().cpu() for k, v in tensors.items()}


def bound(dtype, ref):
    return 1e-5 + 1e-5 * ref.abs() if dtype == "float32" else torch.full_like(ref, 2e-2 * float(ref.abs().max()))


def make_step(needs, entries, page_size=8, num_pages=32):
    from inferloop_b200.cache import CacheManager
    from inferloop_b200.engine.batch import StepStager
    from inferloop_b200.engine.runner import prepare_step
    return CacheManager, StepStager, prepare_step


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rms_norm_part(dtype):
    from inferloop_b200.parts import build_norm
    ctx = env(dtype)
    part = build_norm(PartSpec.make("rms", eps=2e-5), ctx, "some.norm.", width=88)
    w = give(part, dtype)
    assert list(w) == ["some.norm.weight"]
    x = torch.randn(9, 88, device="cuda")
    out = torch.empty(9, 88, dtype=DT[dtype], device="cuda")
    part.forward(x, out)
    ref = plain.rms_norm(x.double().cpu(), w["some.norm.weight"], 2e-5)
    assert ((out.double().cpu() - ref).abs() <= bound(dtype, ref)).all()


def run_mixer(dtype, spec, hidden, entries_tokens, window=None, page_size=8):
    """Build the mixer, run it over a batch of (start position, n tokens) pieces given in
    two steps so that the second reads what the first left in the cache."""
    from inferloop_b200.cache import CacheManager
    from inferloop_b200.engine.batch import StepEntry, StepStager
    from inferloop_b200.engine.runner import prepare_step
    from inferloop_b200.parts import build
    ctx = env(dtype)
    mixer = build("mixer", spec, ctx, "attn.")
    w = give(mixer, dtype, seed=3)
    cache = CacheManager([mixer.cache_needs()], page_size, 32, 4, dtype=DT[dtype], device=ctx.device)
    stager = StepStager(ctx.device)
    lc = cache.layer_cache(RunEntry(0, 0))
    outs = {}
    xs = {rid: torch.randn(n, hidden) for rid, n in entries_tokens.items()}
    cursor = {rid: 0 for rid in xs}
    for cut in ({"a": 19, "b": 5}, {"a": 1, "b": 22, "c": 9}):
        entries = [StepEntry(rid, [0] * n, []) for rid, n in cut.items()]
        step = prepare_step(cache, stager, entries, 10, 4096)
        x = torch.cat([xs[rid][cursor[rid]:cursor[rid] + n] for rid, n in cut.items()]).to(DT[dtype]).cuda()
        residual = torch.zeros(x.shape[0], hidden, device="cuda")
        mixer.forward(x, residual, step, lc)
        off = 0
        for rid, n in cut.items():
            outs.setdefault(rid, []).append(residual[off:off + n].double().cpu())
            off += n
            cache.commit(rid, cache.length(rid) + n)
            cursor[rid] += n
    return w, xs, {rid: torch.cat(v) for rid, v in outs.items()}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nq,nkv,d,hidden,bias,qk_norm,window,rot", [
    (4, 2, 16, 40, False, True, None, 16), (6, 3, 32, 72, True, True, 7, 16), (2, 2, 48, 56, True, False, None, 48)])
def test_attention_part(dtype, nq, nkv, d, hidden, bias, qk_norm, window, rot):
    spec = PartSpec.make("gqa_attention", hidden_size=hidden, num_heads=nq, num_kv_heads=nkv, head_dim=d,
                         qk_norm=qk_norm, qk_norm_eps=1e-5, bias=bias, window=window,
                         position=PartSpec.make("rope_neox", theta=7000.0, rotary_dim=rot, head_dim=d))
    w, xs, got = run_mixer(dtype, spec, hidden, {"a": 20, "b": 27, "c": 9})
    cfg = dict(num_attention_heads=nq, num_key_value_heads=nkv, head_dim=d, attention_bias=bias,
               rms_norm_eps=1e-5, partial_rotary_factor=rot / d, rope_theta=7000.0)
    if not qk_norm:
        w["attn.q_norm.weight"] = torch.ones(d, dtype=torch.float64)
        w["attn.k_norm.weight"] = torch.ones(d, dtype=torch.float64)
    for rid, x in xs.items():
        xin = x.to(DT[dtype]).double()
        if qk_norm:
            ref = plain.attention_block(xin, w, "attn.", cfg, torch.arange(len(x)), window)
        else:   # the plain block always norms; restate it without
            T = len(x)
            lin = lambda n: plain.linear(xin, w[f"attn.{n}_proj.weight"], w.get(f"attn.{n}_proj.bias") if bias else None)
            q = plain.rope_neox(lin("q").view(T, nq, d), torch.arange(T), 7000.0, rot)
            k = plain.rope_neox(lin("k").view(T, nkv, d), torch.arange(T), 7000.0, rot)
            o = plain.causal_attention(q, k, lin("v").view(T, nkv, d), torch.arange(T), window).reshape(T, nq * d)
            ref = plain.linear(o, w["attn.o_proj.weight"], w.get("attn.o_proj.bias") if bias else None)
        assert ((got[rid] - ref).abs() <= bound(dtype, ref)).all(), rid


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("inter", [136, 192])          # 192: a multiple of 64, the fused epilogue in bfloat16
def test_swiglu_part(dtype, inter):
    from inferloop_b200.parts import build
    ctx = env(dtype)
    part = build("feed_forward", PartSpec.make("swiglu", hidden_size=56, intermediate_size=inter), ctx, "ffn.")
    w = give(part, dtype, seed=8)
    assert part.fused == (dtype == "bfloat16" and inter % 64 == 0)
    x = torch.randn(13, 56).to(DT[dtype])
    residual = torch.randn(13, 56)
    out = residual.clone().cuda()
    part.forward(x.cuda(), out, None)
    ref = residual.double() + plain.swiglu_mlp(x.double(), w["ffn.gate_proj.weight"], w["ffn.up_proj.weight"],
                                               w["ffn.down_proj.weight"])
    assert ((out.double().cpu() - ref).abs() <= bound(dtype, ref)).all()


def test_position_part_tables_are_shared_per_step():
    from inferloop_b200.parts import build
    from types import SimpleNamespace
    ctx = env("float32")
    a = build("position", PartSpec.make("rope_neox", theta=1e4, rotary_dim=8, head_dim=8), ctx)
    b = build("position", PartSpec.make("rope_neox", theta=1e4, rotary_dim=8, head_dim=8), ctx)
    c = build("position", PartSpec.make("rope_neox", theta=1e6, rotary_dim=8, head_dim=8), ctx)
    step = SimpleNamespace(n_tokens=3, positions=torch.tensor([0, 5, 9], dtype=torch.int32, device="cuda"),
                           position_tables={})
    ta, tb, tc = a.table(step), b.table(step), c.table(step)
    assert ta.data_ptr() == tb.data_ptr() and ta.data_ptr() != tc.data_ptr()
    ang = torch.tensor([0, 5, 9], dtype=torch.float64)[:, None] * torch.tensor([1e4 ** (-2 * i / 8) for i in range(4)], dtype=torch.float64)
    assert (ta[..., 0].double().cpu() - torch.cos(ang)).abs().max() < 1e-7
    assert build("position", PartSpec.make("none"), ctx).table(step) is None


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_block_part(dtype):
    """A whole pre-norm block with sizes of its own equals the plain layer."""
    from inferloop_b200.cache import CacheManager
    from inferloop_b200.engine.batch import StepEntry, StepStager
    from inferloop_b200.engine.runner import prepare_step
    from inferloop_b200.parts import build_block
    H, nq, nkv, d, I = 48, 3, 1, 16, 104
    norm = PartSpec.make("rms", eps=1e-5)
    layer = LayerSpec(
        prefix="L.", block=PartSpec.make("pre_norm", hidden_size=H), norm=norm,
        mixer=PartSpec.make("gqa_attention", hidden_size=H, num_heads=nq, num_kv_heads=nkv, head_dim=d, qk_norm=True,
                            qk_norm_eps=1e-5, bias=False, window=None,
                            position=PartSpec.make("rope_neox", theta=1e4, rotary_dim=d, head_dim=d)),
        feed_forward=PartSpec.make("swiglu", hidden_size=H, intermediate_size=I))
    ctx = env(dtype)
    block = build_block(layer, ctx, layer.prefix)
    w = give(block, dtype, seed=11)
    cache = CacheManager([block.cache_needs()], 4, 16, 2, dtype=DT[dtype], device=ctx.device)
    step = prepare_step(cache, StepStager(ctx.device), [StepEntry("a", [0] * 21, [])], 10, 4096)
    x = torch.randn(21, H)
    hidden = x.clone().cuda()
    block.forward(hidden, step, cache.layer_cache(RunEntry(0, 0)))
    cfg = dict(num_attention_heads=nq, num_key_value_heads=nkv, head_dim=d, attention_bias=False,
               rms_norm_eps=1e-5, partial_rotary_factor=1.0, rope_theta=1e4)
    ref = plain.decoder_layer(x.double(), w, "L.", cfg, torch.arange(21), None)
    assert ((hidden.double().cpu() - ref).abs() <= bound(dtype, ref)).all()


def test_one_seed_gives_one_model_on_every_device():
    """The random-weights generator is integer arithmetic and IEEE multiply/add only: a
    tensor made on the GPU has the bits of the one made on the CPU, in both dtypes, across
    the generator's chunk edge too."""
    from inferloop_b200.weights import random_init
    from inferloop_b200.weights.decl import WeightDecl
    big = random_init._CHUNK + 12_345
    a = random_init.standard_normal(2024, big, "cuda")
    b = random_init.standard_normal(2024, big, "cpu")
    assert torch.equal(a.cpu(), b)
    for decl in (WeightDecl("x.weight", (130, 77)), WeightDecl("n.weight", (515,), "vector", "norm"),
                 WeightDecl("b.bias", (96,), "vector", "bias")):
        for dtype in (torch.float32, torch.bfloat16):
            on_gpu = random_init.random_tensor(decl, 5, dtype, "cuda")
            on_cpu = random_init.random_tensor(decl, 5, dtype, "cpu")
            assert on_gpu.dtype == dtype and torch.equal(on_gpu.cpu(), on_cpu), decl.name
