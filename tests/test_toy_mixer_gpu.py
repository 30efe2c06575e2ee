"""A mixer with state of its own, defined HERE, is registered, built into a model beside
attention layers, and stepped -- without a change to the framework's files (GPU).

The toy architecture has three layers: [attention, toy recurrence, attention], the
run order names layer 0 twice, and its last entry reads layer 0's cache without writing
it.  The recurrence keeps s <- decay * s + x W per request in its state slot; portions
of changing size must give what the whole sequence gives, which only holds if the slot
carries the state from step to step and is cleared when a new request takes it.
"""
import json
import math

import pytest
import torch

import plain_qwen3 as plain
from helpers import random_tokens
from inferloop_b200.config import Architecture, ArchitectureRegistry, LayerSpec, ModelSpec, PartSpec, RunEntry
from inferloop_b200.parts import CacheNeeds, Mixer, SlotStateNeed, register, unregister
from inferloop_b200.weights.decl import WeightDecl

pytestmark = pytest.mark.gpu

H, V = 40, 97


class DecayMixer(Mixer):
    """y_t = s_t,  s_t = decay * s_{t-1} + W x_t, one state vector per request."""

    def __init__(self, spec, ctx, prefix=""):
        super().__init__(spec, ctx, prefix)
        self.hidden, self.decay = int(spec["hidden_size"]), float(spec["decay"])
        self.name = prefix + "mix.weight"

    def declare_weights(self):
        return [WeightDecl(self.name, (self.hidden, self.hidden))]

    def bind(self, tensors):
        self.w = tensors[self.name].float()

    def cache_needs(self):
        return CacheNeeds(slots=(SlotStateNeed("s", (self.hidden,), torch.float32),))

    def forward(self, x, residual, step, cache):
        state = cache.state["s"]
        proj = x.float() @ self.w.T
        off = 0
        for slot, n in zip(step.h_slots, step.h_q_len):           # each request's tokens, in order
            s = state[slot]
            for t in range(off, off + n):
                s = self.decay * s + proj[t]
                residual[t] += s
            state[slot] = s
            off += n


def toy_spec(cfg):
    norm = PartSpec.make("rms", eps=cfg["eps"])
    attn = PartSpec.make("gqa_attention", hidden_size=H, num_heads=4, num_kv_heads=2, head_dim=16, qk_norm=True,
                         qk_norm_eps=cfg["eps"], bias=False, window=None,
                         position=PartSpec.make("rope_neox", theta=1e4, rotary_dim=16, head_dim=16))
    toy = PartSpec.make("decay_state", hidden_size=H, decay=cfg["decay"])
    ffn = PartSpec.make("swiglu", hidden_size=H, intermediate_size=72)
    block = PartSpec.make("pre_norm", hidden_size=H)
    layers = tuple(LayerSpec(f"layers.{i}.", block, m, ffn, norm) for i, m in enumerate((attn, toy, attn)))
    order = (RunEntry(0, 0), RunEntry(1, 1), RunEntry(2, 2), RunEntry(0, 0, writes_cache=False))
    return ModelSpec("ToyForCausalLM", V, H, 512, "embed_tokens.weight", "lm_head.weight", "norm.weight", norm,
                     layers, run_order=order, weight_prefixes=("model.",))


def plain_toy(w, cfg, tokens):
    """The same model, whole sequence, 64-bit, from the plain parts."""
    x = w["embed_tokens.weight"][torch.tensor(tokens)]
    T = len(tokens)
    pos = torch.arange(T)
    acfg = dict(num_attention_heads=4, num_key_value_heads=2, head_dim=16, attention_bias=False,
                rms_norm_eps=cfg["eps"], partial_rotary_factor=1.0, rope_theta=1e4)

    def ffn(x, p):
        n = plain.rms_norm(x, w[p + "post_attention_layernorm.weight"], cfg["eps"])
        return x + plain.swiglu_mlp(n, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])

    def attn_layer(x, p):
        n = plain.rms_norm(x, w[p + "input_layernorm.weight"], cfg["eps"])
        return ffn(x + plain.attention_block(n, w, p + "self_attn.", acfg, pos, None), p)

    def attn_layer_reading(x, p, kv_from):
        """Layer p's weights for q and o, but keys and values as layer p wrote them
        earlier in the run order (from `kv_from`, the layer's input at that time)."""
        n = plain.rms_norm(x, w[p + "input_layernorm.weight"], cfg["eps"])
        nk = plain.rms_norm(kv_from, w[p + "input_layernorm.weight"], cfg["eps"])
        a = p + "self_attn."
        q = plain.rope_neox(plain.rms_norm(plain.linear(n, w[a + "q_proj.weight"]).view(T, 4, 16), w[a + "q_norm.weight"], cfg["eps"]), pos, 1e4, 16)
        k = plain.rope_neox(plain.rms_norm(plain.linear(nk, w[a + "k_proj.weight"]).view(T, 2, 16), w[a + "k_norm.weight"], cfg["eps"]), pos, 1e4, 16)
        v = plain.linear(nk, w[a + "v_proj.weight"]).view(T, 2, 16)
        o = plain.causal_attention(q, k, v, pos, None).reshape(T, 64)
        return ffn(x + plain.linear(o, w[a + "o_proj.weight"]), p)

    x0 = x
    x = attn_layer(x, "layers.0.")
    n = plain.rms_norm(x, w["layers.1.input_layernorm.weight"], cfg["eps"])
    proj = n @ w["layers.1.self_attn.mix.weight"].T
    s = torch.zeros(H, dtype=torch.float64)
    y = []
    for t in range(T):
        s = cfg["decay"] * s + proj[t]
        y.append(s)
    x = ffn(x + torch.stack(y), "layers.1.")
    x = attn_layer(x, "layers.2.")
    x = attn_layer_reading(x, "layers.0.", x0)
    return plain.linear(plain.rms_norm(x, w["norm.weight"], cfg["eps"]), w["lm_head.weight"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_mixer_registered_built_and_stepped(dtype):
    from inferloop_b200.engine import ModelRunner, StepEntry
    register("mixer", "decay_state", DecayMixer)
    try:
        registry = ArchitectureRegistry()
        registry.register(Architecture("toy", ("ToyForCausalLM",), dict, toy_spec))
        cfg = {"architectures": ["ToyForCausalLM"], "eps": 1e-5, "decay": 0.9}
        runner = ModelRunner.from_config(cfg, seed=4, dtype=dtype, page_size=4, num_pages=64, max_requests=2,
                                         registry=registry)
        # one page group (layers 0 and 2), one slot tensor for layer 1; the borrowed entry owns nothing
        assert [g.layers for g in runner.cache.groups] == [[0, 2]]
        tensors = {}
        from inferloop_b200.models.decoder import declare_weights
        from inferloop_b200.weights import random_tensor, target_dtype
        DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
        for d in declare_weights(toy_spec(cfg)):
            tensors[d.name] = random_tensor(d, 4, target_dtype(d.role, DT), "cuda").double().cpu()
        for rid, n, cuts in (("a", 45, [45]), ("b", 45, [7, 2, 13, 1, 1, 21]), ("c", 30, [3, 27])):
            toks = random_tokens(n, V, 5)          # same tokens for a and b: same logits, and b
            got, i = [], 0                          # reuses a's slot, which must have been cleared
            for c in cuts:
                got.append(runner.step([StepEntry(rid, toks[i:i + c], list(range(c)))]).double().cpu().clone())
                i += c
            runner.end(rid)
            ref = plain_toy(tensors, cfg, toks)
            err = (torch.cat(got) - ref).abs()
            lim = 1e-5 + 1e-5 * ref.abs() if dtype == "float32" else torch.full_like(ref, 1e-2 * float(ref.abs().max()))
            assert (err <= lim).all(), (rid, err.max().item())
        # Two requests decoding side by side, one token each per step: the attention layers
        # around the toy mixer are replayed as recorded graph segments, the toy mixer (which
        # loops over the batch on the host) runs kernel by kernel between them.
        assert runner.graphs is not None and not runner.graphs.whole
        assert [safe for safe, _, _ in runner.graphs.plan] == [True, False, True]
        seqs = {"d": random_tokens(34, V, 8), "e": random_tokens(29, V, 9)}
        refs = {rid: plain_toy(tensors, cfg, toks) for rid, toks in seqs.items()}
        runner.step([StepEntry("d", seqs["d"][:14], []), StepEntry("e", seqs["e"][:9], [])])
        before = runner.graphs.replays
        for i in range(20):
            out = runner.step([StepEntry("d", [seqs["d"][14 + i]], [0]), StepEntry("e", [seqs["e"][9 + i]], [0])]).double().cpu()
            ref = torch.stack([refs["d"][14 + i], refs["e"][9 + i]])
            err = (out - ref).abs()
            lim = 1e-5 + 1e-5 * ref.abs() if dtype == "float32" else torch.full_like(ref, 1e-2 * float(ref.abs().max()))
            assert (err <= lim).all(), (i, err.max().item())
        assert runner.graphs.replays - before >= 18
        rec = next(iter(runner.graphs._recorded.values()))
        assert [seg[0] for seg in rec.segments] == ["graph", "entries", "graph"]
    finally:
        unregister("mixer", "decay_state")
