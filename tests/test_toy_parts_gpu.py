"""More toy parts, defined HERE and registered without a change to the framework's files
(GPU): a feed-forward that routes every token to one of three small experts, and a position
encoding other than the architecture's (rotary angles of positions divided by a factor);
further down a position encoding of two axes with what sits around the layers, and a norm
and a block of another kind.

The toy architecture alternates them layer by layer: layer 0 has the stock attention with the
stock rotary encoding and the routed feed-forward, layer 1 the stock attention with the scaled
encoding and the stock SwiGLU.  Whole prompts, portions and single tokens must agree with the
plain 64-bit statement of the same model.
"""
import pytest
import torch

import plain_qwen3 as plain
from helpers import random_tokens
from inferloop_b200.config import Architecture, ArchitectureRegistry, LayerSpec, ModelSpec, PartSpec, RunEntry
from inferloop_b200.parts import Block, FeedForward, Norm, PositionEncoding, register, unregister
from inferloop_b200.parts import registry as parts_registry
from inferloop_b200.weights.decl import WeightDecl

pytestmark = pytest.mark.gpu

H, V, E, I = 48, 131, 3, 40


class RoutedFeedForward(FeedForward):
    """Router logits in 32-bit from the normed input; the best expert alone runs (ties to the
    lower index); its output, scaled by its softmax weight among all experts, is added to the
    residual.  Each expert is y = W2 relu(W1 x)."""

    def __init__(self, spec, ctx, prefix=""):
        super().__init__(spec, ctx, prefix)
        self.hidden, self.experts, self.inter = int(spec["hidden_size"]), int(spec["experts"]), int(spec["inter"])
        self.p = prefix

    def declare_weights(self):
        out = [WeightDecl(self.p + "router.weight", (self.experts, self.hidden))]
        for e in range(self.experts):
            out += [WeightDecl(f"{self.p}experts.{e}.w1.weight", (self.inter, self.hidden)),
                    WeightDecl(f"{self.p}experts.{e}.w2.weight", (self.hidden, self.inter))]
        return out

    def bind(self, tensors):
        self.router = tensors[self.p + "router.weight"].float()
        self.w1 = [tensors[f"{self.p}experts.{e}.w1.weight"].float() for e in range(self.experts)]
        self.w2 = [tensors[f"{self.p}experts.{e}.w2.weight"].float() for e in range(self.experts)]

    def forward(self, x, residual, step):
        xf = x.float()
        logits = xf @ self.router.T                       # [T, E], 32-bit
        weight = torch.softmax(logits, dim=-1)
        choice = logits.argmax(dim=-1)
        for e in range(self.experts):
            rows = torch.nonzero(choice == e).flatten()
            if rows.numel():
                y = torch.relu(xf[rows] @ self.w1[e].T) @ self.w2[e].T
                residual[rows] += y * weight[rows, e:e + 1]


class ScaledRope(PositionEncoding):
    """The stock table format ([T, rd/2, 2] cos/sin), but of positions divided by `factor`."""

    def __init__(self, spec, ctx, prefix=""):
        super().__init__(spec, ctx, prefix)
        self.theta, self.rd, self.factor = float(spec["theta"]), int(spec["rotary_dim"]), float(spec["factor"])

    def table(self, step):
        key = ("scaled_rope", self.theta, self.rd, self.factor)
        t = step.position_tables.get(key)
        if t is None:
            half = self.rd // 2
            inv = torch.tensor([self.theta ** (-(2.0 * i) / self.rd) for i in range(half)], dtype=torch.float64,
                               device=step.positions.device)
            ang = step.positions.double()[:, None] / self.factor * inv[None, :]
            t = torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).float().contiguous()
            step.position_tables[key] = t
        return t


def toy_spec(cfg):
    norm = PartSpec.make("rms", eps=cfg["eps"])

    def attn(position):
        return PartSpec.make("gqa_attention", hidden_size=H, num_heads=3, num_kv_heads=3, head_dim=16, qk_norm=True,
                             qk_norm_eps=cfg["eps"], bias=False, window=None, position=position)

    rope = PartSpec.make("rope_neox", theta=1e4, rotary_dim=16, head_dim=16)
    scaled = PartSpec.make("scaled_rope", theta=1e4, rotary_dim=16, head_dim=16, factor=cfg["factor"])
    routed = PartSpec.make("routed_relu", hidden_size=H, experts=E, inter=I)
    dense = PartSpec.make("swiglu", hidden_size=H, intermediate_size=64)
    block = PartSpec.make("pre_norm", hidden_size=H)
    layers = (LayerSpec("layers.0.", block, attn(rope), routed, norm), LayerSpec("layers.1.", block, attn(scaled), dense, norm))
    return ModelSpec("Toy2ForCausalLM", V, H, 512, "embed_tokens.weight", "lm_head.weight", "norm.weight", norm,
                     layers, run_order=(RunEntry(0, 0), RunEntry(1, 1)), weight_prefixes=("model.",))


def plain_toy(w, cfg, tokens):
    T = len(tokens)
    x = w["embed_tokens.weight"][torch.tensor(tokens)]
    pos = torch.arange(T)
    acfg = dict(num_attention_heads=3, num_key_value_heads=3, head_dim=16, attention_bias=False,
                rms_norm_eps=cfg["eps"], partial_rotary_factor=1.0, rope_theta=1e4)
    # layer 0: stock attention, routed feed-forward
    p = "layers.0."
    n = plain.rms_norm(x, w[p + "input_layernorm.weight"], cfg["eps"])
    x = x + plain.attention_block(n, w, p + "self_attn.", acfg, pos, None)
    n = plain.rms_norm(x, w[p + "post_attention_layernorm.weight"], cfg["eps"])
    logits = n @ w[p + "mlp.router.weight"].T
    weight = torch.softmax(logits, dim=-1)
    top2 = logits.topk(2, dim=-1).values
    margin = (top2[:, 0] - top2[:, 1]) / logits.abs().max()      # how decided each token's routing is
    for t in range(T):
        e = int(logits[t].argmax())
        y = torch.relu(n[t] @ w[f"{p}mlp.experts.{e}.w1.weight"].T) @ w[f"{p}mlp.experts.{e}.w2.weight"].T
        x[t] = x[t] + y * weight[t, e]
    # layer 1: attention with positions divided by the factor, stock SwiGLU
    p = "layers.1."
    a = p + "self_attn."
    n = plain.rms_norm(x, w[p + "input_layernorm.weight"], cfg["eps"])
    scaled = pos.double() / cfg["factor"]
    q = plain.rope_neox(plain.rms_norm(plain.linear(n, w[a + "q_proj.weight"]).view(T, 3, 16), w[a + "q_norm.weight"], cfg["eps"]), scaled, 1e4, 16)
    k = plain.rope_neox(plain.rms_norm(plain.linear(n, w[a + "k_proj.weight"]).view(T, 3, 16), w[a + "k_norm.weight"], cfg["eps"]), scaled, 1e4, 16)
    v = plain.linear(n, w[a + "v_proj.weight"]).view(T, 3, 16)
    o = plain.causal_attention(q, k, v, pos, None).reshape(T, 48)
    x = x + plain.linear(o, w[a + "o_proj.weight"])
    n = plain.rms_norm(x, w[p + "post_attention_layernorm.weight"], cfg["eps"])
    x = x + plain.swiglu_mlp(n, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    return plain.linear(plain.rms_norm(x, w["norm.weight"], cfg["eps"]), w["lm_head.weight"]), margin


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_routed_feed_forward_and_another_position_encoding(dtype):
    from inferloop_b200.engine import ModelRunner, StepEntry
    from inferloop_b200.models.decoder import declare_weights
    from inferloop_b200.weights import random_tensor, target_dtype
    register("feed_forward", "routed_relu", RoutedFeedForward)
    register("position", "scaled_rope", ScaledRope)
    try:
        registry = ArchitectureRegistry()
        registry.register(Architecture("toy2", ("Toy2ForCausalLM",), dict, toy_spec))
        cfg = {"architectures": ["Toy2ForCausalLM"], "eps": 1e-6, "factor": 4.0}
        runner = ModelRunner.from_config(cfg, seed=9, dtype=dtype, page_size=8, num_pages=32, max_requests=3,
                                         registry=registry)
        assert runner.graphs is None          # the toy parts read the batch on the host: no replayed graphs
        DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
        w = {d.name: random_tensor(d, 9, target_dtype(d.role, DT), "cuda").double().cpu() for d in declare_weights(toy_spec(cfg))}
        toks = {"a": random_tokens(50, V, 11), "b": random_tokens(37, V, 12)}
        both = {rid: plain_toy(w, cfg, t) for rid, t in toks.items()}
        ref = {rid: b[0] for rid, b in both.items()}
        margin = {rid: b[1] for rid, b in both.items()}
        # a whole, b in portions beside a's decode steps
        got = {"a": [], "b": []}
        got["a"].append(runner.step([StepEntry("a", toks["a"][:30], list(range(30)))]).double().cpu().clone())
        ia, ib = 30, 0
        for cut in (5, 2, 11, 1, 18):
            entries = [StepEntry("b", toks["b"][ib:ib + cut], list(range(cut)))]
            if ia < 50:
                entries.insert(0, StepEntry("a", [toks["a"][ia]], [0]))
            out = runner.step(entries).double().cpu().clone()
            if ia < 50:
                got["a"].append(out[:1]); out = out[1:]; ia += 1
            got["b"].append(out)
            ib += cut
        while ia < 50:
            got["a"].append(runner.step([StepEntry("a", [toks["a"][ia]], [0])]).double().cpu().clone())
            ia += 1
        for rid in toks:
            runner.end(rid)
            g = torch.cat(got[rid])
            assert g.shape == ref[rid].shape and torch.isfinite(g).all()
            err = (g - ref[rid]).abs()
            if dtype == "float32":
                assert (err <= 1e-5 + 1e-5 * ref[rid].abs()).all(), (rid, err.max().item())
            else:
                # in bfloat16 a router logit within rounding of the best may pick the other
                # expert, and every later token (which attends to that one) then differs for a
                # reason that is no fault: rows are compared up to the first token whose plain
                # routing margin is below 0.5 % of the largest router logit (bfloat16 keeps 8 bits)
                close = (margin[rid] < 0.005).nonzero()
                upto = int(close[0]) if close.numel() else len(margin[rid])
                assert upto >= 5, "the seed gives no decided prefix to compare"
                lim = 1e-2 * float(ref[rid].abs().max())
                assert (err[:upto] <= lim).all(), (rid, upto, err[:upto].max().item())
    finally:
        unregister("feed_forward", "routed_relu")
        unregister("position", "scaled_rope")


# ------------------------------------------------------------------ what sits around the layers
class TwoAxisRope(PositionEncoding):
    """Rotary angles from TWO position axes per token (rows and columns of a grid, say): the
    first half of the rotation pairs turns with axis 0, the second half with axis 1.  The
    axes come as a declared per-token input, `pos2` [tokens, 2], not from the 1-D positions."""

    graph_safe = True        # device operations on device tensors only (its constants are made at construction)

    def __init__(self, spec, ctx, prefix=""):
        super().__init__(spec, ctx, prefix)
        self.theta, self.rd = float(spec["theta"]), int(spec["rotary_dim"])
        half = self.rd // 2
        if ctx.device is not None:
            self.inv = torch.tensor([self.theta ** (-(2.0 * i) / self.rd) for i in range(half)], dtype=torch.float64,
                                    device=ctx.device)
            self.which = (torch.arange(half, device=ctx.device) >= half // 2).long()

    def table(self, step):
        key = ("two_axis_rope", self.theta, self.rd)
        t = step.position_tables.get(key)
        if t is None:
            axes = step.extras["pos2"].double()                        # [T, 2]
            ang = axes[:, self.which] * self.inv[None, :]
            t = torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).float().contiguous()
            step.position_tables[key] = t
        return t


EMBED_SCALE, LOGIT_CAP, LOGIT_SCALE = 1.75, 2.5, 3.0


def toy3_spec(cfg):
    norm = PartSpec.make("rms", eps=cfg["eps"])
    pos = PartSpec.make("two_axis_rope", theta=1e4, rotary_dim=16, head_dim=16)
    attn = PartSpec.make("gqa_attention", hidden_size=H, num_heads=3, num_kv_heads=3, head_dim=16, qk_norm=True,
                         qk_norm_eps=cfg["eps"], bias=False, window=None, position=pos)
    dense = PartSpec.make("swiglu", hidden_size=H, intermediate_size=64)
    block = PartSpec.make("pre_norm", hidden_size=H)
    layers = (LayerSpec("layers.0.", block, attn, dense, norm), LayerSpec("layers.1.", block, attn, dense, norm))
    return ModelSpec("Toy3ForCausalLM", V, H, 512, "embed_tokens.weight", None, "norm.weight", norm, layers,
                     weight_prefixes=("model.",), embedding_scale=EMBED_SCALE,
                     logits_post=PartSpec.make("soft_cap", cap=LOGIT_CAP, scale=LOGIT_SCALE),
                     token_extras=(("pos2", 2),))


def plain_toy3(w, cfg, tokens, pos2):
    T = len(tokens)
    x = w["embed_tokens.weight"][torch.tensor(tokens)] * EMBED_SCALE
    pos = torch.arange(T)
    inv = torch.tensor([1e4 ** (-(2.0 * i) / 16) for i in range(8)], dtype=torch.float64)
    axes = torch.tensor(pos2, dtype=torch.float64)
    ang = axes[:, (torch.arange(8) >= 4).long()] * inv[None, :]             # [T, 8]

    def rotate(v):                                                        # v [T, heads, 16], pairs (i, i + 8)
        a, b = v[..., :8], v[..., 8:]
        c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        return torch.cat([a * c - b * s, a * s + b * c], dim=-1)

    for layer in range(2):
        p = f"layers.{layer}."
        a = p + "self_attn."
        n = plain.rms_norm(x, w[p + "input_layernorm.weight"], cfg["eps"])
        q = rotate(plain.rms_norm(plain.linear(n, w[a + "q_proj.weight"]).view(T, 3, 16), w[a + "q_norm.weight"], cfg["eps"]))
        k = rotate(plain.rms_norm(plain.linear(n, w[a + "k_proj.weight"]).view(T, 3, 16), w[a + "k_norm.weight"], cfg["eps"]))
        v = plain.linear(n, w[a + "v_proj.weight"]).view(T, 3, 16)
        x = x + plain.linear(plain.causal_attention(q, k, v, pos, None).reshape(T, 48), w[a + "o_proj.weight"])
        n = plain.rms_norm(x, w[p + "post_attention_layernorm.weight"], cfg["eps"])
        x = x + plain.swiglu_mlp(n, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    logits = plain.linear(plain.rms_norm(x, w["norm.weight"], cfg["eps"]), w["embed_tokens.weight"])
    return LOGIT_CAP * torch.tanh(logits * LOGIT_SCALE / LOGIT_CAP)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embedding_multiplier_logits_map_and_inputs_per_token(dtype):
    """A description with a multiplier on the embedding rows, a soft cap on the logits (a part of
    role "logits") and a position encoding that reads two axes per token from a declared
    per-token input: portions, single tokens through recorded graphs, and the entry point
    (which continues the axes for generated tokens), all against the plain statement."""
    from inferloop_b200 import Engine, SamplingParams
    from inferloop_b200.engine import ModelRunner, StepEntry
    from inferloop_b200.models.decoder import declare_weights
    from inferloop_b200.weights import random_tensor, target_dtype
    register("position", "two_axis_rope", TwoAxisRope)
    try:
        registry = ArchitectureRegistry()
        registry.register(Architecture("toy3", ("Toy3ForCausalLM",), dict, toy3_spec))
        cfg = {"architectures": ["Toy3ForCausalLM"], "eps": 1e-6}
        runner = ModelRunner.from_config(cfg, seed=13, dtype=dtype, page_size=8, num_pages=32, max_requests=3,
                                         registry=registry)
        DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
        w = {d.name: random_tensor(d, 13, target_dtype(d.role, DT), "cuda").double().cpu() for d in declare_weights(toy3_spec(cfg))}
        toks = random_tokens(40, V, 21)
        pos2 = [[t // 7, t % 7] for t in range(40)]                     # a grid seven wide, row by row
        ref = plain_toy3(w, cfg, toks, pos2)
        flat = lambda a, b: [x for row in pos2[a:b] for x in row]
        got, i = [], 0
        for cut in (9, 2, 12, 1, 1, 1, 14):                            # single tokens: recorded graphs
            got.append(runner.step([StepEntry("a", toks[i:i + cut], list(range(cut)), {"pos2": flat(i, i + cut)})]).double().cpu().clone())
            i += cut
        runner.end("a")
        assert runner.graphs is not None and runner.graphs.replays >= 2
        g = torch.cat(got)
        err = (g - ref).abs()
        lim = 1e-5 + 1e-5 * ref.abs() if dtype == "float32" else torch.full_like(ref, 1e-2 * float(ref.abs().max()))
        assert (err <= lim).all(), err.max().item()
        assert float(g.abs().max()) <= LOGIT_CAP
        with pytest.raises(ValueError, match="must bring"):
            runner.step([StepEntry("b", toks[:3], [2])])
        # through the entry point: generated tokens continue both axes by one each
        engine = Engine(None, runner=runner, max_num_seqs=2, prefill_chunk_tokens=16)
        prompt = toks[:11]
        rid = engine.submit(prompt, SamplingParams(), 6, extras={"pos2": flat(0, 11)})
        while not engine.is_idle():
            engine.step()
        out = engine.result(rid).generated
        seq, axes = list(prompt), [list(r) for r in pos2[:11]]
        for n in range(6):
            axes.append([pos2[10][0] + n + 1, pos2[10][1] + n + 1])
            logits = plain_toy3(w, cfg, seq + [out[n]], axes)[-2]
            if dtype == "float32":
                assert out[n] == int(logits.argmax())
            else:
                assert logits[out[n]] >= logits.max() - 2e-2 * float(logits.abs().max())
            seq.append(out[n])
        with pytest.raises(ValueError, match="values of 'pos2'"):
            engine.submit(prompt, SamplingParams(), 2)
    finally:
        unregister("position", "two_axis_rope")


# ------------------------------------------------------------------ another norm and another arrangement of a block
class CenteredNorm(Norm):
    """(x - mean) / sqrt(var + eps) * weight + bias over the last dimension, in 32-bit: a norm
    with two tensors, written with library elementwise operations (a toy, not a model's)."""

    graph_safe = True

    def __init__(self, spec, ctx, prefix="", width=0):
        super().__init__(spec, ctx, prefix)
        self.eps, self.width, self.p = float(spec["eps"]), int(width), prefix

    def declare_weights(self):
        return [WeightDecl(self.p + "weight", (self.width,), role="vector", init="norm"),
                WeightDecl(self.p + "bias", (self.width,), role="vector", init="bias")]

    def bind(self, tensors):
        self.weight, self.bias = tensors[self.p + "weight"], tensors[self.p + "bias"]

    def forward(self, x, out):
        mean = x.mean(dim=-1, keepdim=True)
        var = ((x - mean) ** 2).mean(dim=-1, keepdim=True)
        out.copy_((x - mean) * torch.rsqrt(var + self.eps) * self.weight + self.bias)


class ParallelBlock(Block):
    """h += mixer(norm(h)) + ffn(norm(h)): ONE norm per layer, both branches read it."""

    def __init__(self, spec, ctx, prefix="", layer=None):
        super().__init__(spec, ctx, prefix)
        self.hidden = int(spec["hidden_size"])
        self.norm = parts_registry.build_norm(layer.norm, ctx, prefix + "ln.", width=self.hidden)
        self.mixer = parts_registry.build("mixer", layer.mixer, ctx, prefix + "self_attn.")
        self.ffn = parts_registry.build("feed_forward", layer.feed_forward, ctx, prefix + "mlp.")

    @property
    def graph_safe(self):
        return all(p.graph_safe for p in (self.norm, self.mixer, self.ffn))

    def declare_weights(self):
        return self.norm.declare_weights() + self.mixer.declare_weights() + self.ffn.declare_weights()

    def bind(self, tensors):
        for part in (self.norm, self.mixer, self.ffn):
            part.bind(tensors)

    def cache_needs(self):
        return self.mixer.cache_needs()

    def scratch_bytes(self, tokens):
        return tokens * self.hidden * 4 + self.mixer.scratch_bytes(tokens) + self.ffn.scratch_bytes(tokens)

    def forward(self, hidden, step, cache):
        normed = self.ctx.workspace.buffer("toy4.normed", hidden.shape, self.ctx.dtype)
        self.norm.forward(hidden, normed)
        self.mixer.forward(normed, hidden, step, cache)       # both branches add into the residual
        self.ffn.forward(normed, hidden, step)


def toy4_spec(cfg):
    norm = PartSpec.make("centered", eps=cfg["eps"])
    pos = PartSpec.make("rope_neox", theta=1e4, rotary_dim=16, head_dim=16)
    attn = PartSpec.make("gqa_attention", hidden_size=H, num_heads=3, num_kv_heads=1, head_dim=16, qk_norm=False,
                         qk_norm_eps=cfg["eps"], bias=False, window=None, position=pos)
    dense = PartSpec.make("swiglu", hidden_size=H, intermediate_size=64)
    block = PartSpec.make("parallel", hidden_size=H)
    layers = tuple(LayerSpec(f"layers.{i}.", block, attn, dense, norm) for i in range(3))
    return ModelSpec("Toy4ForCausalLM", V, H, 512, "embed_tokens.weight", None, "norm.weight", norm, layers,
                     weight_prefixes=("model.",))


def plain_toy4(w, cfg, tokens):
    T = len(tokens)
    x = w["embed_tokens.weight"][torch.tensor(tokens)]
    pos = torch.arange(T)

    def centered(v, p):
        m = v.mean(dim=-1, keepdim=True)
        var = ((v - m) ** 2).mean(dim=-1, keepdim=True)
        return (v - m) / torch.sqrt(var + cfg["eps"]) * w[p + "weight"] + w[p + "bias"]

    for layer in range(3):
        p = f"layers.{layer}."
        a = p + "self_attn."
        n = centered(x, p + "ln.")
        q = plain.rope_neox(plain.linear(n, w[a + "q_proj.weight"]).view(T, 3, 16), pos, 1e4, 16)
        k = plain.rope_neox(plain.linear(n, w[a + "k_proj.weight"]).view(T, 1, 16), pos, 1e4, 16)
        v = plain.linear(n, w[a + "v_proj.weight"]).view(T, 1, 16)
        attn = plain.linear(plain.causal_attention(q, k, v, pos, None).reshape(T, 48), w[a + "o_proj.weight"])
        x = x + attn + plain.swiglu_mlp(n, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    return plain.linear(centered(x, "norm."), w["embed_tokens.weight"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_another_norm_and_another_arrangement_of_a_block(dtype):
    """A norm with a mean and a bias and a block whose two branches read one norm, both defined
    in this file: built by name from the description, stepped in portions and single tokens
    (through recorded graphs) and generated from through the entry point, against the plain
    statement of the same model."""
    from inferloop_b200 import Engine, SamplingParams
    from inferloop_b200.engine import ModelRunner, StepEntry
    from inferloop_b200.models.decoder import declare_weights
    from inferloop_b200.weights import random_tensor, target_dtype
    register("norm", "centered", CenteredNorm)
    register("block", "parallel", ParallelBlock)
    try:
        registry = ArchitectureRegistry()
        registry.register(Architecture("toy4", ("Toy4ForCausalLM",), dict, toy4_spec))
        cfg = {"architectures": ["Toy4ForCausalLM"], "eps": 1e-5}
        runner = ModelRunner.from_config(cfg, seed=17, dtype=dtype, page_size=8, num_pages=32, max_requests=3,
                                         registry=registry)
        DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
        w = {d.name: random_tensor(d, 17, target_dtype(d.role, DT), "cuda").double().cpu() for d in declare_weights(toy4_spec(cfg))}
        assert "layers.1.ln.bias" in w and "norm.bias" in w and "layers.0.post_attention_layernorm.weight" not in w
        toks = random_tokens(45, V, 23)
        ref = plain_toy4(w, cfg, toks)
        got, i = [], 0
        for cut in (17, 2, 9, 1, 1, 1, 14):
            got.append(runner.step([StepEntry("a", toks[i:i + cut], list(range(cut)))]).double().cpu().clone())
            i += cut
        runner.end("a")
        assert runner.graphs is not None and runner.graphs.replays >= 2
        g = torch.cat(got)
        err = (g - ref).abs()
        lim = 1e-5 + 1e-5 * ref.abs() if dtype == "float32" else torch.full_like(ref, 1e-2 * float(ref.abs().max()))
        assert (err <= lim).all(), err.max().item()
        engine = Engine(None, runner=runner, max_num_seqs=2, prefill_chunk_tokens=16)
        out = engine.generate([toks[:13]], SamplingParams(), 5)[0]
        seq = list(toks[:13])
        for n in range(5):
            logits = plain_toy4(w, cfg, seq)[-1]
            if dtype == "float32":
                assert out[n] == int(logits.argmax())
            else:
                assert logits[out[n]] >= logits.max() - 2e-2 * float(logits.abs().max())
            seq.append(out[n])
    finally:
        unregister("norm", "centered")
        unregister("block", "parallel")
