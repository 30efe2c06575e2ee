"""A plain, slow Qwen3 dense decoder used as the oracle of the tests.

Whole sequences, no cache, 64-bit arithmetic on the CPU, one function per part.  It
shares no code with `inferloop_b200`: it reads config.json with `json`, the weights with
the `safetensors` package, and names tensors itself.

It rests on the reference's FORMULAS, not on running the reference: 1994/inferloop is a
Rust workspace (no `cargo`/`rustc` here), contains no Python model code, and rejects
`attention_bias: true`, so it can neither be imported nor compiled on this machine.
Every function cites the file and lines (paths within the reference project) that it
restates.  Biases and the sliding window are this build's own extensions and say so.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch

F64 = torch.float64


# --------------------------------------------------------------------------- loading
def read_config(folder: str) -> dict:
    """Keys and defaults: crates/model/package/src/providers/qwen/mod.rs:101-165
    (head_dim 128, rms_norm_eps 1e-6, rope_theta 10000: mod.rs:79-95)."""
    with open(os.path.join(folder, "config.json")) as fh:
        raw = json.load(fh)
    cfg = dict(raw)
    cfg.setdefault("head_dim", 128)
    cfg.setdefault("rms_norm_eps", 1e-6)
    cfg.setdefault("rope_theta", 10000.0)
    cfg.setdefault("partial_rotary_factor", 1.0)
    cfg.setdefault("tie_word_embeddings", False)
    cfg.setdefault("attention_bias", False)
    cfg.setdefault("layer_types", ["full_attention"] * cfg["num_hidden_layers"])
    cfg.setdefault("sliding_window", None)
    return cfg


def load_tensors(folder: str, round_to_bf16: bool = False) -> Dict[str, torch.Tensor]:
    """All tensors as float64.  With `round_to_bf16`, every tensor of two or more
    dimensions is first rounded to bfloat16, which is what a bfloat16 engine holds
    (the reference converts every projection to BF16 on upload and keeps norm vectors in
    F32: crates/backend/cuda/src/loading/weights.rs:151-161, bindings.rs:230-237)."""
    from safetensors import safe_open
    out = {}
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt") as f:
        for name in f.keys():
            t = f.get_tensor(name)
            if round_to_bf16 and t.dim() >= 2:
                t = t.to(torch.bfloat16)
            out[name] = t.to(F64)
    return out


def weight_prefix(tensors: Dict[str, torch.Tensor]) -> str:
    """First prefix under which the token table exists
    (crates/model/package/src/providers/qwen/mod.rs:371-374;
    crates/model/package/src/storage/package.rs:231-237)."""
    for p in ("model.language_model.", "model.", ""):
        if p + "embed_tokens.weight" in tensors:
            return p
    raise KeyError("embed_tokens.weight")


# --------------------------------------------------------------------------- parts
def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) * (w + 0) over the last dimension
    (crates/testing/cpu/reference-ops/src/kernels.rs:38-54; offset 0 for this family,
    crates/model/package/src/providers/qwen/mod.rs:252)."""
    scale = torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return x / scale * weight


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = W x with W stored [out, in] (kernels.rs:168-183).  The bias is this build's
    extension: the reference rejects attention_bias (qwen/mod.rs:416-424)."""
    y = x @ weight.T
    return y if bias is None else y + bias


def rope_neox(x: torch.Tensor, positions: torch.Tensor, theta: float, rotary_dim: int) -> torch.Tensor:
    """x: [T, heads, d].  For i < rd/2: angle = pos / theta^(2i/rd);
    x[i] = a cos - b sin; x[i + rd/2] = a sin + b cos with (a, b) = (x[i], x[i + rd/2]);
    the rest passes through (kernels.rs:217-241)."""
    half = rotary_dim // 2
    i = torch.arange(half, dtype=F64)
    angle = positions.to(F64)[:, None] / torch.pow(torch.tensor(theta, dtype=F64), 2.0 * i / rotary_dim)
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    a, b = x[..., :half], x[..., half:rotary_dim]
    out = x.clone()
    out[..., :half] = a * cos - b * sin
    out[..., half:rotary_dim] = a * sin + b * cos
    return out


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, positions: torch.Tensor,
                     window: Optional[int]) -> torch.Tensor:
    """q: [T, nq, d], k, v: [T, nkv, d] of ONE sequence whose token t has position
    positions[t].  Head h reads kv head h // (nq // nkv); s_j = q.k_j / sqrt(d) over the
    keys start..pos, start = (pos + 1).saturating_sub(window) or 0; softmax with the
    maximum subtracted; o = sum p_j v_j (kernels.rs:251-297)."""
    T, nq, d = q.shape
    nkv = k.shape[1]
    group = nq // nkv
    out = torch.zeros_like(q)
    pos = positions.tolist()
    for h in range(nq):
        kh = h // group
        scores = (q[:, h, :] @ k[:, kh, :].T) / math.sqrt(d)          # [T, T]
        for t in range(T):
            start = max(0, pos[t] + 1 - window) if window else 0
            visible = [j for j in range(T) if start <= pos[j] <= pos[t]]
            s = scores[t, visible]
            p = torch.exp(s - s.max())
            p = p / p.sum()
            out[t, h, :] = p @ v[visible, kh, :]
    return out


def silu(z: torch.Tensor) -> torch.Tensor:
    """z * sigmoid(z) (kernels.rs:12-22)."""
    return z * torch.sigmoid(z)


def swiglu_mlp(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor) -> torch.Tensor:
    """W_down (silu(W_gate x) * (W_up x)) (crates/model/recipes/src/decoder.rs:481-501)."""
    return linear(silu(linear(x, w_gate)) * linear(x, w_up), w_down)


def attention_block(x: torch.Tensor, w: Dict[str, torch.Tensor], p: str, cfg: dict,
                    positions: torch.Tensor, window: Optional[int]) -> torch.Tensor:
    """Projections, per-head q/k RMSNorm over head_dim BEFORE the rotation, rotation of q
    and k, attention, output projection (crates/model/recipes/src/decoder.rs:229-364;
    q/k norm :278-293, rope :315-335)."""
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    T = x.shape[0]
    bias = cfg["attention_bias"]
    q = linear(x, w[p + "q_proj.weight"], w.get(p + "q_proj.bias") if bias else None).view(T, nq, d)
    k = linear(x, w[p + "k_proj.weight"], w.get(p + "k_proj.bias") if bias else None).view(T, nkv, d)
    v = linear(x, w[p + "v_proj.weight"], w.get(p + "v_proj.bias") if bias else None).view(T, nkv, d)
    q = rms_norm(q, w[p + "q_norm.weight"], cfg["rms_norm_eps"])
    k = rms_norm(k, w[p + "k_norm.weight"], cfg["rms_norm_eps"])
    rd = int(math.floor(d * cfg["partial_rotary_factor"]))          # decoder.rs:516-522
    q = rope_neox(q, positions, cfg["rope_theta"], rd)
    k = rope_neox(k, positions, cfg["rope_theta"], rd)
    o = causal_attention(q, k, v, positions, window).reshape(T, nq * d)
    return linear(o, w[p + "o_proj.weight"], w.get(p + "o_proj.bias") if bias else None)


def decoder_layer(x: torch.Tensor, w: Dict[str, torch.Tensor], p: str, cfg: dict,
                  positions: torch.Tensor, window: Optional[int]) -> torch.Tensor:
    """x += attn(norm(x)); x += mlp(norm(x)) (decoder.rs:112-120, :474-501)."""
    eps = cfg["rms_norm_eps"]
    x = x + attention_block(rms_norm(x, w[p + "input_layernorm.weight"], eps), w,
                            p + "self_attn.", cfg, positions, window)
    n = rms_norm(x, w[p + "post_attention_layernorm.weight"], eps)
    return x + swiglu_mlp(n, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                          w[p + "mlp.down_proj.weight"])


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int]) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence starting at position 0
    (embedding decoder.rs:104-108; final norm :143; output matrix, tied or
    `lm_head.weight` at the file's root :144-149, crates/foundation/spi/src/model.rs:220-226)."""
    p = weight_prefix(w)
    ids = torch.tensor(list(tokens), dtype=torch.long)
    positions = torch.arange(len(ids))
    x = w[p + "embed_tokens.weight"][ids]
    for layer in range(cfg["num_hidden_layers"]):
        window = cfg["sliding_window"] if cfg["layer_types"][layer] == "sliding_attention" else None
        x = decoder_layer(x, w, f"{p}layers.{layer}.", cfg, positions, window)
    x = rms_norm(x, w[p + "norm.weight"], cfg["rms_norm_eps"])
    head = w[p + "embed_tokens.weight"] if cfg["tie_word_embeddings"] else w["lm_head.weight"]
    return linear(x, head)


class PlainModel:
    def __init__(self, folder: str, round_to_bf16: bool = False) -> None:
        self.cfg = read_config(folder)
        self.w = load_tensors(folder, round_to_bf16)

    def logits(self, tokens: Sequence[int]) -> torch.Tensor:
        return forward(self.cfg, self.w, tokens)


# --------------------------------------------------------------------------- sampling
MASK64 = (1 << 64) - 1


def uniform_for(seed: int, request: int, position: int) -> float:
    """Stateless 53-bit uniform from (seed, request, position)
    (crates/engine/workloads/src/sampling.rs:9-23 constants, :197-205)."""
    x = (seed + ((request * 0x9E3779B97F4A7C15) & MASK64) + position) & MASK64
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & MASK64
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & MASK64
    x ^= x >> 31
    return (x >> 11) / float(1 << 53)


def greedy(logits: Sequence[float]) -> int:
    """Highest logit, lowest index among equals (sampling.rs:175-192)."""
    best, best_v = 0, None
    for i, v in enumerate(logits):
        if not math.isfinite(v):
            raise ValueError("invalid sampling logits")
        if best_v is None or _total_key(v) > _total_key(best_v):
            best, best_v = i, v
    if best_v is None:
        raise ValueError("invalid sampling logits")
    return best


def _total_key(v: float):
    """Sort key of f32::total_cmp for finite values: by value, -0.0 below +0.0."""
    return (v, math.copysign(1.0, v))


def sample(logits: Sequence[float], temperature: float, seed: int, request: int, position: int,
           top_k: Optional[int] = None, top_p: float = 1.0, min_p: float = 0.0) -> int:
    """Temperature / top-k / top-p / min-p draw (sampling.rs:146-168 order of steps,
    :282-298 filters, :210-226 cumulative draw over F32-rounded normalised weights)."""
    if temperature == 0.0:
        return greedy(logits)
    cand = sorted(((i, float(v)) for i, v in enumerate(logits)), key=lambda c: (-c[1], -math.copysign(1.0, c[1]), c[0]))
    if top_k is not None and 0 < top_k < len(cand):
        cand = cand[:top_k]
    mx = cand[0][1]
    # logits are F32, the temperature is F32 widened to F64 (sampling.rs:160-163)
    t = float(torch.tensor(temperature, dtype=torch.float32).item())
    weights = [math.exp((v - mx) / t) for _, v in cand]
    keep = 0
    for wgt in weights:
        if wgt >= min_p:
            keep += 1
        else:
            break
    keep = max(keep, 1)
    cand, weights = cand[:keep], weights[:keep]
    if top_p < 1.0:
        threshold = sum(weights) * top_p
        c, n = 0.0, 0
        for wgt in weights:
            c += wgt
            n += 1
            if c >= threshold:
                break
        cand, weights = cand[:n], weights[:n]
    total = sum(weights)
    u = uniform_for(seed, request, position)
    c = 0.0
    for (i, _), wgt in zip(cand, weights):
        c += float(torch.tensor(wgt / total, dtype=torch.float32).item())
        if u < c:
            return i
    return cand[-1][0]


def generate(model: PlainModel, prompt: Sequence[int], max_new_tokens: int, temperature: float = 0.0,
             seed: int = 0, request: int = 0, eos: Sequence[int] = (), logits_dtype=torch.float32) -> List[int]:
    """Recompute the whole sequence for every new token; `position` of a draw is the
    index of the token being generated (crates/engine/runtime/src/pipeline/completion/cpu.rs:104)."""
    seq = list(prompt)
    out: List[int] = []
    for n in range(max_new_tokens):
        last = model.logits(seq)[-1].to(logits_dtype).tolist()
        tok = sample(last, temperature, seed, request, n)
        out.append(tok)
        seq.append(tok)
        if tok in eos:
            break
    return out
