"""The plain implementation itself (no GPU): its parts against hand-computed cases, a
second, scalar, token-at-a-time statement of the same formulas, and committed outputs."""
import json
import math
import os

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from helpers import CONFIGS, make_model_folder, random_tokens


def test_rms_norm_by_hand():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    w = torch.tensor([2.0, 0.5], dtype=torch.float64)
    got = plain.rms_norm(x, w, 1e-6)
    scale = math.sqrt((9 + 16) / 2 + 1e-6)
    assert torch.allclose(got, torch.tensor([[3 / scale * 2, 4 / scale * 0.5]], dtype=torch.float64))


def test_rope_by_hand_and_partial():
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0, 5.0, 6.0]]], dtype=torch.float64)       # d = 6, rd = 4
    out = plain.rope_neox(x, torch.tensor([3]), theta=100.0, rotary_dim=4)[0, 0]
    a0, a1 = 3 / 100.0 ** 0.0, 3 / 100.0 ** 0.5
    want = [1 * math.cos(a0) - 3 * math.sin(a0), 2 * math.cos(a1) - 4 * math.sin(a1),
            1 * math.sin(a0) + 3 * math.cos(a0), 2 * math.sin(a1) + 4 * math.cos(a1), 5.0, 6.0]
    assert torch.allclose(out, torch.tensor(want, dtype=torch.float64))
    assert torch.equal(plain.rope_neox(x, torch.tensor([0]), 100.0, 4), x)       # position 0 is the identity


def test_attention_causal_window_and_groups():
    torch.manual_seed(0)
    T, nq, nkv, d = 6, 4, 2, 8
    q, k, v = (torch.randn(T, h, d, dtype=torch.float64) for h in (nq, nkv, nkv))
    pos = torch.arange(T)
    full = plain.causal_attention(q, k, v, pos, None)
    assert torch.allclose(full[0, 1], v[0, 0])                   # one key: its value, whatever q is
    assert torch.allclose(full[0, 3], v[0, 1])                   # head 3 reads kv head 1
    s = (q[4, 2] @ k[:5, 1].T) / math.sqrt(d)
    assert torch.allclose(full[4, 2], torch.softmax(s, 0) @ v[:5, 1])
    win = plain.causal_attention(q, k, v, pos, 2)                # keys p-1..p
    s = (q[4, 2] @ k[3:5, 1].T) / math.sqrt(d)
    assert torch.allclose(win[4, 2], torch.softmax(s, 0) @ v[3:5, 1])
    assert torch.allclose(plain.causal_attention(q, k, v, pos, 100), full)


def test_sampling_rules():
    assert plain.greedy([0.5, 2.0, 2.0, -1.0]) == 1                 # lowest index among equals
    with pytest.raises(ValueError):
        plain.greedy([0.0, float("nan")])
    u = [plain.uniform_for(7, r, p) for r in range(3) for p in range(3)]
    assert all(0.0 <= x < 1.0 for x in u) and len(set(u)) == 9
    assert plain.uniform_for(7, 1, 2) == plain.uniform_for(7, 1, 2)
    logits = [0.0, 1.0, 3.0, 2.5, -2.0]
    draws = [plain.sample(logits, 0.7, seed=s, request=0, position=0) for s in range(400)]
    counts = np.bincount(draws, minlength=5) / 400
    p = np.exp(np.array(logits) / 0.7); p /= p.sum()
    assert np.abs(counts - p).max() < 0.08
    assert all(plain.sample(logits, 0.7, s, 0, 0, top_k=1) == 2 for s in range(20))
    assert set(plain.sample(logits, 1.0, s, 0, 0, top_p=0.5) for s in range(50)) <= {2, 3}
    assert set(plain.sample(logits, 1.0, s, 0, 0, min_p=0.5) for s in range(50)) <= {2, 3}


# ------------------------------------------------------------------ the scalar twin
def scalar_forward(cfg, w, tokens):
    """One token at a time with growing key/value lists, scalar loops, in the manner of
    the reference's CPU ops (crates/testing/cpu/reference-ops/src/kernels.rs:38-54 norm,
    :168-183 linear, :217-241 rope, :251-297 attention with its own cache)."""
    p = plain.weight_prefix(w)
    W = {k: v.numpy() for k, v in w.items()}
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    rd = int(math.floor(d * cfg["partial_rotary_factor"]))
    eps, theta = cfg["rms_norm_eps"], cfg["rope_theta"]
    L = cfg["num_hidden_layers"]
    keys = [[] for _ in range(L)]
    values = [[] for _ in range(L)]

    def norm(x, weight, dim):
        out = np.empty_like(x)
        for s in range(0, len(x), dim):
            head = x[s:s + dim]
            scale = math.sqrt(sum(float(v) ** 2 for v in head) / dim + eps)
            out[s:s + dim] = [float(v) / scale * float(g) for v, g in zip(head, weight)]
        return out

    def lin(x, name, bias=None):
        y = np.array([sum(float(a) * float(b) for a, b in zip(row, x)) for row in W[name]])
        return y + W[bias] if bias else y

    def rope(x, heads, pos):
        x = x.copy()
        for h in range(heads):
            for i in range(rd // 2):
                angle = pos / theta ** ((2 * i) / rd)
                s, c = math.sin(angle), math.cos(angle)
                a, b = x[h * d + i], x[h * d + i + rd // 2]
                x[h * d + i], x[h * d + i + rd // 2] = a * c - b * s, a * s + b * c
        return x

    out = []
    for pos, tok in enumerate(tokens):
        x = W[p + "embed_tokens.weight"][tok].copy()
        for l in range(L):
            lp = f"{p}layers.{l}."
            ap = lp + "self_attn."
            b = cfg["attention_bias"]
            n = norm(x, W[lp + "input_layernorm.weight"], len(x))
            q = lin(n, ap + "q_proj.weight", ap + "q_proj.bias" if b else None)
            k = lin(n, ap + "k_proj.weight", ap + "k_proj.bias" if b else None)
            v = lin(n, ap + "v_proj.weight", ap + "v_proj.bias" if b else None)
            q = rope(norm(q, W[ap + "q_norm.weight"], d), nq, pos)
            k = rope(norm(k, W[ap + "k_norm.weight"], d), nkv, pos)
            keys[l].append(k); values[l].append(v)
            window = cfg["sliding_window"] if cfg["layer_types"][l] == "sliding_attention" else None
            start = max(0, pos + 1 - window) if window else 0
            o = np.zeros(nq * d)
            for h in range(nq):
                kh = h // (nq // nkv)
                sc = [sum(q[h * d + i] * keys[l][j][kh * d + i] for i in range(d)) / math.sqrt(d)
                      for j in range(start, pos + 1)]
                m = max(sc)
                pr = [math.exp(s - m) for s in sc]
                z = sum(pr)
                for jj, j in enumerate(range(start, pos + 1)):
                    for i in range(d):
                        o[h * d + i] += pr[jj] / z * values[l][j][kh * d + i]
            x = x + lin(o, ap + "o_proj.weight", ap + "o_proj.bias" if b else None)
            n = norm(x, W[lp + "post_attention_layernorm.weight"], len(x))
            g = lin(n, lp + "mlp.gate_proj.weight")
            u = lin(n, lp + "mlp.up_proj.weight")
            act = np.array([gi * (1 / (1 + math.exp(-gi)) if gi >= 0 else math.exp(gi) / (1 + math.exp(gi))) * ui
                            for gi, ui in zip(g, u)])
            x = x + lin(act, lp + "mlp.down_proj.weight")
        x = norm(x, W[p + "norm.weight"], len(x))
        head = p + "embed_tokens.weight" if cfg["tie_word_embeddings"] else "lm_head.weight"
        out.append(lin(x, head))
    return np.stack(out)


@pytest.mark.parametrize("name,n", [("A", 9), ("B", 7), ("C", 26)])
def test_vectorised_and_scalar_forms_agree(tmp_path, name, n):
    cfg, seed, _ = CONFIGS[name]
    d = make_model_folder(str(tmp_path / name), cfg, seed)
    model = plain.PlainModel(d)
    toks = random_tokens(n, cfg["vocab_size"], 3)
    a = model.logits(toks).numpy()
    b = scalar_forward(model.cfg, model.w, toks)
    assert np.abs(a - b).max() < 1e-12 * max(1.0, np.abs(a).max())


def test_committed_outputs_have_not_drifted(tmp_path):
    """tests/golden/make_golden.py wrote the plain implementation's logits for tiny A and
    B; a change to it, to the random-weights mode or to the container shows here."""
    path = os.path.join(os.path.dirname(__file__), "golden", "plain_logits.json")
    with open(path) as fh:
        golden = json.load(fh)
    for name, rec in golden.items():
        cfg, seed, _ = CONFIGS[name]
        d = make_model_folder(str(tmp_path / name), cfg, seed)
        got = plain.PlainModel(d).logits(rec["tokens"])[-1, :16].tolist()
        assert np.allclose(got, rec["last_logits_first16"], rtol=0, atol=1e-12), name
        assert plain.generate(plain.PlainModel(d), rec["tokens"], 4) == rec["greedy4"]
