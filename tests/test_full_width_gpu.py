"""Two layers at the serving configuration's own layer sizes (width 4096, 32 query heads over
8 key/value heads of size 128, feed-forward 12288) against the plain implementation, in 32-bit
and in bfloat16 (GPU).  The tiny configurations never reach the shapes the serving kernels are
tuned for: K ranges of a tile spread over a cluster, the widest SwiGLU epilogue, sums of 12288
terms.  The vocabulary is kept small and odd; the output matrix is not what differs at size.

The noise that rounding activations to bfloat16 leaves on the logits grows with the width:
measured here over a whole prompt, root-mean-square 2.0e-3 of the largest reference logit and
1.0e-2 for the worst of 600,000 elements (4.5 to 5 times the root-mean-square, as at the
small configurations, whose figures are 0.9e-3 and 4.3e-3).  This file's bfloat16 bound is
therefore 2e-2 per element and 5e-3 for the root-mean-square; the 32-bit bound is the common one."""
import pytest
import torch

import plain_qwen3 as plain
from helpers import Trace, check_trace, make_model_folder, random_tokens, run_trace_inprocess

pytestmark = pytest.mark.gpu

CONFIG_WIDE = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=2, hidden_size=4096,
    num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288,
    vocab_size=4099, rope_theta=1000000.0, rms_norm_eps=1e-6, attention_bias=False,
    tie_word_embeddings=False, max_position_embeddings=4096, hidden_act="silu")
LENGTHS = {"a": 150, "b": 70}


@pytest.fixture(scope="module")
def folder(tmp_path_factory):
    return make_model_folder(str(tmp_path_factory.mktemp("model") / "wide"), CONFIG_WIDE, 21)


def wide_trace(reqs):
    """a: portions of 64, 2 and 52 tokens, then its last 32 tokens one by one; b arrives
    beside a's single tokens in portions of 17, 2, 30 and then decodes too."""
    trace = Trace()
    a, b = reqs["a"], reqs["b"]
    ia = 0
    for n in (64, 2, 52):
        trace.step([("a", a[ia:ia + n], list(range(n)))])
        ia += n
    ib, cuts = 0, [17, 2, 30]
    while ia < len(a) or ib < len(b):
        entries, ended = [], []
        if ia < len(a):
            entries.append(("a", [a[ia]], [0]))
            ia += 1
            if ia == len(a):
                ended.append("a")
        if ib < len(b):
            n = cuts.pop(0) if cuts else 1
            entries.append(("b", b[ib:ib + n], list(range(n))))
            ib += n
            if ib == len(b):
                ended.append("b")
        trace.step(entries, end=ended)
    return trace


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_two_layers_of_serving_width(folder, dtype):
    from inferloop_b200.engine import ModelRunner
    reqs = {rid: random_tokens(n, CONFIG_WIDE["vocab_size"], 300 + n) for rid, n in LENGTHS.items()}
    model = plain.PlainModel(folder, round_to_bf16=(dtype == "bfloat16"))
    ref = {rid: model.logits(toks) for rid, toks in reqs.items()}
    del model
    runner = ModelRunner.from_folder(folder, dtype=dtype, page_size=16, num_pages=24, max_requests=4)
    trace = wide_trace(reqs)
    check_trace(run_trace_inprocess(runner, trace), trace, ref, dtype, f"wide {dtype}", bf16_rel_of_max=2e-2)
    runner.cache.check()
    from inferloop_b200.csrc import ops
    ops.check_device_errors()
    del runner
    torch.cuda.empty_cache()
