"""Decisions that the kernels' Python face takes on the host (no GPU needed)."""
from inferloop_b200.csrc.ops import tc_row_blocks

SMS = 148


def ctas(tokens, heads, kv_heads, blocks):
    per = blocks * (128 // (heads // kv_heads))
    return -(-tokens // per) * kv_heads


def test_row_blocks_of_the_prefill_attention_kernel():
    # prompts from their start: two blocks once there is a CTA pair for every SM
    assert tc_row_blocks(ctas(1024, 32, 8, 1), ctas(1024, 32, 8, 2), SMS, False) == 1
    assert tc_row_blocks(ctas(2048, 32, 8, 1), ctas(2048, 32, 8, 2), SMS, False) == 2
    # portions behind a long cached prefix run in rounds: 512 tokens of 40 / 8 heads are 168 CTAs
    # (two rounds) or 88 pairs (one round of dearer tiles); 512 tokens of 32 / 8 heads fit one round
    assert tc_row_blocks(ctas(512, 40, 8, 1), ctas(512, 40, 8, 2), SMS, True) == 2
    assert tc_row_blocks(ctas(512, 32, 8, 1), ctas(512, 32, 8, 2), SMS, True) == 1
    assert tc_row_blocks(ctas(384, 40, 8, 1), ctas(384, 40, 8, 2), SMS, True) == 1
    # three rounds of one block against two of pairs: one block
    assert tc_row_blocks(ctas(1536, 32, 8, 1), ctas(1536, 32, 8, 2), SMS, True) == 1
