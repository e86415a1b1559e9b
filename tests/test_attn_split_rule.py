"""The KV-split rule of the decode attention (pure host logic)."""


def test_pick_nsplit_shapes(monkeypatch):
    from ipex_llm_b200.ops.cuda_ops import pick_nsplit
    monkeypatch.delenv("IPEX_LLM_ATTN_STEPS", raising=False)
    monkeypatch.delenv("IPEX_LLM_ATTN_MIN_CTAS", raising=False)
    # one query row per kv head (Llama-2-7B): 8 steps of 16 tokens per split
    assert pick_nsplit(1, 32, 1024, rows=1) == 8
    # grouped-query heads, 8 rows per kv head: every warp walks all tokens of a split, 32 steps of 4
    assert pick_nsplit(1, 8, 2304, rows=8) == 18
    assert pick_nsplit(1, 1, 2304, rows=8) == 18
    # short contexts never split below one block
    assert pick_nsplit(2, 4, 40, rows=8) == 1
    assert pick_nsplit(1, 1, 1 << 20, rows=1) == 128          # capped
    # opt-in floor on the CTA count: splits down to 8 steps per walk
    monkeypatch.setenv("IPEX_LLM_ATTN_MIN_CTAS", "64")
    assert pick_nsplit(1, 1, 2304, rows=8) == 64
    assert pick_nsplit(1, 8, 2304, rows=8) == 18               # already above the floor
    assert pick_nsplit(1, 1, 40, rows=8) == 1
