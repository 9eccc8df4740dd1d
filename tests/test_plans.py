"""How products and attention are cut (host-side choices, no GPU): every plan must be one the kernels take,
for any size, and must stay inside the scratch that was set aside for it."""
import pytest

import locus_b200.kernels as K


@pytest.fixture(autouse=True)
def _b200(monkeypatch):
    monkeypatch.setattr(K, "_N_SM", 148)
    monkeypatch.setattr(K, "_PLANS", {})


def test_product_plans_are_ones_the_kernel_takes():
    for m in list(range(1, 70)) + [100, 127, 128, 129, 255, 256, 257, 500, 512, 1000, 2048, 4096, 100000]:
        for n, k in ((8, 8), (61, 2048), (100, 72), (2048, 2048), (6144, 2048), (2048, 5632), (5632, 2048),
                     (151936, 2048), (130, 120)):
            for dual in (False, True):
                tile, splits = K.tc_plan(m, n, k, dual)
                assert tile in (16, 32, 64, 128, 256) and tile <= (128 if dual else 256)
                assert 1 <= splits <= 16
                if splits > 1:
                    assert not dual and n % 4 == 0
                    assert splits * m * n * 4 <= K.SPLIT_SCRATCH_BYTES
                    k_blocks = -(-k // 64)
                    per_part = -(-k_blocks // splits)
                    assert -(-k_blocks // per_part) == splits   # no part is empty
                if m <= 16:
                    assert tile >= m   # one tile holds the rows of a decode-sized product
    # the cases the plan was fitted on: few weight tiles are cut along K, many tiles are not
    assert K.tc_plan(64, 2048, 5632, False)[1] > 1 and K.tc_plan(2048, 2048, 5632, False)[1] == 1
    assert K.tc_plan(2048, 6144, 2048, False) == (256, 1) and K.tc_plan(2048, 5632, 2048, True) == (128, 1)


def test_expert_tiles_and_attention_ranges():
    assert all(K.expert_tile(p, e) == 128 for p in (9, 64, 8192, 10 ** 6) for e in (1, 60, 512))
    for items in (1, 2, 4, 9, 10, 64, 200):
        for heads in (1, 3, 16, 64):
            for ctx in (1, 64, 255, 256, 1000, 4096, 30000, 10 ** 6):
                s = K.attn_chunk_mma_splits(items, heads, ctx)
                assert 1 <= s <= K.MMA_ATTN_MAX_SPLITS
                if s > 1:
                    assert items * heads < 148 and s <= -(-ctx // K.MMA_QUERY_TILE)
                    n_o, n_ml = K.attn_chunk_mma_scratch(128)
                    units = items * heads * s * K.MMA_QUERY_TILE
                    assert units * 128 <= n_o and units * 2 <= n_ml   # the scratch the attention part allocates


def test_tensor_core_attention_ranges_stay_inside_their_scratch():
    """The key ranges of the tcgen05 attention: 1 to 16, only while the step's blocks leave half the SMs idle and
    the context has at least eight key tiles, never fewer than four tiles to a range, and one partial result per
    (token, head, range) always fits the scratch, which is sized once from the SM count."""
    n_o, n_ml = K.attn_chunk_tc_scratch()
    assert n_o == 128 * 148 * K.TC_ATTN_HEAD_DIM and n_ml == 128 * 148 * 2
    for items in list(range(1, 40)) + [64, 147, 148, 149, 300, 1000]:
        for heads in (1, 2, 3, 7, 16, 28, 64, 128):
            for ctx in (1, 128, 1023, 1024, 1025, 2048, 4096, 30000, 131072, 10 ** 6):
                s = K.attn_chunk_tc_splits(items, heads, ctx)
                assert 1 <= s <= K.TC_ATTN_MAX_SPLITS
                blocks = -(-items // 2) * heads
                if s > 1:
                    assert 2 * blocks <= 148 and blocks * s <= 148
                    assert s * 4 <= -(-ctx // K.TC_ATTN_QUERY_BLOCK)
                    tokens = 64 * items   # at most: every tile of the item list full
                    assert tokens * heads * s * K.TC_ATTN_HEAD_DIM <= n_o and tokens * heads * s * 2 <= n_ml
    # the cases it was made for: a short portion behind a long context is cut, a long portion is not
    assert K.attn_chunk_tc_splits(4, 16, 30000) > 1 and K.attn_chunk_tc_splits(32, 16, 30000) == 1


def test_which_portions_the_tensor_core_attention_takes():
    import torch

    q = torch.empty(1, dtype=torch.bfloat16)
    takes = lambda **kw: K.attn_chunk_tc_takes(q, kw.get("hd", 128), kw.get("page", 64), kw["n"], kw.get("ctx", 0))
    if not (K.USE_TENSOR_CORES and getattr(K, "USE_TC_ATTENTION", True)):
        pytest.skip("tensor-core attention switched off")
    assert takes(n=256) and takes(n=2048) and not takes(n=255) and not takes(n=64)
    assert takes(n=128, ctx=2048) and not takes(n=128, ctx=2047)          # 128 to 255 tokens: behind 2,048 and more
    assert takes(n=2, ctx=4096) and not takes(n=2, ctx=4095)              # fewer: behind 4,096 and more
    assert not takes(n=2048, hd=64) and not takes(n=2048, page=16) and takes(n=2048, page=128)
    assert not K.attn_chunk_tc_takes(torch.empty(1, dtype=torch.float32), 128, 64, 2048, 0)
