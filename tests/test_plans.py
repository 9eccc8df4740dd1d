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
