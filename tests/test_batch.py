"""The layout of a step's batch (host logic, no GPU): token rows in request order, positions, request index
per row, wanted rows, block tables and slots in one buffer, and the query blocks of the attention kernels."""
import numpy as np
import torch

from beglin_b200.cache import CacheManager
from beglin_b200.engine.batch import ALIGN, Entry, StepBatch
from beglin_b200.parts.cache_need import FixedStateNeed, PagedKVNeed


def test_rows_positions_wanted_rows_and_tables():
    cache = CacheManager([PagedKVNeed(2, 16), PagedKVNeed(2, 16, window=6), FixedStateNeed((3,), "float32")],
                         page_size=4, num_pages=16, max_requests=3, max_context=40)
    for rid, n in (("a", 9), ("b", 0), ("c", 5)):
        cache.add_request(rid)
        if n:
            cache.reserve([(rid, n)])
            cache.commit([(rid, n)])
    ents = [Entry("a", [7], [0]), Entry("b", [1, 2, 3, 4, 5], [1, 4]), Entry("c", [8, 9], [])]
    starts = [cache.length(e.rid) for e in ents]
    assert starts == [9, 0, 5]
    cache.reserve([(e.rid, s + len(e.tokens)) for e, s in zip(ents, starts)])
    b = StepBatch(ents, starts, "cpu", cache)
    assert (b.n_rows, b.n_req, b.n_logit_rows, b.max_position, b.decode_only) == (8, 3, 3, 9, False)
    assert b.row_start == [0, 1, 6] and b.lens == [1, 5, 2]
    assert b.token_ids.tolist() == [7, 1, 2, 3, 4, 5, 8, 9] and b.token_ids.dtype == torch.int32
    assert b.positions.tolist() == [9, 0, 1, 2, 3, 4, 5, 6]
    assert b.row_req.tolist() == [0, 1, 1, 1, 1, 1, 2, 2]
    assert b.logit_rows.tolist() == [0, 2, 5]                        # entry order, then the order of `want`
    # one block table per group of layers, a row per request of the step, in the step's order
    assert set(b.block_tables) == {0, 1}
    for gi in (0, 1):
        assert np.array_equal(b.block_tables[gi].numpy(), cache.block_table(gi, ["a", "b", "c"]))
        assert b.block_tables[gi].shape == (3, cache.max_pages)
    full = b.block_tables[0].numpy()
    assert (full[0, :3] >= 0).all() and (full[0, 3:] == -1).all()    # 10 positions: three pages
    windowed = b.block_tables[1].numpy()
    assert windowed[0, 0] == -1 and (windowed[0, 1:3] >= 0).all()    # the window of 6 has passed the first page
    assert b.slots.tolist() == cache.slot_ids(["a", "b", "c"]).tolist()
    # every array starts on a 128-byte boundary of the one buffer
    base = b.token_ids.data_ptr()
    for t in (b.positions, b.row_req, b.logit_rows, b.block_tables[0], b.block_tables[1], b.slots):
        assert (t.data_ptr() - base) % (4 * ALIGN) == 0
    cache.check()


def test_query_blocks_cut_rows_of_one_request_only():
    ents = [Entry("a", list(range(7)), []), Entry("b", [1], [0]), Entry("c", list(range(4)), [3])]
    b = StepBatch(ents, [0, 30, 2], "cpu")
    blocks, n = b.query_blocks(3)
    assert n == 6 and blocks.tolist() == [[0, 0, 3], [0, 3, 3], [0, 6, 1], [1, 7, 1], [2, 8, 3], [2, 11, 1]]
    assert b.query_blocks(3)[0] is blocks                            # made once per block size
    blocks, n = b.query_blocks(16)
    assert blocks.tolist() == [[0, 0, 7], [1, 7, 1], [2, 8, 4]]
    single = StepBatch([Entry("a", [5], [0]), Entry("b", [6], [0])], [3, 9], "cpu")
    assert single.decode_only and single.max_position == 9


def test_ids_beyond_int32_become_a_value_the_embedding_kernel_reports():
    b = StepBatch([Entry("a", [3, 2 ** 40, -7], [])], [0], "cpu")
    assert b.token_ids.tolist() == [3, -1, -1]
