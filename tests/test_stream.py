"""The residual stream's bookkeeping (host logic only): what is owed, when sums of squares are valid, and
when a norm may be applied inside a product."""
import torch

from beglin_b200.parts.stream import NormedInput, ResidualStream


class FakeNorm:
    def __init__(self, fusable=True):
        self.calls = []
        self._fusable = fusable

    def add_norm(self, x, delta):
        self.calls.append(None if delta is None else delta.clone())
        if delta is not None:
            x += delta
        return x * 2.0

    def fusion(self):
        return ("weight", 1e-6) if self._fusable else None


def test_owed_addend_is_added_by_the_next_norm_and_invalidates_the_squares():
    s = ResidualStream(torch.ones(3, 4))
    s.updated(torch.full((2, 64), 0.5))
    assert s.pending is None and s.ssq is not None
    s.owe(torch.full((3, 4), 2.0))
    assert s.ssq is None                                   # x is no longer what the squares describe
    norm = FakeNorm()
    h = NormedInput(s, norm)
    assert h.fusable() is None                             # an addend is owed: the norm kernel has to add it
    out = h.tensor()
    assert torch.equal(s.x, torch.full((3, 4), 3.0)) and torch.equal(out, torch.full((3, 4), 6.0))
    assert s.pending is None and len(norm.calls) == 1
    assert h.tensor() is out and len(norm.calls) == 1      # computed once


def test_norm_is_left_to_the_product_only_with_valid_squares_and_a_willing_norm():
    s = ResidualStream(torch.ones(2, 8))
    assert NormedInput(s, FakeNorm()).fusable() is None    # nothing is known about x's rows yet
    s.updated(torch.ones(1, 64))
    assert NormedInput(s, FakeNorm()).fusable() == ("weight", 1e-6)
    assert NormedInput(s, FakeNorm(fusable=False)).fusable() is None
    assert NormedInput(s, object()).fusable() is None      # a norm without `fusion`
    h = NormedInput(s, FakeNorm())
    h.tensor()
    assert h.fusable() is None                             # already computed: use the tensor
    assert s.ssq is not None                               # x did not change, the squares still hold


def test_decode_splits_make_one_wave():
    from beglin_b200.csrc.ops import decode_splits
    for sms in (148, 132, 20):
        for streams in (1, 2, 7, 16, 32, 100, 148, 500):
            for context in (1, 200, 256, 257, 4096, 100000):
                n = decode_splits(streams, context, sms=sms)
                assert n >= 1 and (streams * n <= sms or n == 1)
                assert n <= max(1, -(-context // 256))
    assert decode_splits(16, 4096, sms=148) == 8 and decode_splits(2, 4096, sms=148) == 16
    assert decode_splits(128, 4096, sms=148) == 1


def test_which_steps_a_portion_graph_stands_for_and_which_graphs_are_kept():
    """Host logic of the portion graphs: one request, enough rows, few wanted places; the bound on positions
    grows in steps; a shape is captured at its second sighting; the graph used least recently goes first."""
    from types import SimpleNamespace
    from beglin_b200.engine import portion_graph as pg
    from beglin_b200.engine.batch import Entry

    engine = SimpleNamespace(cache=SimpleNamespace(max_context=10000))
    graphs = pg.PortionGraphs(engine, min_rows=16, max_wanted=2, keep=2)
    e = lambda n, w=(): Entry("r", list(range(n)), list(w))
    assert graphs.key_of([e(16), e(16)], [0, 0]) is None                    # two requests
    assert graphs.key_of([e(15)], [0]) is None                              # too few rows
    assert graphs.key_of([e(16, (0, 1, 2))], [0]) is None                   # too many wanted places
    assert graphs.key_of([e(16, (15,))], [0]) == (16, 1, 4095)
    assert graphs.key_of([e(16)], [4080]) == (16, 0, 4095)                  # the last position is 4095
    assert graphs.key_of([e(16)], [4081]) == (16, 0, 8191)
    assert graphs.key_of([e(16)], [9000]) == (16, 0, 9999)                  # never beyond the context limit

    made = []
    pg_class, pg.PortionGraph = pg.PortionGraph, lambda eng, *key: made.append(key) or ("graph", key)
    try:
        a, b, c = (16, 0, 4095), (32, 0, 4095), (48, 1, 4095)
        assert graphs.get(a) is None and made == []                         # first sighting: no graph yet
        assert graphs.get(a) == ("graph", a) and made == [a]
        assert graphs.get(a) == ("graph", a) and made == [a]                # kept
        assert graphs.get(b) is None and graphs.get(b) == ("graph", b)
        assert graphs.get(a) == ("graph", a)                                # a is now the one used last
        assert graphs.get(c) is None and graphs.get(c) == ("graph", c)      # b goes
        assert list(graphs.graphs) == [a, c]
        assert graphs.get(b) == ("graph", b) and made == [a, b, c, b]       # seen before: made again at once
        assert list(graphs.graphs) == [c, b]
    finally:
        pg.PortionGraph = pg_class


def test_no_collection_collects_first_and_keeps_the_collector_off():
    """A dropped cycle (an engine and its graphs are one) is collected before the block begins, not inside it."""
    import gc
    from beglin_b200.engine.capture import no_collection

    freed = []

    class Node:
        def __del__(self):
            freed.append(gc.isenabled())

    def cycle():
        a, b = Node(), Node()
        a.other, b.other = b, a

    assert gc.isenabled()
    gc.disable()
    cycle()                                   # garbage that only the collector can free
    gc.enable()
    with no_collection():
        assert len(freed) == 2                # gone before the block began
        assert not gc.isenabled()
        cycle()
        for _ in range(3):
            [[] for _ in range(100000)]       # enough allocations to start the collector if it were on
        assert len(freed) == 2
    assert gc.isenabled()
    gc.collect()
    assert len(freed) == 4
    gc.disable()
    try:
        with no_collection():
            pass
        assert not gc.isenabled()             # left as it was found
    finally:
        gc.enable()
