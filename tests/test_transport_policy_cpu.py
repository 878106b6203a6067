"""Host-side choices of the halo path that need no GPU: which peers a push group serves, which receive-side
form a packed halo takes at a given width, and the arguments Communicator accepts."""
from types import SimpleNamespace

import pytest


@pytest.mark.parametrize("P,n_groups", [(2, 1), (2, 3), (4, 3), (5, 2), (8, 3), (8, 7), (8, 1), (3, 9)])
def test_push_groups_cover_every_peer_once_and_mirror(P, n_groups):
    """Group g of rank r serves the peers r+1+g*k ...; the rows that arrive with group g come from r-1-g*k ...
    Every peer is served exactly once, and `q is served by r in group g` <=> `r receives from ... ` mirrored:
    if r sends to q in its group g, then q lists r among the sources of ITS group g (that is what lets one
    signal per group cover both directions)."""
    from gnn_benchmark_b200.aggregator_push import _groups

    tables = [_groups(P, r, n_groups) for r in range(P)]
    for r in range(P):
        served = []
        for first, cnt, sources in tables[r]:
            served += [(first + j) % P for j in range(cnt)]
            assert len(sources) == cnt
        assert sorted(served) == [q for q in range(P) if q != r]
        assert len(tables[r]) == len(tables[0]) <= max(1, min(n_groups, P - 1))
    for r in range(P):
        for g, (first, cnt, _) in enumerate(tables[r]):
            for j in range(cnt):
                q = (first + j) % P
                assert r in tables[q][g][2]


def test_fused_unpack_policy_by_width(monkeypatch):
    import gnn_benchmark_b200.aggregator as agg

    plain = SimpleNamespace(comm_buf=SimpleNamespace(lean=False))
    lean = SimpleNamespace(comm_buf=SimpleNamespace(lean=True))
    assert agg._fuse_unpack_forward(plain, 256) and agg._fuse_unpack_forward(plain, agg.FUSE_UNPACK_MIN_WIDTH)
    assert not agg._fuse_unpack_forward(plain, 128) and not agg._fuse_unpack_forward(plain, 32)
    assert agg._fuse_unpack_forward(lean, 32)           # no fp32 halo buffer to unpack into
    assert not agg._fuse_unpack_forward(lean, 30)       # the packed SpMM needs F % 4 == 0
    monkeypatch.setattr(agg, "FUSE_UNPACK", False)
    assert not agg._fuse_unpack_forward(plain, 256)


def test_communicator_rejects_unknown_transport_and_engine():
    from gnn_benchmark_b200 import Communicator

    saved = Communicator.ctx
    try:
        with pytest.raises(ValueError):
            Communicator(32, transport="mpi")
        with pytest.raises(ValueError):
            Communicator(32, transport="push", push_engine="dma")
        c = Communicator(2, transport="push", push_groups=2, push_engine="auto")
        assert (c.transport, c.push_groups, c.push_engine) == ("push", 2, "auto")
    finally:
        Communicator.ctx = saved
