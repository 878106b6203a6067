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


class _FakePeers(object):
    """Peer service without any device: every rank's buffer 'lives' at a made-up base address."""
    engine = "auto"

    def __init__(self, rank, world, info):
        self.rank, self.world, self._info = rank, world, info

    def gather_objects(self, obj):
        assert obj == self._info[self.rank]
        return list(self._info)

    def share(self, nbytes):
        import torch
        self.nbytes = nbytes
        return torch.zeros(nbytes, dtype=torch.uint8), [(p + 1) << 40 for p in range(self.world)]


@pytest.mark.parametrize("bits", [32, 2, 8])
def test_push_plan_blocks_tile_every_receive_buffer(bits):
    """The destination tables of the push transport: for every peer p, the blocks the other ranks store into
    p's receive buffer must tile it in rank order without overlap -- forward rows into recv_buf (or the packed
    pair), backward rows into send_buf -- and every rank must compute the same region layout."""
    from gnn_benchmark_b200.peer import PushPlan

    P, F = 4, 24
    # rows[r][q]: rows r sends to q in forward (= rows q receives from r); some peers exchange nothing
    rows = [[0, 5, 0, 9], [7, 0, 3, 1], [2, 2, 0, 0], [4, 0, 6, 0]]
    info = [([rows[q][r] for q in range(P)], list(rows[r])) for r in range(P)]   # (recv_splits, send_splits) of rank r
    epb = 8 // bits if bits in (2, 4, 8) else 1
    pk = lambda n: (n + epb - 1) // epb
    plans = []
    for r in range(P):
        splits = SimpleNamespace(recv_splits=info[r][0], send_splits=info[r][1])
        plans.append(PushPlan(_FakePeers(r, P, info), splits, F, bits, lean=False))
    assert len({tuple(sorted(pl.offset.items())) for pl in plans}) == 1 and len({pl.peers.nbytes for pl in plans}) == 1
    cases = [("forward", "rows", "recv_buf", 4 * F, lambda src, dst: rows[src][dst], False),
             ("backward", "rows", "send_buf", 4 * F, lambda src, dst: rows[dst][src], False)]
    if bits != 32:
        cases += [("forward", "codes", "q_recv_data", F, lambda src, dst: rows[src][dst], True),
                  ("backward", "codes", "q_send_data", F, lambda src, dst: rows[dst][src], True),
                  ("forward", "params", "q_recv_params", 4, lambda src, dst: rows[src][dst], False),
                  ("backward", "params", "q_send_params", 4, lambda src, dst: rows[dst][src], False)]
    for direction, payload, region, ld, count, packed_rows in cases:
        for p in range(P):   # the receiver
            base = ((p + 1) << 40) + plans[0].offset[region]
            cursor = base
            for r in range(P):   # senders in rank order
                n = count(r, p)
                n = pk(n) if packed_rows else n
                assert int(plans[r].dst_table(direction, payload, ld)[p]) == cursor, (direction, payload, p, r)
                assert plans[r].counts[direction, payload][p] == n
                cursor += n * ld
            # the region is large enough for what lands in it
            nxt = min([o for o in plans[0].offset.values() if o > plans[0].offset[region]] + [plans[0].peers.nbytes])
            assert cursor - base <= nxt - plans[0].offset[region]
