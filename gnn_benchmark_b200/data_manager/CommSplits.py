import math


class CommSplits(object):
    """Per-peer row counts of the halo exchange (data_manager/CommSplits.py:7-19 of the reference).

    recv_splits[p] rows arrive from peer p, send_splits[p] rows go to peer p (forward direction;
    backward swaps them).  For a packed exchange (bits 2, and here also 4 and 8) the `_int2`
    lists hold the packed row counts ceil(split / (8 / bits)); the attribute names are the
    reference's, whatever the bit width."""

    def __init__(self, recv_splits: list, send_splits: list, world_size: int, bits: int) -> None:
        self.recv_splits = [int(x) for x in recv_splits]
        self.send_splits = [int(x) for x in send_splits]
        if bits in (2, 4, 8):
            per_byte = 8 // bits
            self.recv_splits_int2 = [math.ceil(self.recv_splits[r] / per_byte) for r in range(world_size)]
            self.send_splits_int2 = [math.ceil(self.send_splits[r] / per_byte) for r in range(world_size)]
