"""One rank's share of the partitioned graph.

`DistributedGraph` (plain halo path) and `DistributedGraphForPre` (pre/post-aggregation path) carry the
attribute names of the reference's classes of the same names
(self_benchmark/a64fx/data_manager/DistributedGraph.py:8-59) and accept the same positional or keyword
arguments; the aggregation op reads nothing else from them.
"""
from typing import Tuple


class _GraphRecord(object):
    """Record whose constructor binds positional / keyword arguments to `_fields`, in order."""

    _fields: Tuple[str, ...] = ()
    _derived: Tuple[str, ...] = ()

    def __init__(self, *args, **kwargs) -> None:
        if len(args) > len(self._fields):
            raise TypeError(f"{type(self).__name__} takes {len(self._fields)} arguments, {len(args)} given")
        values = dict(zip(self._fields, args))
        for name, value in kwargs.items():
            if name not in self._fields:
                raise TypeError(f"{type(self).__name__} has no field {name!r}")
            if name in values:
                raise TypeError(f"{type(self).__name__}: {name!r} given twice")
            values[name] = value
        missing = [f for f in self._fields if f not in values]
        if missing:
            raise TypeError(f"{type(self).__name__} missing {missing}")
        for name in self._fields:
            setattr(self, name, values[name])
        for name in self._derived:
            setattr(self, name, None)

    def __repr__(self) -> str:
        return f"{type(self).__name__}(local_adj_t={self.local_adj_t!r})"


_COMMON_TAIL = ("in_degrees", "comm_splits", "comm_buf", "comm_buf_for_quantization")


class DistributedGraph(_GraphRecord):
    """Plain halo path: local and remote adjacency (rows = local destinations; remote columns = halo
    slots), the local ids to send (concatenated per requesting peer) and the per-peer counts.

    Derived once by the CUDA path and cached here: `idx_nodes_send_to_others_i32` (int32 copy of the
    send index) and `scatter_adj_t`, the (n_local x n_send) unit matrix whose accumulating SpMM is the
    deterministic form of grad.index_add_(0, idx_nodes_send_to_others, buf)
    (model/layers/aggregator.py:197-199 of the reference)."""

    _fields = ("local_adj_t", "remote_adj_t", "idx_nodes_send_to_others", "num_nodes_send_to_others",
               "num_nodes_recv_from_others") + _COMMON_TAIL
    _derived = ("idx_nodes_send_to_others_i32", "scatter_adj_t")


class DistributedGraphForPre(_GraphRecord):
    """Pre/post-aggregation path: `adj_t_pre_post_aggr_to` (send slots x n_local) builds the send buffer,
    `adj_t_pre_post_aggr_from` (n_local x receive slots) consumes the receive buffer; the two split
    lists repeat comm_splits.recv_splits / send_splits."""

    _fields = ("local_adj_t", "adj_t_pre_post_aggr_from", "adj_t_pre_post_aggr_to", "pre_post_aggr_from_splits",
               "pre_post_aggr_to_splits") + _COMMON_TAIL
