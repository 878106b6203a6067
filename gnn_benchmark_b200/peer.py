"""Halo exchange by direct stores into the receivers' buffers (the "push" transport).

The reference moves halo rows with an MPI all-to-all between send and receive buffers
(self_benchmark/a64fx/communicator.py:85-109, :297-311).  On one NVSwitch box every GPU can address
every other GPU's memory, so here the kernel that produces (or gathers) the rows stores them straight
into the owner's receive buffer (`gnnagg_push_rows`): no send-side staging pass, no library
all-to-all, and the peers can be served group by group so that the receive-side SpMM of one group
runs while the next group's rows are still crossing NVLink.

Pieces:
  NcclPeers   how ranks find each other's buffers and tell each other "your rows are in":
              buffers come from torch's symmetric-memory allocator (every rank maps every other rank's
              allocation), and a signal is a 4-byte NCCL all-reduce queued behind the stores -- no kernel
              of this package ever waits on another GPU.
  PushPlan    per graph: the six receive buffers carved out of one shared allocation, and for every
              direction / payload the table of destination addresses (where this rank's block starts
              inside each peer's buffer).
"""
import torch
import torch.distributed as dist

from . import _lib

_ALIGN = 256


def _round_up(x: int, a: int = _ALIGN) -> int:
    return (x + a - 1) // a * a


def _prefix_i32(counts, device) -> torch.Tensor:
    out = [0]
    for c in counts:
        out.append(out[-1] + int(c))
    return torch.tensor(out, dtype=torch.int32, device=device)


class NcclPeers(object):
    """One process per GPU on one node, NCCL process group initialised."""

    def __init__(self, device, engine="auto"):
        self.device = torch.device(device)
        # "kernel": the store kernel moves everything (gather fused in); "copy": device-to-device copies per
        # peer, rows gathered into the send buffer first where needed; "auto": copies for blocks that are
        # contiguous as they are, the store kernel where a gather is needed
        self.engine = engine
        self.rank, self.world = dist.get_rank(), dist.get_world_size()
        # signals travel on a communicator of their own: they never queue behind a large collective of
        # the default group (e.g. a gradient all-reduce) and keep their own issue order
        self.group = dist.new_group(backend="nccl")
        self._token = torch.zeros(1, dtype=torch.int32, device=self.device)

    def gather_objects(self, obj):
        out = [None] * self.world
        dist.all_gather_object(out, obj)
        return out

    def share(self, nbytes: int):
        """-> (this rank's zero-filled uint8 buffer of nbytes, [address of every rank's buffer as seen from
        this device]).  nbytes must be the same on every rank.  The fill is complete before any peer can
        learn the address: once it is published, rows may arrive at any time."""
        import torch.distributed._symmetric_memory as symm_mem

        buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=self.device)
        buf.zero_()
        torch.cuda.synchronize(self.device)
        handle = symm_mem.rendezvous(buf, dist.group.WORLD.group_name)
        dist.barrier()  # nobody stores before every rank is through its rendezvous
        ptrs = [int(p) for p in handle.buffer_ptrs]
        self._keep = getattr(self, "_keep", []) + [handle]
        return buf, ptrs

    def signal(self):
        """Queue a signal behind the work already on the current stream; the returned handle's wait()
        makes the (then) current stream wait until EVERY rank has raised the same signal."""
        return dist.all_reduce(self._token, group=self.group, async_op=True)


class PushPlan(object):
    """Receive buffers of one DistributedGraph in peer-visible memory + destination tables.

    Buffer roles (the reference's names): forward rows land in comm_buf.recv_buf (or the packed
    quantized_recv_* pair), backward rows in comm_buf.send_buf (or quantized_send_*)."""

    def __init__(self, peers, comm_splits, feat_len: int, bits: int, lean: bool):
        self.peers = peers
        P, r = peers.world, peers.rank
        self.P, self.rank = P, r
        packed = bits in (2, 4, 8)
        epb = 8 // bits if packed else 1
        info = peers.gather_objects((list(comm_splits.recv_splits), list(comm_splits.send_splits)))
        recv_all = [i[0] for i in info]   # recv_all[p][q]: rows p receives from q (forward)
        send_all = [i[1] for i in info]
        n_recv = [sum(x) for x in recv_all]
        n_send = [sum(x) for x in send_all]
        pk = lambda rows: sum((x + epb - 1) // epb for x in rows)
        # one layout for every rank: each region sized for the largest rank
        regions = {}
        if not (lean and packed):
            regions["recv_buf"] = max(n_recv) * feat_len * 4
            regions["send_buf"] = max(n_send) * feat_len * 4
        if packed:
            regions["q_recv_data"] = max(pk(x) for x in recv_all) * feat_len
            regions["q_send_data"] = max(pk(x) for x in send_all) * feat_len
            regions["q_recv_params"] = max(n_recv) * 4
            regions["q_send_params"] = max(n_send) * 4
        self.offset, total = {}, 0
        for name, nbytes in regions.items():
            self.offset[name] = total
            total += _round_up(max(nbytes, 16))
        self.pool, self.bases = peers.share(_round_up(max(total, _ALIGN)))
        dev = self.pool.device

        def before(rows_of_peer, me, packed_rows):
            """Rows (or packed rows) that precede rank `me`'s block in a peer's buffer."""
            rows = rows_of_peer[:me]
            return pk(rows) if packed_rows else sum(rows)

        # tables[(direction, payload)] = (region, row offset of my block in every peer's buffer)
        t = {}
        t["forward", "rows"] = ("recv_buf", [before(recv_all[p], r, False) for p in range(P)])
        t["backward", "rows"] = ("send_buf", [before(send_all[p], r, False) for p in range(P)])
        t["forward", "codes"] = ("q_recv_data", [before(recv_all[p], r, True) for p in range(P)])
        t["backward", "codes"] = ("q_send_data", [before(send_all[p], r, True) for p in range(P)])
        t["forward", "params"] = ("q_recv_params", [before(recv_all[p], r, False) for p in range(P)])
        t["backward", "params"] = ("q_send_params", [before(send_all[p], r, False) for p in range(P)])
        self._tables, self._host_tables = {}, {}
        for key, (region, offs) in t.items():
            if region in self.offset:
                self._host_tables[key] = ([self.bases[p] + self.offset[region] for p in range(P)], offs)
                base = torch.tensor([self.bases[p] + self.offset[region] for p in range(P)], dtype=torch.int64, device=dev)
                self._tables[key] = (base, torch.tensor(offs, dtype=torch.int64, device=dev))
        # send-list prefixes on the device: forward sends follow send_splits, backward sends recv_splits
        mk = lambda xs: _prefix_i32(xs, dev)
        pks = lambda xs: [(x + epb - 1) // epb for x in xs]
        self.seg = {("forward", "rows"): mk(comm_splits.send_splits), ("backward", "rows"): mk(comm_splits.recv_splits),
                    ("forward", "codes"): mk(pks(comm_splits.send_splits)),
                    ("backward", "codes"): mk(pks(comm_splits.recv_splits))}
        self.seg["forward", "params"] = self.seg["forward", "rows"]
        self.seg["backward", "params"] = self.seg["backward", "rows"]
        self.counts = {("forward", "rows"): list(comm_splits.send_splits), ("backward", "rows"): list(comm_splits.recv_splits),
                       ("forward", "codes"): pks(comm_splits.send_splits), ("backward", "codes"): pks(comm_splits.recv_splits)}
        self.counts["forward", "params"] = self.counts["forward", "rows"]
        self.counts["backward", "params"] = self.counts["backward", "rows"]
        self._dst_cache = {}
        self.src_offset = {k: [0] + [sum(v[:i + 1]) for i in range(P)] for k, v in self.counts.items()}  # host prefixes
        self.free = {"forward": None, "backward": None}  # last "receivers are done with this buffer" signal

    def region(self, name: str, shape, dtype) -> torch.Tensor:
        """This rank's buffer `name` as a tensor of `shape` (a view into the shared allocation)."""
        nbytes = 1
        for s in shape:
            nbytes *= int(s)
        nbytes *= torch.empty(0, dtype=dtype).element_size()
        off = self.offset[name]
        return self.pool[off: off + nbytes].view(dtype).view(*shape)

    def dst_table(self, direction: str, payload: str, ld_bytes: int) -> torch.Tensor:
        key = (direction, payload, ld_bytes)
        tab = self._dst_cache.get(key)
        if tab is None:
            base, offs = self._tables[direction, payload]
            tab = (base + offs * ld_bytes).contiguous()
            self._dst_cache[key] = tab
        return tab

    def push(self, direction: str, payload: str, src: torch.Tensor, row_bytes: int, first_peer: int, num_peers: int,
             idx: torch.Tensor = None) -> None:
        """Store this rank's blocks for peers first_peer .. first_peer+num_peers-1 (mod P) into their
        buffers; queued on the current stream."""
        counts = self.counts[direction, payload]
        rows = sum(counts[(first_peer + j) % self.P] for j in range(num_peers))
        if rows == 0:
            return
        ld_src = src.stride(0) * src.element_size()
        if idx is None and ld_src == row_bytes and self.peers.engine in ("copy", "auto"):
            # contiguous on both sides: one device-to-device copy per peer, on the copy engines
            base, offs = self._host_tables[direction, payload]
            start = self.src_offset[direction, payload]
            lib, stream = _lib.lib(), _lib.stream_ptr(src.device)
            for j in range(num_peers):
                p = (first_peer + j) % self.P
                if counts[p]:
                    rc = lib.gnnagg_push_block(src.data_ptr() + start[p] * row_bytes, base[p] + offs[p] * row_bytes,
                                               counts[p] * row_bytes, stream)
                    _lib.check(rc, "push_block")
            return
        dst = self.dst_table(direction, payload, row_bytes)
        rc = _lib.lib().gnnagg_push_rows(src.data_ptr(), ld_src, _lib.ptr(idx), row_bytes,
                                         self.seg[direction, payload].data_ptr(), self.P, first_peer, num_peers,
                                         dst.data_ptr(), row_bytes, rows, _lib.stream_ptr(src.device))
        _lib.check(rc, "push_rows")
