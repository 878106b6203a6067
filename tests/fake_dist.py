"""In-process stand-in for torch.distributed so that P ranks of the aggregation path can run as P
threads on ONE GPU (NCCL refuses two ranks on one device, and kernels of different ranks must not
spin on one another on a shared GPU -- here they never wait on the device, only on host barriers).

Only what the path uses is provided: get_rank / get_world_size / is_initialized / get_backend /
barrier / all_to_all_single (row splits, sync or "async").  Each rank runs on its own CUDA stream.
"""
import threading
from contextlib import contextmanager

import torch
import torch.distributed as dist


class _Work:
    def wait(self):
        return True


class _P2POp:
    """Stand-in for dist.P2POp (the real one insists on an initialised process group)."""

    def __init__(self, op, tensor, peer=None, group=None, tag=0, group_peer=None):
        self.op, self.tensor, self.peer = op, tensor, peer

_REAL_ISEND, _REAL_IRECV = dist.isend, dist.irecv


class ThreadPeers:
    """Stand-in for gnn_benchmark_b200.peer.NcclPeers when the ranks are threads on one GPU: every rank's
    buffer is ordinary memory of the same device, so its address IS the peer address; a signal is a
    stream synchronisation followed by a host barrier (nothing on the device waits for another rank)."""

    def __init__(self, world: "FakeWorld", rank: int):
        self.w, self.rank, self.world = world, rank, world.P
        self.engine = getattr(world, "push_engine", "auto")
        self._bufs = []

    def gather_objects(self, obj):
        self.w._objs[self.rank] = obj
        self.w._barrier.wait()
        out = list(self.w._objs)
        self.w._barrier.wait()
        return out

    def share(self, nbytes: int):
        buf = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
        self._bufs.append(buf)
        torch.cuda.current_stream().synchronize()
        return buf, self.gather_objects(buf.data_ptr())

    def signal(self):
        torch.cuda.current_stream().synchronize()
        self.w._barrier.wait()
        return _Work()


class FakeWorld:
    def __init__(self, world_size: int, push_engine: str = "auto"):
        self._objs = [None] * world_size
        self.P = world_size
        self.push_engine = push_engine
        self._barrier = threading.Barrier(world_size)
        self._slots = [None] * world_size
        self._local = threading.local()
        self._mail = {}
        self._cond = threading.Condition()

    # ---- torch.distributed surface ----
    def get_rank(self, group=None):
        return self._local.rank

    def get_world_size(self, group=None):
        return self.P

    def is_initialized(self):
        return True

    def is_available(self):
        return True

    def get_backend(self, group=None):
        return "nccl"  # plans are built on the tensors' own device

    def barrier(self, *a, **k):
        self._barrier.wait()

    def all_to_all_single(self, output, input, output_split_sizes=None, input_split_sizes=None, group=None,
                          async_op=False):
        r, P = self._local.rank, self.P
        if input_split_sizes is None:
            input_split_sizes = [input.size(0) // P] * P
        if output_split_sizes is None:
            output_split_sizes = [output.size(0) // P] * P
        if input.is_cuda:
            torch.cuda.current_stream().synchronize()  # producers of `input` are done
        self._slots[r] = (input, list(input_split_sizes))
        self._barrier.wait()
        off_out = 0
        for q in range(P):
            src, splits = self._slots[q]
            off_in = sum(splits[:r])
            n = splits[r]
            assert n == output_split_sizes[q], f"rank {r}: peer {q} sends {n} rows, expected {output_split_sizes[q]}"
            if n:
                output[off_out:off_out + n].copy_(src[off_in:off_in + n])
            off_out += n
        if output.is_cuda:
            torch.cuda.current_stream().synchronize()
        self._barrier.wait()  # nobody overwrites a send buffer before every peer has copied from it
        return _Work() if async_op else None

    def batch_isend_irecv(self, ops):
        """Grouped point-to-point operations: sends post a copy into the receiver's mailbox, receives
        block (on the host) until the matching send has been posted."""
        r = self._local.rank
        if any(o.tensor.is_cuda for o in ops):
            torch.cuda.current_stream().synchronize()
        for o in ops:
            if o.op is _REAL_ISEND:
                with self._cond:
                    self._mail.setdefault((r, o.peer), []).append(o.tensor.clone())
                    self._cond.notify_all()
        for o in ops:
            if o.op is _REAL_IRECV:
                with self._cond:
                    ok = self._cond.wait_for(lambda: self._mail.get((o.peer, r)), timeout=60)
                    if not ok:
                        raise RuntimeError(f"rank {r}: no message from rank {o.peer}")
                    src = self._mail[(o.peer, r)].pop(0)
                assert src.shape == o.tensor.shape, f"rank {r}: size mismatch with rank {o.peer}"
                o.tensor.copy_(src)
        if any(o.tensor.is_cuda for o in ops):
            torch.cuda.current_stream().synchronize()
        return [_Work()]

    # ---- harness ----
    @contextmanager
    def patched(self):
        names = ("get_rank", "get_world_size", "is_initialized", "is_available", "get_backend", "barrier",
                 "all_to_all_single", "batch_isend_irecv")
        from gnn_benchmark_b200.communicator import Communicator

        saved = {n: getattr(dist, n) for n in names}
        saved["P2POp"] = dist.P2POp
        real_peers = Communicator.peers
        try:
            for n in names:
                setattr(dist, n, getattr(self, n))
            dist.P2POp = _P2POp
            Communicator.peers = lambda comm: self._local.peers  # one peer service per rank (thread)
            yield self
        finally:
            Communicator.peers = real_peers
            for n, f in saved.items():
                setattr(dist, n, f)

    def run(self, fn):
        """fn(rank) on P threads, each on its own CUDA stream; returns the list of results."""
        results, errors = [None] * self.P, []

        def target(rank):
            self._local.rank = rank
            self._local.peers = ThreadPeers(self, rank)
            try:
                if torch.cuda.is_available():
                    stream = torch.cuda.Stream()
                    with torch.cuda.stream(stream):
                        results[rank] = fn(rank)
                        stream.synchronize()
                else:
                    results[rank] = fn(rank)
            except BaseException as e:  # noqa: BLE001
                errors.append((rank, e))
                self._barrier.abort()

        with self.patched():
            threads = [threading.Thread(target=target, args=(r,)) for r in range(self.P)]
            for t in threads:
                t.start()
            for t in threads:
                t.join()
        if errors:
            errors.sort(key=lambda x: isinstance(x[1], threading.BrokenBarrierError))
            raise errors[0][1]
        return results
