"""TEST INFRASTRUCTURE: the reference's partitioned aggregation on the host, for the CPU baseline.

A restatement, on CPU tensors, of what the reference's ranks do for one `Aggregator` forward +
backward with the fp32 halo (model/layers/aggregator.py:17-119 and :122-208 of the reference): the
plain communication plan (data_manager/DataProcessor.py:20-118), the send-side row gather
(aggregator.py:51), the local and remote SpMM (spmm_kernel.py:45-90 -> model/ops/src/spmm.cpp),
the backward transposed products and the scatter-add of the returned halo gradients
(aggregator.py:197-199).  All P ranks are emulated by ONE process that walks through them in turn
with every host thread; the all-to-all between them is a block copy in host memory.  The sparse
products run on the reference's own compiled kernel (oracle/_ref) when it is there, else on the C
port.  Only bench.py's reference arm and the tests use this module.
"""
import torch

from . import distribute_work_for_row, load_reference_module, spmm as port_spmm


class _Csr(object):
    """CSR arrays in the types the reference's kernel takes, with the greedy per-thread row splits
    of spmm_kernel.py:7-28 computed once (the reference caches them on the matrix)."""

    def __init__(self, rowptr, col, val, n_cols, threads):
        self.rowptr = rowptr.to(torch.int64).cpu().contiguous()
        self.col = col.to(torch.int64).cpu().contiguous()
        self.val = val.to(torch.float32).cpu().contiguous()
        self.M, self.K = self.rowptr.numel() - 1, n_cols
        self.row_split = torch.from_numpy(distribute_work_for_row(self.rowptr.numpy(), self.val.numpy(), threads))

    @staticmethod
    def pair_from_coo(row, col, M, K, threads):
        """(A, A^T) of the unit-valued matrix with entries (row, col): canonical CSR order (columns
        ascending inside a row, duplicates kept) and the CSC twin with rows ascending inside a column.
        The index work runs on the device the lists live on; the results are host arrays."""
        dev = row.device

        def compress(major, minor, n_major):
            order = torch.sort(major * max(int(minor.max()) + 1 if minor.numel() else 1, 1) + minor, stable=True)[1]
            ptr = torch.zeros(n_major + 1, dtype=torch.int64, device=dev)
            torch.cumsum(torch.bincount(major, minlength=n_major), 0, out=ptr[1:])
            return ptr, minor[order]

        ones = torch.ones(row.numel())
        rowptr, cols = compress(row, col, M)
        colptr, rows = compress(col, row, K)
        return _Csr(rowptr, cols, ones, K, threads), _Csr(colptr, rows, ones, M, threads)


class Partition(object):
    """One emulated rank: local / remote adjacency (+ transposes), the send index, the splits."""


def build_partitions(src, dst, begin, threads):
    """The plain halo plan of every rank (DataProcessor.py:20-118): remote sources renumbered to halo
    slots in ascending id order; every owner learns, per requesting rank, which of its rows to send."""
    P = len(begin) - 1
    parts, wanted = [], []
    for r in range(P):
        b0, b1 = int(begin[r]), int(begin[r + 1])
        mine = (dst >= b0) & (dst < b1)
        s, d = src[mine], dst[mine] - b0
        loc = (s >= b0) & (s < b1)
        p = Partition()
        p.n = b1 - b0
        p.local, p.local_T = _Csr.pair_from_coo(d[loc], s[loc] - b0, p.n, p.n, threads)
        halo_ids, slot = torch.unique(s[~loc], return_inverse=True)  # sorted: slot = rank among the sources
        p.remote, p.remote_T = _Csr.pair_from_coo(d[~loc], slot, p.n, halo_ids.numel(), threads)
        owner = torch.searchsorted(torch.as_tensor(begin, device=halo_ids.device), halo_ids, right=True) - 1
        p.recv_splits = torch.bincount(owner, minlength=P)[:P].tolist()
        p.nnz = p.local.col.numel() + p.remote.col.numel()
        wanted.append((halo_ids, p.recv_splits))
        parts.append(p)
    for r in range(P):  # what the others need from r, concatenated in requesting-rank order
        blocks, counts = [], []
        for q in range(P):
            ids, splits = wanted[q]
            off = sum(splits[:r])
            blocks.append(ids[off: off + splits[r]] - int(begin[r]))
            counts.append(splits[r])
        parts[r].send_idx = torch.cat(blocks).cpu()
        parts[r].send_splits = counts
    return parts


class CpuAggregator(object):
    def __init__(self, parts, threads):
        self.parts, self.threads = parts, threads
        # the compiled kernel opens an OpenMP region of the current thread count and indexes the row
        # splits by thread id: the count must be the one the splits were made for
        torch.set_num_threads(threads)
        self.ref = load_reference_module()
        self.kind = "reference" if self.ref is not None else "port"

    def _spmm(self, A, X, out):
        """out += A @ X (the reference's accumulating call)."""
        if A.col.numel() == 0:
            return
        if self.ref is not None:
            self.ref.spmm(A.rowptr, A.col, A.val, X, out, A.M, A.row_split, torch.tensor([0, X.size(1)], dtype=torch.int32))
        else:
            port_spmm(A.rowptr.numpy(), A.col.numpy(), A.val.numpy(), X.numpy(), out.numpy())

    def _exchange(self, send_bufs, send_key, recv_key):
        """all-to-all with row splits between the emulated ranks: rank q's block for rank r lands in r's
        receive buffer at the offset of q."""
        P = len(self.parts)
        out = []
        for r in range(P):
            rs = getattr(self.parts[r], recv_key)
            blocks = []
            for q in range(P):
                ss = getattr(self.parts[q], send_key)
                off = sum(ss[:r])
                blocks.append(send_bufs[q][off: off + ss[r]])
                assert ss[r] == rs[q]
            out.append(torch.cat(blocks))
        return out

    def forward(self, X):
        send = [torch.index_select(x, 0, p.send_idx) for p, x in zip(self.parts, X)]
        recv = self._exchange(send, "send_splits", "recv_splits")
        outs = []
        for p, x, h in zip(self.parts, X, recv):
            out = torch.zeros(p.n, x.size(1))
            self._spmm(p.local, x, out)
            self._spmm(p.remote, h, out)
            outs.append(out)
        return outs

    def backward(self, G):
        halo_grad = []
        for p, g in zip(self.parts, G):
            buf = torch.zeros(p.remote.K, g.size(1))
            self._spmm(p.remote_T, g, buf)
            halo_grad.append(buf)
        back = self._exchange(halo_grad, "recv_splits", "send_splits")
        grads = []
        for p, g, b in zip(self.parts, G, back):
            grad = torch.zeros(p.n, g.size(1))
            self._spmm(p.local_T, g, grad)
            grad.index_add_(0, p.send_idx, b)
            grads.append(grad)
        return grads

    def edges_per_pass(self):
        return sum(p.nnz for p in self.parts)
