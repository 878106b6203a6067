"""SparseTensor: the adjacency container the aggregation path works on.

The reference uses a fork of `torch_sparse.SparseTensor` that is not part of its repository
(self_benchmark/a64fx/model/ops/spmm_kernel.py:3,46-57,76-87 show the surface it needs:
`csr()`, `storage.colptr()/row_T()/value_T()`, `sparse_size()`, and cached per-matrix
"work ranges").  This class offers that surface over device-resident arrays laid out for the
CUDA kernels: int64 row pointers, int32 column indices, fp32 values, CSR in canonical order
(row-major, columns ascending, duplicates kept) and, on demand, the CSC twin with rows
ascending inside a column (the operand of the transposed product).
"""
from typing import Optional, Tuple

import torch

from . import _lib


class _Storage:
    """`src.storage.*` accessors used by SPMM_backward (spmm_kernel.py:76-78)."""

    def __init__(self, owner: "SparseTensor"):
        self._o = owner

    def rowptr(self):
        return self._o._rowptr

    def col(self):
        return self._o._col

    def value(self):
        return self._o._value

    def colptr(self):
        self._o._build_csc()
        return self._o._colptr

    def row_T(self):
        self._o._build_csc()
        return self._o._row_T

    def value_T(self):
        self._o._build_csc()
        return self._o._value_T


def _compress(sorted_major: torch.Tensor, n_major: int) -> torch.Tensor:
    counts = torch.bincount(sorted_major, minlength=n_major) if sorted_major.numel() else torch.zeros(
        n_major, dtype=torch.int64, device=sorted_major.device)
    ptr = torch.zeros(n_major + 1, dtype=torch.int64, device=sorted_major.device)
    torch.cumsum(counts, 0, out=ptr[1:])
    return ptr


class SparseTensor:
    def __init__(self, row: Optional[torch.Tensor] = None, col: Optional[torch.Tensor] = None,
                 value: Optional[torch.Tensor] = None, sparse_sizes: Optional[Tuple[int, int]] = None,
                 rowptr: Optional[torch.Tensor] = None, is_sorted: bool = False):
        """COO (row, col[, value]) or CSR (rowptr, col[, value]) in; canonical CSR kept.

        value defaults to ones (the reference always passes ones, DataProcessor.py:107,114)."""
        if sparse_sizes is None:
            raise ValueError("sparse_sizes=(rows, cols) is required")
        self._M, self._K = int(sparse_sizes[0]), int(sparse_sizes[1])
        if rowptr is not None:
            assert col is not None
            self._rowptr = rowptr.to(torch.int64).contiguous()
            self._col = col.to(torch.int32).contiguous()
            self._value = (torch.ones(col.numel(), dtype=torch.float32, device=col.device) if value is None
                           else value.to(torch.float32).contiguous())
        else:
            assert row is not None and col is not None
            row = row.to(torch.int64)
            col = col.to(torch.int64)
            if value is None:
                value = torch.ones(row.numel(), dtype=torch.float32, device=row.device)
            value = value.to(torch.float32)
            if not is_sorted and row.numel() > 0:
                key = row * self._K + col
                perm = torch.sort(key, stable=True)[1]
                row, col, value = row[perm], col[perm], value[perm]
            self._rowptr = _compress(row, self._M)
            self._col = col.to(torch.int32).contiguous()
            self._value = value.contiguous()
        self._colptr = None
        self._row_T = None
        self._value_T = None
        # cached per-matrix launch plans (the GPU counterpart of the reference's cached row splits)
        self._plan = None
        self._plan_T = None
        self.storage = _Storage(self)

    # ---- torch_sparse-like surface --------------------------------------------------------
    def csr(self):
        return self._rowptr, self._col, self._value

    def sparse_size(self, dim: int) -> int:
        return (self._M, self._K)[dim]

    def sparse_sizes(self):
        return (self._M, self._K)

    def nnz(self) -> int:
        return int(self._col.numel())

    @property
    def device(self):
        return self._rowptr.device

    def to_dense(self) -> torch.Tensor:
        out = torch.zeros(self._M, self._K, dtype=torch.float32, device=self.device)
        if self.nnz():
            rows = torch.repeat_interleave(torch.arange(self._M, device=self.device),
                                           self._rowptr[1:] - self._rowptr[:-1])
            out.index_put_((rows, self._col.to(torch.int64)), self._value, accumulate=True)
        return out

    def to(self, device) -> "SparseTensor":
        device = torch.device(device)
        if device == self.device:
            return self
        new = SparseTensor(rowptr=self._rowptr.to(device), col=self._col.to(device), value=self._value.to(device),
                           sparse_sizes=(self._M, self._K))
        if self._colptr is not None:
            new._colptr, new._row_T, new._value_T = (self._colptr.to(device), self._row_T.to(device),
                                                     self._value_T.to(device))
        return new

    def cuda(self, device=None) -> "SparseTensor":
        return self.to(torch.device("cuda", torch.cuda.current_device() if device is None else device))

    def set_value_(self, value: torch.Tensor) -> "SparseTensor":
        """Replace the per-nonzero values (CSR order); drops the cached CSC values."""
        assert value.numel() == self.nnz()
        self._value = value.to(torch.float32).contiguous()
        self._value_T = None
        if self._colptr is not None:
            self._colptr = None
            self._row_T = None
        return self

    # ---- work ranges (spmm_kernel.py:48,57,80,87) --------------------------------------------
    def get_work_range(self):
        return self._plan if self._plan is not None else torch.empty(0, dtype=torch.uint8, device=self.device)

    def set_work_range(self, plan: torch.Tensor) -> None:
        self._plan = plan

    def get_work_range_for_transpose(self):
        return self._plan_T if self._plan_T is not None else torch.empty(0, dtype=torch.uint8, device=self.device)

    def set_work_range_for_transpose(self, plan: torch.Tensor) -> None:
        self._plan_T = plan

    # ---- CSC twin ---------------------------------------------------------------------------
    def _build_csc(self) -> None:
        if self._colptr is not None:
            return
        dev = self.device
        nnz = self.nnz()
        if nnz == 0:
            self._colptr = torch.zeros(self._K + 1, dtype=torch.int64, device=dev)
            self._row_T = torch.zeros(0, dtype=torch.int32, device=dev)
            self._value_T = torch.zeros(0, dtype=torch.float32, device=dev)
            return
        if self._rowptr.is_cuda:
            # the library's transpose: a stable radix sort of the nonzeros by column
            lib = _lib.lib()
            ws = torch.empty(lib.gnnagg_csr_to_csc_workspace_bytes(self._M, self._K, nnz), dtype=torch.uint8, device=dev)
            self._colptr = torch.empty(self._K + 1, dtype=torch.int64, device=dev)
            self._row_T = torch.empty(nnz, dtype=torch.int32, device=dev)
            self._value_T = torch.empty(nnz, dtype=torch.float32, device=dev)
            rc = lib.gnnagg_csr_to_csc(self._rowptr.data_ptr(), self._col.data_ptr(), self._value.data_ptr(), self._M,
                                       self._K, nnz, self._colptr.data_ptr(), self._row_T.data_ptr(),
                                       self._value_T.data_ptr(), ws.data_ptr(), ws.numel(), _lib.stream_ptr(dev))
            _lib.check(rc, "csr_to_csc")
            return
        # host tensors (plan tests on CPU): CSR order is row-ascending, so a stable sort by column leaves
        # rows ascending in a column
        col64 = self._col.to(torch.int64)
        sorted_col, perm = torch.sort(col64, stable=True)
        rows = torch.repeat_interleave(torch.arange(self._M, device=dev, dtype=torch.int32),
                                       self._rowptr[1:] - self._rowptr[:-1])
        self._row_T = rows[perm].contiguous()
        self._value_T = self._value[perm].contiguous()
        self._colptr = _compress(sorted_col, self._K)

    def validate(self) -> None:
        """Device-side check of rowptr monotonicity and column range; raises on a bad matrix."""
        _lib.require_cuda(self._rowptr)
        status = torch.zeros(1, dtype=torch.int32, device=self.device)
        rc = _lib.lib().gnnagg_csr_validate(self._rowptr.data_ptr(), _lib.ptr(self._col), self._M, self._K, self.nnz(),
                                            status.data_ptr(), _lib.stream_ptr(self.device))
        _lib.check(rc, "csr_validate")
        s = int(status.item())
        if s:
            raise RuntimeError(f"malformed CSR matrix (status mask {s}: 1 = rowptr, 2 = column index out of range)")

    def __repr__(self):
        return f"SparseTensor(sizes=({self._M}, {self._K}), nnz={self.nnz()}, device={self.device})"
