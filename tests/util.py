"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch


def random_csr(rng, M, K, avg_deg, hubs=0, hub_len=3000, empty_frac=0.2):
    """Random CSR with empty rows, duplicate-free sorted columns and a few very long rows."""
    deg = rng.poisson(avg_deg, size=M)
    deg[rng.random(M) < empty_frac] = 0
    if hubs and M > 0:
        idx = rng.choice(M, size=min(hubs, M), replace=False)
        deg[idx] = min(hub_len, K)
    deg = np.minimum(deg, K)
    rowptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    col = np.empty(int(rowptr[-1]), dtype=np.int64)
    for m in range(M):
        if deg[m]:
            col[rowptr[m]:rowptr[m + 1]] = np.sort(rng.choice(K, size=deg[m], replace=False))
    val = rng.standard_normal(col.shape[0]).astype(np.float32)
    return rowptr, col, val


def to_dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()


def rel_err(a, b):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return np.abs(a - b).max() / max(np.abs(b).max(), 1e-30)
