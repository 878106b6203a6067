"""Seeded synthetic graphs on the GPU (or CPU): R-MAT, Erdos-Renyi G(n,m), Chung-Lu power law;
symmetrise / deduplicate / self-loops, GCN normalisation, random relabelling and the split into
contiguous 1-D vertex partitions in the reference's per-rank form (local edges with both ends
localised, remote edges as [global source, local destination]; data_manager/DataLoader.py:12-40
of the reference).  These stand in for the public datasets whose shapes the benchmark
configurations copy; every generator takes an explicit seed and is pure torch, so the same seed
gives the same graph on every rank.
"""
import math
from typing import Tuple

import torch


def _gen(seed: int, device) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(int(seed))
    return g


def rmat_edges(scale: int, edge_factor: int = 16, a: float = 0.57, b: float = 0.19, c: float = 0.19,
               seed: int = 0, device="cpu", chunk: int = 1 << 25) -> Tuple[torch.Tensor, torch.Tensor]:
    """Directed R-MAT edge list (src, dst), 2^scale vertices, edge_factor * 2^scale edges.
    Per bit level one uniform draw picks the quadrant with probabilities (a, b, c, 1-a-b-c)."""
    n_edges = edge_factor << scale
    g = _gen(seed, device)
    srcs, dsts = [], []
    for start in range(0, n_edges, chunk):
        m = min(chunk, n_edges - start)
        src = torch.zeros(m, dtype=torch.int64, device=device)
        dst = torch.zeros(m, dtype=torch.int64, device=device)
        for _ in range(scale):
            r = torch.rand(m, generator=g, device=device)
            src_bit = r >= (a + b)
            dst_bit = ((r >= a) & (r < a + b)) | (r >= a + b + c)
            src = (src << 1) | src_bit.to(torch.int64)
            dst = (dst << 1) | dst_bit.to(torch.int64)
        srcs.append(src)
        dsts.append(dst)
    return torch.cat(srcs), torch.cat(dsts)


def erdos_renyi_edges(n: int, m: int, seed: int = 0, device="cpu") -> Tuple[torch.Tensor, torch.Tensor]:
    """m undirected edges sampled uniformly (duplicates and loops are removed later by
    `symmetrize`, so slightly fewer than m may remain)."""
    g = _gen(seed, device)
    src = torch.randint(0, n, (m,), generator=g, device=device, dtype=torch.int64)
    dst = torch.randint(0, n, (m,), generator=g, device=device, dtype=torch.int64)
    return src, dst


def _power_law_cdf(n: int, m: int, gamma: float, device) -> torch.Tensor:
    """Integer cumulative weights of the Chung-Lu endpoint distribution: expected degrees
    w_i ~ (i + 1)^(-1/(gamma-1)), scaled to sum 2m and capped at sqrt(2m), then put on a fixed-point
    grid of about 2^52 units in total.  The running sum is taken over INTEGERS, so it is exact and the
    same whatever order a parallel scan adds in: a floating-point prefix sum on the GPU differs in
    the last bit from run to run, which at 10^8 vertices and 10^9 draws moves a dozen edges."""
    i = torch.arange(n, dtype=torch.float64, device=device)
    w = (i + 1.0).pow(-1.0 / (gamma - 1.0))
    w = w * (2.0 * m / w.sum())
    w = torch.clamp(w, max=math.sqrt(2.0 * m))
    units = (w * (float(1 << 52) / float(w.sum()))).floor().to(torch.int64).clamp_(min=1)
    return torch.cumsum(units, 0)


def _draw_endpoints(cdf: torch.Tensor, k: int, g: torch.Generator) -> torch.Tensor:
    """k vertex ids with probability proportional to the weights behind the integer `cdf`."""
    u = torch.randint(0, int(cdf[-1]), (k,), generator=g, device=cdf.device, dtype=torch.int64)
    return torch.searchsorted(cdf, u, right=True).clamp_(max=cdf.numel() - 1)


def chung_lu_edges(n: int, m: int, gamma: float = 2.1, seed: int = 0, device="cpu",
                   chunk: int = 1 << 26) -> Tuple[torch.Tensor, torch.Tensor]:
    """m edges whose endpoints are drawn independently with probability proportional to the
    expected degrees w_i ~ (i + 1)^(-1/(gamma-1)), w_max capped at sqrt(sum w)."""
    g = _gen(seed, device)
    cdf = _power_law_cdf(n, m, gamma, device)
    out = []
    for _ in range(2):
        out.append(torch.cat([_draw_endpoints(cdf, min(chunk, m - start), g) for start in range(0, m, chunk)]))
    return out[0], out[1]


def symmetrize(src: torch.Tensor, dst: torch.Tensor, n: int, self_loops: bool = True,
               drop_loops: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    """Both directions of every edge, duplicates removed, optional self-loop on every vertex.
    Returned sorted by (dst, src): row-major order of the adjacency A[dst, src]."""
    if drop_loops:
        keep = src != dst
        src, dst = src[keep], dst[keep]
    key = torch.cat([dst * n + src, src * n + dst])
    if self_loops:
        d = torch.arange(n, dtype=torch.int64, device=key.device)
        key = torch.cat([key, d * n + d])
    key = torch.unique(key)  # sorted
    return key % n, key // n  # (src, dst)


def relabel(src: torch.Tensor, dst: torch.Tensor, n: int, seed: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Apply one seeded random permutation of the vertex ids to both ends."""
    perm = torch.randperm(n, generator=_gen(seed, src.device), device=src.device)
    return perm[src], perm[dst]


def csr_from_edges(src: torch.Tensor, dst: torch.Tensor, n_rows: int, n_cols: int, gcn_normalize: bool = False):
    """CSR of A[dst, src] (row = destination).  Returns (rowptr int64, col int32, val fp32).
    gcn_normalize: val = d_dst^-1/2 * d_src^-1/2 with d = row degree (self-loops included if
    present in the edge list); else all ones."""
    key = dst * n_cols + src
    key = torch.sort(key)[0]
    row = key // n_cols
    col = key % n_cols
    counts = torch.bincount(row, minlength=n_rows)
    rowptr = torch.zeros(n_rows + 1, dtype=torch.int64, device=src.device)
    torch.cumsum(counts, 0, out=rowptr[1:])
    if gcn_normalize:
        dinv = counts.clamp(min=1).to(torch.float32).rsqrt()
        val = dinv[row] * dinv[col]
    else:
        val = torch.ones(col.numel(), dtype=torch.float32, device=src.device)
    return rowptr, col.to(torch.int32), val


def contiguous_partitions(n: int, parts: int) -> torch.Tensor:
    """begin_node_on_each_partition: P+1 int64, blocks as equal as possible."""
    base, rem = divmod(n, parts)
    sizes = torch.tensor([base + (1 if r < rem else 0) for r in range(parts)], dtype=torch.int64)
    return torch.cat([torch.zeros(1, dtype=torch.int64), torch.cumsum(sizes, 0)])


def partition_edges(src: torch.Tensor, dst: torch.Tensor, begin: torch.Tensor, rank: int):
    """The reference's per-rank edge lists for the block [begin[rank], begin[rank+1]):
    local_edges (2, E_l) both ends localised; remote_edges (2, E_r) [global src, localised dst]."""
    b0, b1 = int(begin[rank]), int(begin[rank + 1])
    mine = (dst >= b0) & (dst < b1)
    s, d = src[mine], dst[mine]
    loc = (s >= b0) & (s < b1)
    local_edges = torch.stack([s[loc] - b0, d[loc] - b0])
    remote_edges = torch.stack([s[~loc], d[~loc] - b0])
    return local_edges, remote_edges


def write_partition_files(out_dir: str, graph_name: str, rank: int, begin: torch.Tensor, local_edges, remote_edges,
                          feat, label, train_idx, valid_idx, test_idx) -> None:
    """Write one rank's files in the reference's on-disk format (see data_manager/DataLoader.py)."""
    import os

    import numpy as np

    os.makedirs(out_dir, exist_ok=True)
    b0, b1 = int(begin[rank]), int(begin[rank + 1])
    ids = np.arange(b0, b1, dtype=np.int64)

    def f(what):
        return os.path.join(out_dir, "p{:0>3d}-{}_{}.npy".format(rank, graph_name, what))

    np.save(f("nodes"), np.stack([ids, ids], axis=1))
    np.save(f("local_edges"), local_edges.cpu().numpy().astype(np.int64))
    np.save(f("remote_edges"), remote_edges.cpu().numpy().astype(np.int64))
    np.save(f("nodes_feat"), feat.cpu().numpy().astype(np.float32))
    np.save(f("nodes_label"), label.cpu().numpy().astype(np.int64))
    np.save(f("nodes_train_idx"), train_idx.cpu().numpy().astype(np.int64))
    np.save(f("nodes_valid_idx"), valid_idx.cpu().numpy().astype(np.int64))
    np.save(f("nodes_test_idx"), test_idx.cpu().numpy().astype(np.int64))
    if rank == 0:
        with open(os.path.join(out_dir, "begin_node_on_each_partition.txt"), "w") as fh:
            fh.write(" ".join(str(int(x)) for x in begin.tolist()) + "\n")


def partitioned_in_edges(kind: str, n: int, n_edges: int, seed: int, rank: int, world: int, device, relabel: bool = True,
                         chunk: int = 1 << 25, scale: int = 0, gamma: float = 2.1, self_loops: bool = True):
    """In-edges (src, dst; global ids) of rank `rank`'s contiguous vertex block of a symmetrised,
    deduplicated synthetic graph, generated chunk by chunk from one seed so that every rank sees the
    same global edge stream without any rank holding the whole graph.

    kind "rmat": 2^scale vertices, (a,b,c,d) = (.57,.19,.19,.05); kind "chung_lu": expected degrees
    ~ (i+1)^(-1/(gamma-1)).  relabel applies one seeded random permutation of the vertex ids (keeps
    the partitions balanced: both generators put their hubs at low ids).  Returns (src, dst, begin)."""
    begin = contiguous_partitions(n, world)
    b0, b1 = int(begin[rank]), int(begin[rank + 1])
    perm = torch.randperm(n, generator=_gen(seed + 1, device), device=device) if relabel else None
    g = _gen(seed, device)
    cdf = None
    if kind == "chung_lu":
        cdf = _power_law_cdf(n, n_edges, gamma, device)
    keys = []
    for start in range(0, n_edges, chunk):
        m = min(chunk, n_edges - start)
        if kind == "rmat":
            a, b, c = 0.57, 0.19, 0.19
            src = torch.zeros(m, dtype=torch.int64, device=device)
            dst = torch.zeros(m, dtype=torch.int64, device=device)
            for _ in range(scale):
                r = torch.rand(m, generator=g, device=device)
                src = (src << 1) | (r >= (a + b)).to(torch.int64)
                dst = (dst << 1) | (((r >= a) & (r < a + b)) | (r >= a + b + c)).to(torch.int64)
        elif kind == "chung_lu":
            src = _draw_endpoints(cdf, m, g)
            dst = _draw_endpoints(cdf, m, g)
        else:
            raise ValueError(kind)
        keep = src != dst
        src, dst = src[keep], dst[keep]
        if perm is not None:
            src, dst = perm[src], perm[dst]
        for s_, d_ in ((src, dst), (dst, src)):  # both directions; keep what lands in this rank's rows
            mine = (d_ >= b0) & (d_ < b1)
            keys.append(torch.unique(d_[mine] * n + s_[mine]))
        del src, dst, keep
    if self_loops:
        diag = torch.arange(b0, b1, dtype=torch.int64, device=device)
        keys.append(diag * n + diag)
    key = torch.unique(torch.cat(keys)) if keys else torch.zeros(0, dtype=torch.int64, device=device)
    del keys, cdf
    return key % n, key // n, begin
