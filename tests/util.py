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


def philox4x32_10(counter, key):
    """Philox-4x32-10 (Salmon et al., SC'11) on numpy uint32 arrays: counter (..., 4), key (2,).
    The keep-bits of the fused dropout kernels are defined on this generator."""
    import numpy as np

    c = [np.asarray(counter[..., i], dtype=np.uint64) for i in range(4)]
    k0, k1 = np.uint64(int(key[0]) & 0xFFFFFFFF), np.uint64(int(key[1]) & 0xFFFFFFFF)
    m0, m1, mask = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57), np.uint64(0xFFFFFFFF)
    for _ in range(10):
        p0, p1 = m0 * c[0], m1 * c[2]
        hi0, lo0, hi1, lo1 = p0 >> np.uint64(32), p0 & mask, p1 >> np.uint64(32), p1 & mask
        c = [hi1 ^ c[1] ^ k0, lo1, hi0 ^ c[3] ^ k1, lo0]
        k0 = (k0 + np.uint64(0x9E3779B9)) & mask
        k1 = (k1 + np.uint64(0xBB67AE85)) & mask
    return np.stack([x.astype(np.uint32) for x in c], axis=-1)


def dropout_keep_bits(rows, chunks, seed, p):
    """(rows, chunks) uint8: the 4 keep-bits of every float4 chunk as the kernels draw them:
    counter = (row low, row high, chunk, 0x6e6f726d), key = (seed low, seed high); element i of a chunk
    is kept when its 16-bit draw (x low, x high, y low, y high) is >= round(p * 65536)."""
    import numpy as np

    thresh = max(int(p * 65536.0 + 0.5), 1 if p > 0 else 0)
    r = np.arange(rows, dtype=np.uint64)[:, None] + np.zeros((1, chunks), dtype=np.uint64)
    c = np.arange(chunks, dtype=np.uint64)[None, :] + np.zeros((rows, 1), dtype=np.uint64)
    ctr = np.stack([r & np.uint64(0xFFFFFFFF), r >> np.uint64(32), c, np.full_like(r, 0x6E6F726D)], axis=-1)
    out = philox4x32_10(ctr, (seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF))
    x, y = out[..., 0], out[..., 1]
    draws = [x & 0xFFFF, x >> 16, y & 0xFFFF, y >> 16]
    bits = np.zeros((rows, chunks), dtype=np.uint8)
    for i, d in enumerate(draws):
        bits |= ((d >= thresh).astype(np.uint8) << i)
    return bits


def synthetic_problem(cfg, device="cpu"):
    """Graph, features, labels and train mask of a scaled BASELINE configuration, from the seeds in
    `cfg` (nodes, edges, P, dims, graph_seed, self_loops, train_frac).  Used by the script that runs the
    reference (tests/golden/make_config_golden.py) and by the tests that replay its runs, so that both
    sides see exactly the same inputs."""
    from gnn_benchmark_b200 import graphgen

    n, P = cfg["nodes"], cfg["P"]
    src, dst = graphgen.chung_lu_edges(n, cfg["edges"], gamma=2.1, seed=cfg["graph_seed"], device=device)
    src, dst = graphgen.relabel(src, dst, n, cfg["graph_seed"] + 7)
    src, dst = graphgen.symmetrize(src, dst, n, self_loops=bool(cfg["self_loops"]))
    begin = graphgen.contiguous_partitions(n, P)
    g = torch.Generator().manual_seed(cfg["graph_seed"] + 1)
    X = torch.randn(n, cfg["dims"][0], generator=g)
    labels = torch.randint(0, cfg["dims"][-1], (n,), generator=g)
    train_mask = torch.rand(n, generator=g) < cfg["train_frac"]
    return src, dst, begin, X, labels, train_mask
