"""Generate the golden fixtures under tests/golden/ by running the REFERENCE's own code.

Run once, in a container that has the reference checkout (its root is the optional argument) and the
compiled reference module (python oracle/build_ref.py):

    python tests/golden/make_golden.py [reference_root]

The reference's Python imports a forked torch_sparse that is not available; a minimal stand-in
(row/col/value holder) is registered for the import to succeed -- no arithmetic of the path
goes through it.  The multi-rank plan exchange is simulated in-process by handing each rank's
"sent" lists to the receiving rank, which is exactly what the two all-to-alls of the reference
do (data_manager/DataProcessor.py:63-98, 329-382).

Outputs (small .npz files, committed):
  plan_plain_*.npz, plan_prepost_*.npz  comm plans of the reference's DataProcessor classes
  quant_v1.npz, quant_rowpacked.npz     bytes of the compiled x86 quantisers
  spmm_ref.npz                          output of the compiled reference spmm
  ref_test_vectors.json                 the literal vectors of the reference's own unit tests
"""
import json
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, REPO)


def install_shims(ref_root):
    import oracle

    class SparseTensor:  # holder only
        def __init__(self, row=None, col=None, value=None, sparse_sizes=None, **kw):
            self.row, self.col, self.value, self.sizes = row, col, value, sparse_sizes

        def sparse_size(self, i):
            return self.sizes[i]

    ts = types.ModuleType("torch_sparse")
    ts.SparseTensor = SparseTensor
    sys.modules["torch_sparse"] = ts
    ref_mod = oracle.load_reference_module()
    if ref_mod is None:
        raise SystemExit("build oracle/_ref first: python oracle/build_ref.py")
    sys.modules["computation_ops"] = ref_mod
    sys.path.insert(0, os.path.join(ref_root, "self_benchmark", "a64fx"))
    return ref_mod


def random_partitioned_graph(rng, P, n_per, deg, dup_frac=0.1):
    """Directed edge list over P contiguous blocks; returns begin and per-rank (local, remote)."""
    sizes = rng.integers(max(1, n_per // 2), n_per + 1, size=P)
    begin = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64)
    N = int(begin[-1])
    E = N * deg
    src = rng.integers(0, N, size=E)
    # skew: a few hub sources and hub destinations so that pre and post both occur
    hubs = rng.integers(0, N, size=max(2, N // 20))
    src[: E // 4] = rng.choice(hubs, size=E // 4)
    dst = rng.integers(0, N, size=E)
    dst[E // 4: E // 2] = rng.choice(hubs, size=E // 2 - E // 4)
    ndup = int(E * dup_frac)
    src = np.concatenate([src, src[:ndup]])
    dst = np.concatenate([dst, dst[:ndup]])
    parts = []
    for r in range(P):
        m = (dst >= begin[r]) & (dst < begin[r + 1])
        s, d = src[m], dst[m]
        loc = (s >= begin[r]) & (s < begin[r + 1])
        local = np.stack([s[loc] - begin[r], d[loc] - begin[r]]).astype(np.int64)
        remote = np.stack([s[~loc], d[~loc] - begin[r]]).astype(np.int64)
        parts.append((local, remote))
    return begin, parts


def plain_plan(DataProcessor, begin, parts):
    P = len(parts)
    per_rank = []
    for r in range(P):
        local, remote = parts[r]
        n = int(begin[r + 1] - begin[r])
        rem = [torch.from_numpy(remote[0].copy()), torch.from_numpy(remote[1].copy())]
        indeg = DataProcessor.get_in_degrees([torch.from_numpy(local[0]), torch.from_numpy(local[1])], rem, n)
        rem = DataProcessor.sort_remote_edges_list_based_on_remote_nodes(rem)
        nodes, rng_, cnt = DataProcessor.obtain_remote_nodes_list(rem, n, torch.from_numpy(begin), P)
        per_rank.append(dict(n=n, rem=rem, nodes=nodes, rng=rng_, cnt=cnt, indeg=indeg))
    out = {}
    for r in range(P):
        # what rank r receives: from every q, q's needed-node list restricted to r's range
        recv = [per_rank[q]["nodes"][per_rank[q]["rng"][r]: per_rank[q]["rng"][r + 1]] for q in range(P)]
        idx = torch.cat(recv) - int(begin[r])
        pr = per_rank[r]
        out[f"r{r}_remote_nodes_list"] = pr["nodes"].numpy()
        out[f"r{r}_range"] = pr["rng"].numpy()
        out[f"r{r}_recv_splits"] = pr["cnt"].numpy()
        out[f"r{r}_send_splits"] = np.array([len(x) for x in recv], dtype=np.int64)
        out[f"r{r}_idx_nodes_send_to_others"] = idx.numpy()
        out[f"r{r}_in_degrees"] = pr["indeg"].numpy()
        # remote_adj_t as COO (row = local dst, col = halo slot - n), before canonical sorting
        out[f"r{r}_remote_row"] = pr["rem"][1].numpy()
        out[f"r{r}_remote_col"] = (pr["rem"][0] - pr["n"]).numpy()
    return out


def prepost_plan(DP, begin, parts):
    P = len(parts)
    stage1 = []
    for r in range(P):
        local, remote = parts[r]
        rem = [torch.from_numpy(remote[0].copy()), torch.from_numpy(remote[1].copy()) + int(begin[r])]
        sent, on_recv, begin_from, recv_splits = DP.split_remote_edges_for_aggr_and_graph_exchange(
            torch.from_numpy(begin), rem, P)
        stage1.append(dict(sent=sent, on_recv=on_recv, begin_from=begin_from, recv_splits=recv_splits))
    out = {}
    for r in range(P):
        got = [stage1[q]["sent"][r] for q in range(P)]
        for_send, begin_to, send_splits = DP.split_remote_edges_recv_from_graph_exchange(got, P)
        s1 = stage1[r]
        frm = [s1["on_recv"][0].clone(), s1["on_recv"][1].clone()]
        frm[1] -= int(begin[r])
        n_from = DP.remap_remote_nodes_id(frm[0], s1["begin_from"])
        to = [for_send[0].clone(), for_send[1].clone()]
        to[0] -= int(begin[r])
        n_to = DP.remap_remote_nodes_id(to[1], begin_to)
        out[f"r{r}_recv_splits"] = np.array(s1["recv_splits"], dtype=np.int64)
        out[f"r{r}_send_splits"] = np.array(send_splits, dtype=np.int64)
        out[f"r{r}_from_row"] = frm[1].numpy()   # local destination
        out[f"r{r}_from_col"] = frm[0].numpy()   # wire slot
        out[f"r{r}_n_from"] = np.array(n_from)
        out[f"r{r}_to_row"] = to[1].numpy()      # wire slot
        out[f"r{r}_to_col"] = to[0].numpy()      # local source
        out[f"r{r}_n_to"] = np.array(n_to)
    return out


def save_parts(out, begin, parts):
    out["begin"] = begin
    for r, (local, remote) in enumerate(parts):
        out[f"r{r}_local_edges"] = local
        out[f"r{r}_remote_edges"] = remote


def main():
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("GNNAGG_REFERENCE_ROOT")
    if not ref_root:
        raise SystemExit("usage: python tests/golden/make_golden.py <reference_root>  (or set GNNAGG_REFERENCE_ROOT)")
    ref = install_shims(ref_root)
    from data_manager.DataProcessor import DataProcessor, DataProcessorForPreAggresive

    rng = np.random.default_rng(20261125)
    for name, P, n_per, deg in (("a", 3, 12, 3), ("b", 4, 40, 4), ("c", 2, 64, 6), ("d", 5, 9, 2)):
        begin, parts = random_partitioned_graph(rng, P, n_per, deg)
        o = plain_plan(DataProcessor, begin, parts)
        save_parts(o, begin, parts)
        np.savez_compressed(os.path.join(HERE, f"plan_plain_{name}.npz"), **o)
        o = prepost_plan(DataProcessorForPreAggresive, begin, parts)
        save_parts(o, begin, parts)
        np.savez_compressed(os.path.join(HERE, f"plan_prepost_{name}.npz"), **o)

    # --- compiled x86 quantisers ---------------------------------------------------------
    rows, F = 61, 37
    x = rng.standard_normal((rows, F)).astype(np.float32)
    x[5] = 0.25            # constant row: scale 0 -> 1
    x[6, :] = np.abs(x[6])  # a row with an exact zero minimum
    x[6, 3] = 0.0
    bits = rng.choice([2, 4, 8], size=rows).astype(np.float32)
    import oracle
    r = oracle.quantized_nodes_feat_range(bits.astype(np.int64), F)
    params = torch.zeros(rows, 3)
    params[:, 0] = torch.from_numpy(bits)
    codes = torch.zeros(int(r[-1]), dtype=torch.uint8)
    ref.quantize_tensor_v1(torch.from_numpy(x), codes, torch.from_numpy(r), params)
    deq = torch.zeros(rows, F)
    ref.dequantize_tensor_v1(codes, deq, torch.from_numpy(r), params)
    np.savez_compressed(os.path.join(HERE, "quant_v1.npz"), x=x, bits=bits, range=r, params=params.numpy(),
                        codes=codes.numpy(), deq=deq.numpy())

    o = {"x": x}
    for b in (2, 4, 8):
        mn = x.min(1)
        sc = ((x.max(1) - mn) / np.float32(2 ** b - 1)).astype(np.float32)
        sc[sc == 0] = 1.0
        epb = 8 // b
        c = torch.zeros(((rows + epb - 1) // epb, F), dtype=torch.uint8)
        ref.quantize_tensor(torch.from_numpy(x), c, torch.from_numpy(mn), torch.from_numpy(sc), b)
        d = torch.zeros(rows, F)
        ref.dequantize_tensor(c, d, torch.from_numpy(mn), torch.from_numpy(sc), b)
        o[f"min{b}"], o[f"scale{b}"], o[f"codes{b}"], o[f"deq{b}"] = mn, sc, c.numpy(), d.numpy()
    np.savez_compressed(os.path.join(HERE, "quant_rowpacked.npz"), **o)

    # --- compiled reference spmm (accumulating) ---------------------------------------------
    import scipy.sparse as sp
    A = sp.random(300, 211, density=0.03, format="csr", dtype=np.float32, random_state=7)
    A.sort_indices()
    X = rng.standard_normal((211, 47)).astype(np.float32)
    out0 = rng.standard_normal((300, 47)).astype(np.float32)
    out = torch.from_numpy(out0.copy())
    T = 4
    splits = oracle.distribute_work_for_row(A.indptr, np.ones_like(A.data), T)
    torch.set_num_threads(T)
    ref.spmm(torch.from_numpy(A.indptr.astype(np.int64)), torch.from_numpy(A.indices.astype(np.int64)),
             torch.from_numpy(A.data), torch.from_numpy(X), out, 300, torch.from_numpy(splits),
             torch.tensor([0, 47], dtype=torch.int32))
    np.savez_compressed(os.path.join(HERE, "spmm_ref.npz"), rowptr=A.indptr.astype(np.int64),
                        col=A.indices.astype(np.int64), val=A.data, X=X, out0=out0, out=out.numpy())

    # --- literal vectors of the reference's unit tests (tests/test_quantizer.py:57-84,
    #     tests/test_data_preprocessor.py:15-30), for the record ---------------------------------
    vec = {
        "quantizer_v1": {
            "source": "tests/test_quantizer.py:57-84",
            "data": [[0.2, 0.1, 0.3], [0.4, 0.5, 0.6], [0.7, 0.8, 0.9], [1.0, 1.1, 1.2], [0.3, 0.1, 0.7]],
            "bits": [8, 4, 2, 4, 4],
            "codes": [127, 0, 255, 7, 240, 44, 8, 240, 80, 240],
            "range": [0, 3, 5, 6, 8, 10],
        },
        "feat_range": {
            "source": "tests/test_quantizer.py:29-55",
            "cases": [[6, 4, [8, 4, 2, 8, 4, 2], [0, 4, 6, 7, 11, 13, 14]], [3, 1, [2, 2, 2], [0, 1, 2, 3]],
                      [3, 3, [4, 4, 2], [0, 2, 4, 5]]],
        },
    }
    with open(os.path.join(HERE, "ref_test_vectors.json"), "w") as f:
        json.dump(vec, f, indent=1)
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    main()
