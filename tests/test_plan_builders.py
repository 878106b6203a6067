"""Communication-plan parity (bit-exact): the vectorised builders of
gnn_benchmark_b200.data_manager against (a) the literal cases of the reference's unit tests
(tests/test_data_preprocessor.py, tests/test_data_preprocessor_pre_aggr.py) and (b) golden plans
produced by running the reference's per-edge-loop builders (tests/golden/make_golden.py)."""
import glob
import os

import numpy as np
import pytest
import torch

from gnn_benchmark_b200.data_manager import DataProcessor, DataProcessorForPreAggresive

T = torch.tensor
DP = DataProcessor
DPP = DataProcessorForPreAggresive


# ---- reference tests/test_data_preprocessor.py ------------------------------------------------
def test_sort_remote_edges_list_based_on_remote_nodes():
    out = DP.sort_remote_edges_list_based_on_remote_nodes(T([[3, 2, 1, 4, 0, 0], [6, 5, 8, 7, 9, 10]]))
    assert torch.equal(out, T([[0, 0, 1, 2, 3, 4], [9, 10, 8, 5, 6, 7]]))


def test_obtain_remote_nodes_list():
    edges = T([[2, 5, 5, 4, 4, 4, 1], [6, 5, 7, 8, 9, 10, 8]])
    edges = DP.sort_remote_edges_list_based_on_remote_nodes(edges)
    nodes, rng, cnt = DP.obtain_remote_nodes_list(edges, 2, T([0, 3, 6, 9]), 3)
    assert torch.equal(edges, T([[2, 3, 4, 4, 4, 5, 5], [8, 6, 8, 9, 10, 5, 7]]))
    assert torch.equal(nodes, T([1, 2, 4, 5]))
    assert torch.equal(rng, T([0, 2, 4, 4]))
    assert torch.equal(cnt, T([2, 2, 0]))


def test_transform_edge_index_to_sparse_tensor():
    local = [T([1, 2, 3]), T([2, 3, 4])]
    remote = [T([7, 7, 7]), T([2, 0, 1])]
    la, ra = DP.transform_edge_index_to_sparse_tensor(local, remote, 5, 3)
    el = torch.zeros(5, 5)
    el[[2, 3, 4], [1, 2, 3]] = 1
    er = torch.zeros(5, 3)
    er[[2, 0, 1], [2, 2, 2]] = 1
    assert torch.equal(la.to_dense(), el) and torch.equal(ra.to_dense(), er)

    local = T([[0, 1, 1], [0, 0, 1]])
    remote = T([[2, 5, 5, 4, 4, 4, 2], [0, 0, 0, 1, 0, 1, 0]])
    remote = DP.sort_remote_edges_list_based_on_remote_nodes(remote)
    DP.obtain_remote_nodes_list(remote, 2, T([0, 3, 6, 9]), 3)
    assert torch.equal(remote[0], T([2, 2, 3, 3, 3, 4, 4]))
    assert sorted(zip(remote[0].tolist(), remote[1].tolist())) == sorted(
        zip([2, 2, 3, 3, 3, 4, 4], [0, 0, 1, 0, 1, 0, 0]))
    la, ra = DP.transform_edge_index_to_sparse_tensor(local, remote, 2, 3)
    assert torch.equal(la.to_dense(), T([[1., 1.], [0., 1.]]))
    # duplicated edges stay duplicated: (row 0, col 0) and (row 0, col 2) occur twice
    assert torch.equal(ra.to_dense(), T([[2., 1., 2.], [0., 2., 0.]]))


def test_get_in_degrees():
    d = DP.get_in_degrees([T([1, 2, 3]), T([0, 0, 1])], [T([2, 3, 4]), T([2, 3, 3])], 5)
    assert torch.equal(d, T([[2.], [1.], [1.], [2.], [1.]]))


# ---- reference tests/test_data_preprocessor_pre_aggr.py ---------------------------------------
def test_get_degrees():
    assert DPP.get_degrees(T([], dtype=torch.int64)) == {}
    assert DPP.get_degrees(T([1])) == {1: 1}
    assert DPP.get_degrees(T([1, 2, 3, 2, 1, 3, 3])) == {1: 2, 2: 2, 3: 3}
    nodes = torch.randint(0, 100, (10000,), generator=torch.Generator().manual_seed(0))
    assert DPP.get_degrees(nodes) == {v: nodes.tolist().count(v) for v in torch.unique(nodes).tolist()}


def test_decide_pre_or_post_aggr():
    pre, post = 1, 0
    assert torch.equal(DPP.decide_pre_or_post_aggr(T([1, 3, 1, 1]), T([2, 1, 2, 3]), pre, post),
                       T([post, pre, post, post]))
    assert torch.equal(DPP.decide_pre_or_post_aggr(T([2, 1, 2, 1, 0]), T([1, 4, 1, 1, 1]), pre, post),
                       T([pre, post, pre, pre, pre]))
    e = T([], dtype=torch.int64)
    assert torch.equal(DPP.decide_pre_or_post_aggr(e, e, pre, post), e)
    assert torch.equal(DPP.decide_pre_or_post_aggr(T([0, 2, 2, 2, 4, 4, 5, 5]), T([1, 1, 2, 4, 4, 3, 6, 3]), pre, post),
                       T([pre, post, post, post, pre, pre, post, pre]))


@pytest.mark.parametrize("src,dst,pre,post,exp_src,exp_dst", [
    ([0, 2, 2, 2, 4, 4, 5, 5], [1, 1, 2, 4, 4, 3, 6, 3], [0, 4, 5, 7], [1, 2, 3, 6],
     [0, 2, 4, 5, 4, 5], [1, 2, 3, 3, 4, 5]),
    ([0, 2, 2, 2, 4, 4, 5, 5], [1, 1, 2, 4, 4, 3, 6, 3], [0, 1, 2, 3, 4, 5, 6, 7], [],
     [0, 2, 2, 4, 5, 2, 4, 5], [1, 1, 2, 3, 3, 4, 4, 6]),
    ([0, 2, 9, 3, 4, 1, 5, 3], [1, 1, 2, 4, 4, 3, 6, 3], [], [0, 1, 2, 3, 4, 5, 6, 7],
     [0, 1, 2, 3, 4, 5, 9], [0, 1, 2, 3, 4, 5, 9]),
])
def test_collect_edges_sent_to_other_subgraphs(src, dst, pre, post, exp_src, exp_dst):
    out = []
    DPP.collect_edges_sent_to_other_subgraphs(T(src), T(dst), T(pre, dtype=torch.int64), T(post, dtype=torch.int64), out)
    half = out[0].numel() // 2
    assert out[0][:half].tolist() == exp_src and out[0][half:].tolist() == exp_dst


@pytest.mark.parametrize("dst,pre,post,exp_src,exp_dst,exp_split,exp_begin", [
    ([0, 2, 2, 2, 4, 4, 5, 5], [1, 2, 3, 6], [0, 4, 5, 7], [1, 2, 3, 3, 4, 5], [0, 2, 4, 5, 4, 5], [5], [0, 6]),
    ([0, 2, 2, 2, 4, 4, 5, 5], [], [0, 1, 2, 3, 4, 5, 6, 7], [1, 1, 2, 3, 3, 4, 4, 6], [0, 2, 2, 4, 5, 2, 4, 5],
     [5], [0, 8]),
    ([0, 2, 9, 3, 4, 1, 5, 3], [0, 1, 2, 3, 4, 5, 6, 7], [], [0, 1, 2, 3, 4, 5, 9], [0, 1, 2, 3, 4, 5, 9], [7],
     [0, 7]),
])
def test_collect_edges_for_aggregation(dst, pre, post, exp_src, exp_dst, exp_split, exp_begin):
    src = T([1, 1, 2, 4, 4, 3, 6, 3])
    lists = [T([], dtype=torch.int64), T([], dtype=torch.int64)]
    splits, begin = [], torch.zeros(2, dtype=torch.int64)
    DPP.collect_edges_for_aggregation(src, T(dst), T(pre, dtype=torch.int64), T(post, dtype=torch.int64), lists,
                                      splits, begin, 0)
    assert lists[0].tolist() == exp_src and lists[1].tolist() == exp_dst
    assert splits == exp_split and begin.tolist() == exp_begin


def test_split_remote_edges_for_aggr_and_graph_exchange():
    begin = T([0, 2, 5, 10, 14])
    edges = [T([8, 9, 3, 6, 6, 7, 1, 0, 3, 5]), T([9, 7, 10, 8, 4, 7, 10, 10, 8, 11])]
    sent, on_recv, begin_from, recv_splits = DPP.split_remote_edges_for_aggr_and_graph_exchange(begin, edges, 4)
    expect_sent = [[1, 0, 10, 10], [3, 3], [6, 9, 7, 8, 5, 6, 7, 7, 9, 11], []]
    assert [s.tolist() for s in sent] == expect_sent
    assert on_recv[0].tolist() == [10, 3, 3, 6, 6, 7, 9, 11]
    assert on_recv[1].tolist() == [10, 10, 8, 8, 4, 7, 9, 11]
    assert begin_from.tolist() == [0, 1, 3, 8, 8]
    assert recv_splits == [1, 1, 4, 0]


@pytest.mark.parametrize("got,exp0,exp1,exp_begin,exp_splits", [
    ([[], [1, 2, 3, 4], [7, 8, 9, 10, 11, 12]], [1, 2, 7, 8, 9], [3, 4, 10, 11, 12], [0, 0, 2, 5], [0, 2, 3]),
    ([[2, 2, 3, 4], [], [7, 8, 9, 9]], [2, 2, 7, 8], [3, 4, 9, 9], [0, 2, 2, 4], [2, 0, 1]),
    ([[], []], [], [], [0, 0, 0], [0, 0]),
])
def test_split_remote_edges_recv_from_graph_exchange(got, exp0, exp1, exp_begin, exp_splits):
    lists, begin_to, splits = DPP.split_remote_edges_recv_from_graph_exchange(
        [T(g, dtype=torch.int64) for g in got], len(got))
    assert lists[0].tolist() == exp0 and lists[1].tolist() == exp1
    assert begin_to.tolist() == exp_begin and splits == exp_splits


@pytest.mark.parametrize("keys,begin,count,remapped", [
    ([0, 0, 1, 1, 2, 2, 3, 3], [0, 2, 4, 6, 8], 4, [0, 0, 1, 1, 2, 2, 3, 3]),
    ([0, 0, 1, 1, 2, 2, 3, 3, 4, 4], [0, 2, 4, 6, 8, 10], 5, [0, 0, 1, 1, 2, 2, 3, 3, 4, 4]),
    ([0, 0, 0, 1, 1, 2, 2, 3, 3, 3], [0, 3, 5, 7, 10], 4, [0, 0, 0, 1, 1, 2, 2, 3, 3, 3]),
    ([0, 1, 2, 3, 4, 5], [0, 1, 2, 3, 4, 5, 6], 6, [0, 1, 2, 3, 4, 5]),
    ([0, 0, 0, 0, 0], [0, 5], 1, [0, 0, 0, 0, 0]),
    ([0, 0, 2, 2, 4, 5, 10, 11, 11, 12], [0, 2, 4, 6, 9, 10], 7, [0, 0, 1, 1, 2, 3, 4, 5, 5, 6]),
    ([0, 0, 2, 2, 4, 5, 10, 11, 13, 13], [0, 0, 2, 4, 6, 8, 10], 7, [0, 0, 1, 1, 2, 3, 4, 5, 6, 6]),
    ([3, 3, 4, 7, 7, 9], [0, 0, 2, 3, 5, 6], 4, [0, 0, 1, 2, 2, 3]),
    # same key on both sides of a peer boundary: a new slot starts at the boundary
    ([5, 5, 5, 5], [0, 2, 4], 2, [0, 0, 1, 1]),
    ([], [0, 0], 0, []),
])
def test_remap_remote_nodes_id(keys, begin, count, remapped):
    k = T(keys, dtype=torch.int64)
    assert DPP.remap_remote_nodes_id(k, T(begin, dtype=torch.int64)) == count
    assert k.tolist() == remapped


# ---- golden plans from the reference's own builders ----------------------------------------------
def _coo_sorted(row, col, ncol):
    key = np.asarray(row, dtype=np.int64) * max(int(ncol), 1) + np.asarray(col, dtype=np.int64)
    return np.sort(key)


def _csr_as_keys(sp):
    rowptr, col, _ = sp.csr()
    rows = np.repeat(np.arange(sp.sparse_size(0)), np.diff(rowptr.numpy()))
    return rows * max(sp.sparse_size(1), 1) + col.numpy().astype(np.int64)


GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLD, "plan_plain_*.npz"))))
def test_plain_plan_against_reference_golden(path):
    g = np.load(path)
    begin = torch.from_numpy(g["begin"])
    P = len(begin) - 1
    stage = []
    for r in range(P):
        n = int(begin[r + 1] - begin[r])
        local = torch.from_numpy(g[f"r{r}_local_edges"])
        remote = torch.from_numpy(g[f"r{r}_remote_edges"].copy())
        rem = [remote[0].clone(), remote[1].clone()]
        indeg = DP.get_in_degrees([local[0], local[1]], rem, n)
        rem = DP.sort_remote_edges_list_based_on_remote_nodes(rem)
        nodes, rng, cnt = DP.obtain_remote_nodes_list(rem, n, begin, P)
        stage.append((n, rem, nodes, rng, cnt, indeg, local))
    for r in range(P):
        n, rem, nodes, rng, cnt, indeg, local = stage[r]
        np.testing.assert_array_equal(nodes.numpy(), g[f"r{r}_remote_nodes_list"])
        np.testing.assert_array_equal(rng.numpy(), g[f"r{r}_range"])
        np.testing.assert_array_equal(cnt.numpy(), g[f"r{r}_recv_splits"])
        np.testing.assert_array_equal(indeg.numpy(), g[f"r{r}_in_degrees"])
        recv = [stage[q][2][stage[q][3][r]: stage[q][3][r + 1]] for q in range(P)]
        idx = torch.cat(recv) - int(begin[r])
        np.testing.assert_array_equal(idx.numpy(), g[f"r{r}_idx_nodes_send_to_others"])
        np.testing.assert_array_equal(np.array([len(x) for x in recv]), g[f"r{r}_send_splits"])
        la, ra = DP.transform_edge_index_to_sparse_tensor([local[0], local[1]], rem, n, nodes.numel())
        np.testing.assert_array_equal(_csr_as_keys(ra),
                                      _coo_sorted(g[f"r{r}_remote_row"], g[f"r{r}_remote_col"], nodes.numel()))
        assert la.nnz() == local.shape[1]


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLD, "plan_prepost_*.npz"))))
def test_prepost_plan_against_reference_golden(path):
    g = np.load(path)
    begin = torch.from_numpy(g["begin"])
    P = len(begin) - 1
    s1 = []
    for r in range(P):
        remote = torch.from_numpy(g[f"r{r}_remote_edges"].copy())
        rem = [remote[0].clone(), remote[1].clone() + int(begin[r])]
        s1.append(DPP.split_remote_edges_for_aggr_and_graph_exchange(begin, rem, P))
    for r in range(P):
        n = int(begin[r + 1] - begin[r])
        sent, on_recv, begin_from, recv_splits = s1[r]
        got = [s1[q][0][r] for q in range(P)]
        for_send, begin_to, send_splits = DPP.split_remote_edges_recv_from_graph_exchange(got, P)
        local = torch.from_numpy(g[f"r{r}_local_edges"])
        la, a_from, a_to = DPP.transform_edge_index_to_sparse_tensor(
            [local[0], local[1]], [on_recv[0].clone(), on_recv[1].clone()], [for_send[0].clone(), for_send[1].clone()],
            begin_from, begin_to, n, int(begin[r]))
        assert recv_splits == g[f"r{r}_recv_splits"].tolist()
        assert send_splits == g[f"r{r}_send_splits"].tolist()
        assert a_from.sparse_sizes() == (n, int(g[f"r{r}_n_from"]))
        assert a_to.sparse_sizes() == (int(g[f"r{r}_n_to"]), n)
        np.testing.assert_array_equal(_csr_as_keys(a_from),
                                      _coo_sorted(g[f"r{r}_from_row"], g[f"r{r}_from_col"], int(g[f"r{r}_n_from"])))
        np.testing.assert_array_equal(_csr_as_keys(a_to), _coo_sorted(g[f"r{r}_to_row"], g[f"r{r}_to_col"], n))
        # slot counts and splits are consistent
        assert sum(recv_splits) == int(g[f"r{r}_n_from"]) and sum(send_splits) == int(g[f"r{r}_n_to"])
