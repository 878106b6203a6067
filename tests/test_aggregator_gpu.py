"""Aggregator parity on one GPU: P ranks run as threads over an in-process exchange
(tests/fake_dist.py).  Checked against (a) the product of the GLOBAL adjacency (plans + kernels +
exchange together) and (b) the reference's order of operations restated with the CPU oracle on the
same per-rank matrices: zeros -> local SpMM -> [quantise -> bf16 params -> dequantise] -> remote
SpMM, which the CUDA path reproduces bit for bit at F >= 128 (one nonzero per warp instruction)."""
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import oracle
from fake_dist import FakeWorld

pytestmark = pytest.mark.gpu


def make_graph(seed, P, n_per, deg):
    """Directed multigraph over P contiguous blocks, with hubs; returns begin, global (src, dst)."""
    rng = np.random.default_rng(seed)
    sizes = rng.integers(max(1, n_per // 2), n_per + 1, size=P)
    begin = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64)
    N = int(begin[-1])
    E = N * deg
    src = rng.integers(0, N, size=E)
    dst = rng.integers(0, N, size=E)
    hubs = rng.integers(0, N, size=max(2, N // 50))
    src[: E // 5] = rng.choice(hubs, size=E // 5)
    dst[E // 5: 2 * E // 5] = rng.choice(hubs, size=2 * E // 5 - E // 5)
    src = np.concatenate([src, src[: E // 20]])  # duplicated edges stay duplicated
    dst = np.concatenate([dst, dst[: E // 20]])
    return begin, src.astype(np.int64), dst.astype(np.int64)


def global_csr(src, dst, N, transpose=False):
    r, c = (src, dst) if transpose else (dst, src)
    order = np.lexsort((c, r))
    r, c = r[order], c[order]
    rowptr = np.concatenate([[0], np.cumsum(np.bincount(r, minlength=N))]).astype(np.int64)
    return rowptr, c.astype(np.int64), np.ones(len(c), np.float32)


def csr_np(sp):
    rp, c, v = sp.csr()
    return rp.cpu().numpy(), c.cpu().numpy().astype(np.int64), v.cpu().numpy()


def csc_np(sp):
    return (sp.storage.colptr().cpu().numpy(), sp.storage.row_T().cpu().numpy().astype(np.int64),
            sp.storage.value_T().cpu().numpy())


def close(got, want, scale, rtol=1e-5):
    err = np.abs(got.astype(np.float64) - want.astype(np.float64))
    assert (err <= rtol * scale + 1e-30).all(), f"worst ratio {np.max(err / (scale + 1e-30)):.3e}"


@pytest.mark.parametrize("P,num_bits,is_pre,F", [
    (1, 32, False, 128), (2, 32, False, 128), (4, 32, False, 64), (3, 32, True, 128), (4, 32, True, 32),
    (2, 2, False, 128), (4, 2, False, 256), (3, 2, True, 128), (4, 16, False, 128), (3, 8, False, 100),
    (2, 4, True, 64),
])
@pytest.mark.parametrize("fuse", [False, True], ids=["unpack_then_spmm", "fused_unpack"])
def test_aggregator_forward_backward(cuda_lib, monkeypatch, fuse, P, num_bits, is_pre, F):
    from gnn_benchmark_b200 import Communicator, Quantizer_for_all_procs, TimeRecorder, graphgen
    from gnn_benchmark_b200.aggregator import Aggregator
    from gnn_benchmark_b200.data_manager.DataLoader import build_graph

    begin_np, src, dst = make_graph(100 * P + F + num_bits, P, 700, 6)
    N = int(begin_np[-1])
    begin = torch.from_numpy(begin_np)
    rng = np.random.default_rng(1)
    X = rng.standard_normal((N, F)).astype(np.float32)
    G = rng.standard_normal((N, F)).astype(np.float32)
    s_t, d_t = torch.from_numpy(src).cuda(), torch.from_numpy(dst).cuda()

    import gnn_benchmark_b200.aggregator as agg_mod
    monkeypatch.setattr(agg_mod, "FUSE_UNPACK", fuse)
    monkeypatch.setattr(agg_mod, "FUSE_UNPACK_MIN_WIDTH", 0)  # the fused forward at every width
    Communicator(num_bits, is_async=True)
    Quantizer_for_all_procs(P, num_bits)
    TimeRecorder(1, 1, enabled=False)
    world = FakeWorld(P)

    def rank_fn(rank):
        local, remote = graphgen.partition_edges(s_t, d_t, begin, rank)
        graph = build_graph(local, remote, begin, rank, P, F, num_bits, is_pre, device="cuda")
        b0, b1 = int(begin[rank]), int(begin[rank + 1])
        x = torch.from_numpy(X[b0:b1]).cuda()
        g = torch.from_numpy(G[b0:b1]).cuda()
        ctx = SimpleNamespace()
        out = Aggregator.forward(ctx, graph, x, 0, num_bits, is_pre, True)
        snap = {}
        if P > 1:
            snap["recv_fwd"] = graph.comm_buf.recv_buf.clone()
            if num_bits in (2, 4, 8):
                q = graph.comm_buf_for_quantization
                snap["codes_fwd"] = q.quantized_send_data_buf.clone()
                snap["params_fwd"] = q.quantized_send_params_buf_fp32.clone()
        grad = Aggregator.backward(ctx, g)[1]
        torch.cuda.current_stream().synchronize()
        return graph, out.cpu().numpy(), grad.cpu().numpy(), {k: v.cpu().numpy() for k, v in snap.items()}

    res = world.run(rank_fn)

    # (a) against the global adjacency
    rp, c, v = global_csr(src, dst, N)
    want_out = oracle.spmm(rp, c, v, X)
    scale_out = oracle.spmm(rp, c, v, np.abs(X))
    rpt, ct, vt = global_csr(src, dst, N, transpose=True)
    want_grad = oracle.spmm(rpt, ct, vt, G)
    scale_grad = oracle.spmm(rpt, ct, vt, np.abs(G))
    exact_halo = num_bits == 32
    for r in range(P):
        b0, b1 = int(begin[r]), int(begin[r + 1])
        _, out, grad, _ = res[r]
        if exact_halo:
            close(out, want_out[b0:b1], scale_out[b0:b1])
            close(grad, want_grad[b0:b1], scale_grad[b0:b1])
        else:
            # lossy halo: bounded by the quantisation step of the rows that crossed (loose sanity bound)
            tol = {16: 2e-2, 8: 5e-2, 4: 0.5, 2: 2.5}[num_bits]
            assert np.abs(out - want_out[b0:b1]).max() <= tol * max(1.0, scale_out[b0:b1].max())
            assert np.abs(grad - want_grad[b0:b1]).max() <= tol * max(1.0, scale_grad[b0:b1].max())

    # (b) the reference's sequence of operations, restated with the oracle on the same plan
    if P > 1 and not is_pre and num_bits in (32, 2):
        for r in range(P):
            graph, out, grad, snap = res[r]
            b0, b1 = int(begin[r]), int(begin[r + 1])
            # what every peer sends to r, in peer order
            recv_rows = []
            for qk in range(P):
                gq = res[qk][0]
                idx = gq.idx_nodes_send_to_others.cpu().numpy()
                offs = np.concatenate([[0], np.cumsum(gq.comm_splits.send_splits)])
                sel = idx[offs[r]:offs[r + 1]]
                qb0 = int(begin[qk])
                rows = X[qb0 + sel]
                if num_bits == 2:
                    # peer qk quantises ALL its send rows in one call; r receives its segment
                    allrows = X[qb0 + idx]
                    codes, params = oracle.quantize_int2_for_all_procs(allrows, offs.astype(np.int32))
                    np.testing.assert_array_equal(res[qk][3]["codes_fwd"], codes)
                    np.testing.assert_array_equal(res[qk][3]["params_fwd"], params)
                    deq = oracle.dequantize_int2_for_all_procs(codes, offs.astype(np.int32), oracle.bf16_round(params))
                    rows = deq[offs[r]:offs[r + 1]]
                recv_rows.append(rows)
            recv = np.concatenate(recv_rows) if recv_rows else np.zeros((0, F), np.float32)
            if not (fuse and num_bits == 2):
                np.testing.assert_array_equal(snap["recv_fwd"], recv)
            want = oracle.spmm(*csr_np(graph.local_adj_t), X[b0:b1])
            if recv.shape[0]:
                want = oracle.spmm(*csr_np(graph.remote_adj_t), recv, want)
            if F >= 128:
                np.testing.assert_array_equal(out, want)  # same FMA chain, same order
            else:
                close(out, want, scale_out[b0:b1])


def test_single_rank_autograd(cuda_lib):
    """world_size 1 through torch.autograd: forward A x, backward A^T g, no exchange."""
    from gnn_benchmark_b200 import Aggregator, Communicator, Quantizer_for_all_procs, TimeRecorder, graphgen
    from gnn_benchmark_b200.data_manager.DataLoader import build_graph

    begin_np, src, dst = make_graph(5, 1, 900, 5)
    N, F = int(begin_np[-1]), 128
    begin = torch.from_numpy(begin_np)
    Communicator(32)
    Quantizer_for_all_procs(1, 32)
    TimeRecorder(2, 1, enabled=True)
    local, remote = graphgen.partition_edges(torch.from_numpy(src).cuda(), torch.from_numpy(dst).cuda(), begin, 0)
    assert remote.shape[1] == 0
    graph = build_graph(local, remote, begin, 0, 1, F, 32, False, device="cuda")
    rng = np.random.default_rng(0)
    X = rng.standard_normal((N, F)).astype(np.float32)
    G = rng.standard_normal((N, F)).astype(np.float32)
    x = torch.from_numpy(X).cuda().requires_grad_()
    out = Aggregator.apply(graph, x, 0, 32, False, True)
    out.backward(torch.from_numpy(G).cuda())
    rp, c, v = global_csr(src, dst, N)
    np.testing.assert_array_equal(out.detach().cpu().numpy(), oracle.spmm(rp, c, v, X))
    rpt, ct, vt = global_csr(src, dst, N, transpose=True)
    np.testing.assert_array_equal(x.grad.cpu().numpy(), oracle.spmm(rpt, ct, vt, G))
    assert TimeRecorder.ctx.get_total_local_aggregate_time() > 0


@pytest.mark.parametrize("P,F", [(2, 128), (3, 64), (4, 256), (5, 32)])
def test_peer_pipelined_exchange(cuda_lib, monkeypatch, P, F):
    """Communicator(pipeline_peers=True): the fp32 halo moves peer by peer and each peer's rows are
    aggregated on arrival.  Same terms as the one-shot exchange, added in arrival order: results agree
    with the one-shot path within fp32 re-association, and with the global product within 1e-5."""
    from gnn_benchmark_b200 import Communicator, Quantizer_for_all_procs, TimeRecorder, graphgen
    from gnn_benchmark_b200.aggregator import Aggregator
    from gnn_benchmark_b200.data_manager.DataLoader import build_graph

    begin_np, src, dst = make_graph(7 * P + F, P, 600, 6)
    N = int(begin_np[-1])
    begin = torch.from_numpy(begin_np)
    rng = np.random.default_rng(2)
    X = rng.standard_normal((N, F)).astype(np.float32)
    G = rng.standard_normal((N, F)).astype(np.float32)
    s_t, d_t = torch.from_numpy(src).cuda(), torch.from_numpy(dst).cuda()
    Quantizer_for_all_procs(P, 32)
    TimeRecorder(1, 1)
    results = {}
    for pipelined in (False, True):
        Communicator(32, is_async=True, pipeline_peers=pipelined)

        def rank_fn(rank):
            local, remote = graphgen.partition_edges(s_t, d_t, begin, rank)
            graph = build_graph(local, remote, begin, rank, P, F, 32, False, device="cuda")
            b0, b1 = int(begin[rank]), int(begin[rank + 1])
            ctx = SimpleNamespace()
            out = Aggregator.forward(ctx, graph, torch.from_numpy(X[b0:b1]).cuda(), 0, 32, False, True)
            grad = Aggregator.backward(ctx, torch.from_numpy(G[b0:b1]).cuda())[1]
            return out.cpu().numpy(), grad.cpu().numpy()

        results[pipelined] = FakeWorld(P).run(rank_fn)
    rp, c, v = global_csr(src, dst, N)
    want_out, scale_out = oracle.spmm(rp, c, v, X), oracle.spmm(rp, c, v, np.abs(X))
    rpt, ct, vt = global_csr(src, dst, N, transpose=True)
    want_grad, scale_grad = oracle.spmm(rpt, ct, vt, G), oracle.spmm(rpt, ct, vt, np.abs(G))
    for r in range(P):
        b0, b1 = int(begin[r]), int(begin[r + 1])
        out, grad = results[True][r]
        close(out, want_out[b0:b1], scale_out[b0:b1])
        close(grad, want_grad[b0:b1], scale_grad[b0:b1])
        close(out, results[False][r][0], scale_out[b0:b1])
        close(grad, results[False][r][1], scale_grad[b0:b1])
        # the backward halo blocks are the same numbers whichever way they travel
        np.testing.assert_array_equal(grad.shape, results[False][r][1].shape)


@pytest.mark.parametrize("P,bits,is_pre", [(1, 32, False), (3, 32, False), (2, 2, False), (3, 32, True), (2, 2, True)])
def test_padded_feature_rows_give_identical_results(cuda_lib, P, bits, is_pre):
    """Features kept in rows padded to 128 floats (row stride > F) go through the path without a copy
    and give bit-identical outputs and gradients."""
    from gnn_benchmark_b200 import Communicator, Quantizer_for_all_procs, TimeRecorder, graphgen
    from gnn_benchmark_b200.aggregator import Aggregator
    from gnn_benchmark_b200.data_manager.DataLoader import build_graph

    F = 100
    begin_np, src, dst = make_graph(31 * P + bits, P, 500, 6)
    N = int(begin_np[-1])
    begin = torch.from_numpy(begin_np)
    rng = np.random.default_rng(4)
    X = rng.standard_normal((N, F)).astype(np.float32)
    G = rng.standard_normal((N, F)).astype(np.float32)
    s_t, d_t = torch.from_numpy(src).cuda(), torch.from_numpy(dst).cuda()
    Quantizer_for_all_procs(P, bits)
    TimeRecorder(1, 1)
    Communicator(bits, is_async=True)
    results = {}
    for padded in (False, True):
        def rank_fn(rank):
            local, remote = graphgen.partition_edges(s_t, d_t, begin, rank)
            graph = build_graph(local, remote, begin, rank, P, F, bits, is_pre, device="cuda")
            b0, b1 = int(begin[rank]), int(begin[rank + 1])
            x = torch.from_numpy(X[b0:b1]).cuda()
            if padded:
                store = torch.full((b1 - b0, 128), float("nan"), device="cuda")
                store[:, :F] = x
                x = store[:, :F]
                assert x.stride(0) == 128
            ctx = SimpleNamespace()
            out = Aggregator.forward(ctx, graph, x, 0, bits, is_pre, True)
            grad = Aggregator.backward(ctx, torch.from_numpy(G[b0:b1]).cuda())[1]
            return out.cpu().numpy(), grad.cpu().numpy()

        results[padded] = FakeWorld(P).run(rank_fn)
    for r in range(P):
        np.testing.assert_array_equal(results[True][r][0], results[False][r][0])
        np.testing.assert_array_equal(results[True][r][1], results[False][r][1])


@pytest.mark.parametrize("P,F,bits,is_pre", [(2, 128, 2, False), (4, 256, 2, False), (3, 96, 8, False),
                                             (3, 128, 2, True), (4, 256, 2, True)])
def test_lean_halo_buffers_give_identical_results(cuda_lib, monkeypatch, P, F, bits, is_pre):
    """lean_halo=True: the fp32 staging buffers of the exchange have no memory (meta tensors).  Forward
    goes gather+pack (plain path) or pre-aggregation SpMM with the packing epilogue (pre/post path) ->
    exchange -> fused unpack SpMM; backward packs the halo gradients in the epilogue of the transposed
    receive-side SpMM.  Outputs, gradients and the codes on the wire are bit-identical to the path that
    stages everything in fp32 (SpMM into the fp32 buffer, then quantise + pack)."""
    import gnn_benchmark_b200.aggregator as agg_mod

    from gnn_benchmark_b200 import Communicator, Quantizer_for_all_procs, TimeRecorder, graphgen
    from gnn_benchmark_b200.aggregator import Aggregator
    from gnn_benchmark_b200.data_manager.DataLoader import build_graph

    begin_np, src, dst = make_graph(31 * P + F, P, 500, 6)
    N = int(begin_np[-1])
    begin = torch.from_numpy(begin_np)
    rng = np.random.default_rng(3)
    X = rng.standard_normal((N, F)).astype(np.float32)
    G = rng.standard_normal((N, F)).astype(np.float32)
    s_t, d_t = torch.from_numpy(src).cuda(), torch.from_numpy(dst).cuda()
    Communicator(bits, is_async=True)
    Quantizer_for_all_procs(P, bits)
    TimeRecorder(1, 1)
    results = {}
    for lean in (False, True):
        monkeypatch.setattr(agg_mod, "FUSE_PACK", "lean")  # staged run: SpMM into the fp32 buffer, then pack

        def rank_fn(rank):
            local, remote = graphgen.partition_edges(s_t, d_t, begin, rank)
            graph = build_graph(local, remote, begin, rank, P, F, bits, is_pre, device="cuda", lean_halo=lean)
            assert graph.comm_buf.send_buf.is_meta == lean and graph.comm_buf.recv_buf.is_meta == lean
            b0, b1 = int(begin[rank]), int(begin[rank + 1])
            ctx = SimpleNamespace()
            out = Aggregator.forward(ctx, graph, torch.from_numpy(X[b0:b1]).cuda(), 0, bits, is_pre, True)
            grad = Aggregator.backward(ctx, torch.from_numpy(G[b0:b1]).cuda())[1]
            q = graph.comm_buf_for_quantization
            return (out.cpu().numpy(), grad.cpu().numpy(), q.quantized_recv_data_buf.cpu().numpy(),
                    q.quantized_recv_params_buf_fp32.cpu().numpy())

        results[lean] = FakeWorld(P).run(rank_fn)
    for r in range(P):
        for a, b in zip(results[False][r], results[True][r]):
            np.testing.assert_array_equal(a, b)


@pytest.mark.parametrize("bits", [2, 8])
def test_config3_downscaled_codes_bit_exact(cuda_lib, monkeypatch, bits):
    """BASELINE configuration 3, down-scaled: R-MAT scale 16 (edge factor 16, symmetrised, randomly
    relabelled), 8 contiguous partitions, F = 256.  The codes and parameters every rank puts on the wire
    -- 2-bit (the reference's live layout, 4 rows per byte) and 8-bit (its generic row-packed layout) --
    are compared byte for byte with the CPU oracle, and the fp32 / quantised aggregation results with the
    global product."""
    import gnn_benchmark_b200.aggregator as agg_mod
    from gnn_benchmark_b200 import Communicator, Quantizer_for_all_procs, TimeRecorder, graphgen
    from gnn_benchmark_b200.aggregator import Aggregator
    from gnn_benchmark_b200.data_manager.DataLoader import build_graph

    monkeypatch.setattr(agg_mod, "FUSE_UNPACK", True)
    monkeypatch.setattr(agg_mod, "FUSE_UNPACK_MIN_WIDTH", 0)
    P, F, scale = 8, 256, 16
    n = 1 << scale
    s_t, d_t = graphgen.rmat_edges(scale, 16, seed=20261128, device="cuda")
    s_t, d_t = graphgen.symmetrize(s_t, d_t, n, self_loops=True)
    s_t, d_t = graphgen.relabel(s_t, d_t, n, seed=20261129)
    begin = graphgen.contiguous_partitions(n, P)
    rng = np.random.default_rng(bits)
    X = rng.standard_normal((n, F)).astype(np.float32)
    Communicator(bits, is_async=True)
    Quantizer_for_all_procs(P, bits)
    TimeRecorder(1, 1)

    def rank_fn(rank):
        local, remote = graphgen.partition_edges(s_t, d_t, begin, rank)
        graph = build_graph(local, remote, begin, rank, P, F, bits, False, device="cuda")
        b0, b1 = int(begin[rank]), int(begin[rank + 1])
        ctx = SimpleNamespace()
        out = Aggregator.forward(ctx, graph, torch.from_numpy(X[b0:b1]).cuda(), 0, bits, False, True)
        q = graph.comm_buf_for_quantization
        return (out.cpu().numpy(), q.quantized_send_data_buf.cpu().numpy(), q.quantized_send_params_buf_fp32.cpu().numpy(),
                graph.idx_nodes_send_to_others.cpu().numpy(), list(graph.comm_splits.send_splits))

    res = FakeWorld(P).run(rank_fn)
    src, dst = s_t.cpu().numpy(), d_t.cpu().numpy()
    rp, c, v = global_csr(src, dst, n)
    want, scale_abs = oracle.spmm(rp, c, v, X), oracle.spmm(rp, c, v, np.abs(X))
    epb = 8 // bits
    for r in range(P):
        out, codes, params, idx, send_splits = res[r]
        b0, b1 = int(begin[r]), int(begin[r + 1])
        rows = X[b0 + idx]
        offs = np.concatenate([[0], np.cumsum(send_splits)]).astype(np.int32)
        if bits == 2:
            wc, wp = oracle.quantize_int2_for_all_procs(rows, offs)
        else:
            mn = rows.min(1)
            sc = ((rows.max(1) - mn) / np.float32(2 ** bits - 1)).astype(np.float32)
            sc[sc == 0] = 1
            wp = np.stack([mn, sc], 1)
            wc = np.concatenate([oracle.quantize_rowpacked(rows[a:b], mn[a:b], sc[a:b], bits)
                                 for a, b in zip(offs[:-1], offs[1:]) if b > a])
        np.testing.assert_array_equal(params, wp)
        np.testing.assert_array_equal(codes, wc)
        # the lossy halo keeps the aggregate within one quantisation step per remote term
        assert np.abs(out - want[b0:b1]).max() <= (2.5 if bits == 2 else 0.05) * max(1.0, scale_abs[b0:b1].max())


@pytest.mark.parametrize("engine", ["kernel", "copy", "auto"])
@pytest.mark.parametrize("P,bits,is_pre,F,groups", [
    (2, 32, False, 128, 1), (4, 32, False, 256, 1), (4, 32, False, 100, 3), (5, 32, False, 32, 2), (8, 32, False, 128, 3),
    (3, 32, True, 128, 1), (2, 2, False, 128, 1), (4, 2, False, 256, 3), (3, 2, True, 128, 1), (3, 8, False, 64, 1),
])
def test_push_transport_matches_all_to_all(cuda_lib, P, bits, is_pre, F, groups, engine):
    """Communicator(transport="push"): halo rows stored straight into the receivers' buffers by
    gnnagg_push_rows (gathered on the way) or, with push_engine="copy", moved there block by block with
    device-to-device copies (gnnagg_push_block); signals instead of a collective.  With one group of peers the
    outputs, gradients and wire codes equal the all-to-all path bit for bit; with several groups (fp32 halo,
    plain path) the peers' contributions are added in arrival order: 1e-5 of the summed magnitudes.  Two
    forward + backward rounds, so that buffers are reused behind their "free" signals."""
    from gnn_benchmark_b200 import Communicator, Quantizer_for_all_procs, TimeRecorder, graphgen
    from gnn_benchmark_b200.aggregator import Aggregator
    from gnn_benchmark_b200.data_manager.DataLoader import build_graph

    begin_np, src, dst = make_graph(17 * P + F + bits, P, 400, 6)
    N = int(begin_np[-1])
    begin = torch.from_numpy(begin_np)
    rng = np.random.default_rng(5)
    X = rng.standard_normal((2, N, F)).astype(np.float32)
    G = rng.standard_normal((2, N, F)).astype(np.float32)
    s_t, d_t = torch.from_numpy(src).cuda(), torch.from_numpy(dst).cuda()
    Quantizer_for_all_procs(P, bits)
    TimeRecorder(1, 1)
    results = {}
    for transport in ("all_to_all", "push"):
        Communicator(bits, is_async=True, transport=transport, push_groups=groups, push_engine=engine)

        def rank_fn(rank):
            local, remote = graphgen.partition_edges(s_t, d_t, begin, rank)
            graph = build_graph(local, remote, begin, rank, P, F, bits, is_pre, device="cuda")
            assert (graph.push_plan is not None) == (transport == "push")
            assert transport != "push" or graph.push_plan.peers.engine == engine
            b0, b1 = int(begin[rank]), int(begin[rank + 1])
            got = []
            for k in range(2):
                ctx = SimpleNamespace()
                out = Aggregator.forward(ctx, graph, torch.from_numpy(X[k, b0:b1]).cuda(), 0, bits, is_pre, True)
                grad = Aggregator.backward(ctx, torch.from_numpy(G[k, b0:b1]).cuda())[1]
                got += [out.cpu().numpy(), grad.cpu().numpy()]
                if bits != 32:
                    q = graph.comm_buf_for_quantization
                    got += [q.quantized_recv_data_buf.cpu().numpy(), q.quantized_send_data_buf.cpu().numpy()]
            return got

        results[transport] = FakeWorld(P, push_engine=engine).run(rank_fn)
    for r in range(P):
        for i, (a, b) in enumerate(zip(results["all_to_all"][r], results["push"][r])):
            if groups == 1 or a.dtype == np.uint8:
                np.testing.assert_array_equal(a, b)
            else:
                bad = np.nonzero(np.abs(a - b).max(axis=1) > 1e-5 * max(1.0, np.abs(a).max()))[0]
                assert bad.size == 0, f"rank {r}, array {i}: {bad.size} of {a.shape[0]} rows differ, first {bad[:8]}"
