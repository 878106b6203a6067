"""Mixed-precision halo exchange (a bit width per row): Communicator.comm_with_mixed_quantization over the
column-packed codec kernels, with the widths drawn by the Assigner, against the CPU oracle's restatement of
the reference's quantize_tensor_v1 / dequantize_tensor_v1 (model/ops/src/quantization_x86.cpp:170-312;
golden bytes of the reference's own test pin that restatement in tests/test_oracle_pins.py)."""
import numpy as np
import pytest
import torch

import oracle
from fake_dist import FakeWorld

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("P,F,num_bits", [(3, 64, -1), (4, 100, -1), (2, 37, 4)])
def test_mixed_bit_exchange_codes_and_rows(cuda_lib, P, F, num_bits):
    from gnn_benchmark_b200 import Assigner, Communicator, QuantizerForMixedBits, TimeRecorder

    rng = np.random.default_rng(P * 100 + F)
    splits = rng.integers(0, 40, size=(P, P))  # splits[r][p]: rows rank r sends to rank p
    np.fill_diagonal(splits, 0)
    rows = [rng.standard_normal((int(splits[r].sum()), F)).astype(np.float32) for r in range(P)]
    Communicator(32, is_async=True)
    TimeRecorder(1, 1)
    torch.manual_seed(7)

    def rank_fn(rank):
        send_splits = [int(x) for x in splits[rank]]
        recv_splits = [int(splits[q][rank]) for q in range(P)]
        a = Assigner(num_bits, 1, [0.3, 0.3, 0.4], 1, sum(send_splits), sum(recv_splits), device="cuda")
        a.reassign_node_dataformat(0)
        bits = a.get_node_dataformat("forward0")
        send_buf = torch.from_numpy(rows[rank]).cuda()
        recv_buf = torch.full((sum(recv_splits), F), float("nan"), device="cuda")
        handle, qrecv, drange, dparams = Communicator.ctx.comm_with_mixed_quantization(
            recv_buf, send_buf, recv_splits, send_splits, bits)
        if handle is not None:
            handle.wait()
        QuantizerForMixedBits.dequantize_intX_to_fp32(qrecv, recv_buf, drange, dparams)
        torch.cuda.synchronize()
        return bits.cpu().numpy(), qrecv.cpu().numpy(), dparams.cpu().numpy(), recv_buf.cpu().numpy()

    res = FakeWorld(P).run(rank_fn)
    for r in range(P):
        assert set(np.unique(res[r][0])) <= {2.0, 4.0, 8.0}
    # what every sender must have produced, per the oracle
    sent = []
    for q in range(P):
        codes, params, rng_q = oracle.quantize_v1(rows[q], res[q][0].astype(np.int64))
        sent.append((codes, params, rng_q, np.concatenate([[0], np.cumsum(splits[q])])))
    for r in range(P):
        want_codes, want_params, want_rows = [], [], []
        for q in range(P):
            codes, params, rng_q, off = sent[q]
            lo, hi = int(off[r]), int(off[r + 1])
            want_codes.append(codes[int(rng_q[lo]):int(rng_q[hi])])
            wire = oracle.bf16_round(params[lo:hi])
            want_params.append(wire)
            if hi > lo:
                sub_rng = rng_q[lo:hi + 1] - rng_q[lo]
                want_rows.append(oracle.dequantize_v1(codes[int(rng_q[lo]):int(rng_q[hi])], hi - lo, F, sub_rng, wire))
        np.testing.assert_array_equal(res[r][1], np.concatenate(want_codes))
        np.testing.assert_array_equal(res[r][2], np.concatenate(want_params))
        if want_rows:
            np.testing.assert_array_equal(res[r][3], np.concatenate(want_rows))
