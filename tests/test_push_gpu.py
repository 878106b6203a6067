"""gnnagg_push_rows / gnnagg_push_block through the C ABI on one device: the "peers" are three ordinary
buffers of the same GPU (a peer address is just an address), so every row must land at
dst[p] + (row inside this rank's block for p) * ld_dst, gathered through idx when given, for every access
width the kernel picks (16-, 4- and 1-byte units), for empty peers and for a peer range that wraps."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _prefix(counts):
    return np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)


@pytest.mark.parametrize("row_bytes,pad_src,pad_dst", [(512, 0, 0), (400, 0, 16), (4, 0, 0), (100, 0, 0), (7, 1, 2),
                                                       (64, 64, 0), (1024, 0, 0)])
@pytest.mark.parametrize("use_idx", [False, True])
@pytest.mark.parametrize("counts,first,num", [([5, 0, 9], 0, 3), ([300, 41, 2], 1, 2), ([0, 0, 7], 2, 3), ([13, 6, 1], 2, 2)])
def test_push_rows_places_every_row(cuda_lib, row_bytes, pad_src, pad_dst, use_idx, counts, first, num):
    from gnn_benchmark_b200 import _lib

    P = len(counts)
    seg = _prefix(counts)
    rows = int(seg[-1])
    ld_src, ld_dst = row_bytes + pad_src, row_bytes + pad_dst
    rng = np.random.default_rng(row_bytes * 7 + rows + first)
    n_src = rows + 17 if use_idx else rows
    src = rng.integers(0, 256, size=(n_src, ld_src), dtype=np.uint8)
    idx = rng.integers(0, n_src, size=rows).astype(np.int32) if use_idx else None
    lead = [3, 0, 11]  # rows of other ranks that precede this rank's block in each peer's buffer
    cap = [lead[p] + counts[p] + 2 for p in range(P)]
    src_d = torch.from_numpy(src).cuda()
    idx_d = torch.from_numpy(idx).cuda() if use_idx else None
    seg_d = torch.from_numpy(seg).cuda()
    bufs = [torch.full((cap[p], ld_dst), 0xEE, dtype=torch.uint8, device="cuda") for p in range(P)]
    dst = torch.tensor([bufs[p].data_ptr() + lead[p] * ld_dst for p in range(P)], dtype=torch.int64, device="cuda")
    served = [(first + j) % P for j in range(num)]
    hint = sum(counts[p] for p in served)
    rc = _lib.lib().gnnagg_push_rows(src_d.data_ptr(), ld_src, _lib.ptr(idx_d), row_bytes, seg_d.data_ptr(), P, first, num,
                                     dst.data_ptr(), ld_dst, hint, _lib.stream_ptr(src_d.device))
    _lib.check(rc, "push_rows")
    torch.cuda.synchronize()
    for p in range(P):
        got = bufs[p].cpu().numpy()
        want = np.full((cap[p], ld_dst), 0xEE, dtype=np.uint8)
        if p in served:
            for i in range(counts[p]):
                r = seg[p] + i
                want[lead[p] + i, :row_bytes] = src[idx[r] if use_idx else r, :row_bytes]
        np.testing.assert_array_equal(got, want, err_msg=f"peer {p}")


def test_push_block_copies_and_checks_arguments(cuda_lib):
    from gnn_benchmark_b200 import _lib

    lib = _lib.lib()
    src = torch.arange(4096, dtype=torch.int32, device="cuda")
    dst = torch.zeros(8192, dtype=torch.int32, device="cuda")
    st = _lib.stream_ptr(src.device)
    _lib.check(lib.gnnagg_push_block(src.data_ptr() + 4 * 100, dst.data_ptr() + 4 * 5000, 4 * 1000, st), "push_block")
    _lib.check(lib.gnnagg_push_block(src.data_ptr(), dst.data_ptr(), 0, st), "push_block")  # nothing to move
    torch.cuda.synchronize()
    want = torch.zeros(8192, dtype=torch.int32)
    want[5000:6000] = torch.arange(100, 1100, dtype=torch.int32)
    assert torch.equal(dst.cpu(), want)
    assert lib.gnnagg_push_block(None, dst.data_ptr(), 16, st) != 0
    assert lib.gnnagg_push_rows(src.data_ptr(), 4, None, 8, src.data_ptr(), 1, 0, 1, dst.data_ptr(), 8, 1, st) != 0  # ld < row
    assert lib.gnnagg_push_rows(src.data_ptr(), 8, None, 8, src.data_ptr(), 2, 2, 1, dst.data_ptr(), 8, 1, st) != 0  # peer range
