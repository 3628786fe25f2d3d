"""Failure reporting and training paths: out-of-range indices are skipped and reported, a bounded
device-side wait that cannot complete gives up and reports, the status word makes later launches
loud (NaN) until it is read, and gradients reach the bias and flow through pooling."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import kernel_map as km
from warpconvnet_b200 import (SPARSE_CONV_BWD_ALGO_MODE as BWD, SPARSE_CONV_FWD_ALGO_MODE as ALGO, ConvEpilogue,
                              IntSearchResult, SparseConv3d, Voxels, generate_kernel_map, spatially_sparse_conv)
from warpconvnet_b200._native import (CONV_AUTO, CONV_SIMT, CONV_TCGEN05, check_device_status, device_status, lib, ptr,
                                      stream_ptr)
from warpconvnet_b200.datasets import synthetic
from warpconvnet_b200.nn.functional.sparse_conv import _gather_rows, _scatter_add_rows, sparse_conv_fused, sparse_conv_wgrad
from warpconvnet_b200.nn.functional.sparse_pool import sparse_avg_pool, sparse_max_pool, sparse_reduce, sparse_unpool
from warpconvnet_b200.nn.functional.sparse_conv import STRIDED_CONV_MODE

from conftest import rel_l2

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
BOUNDS, EXPIRED = "index out of bounds", "bounded device-side wait expired"


def room(n, seed=3):
    xyz = synthetic.room_scene(n, 0.02, seed, "raster_crop")
    coords = np.concatenate([np.zeros((len(xyz), 1), np.int32), xyz], 1)
    return np.ascontiguousarray(coords[np.argsort(km.morton_code(coords[:, 1:]), kind="stable")])


@pytest.mark.parametrize("algo,dtype,c_in,c_out", [(CONV_TCGEN05, torch.float16, 64, 64), (CONV_SIMT, torch.float32, 24, 40),
                                                   (CONV_AUTO, torch.float32, 3, 32), (CONV_AUTO, torch.float16, 96, 20)])
def test_out_of_range_neighbour_is_skipped_and_reported(algo, dtype, c_in, c_out):
    """A caller-supplied compact map with one index past the feature matrix: the kernel treats that
    neighbour as absent (no access), every other number is right, the status word says
    WCN_ERR_BOUNDS, and the next launch on a clean word is clean."""
    n = 6000
    coords = room(n)
    i, o, f, iden = km.generate_kernel_map(coords, coords, (1, 1, 1), (3, 3, 3))
    check_device_status(DEV)
    g = torch.Generator().manual_seed(0)
    x = torch.randn(n, c_in, generator=g).to(dtype).to(DEV)
    w = (torch.randn(27, c_in, c_out, generator=g) * 0.1).to(dtype).to(DEV)
    good = IntSearchResult(torch.from_numpy(i).to(DEV), torch.from_numpy(o).to(DEV), torch.from_numpy(f), iden)
    want = sparse_conv_fused(x, w, good, n, algo=algo, out_dtype=torch.float32)
    check_device_status(DEV)
    bad_i = i.copy()
    p = int(f[5]) + 7  # a pair of offset 5
    victim = int(o[p])
    bad_i[p] = n + 12345
    bad = IntSearchResult(torch.from_numpy(bad_i).to(DEV), torch.from_numpy(o).to(DEV), torch.from_numpy(f), iden)
    got = sparse_conv_fused(x, w, bad, n, algo=algo, out_dtype=torch.float32)
    torch.cuda.synchronize()
    assert torch.isfinite(got).all()
    keep = torch.ones(n, dtype=torch.bool, device=DEV)
    keep[victim] = False
    assert torch.equal(got[keep], want[keep])
    dropped = want[victim] - x[int(i[p])].float() @ w[5].float()
    assert rel_l2(got[victim].cpu().numpy(), dropped.cpu().numpy()) < 1e-3
    with pytest.raises(RuntimeError, match=BOUNDS):
        check_device_status(DEV)
    again = sparse_conv_fused(x, w, good, n, algo=algo, out_dtype=torch.float32)
    check_device_status(DEV)
    assert torch.equal(again, want)


def test_out_of_range_rows_in_gather_scatter_reduce_and_wgrad():
    check_device_status(DEV)
    src = torch.arange(40, dtype=torch.float32, device=DEV).reshape(10, 4)
    idx = torch.tensor([3, 10, 0, -2], dtype=torch.int32, device=DEV)
    got = _gather_rows(src, idx)
    torch.cuda.synchronize()
    assert torch.equal(got[0], src[3]) and torch.equal(got[2], src[0]) and float(got[1].abs().sum() + got[3].abs().sum()) == 0
    with pytest.raises(RuntimeError, match=BOUNDS):
        check_device_status(DEV)
    dst = torch.zeros(5, 4, device=DEV)
    _scatter_add_rows(torch.ones(3, 4, device=DEV), torch.tensor([1, 5, 4], dtype=torch.int32, device=DEV), dst)
    torch.cuda.synchronize()
    assert dst.sum(1).tolist() == [0, 4, 0, 0, 4]
    with pytest.raises(RuntimeError, match=BOUNDS):
        check_device_status(DEV)
    # pooling over a table that names a row past the features
    from warpconvnet_b200.ops.reductions import neighbor_reduction
    nbr = torch.tensor([[0, 1, 2], [3, 99, -1]], dtype=torch.int32, device=DEV)
    table = IntSearchResult.from_neighbor_table(nbr, 10, None, None)
    out = neighbor_reduction(src, table, 3, "sum")
    torch.cuda.synchronize()
    assert torch.equal(out, torch.stack([src[0] + src[3], src[1], src[2]]))
    with pytest.raises(RuntimeError, match=BOUNDS):
        check_device_status(DEV)
    # weight gradient: the bad pair contributes nothing
    n = 4000
    coords = room(n, 9)
    c = torch.from_numpy(coords).to(DEV)
    kmap = generate_kernel_map(c, c, (1, 1, 1), (3, 3, 3))
    nbr = kmap.neighbor_table(n).clone()
    g = torch.Generator().manual_seed(1)
    x = torch.randn(n, 32, generator=g).half().to(DEV)
    gy = torch.randn(n, 32, generator=g).half().to(DEV)
    want = sparse_conv_wgrad(x, gy, IntSearchResult.from_neighbor_table(nbr, n, None, 13), n)
    m = int((nbr[2] >= 0).nonzero()[0])
    lost = torch.outer(x[int(nbr[2, m])].float(), gy[m].float())
    nbr[2, m] = n + 5
    got = sparse_conv_wgrad(x, gy, IntSearchResult.from_neighbor_table(nbr, n, None, 13), n)
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match=BOUNDS):
        check_device_status(DEV)
    want[2] -= lost
    assert rel_l2(got.cpu().numpy(), want.cpu().numpy()) < 1e-4


def test_bounded_wait_gives_up_and_later_launches_are_loud():
    """A wait on a barrier phase that nothing completes runs out of its (short) limit, stores
    WCN_ERR_WAIT_EXPIRED and the kernel ends normally.  While the word is set a tensor-core
    convolution computes nothing and fills its output with NaN; once the host has read (and
    thereby zeroed) the word, the same call gives the right numbers."""
    check_device_status(DEV)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    rc = lib().wcn_selftest_bounded_wait(200_000, ptr(device_status(DEV)), ptr(flag), stream_ptr(DEV))
    assert rc == 0
    torch.cuda.synchronize()
    assert int(flag.item()) == 1
    n = 5000
    coords = room(n, 5)
    c = torch.from_numpy(coords).to(DEV)
    kmap = generate_kernel_map(c, c, (1, 1, 1), (3, 3, 3))
    g = torch.Generator().manual_seed(2)
    x = torch.randn(n, 64, generator=g).half().to(DEV)
    w = (torch.randn(27, 64, 64, generator=g) * 0.1).half().to(DEV)
    for split_k in (1, 4):  # one-pass kernel and the offset-sliced pair of kernels
        y = sparse_conv_fused(x, w, kmap, n, algo=CONV_TCGEN05, split_k=split_k)
        torch.cuda.synchronize()
        assert bool(torch.isnan(y).all())
    with pytest.raises(RuntimeError, match=EXPIRED):
        check_device_status(DEV)
    y = sparse_conv_fused(x, w, kmap, n, algo=CONV_TCGEN05)
    ys = sparse_conv_fused(x, w, kmap, n, algo=CONV_SIMT)
    check_device_status(DEV)
    assert torch.isfinite(y).all() and rel_l2(y.float().cpu().numpy(), ys.float().cpu().numpy()) < 2e-3
    assert lib().wcn_selftest_bounded_wait(10, ptr(device_status(DEV)), None, stream_ptr(DEV)) != 0  # limit too small


def test_input_side_kernel_reports_bad_destinations_and_is_loud_after_an_expired_wait():
    """wcn_conv_rows_fwd: a destination past the output is skipped and reported (every other row is
    right, the rows nobody names keep what they held); while the status word holds an expired wait
    the kernel computes nothing and marks the rows it would have written with NaN."""
    from warpconvnet_b200.nn.functional.sparse_conv import sparse_conv_rows_fused
    check_device_status(DEV)
    g = torch.Generator().manual_seed(4)
    n_in, n_out, c_in, c_out = 3000, 5000, 64, 48
    x = torch.randn(n_in, c_in, generator=g).half().to(DEV)
    w = (torch.randn(1, c_in, c_out, generator=g) * 0.1).half().to(DEV)
    dst = torch.randperm(n_out, generator=g)[:n_in].to(torch.int32).view(1, -1).contiguous()
    bad = dst.clone()
    bad[0, 17] = n_out + 99
    bad[0, 18] = -1            # a pair that names no row: not an error
    out = torch.full((n_out, c_out), -3.0, dtype=torch.float16, device=DEV)
    got = sparse_conv_rows_fused(x, w, bad.to(DEV), n_out, ConvEpilogue(out=out))
    assert got is not None
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match=BOUNDS):
        check_device_status(DEV)
    want = (x.float() @ w[0].float()).half()
    rows = dst[0].long()
    keep = torch.ones(n_in, dtype=torch.bool)
    keep[17] = keep[18] = False
    assert rel_l2(out[rows[keep]].float().cpu().numpy(), want[keep].float().cpu().numpy()) < 2e-3
    untouched = torch.ones(n_out, dtype=torch.bool)
    untouched[rows[keep]] = False
    assert bool((out[untouched.to(DEV)] == -3.0).all())
    # an expired wait on the status word: nothing is computed, the named rows turn NaN
    assert lib().wcn_selftest_bounded_wait(200_000, ptr(device_status(DEV)), None, stream_ptr(DEV)) == 0
    loud = sparse_conv_rows_fused(x, w, dst.to(DEV), n_out, ConvEpilogue(out=torch.zeros_like(out)))
    torch.cuda.synchronize()
    unnamed = torch.ones(n_out, dtype=torch.bool)
    unnamed[rows] = False
    assert bool(torch.isnan(loud[rows]).all()) and bool((loud[unnamed.to(DEV)] == 0).all())
    with pytest.raises(RuntimeError, match=EXPIRED):
        check_device_status(DEV)
    again = sparse_conv_rows_fused(x, w, dst.to(DEV), n_out)
    check_device_status(DEV)
    assert rel_l2(again[rows].float().cpu().numpy(), want.float().cpu().numpy()) < 2e-3


def test_status_word_is_read_where_the_host_waits_anyway():
    """A failure recorded by an earlier kernel surfaces at the next point where the package
    synchronises with the host: sizing strided coordinates, compacting a kernel map."""
    from warpconvnet_b200 import stride_coords
    check_device_status(DEV)
    coords = room(3000, 7)
    c = torch.from_numpy(coords).to(DEV)
    device_status(DEV).fill_(-8)
    with pytest.raises(RuntimeError, match=BOUNDS):
        stride_coords(c, (2, 2, 2), in_offsets=torch.tensor([0, len(coords)]))
    assert int(device_status(DEV).item()) == 0
    kmap = generate_kernel_map(c, c, (1, 1, 1), (3, 3, 3))
    device_status(DEV).fill_(-7)
    with pytest.raises(RuntimeError, match=EXPIRED):
        kmap.offsets
    check_device_status(DEV)


@pytest.mark.parametrize("fwd,bwd", [(ALGO.EXPLICIT_GEMM, BWD.EXPLICIT_GEMM), (ALGO.IMPLICIT_GEMM, BWD.IMPLICIT_GEMM),
                                     (ALGO.AUTO, BWD.AUTO)])
def test_bias_and_weight_gradients_agree_across_algorithms(fwd, bwd):
    """A trainable bias receives its gradient with every forward algorithm (the default module has
    bias=True and algorithm 'auto'), also when it is the only trainable tensor and for the 1x1x1
    shortcut."""
    n = 3000
    coords = room(n, 11)
    g = torch.Generator().manual_seed(3)
    x = torch.randn(n, 8, generator=g)
    go = torch.randn(n, 12, generator=g)
    torch.manual_seed(1)
    ref = SparseConv3d(8, 12, 3, bias=True, fwd_algo=ALGO.EXPLICIT_GEMM, bwd_algo=BWD.EXPLICIT_GEMM).to(DEV)
    vox = Voxels(torch.from_numpy(coords[:, 1:].copy()).to(DEV), x.to(DEV), offsets=torch.tensor([0, n]))
    ref(vox).feature_tensor.backward(go.to(DEV))
    assert ref.bias.grad is not None and rel_l2(ref.bias.grad.cpu().numpy(), go.sum(0).numpy()) < 1e-5
    conv = SparseConv3d(8, 12, 3, bias=True, fwd_algo=fwd, bwd_algo=bwd).to(DEV)
    conv.load_state_dict(ref.state_dict())
    y = conv(vox)
    assert rel_l2(y.feature_tensor.detach().cpu().numpy(), ref(vox).feature_tensor.detach().cpu().numpy()) < 1e-5
    y.feature_tensor.backward(go.to(DEV))
    assert conv.bias.grad is not None and conv.weight.grad is not None
    assert rel_l2(conv.bias.grad.cpu().numpy(), ref.bias.grad.cpu().numpy()) < 1e-5
    assert rel_l2(conv.weight.grad.cpu().numpy(), ref.weight.grad.cpu().numpy()) < 1e-4
    # frozen weight, trainable bias
    conv.zero_grad()
    conv.weight.requires_grad_(False)
    conv(vox).feature_tensor.backward(go.to(DEV))
    assert conv.weight.grad is None and rel_l2(conv.bias.grad.cpu().numpy(), go.sum(0).numpy()) < 1e-5
    # 1x1x1 shortcut with only the bias trainable
    one = SparseConv3d(8, 12, 1, bias=True, fwd_algo=fwd, bwd_algo=bwd).to(DEV)
    one.weight.requires_grad_(False)
    one(vox).feature_tensor.backward(go.to(DEV))
    assert rel_l2(one.bias.grad.cpu().numpy(), go.sum(0).numpy()) < 1e-5


@pytest.mark.parametrize("reduction", ["max", "min", "mean", "sum"])
def test_pooling_is_differentiable(reduction):
    """Gradients through sparse_reduce / sparse_unpool equal those of the same reduction written with
    torch ops over the oracle's kernel map."""
    n, ch = 4000, 6
    coords = room(n, 13)
    g = torch.Generator().manual_seed(4)
    x = torch.randn(n, ch, generator=g)
    out_c, _ = km.stride_coords(coords, (2, 2, 2))
    i, o, f, _ = km.generate_kernel_map(coords, out_c, (2, 2, 2), (2, 2, 2))
    go = torch.randn(len(out_c), ch, generator=g)
    xr = x.clone().requires_grad_(True)
    idx = torch.from_numpy(o).long().unsqueeze(1).expand(-1, ch)
    src = xr[torch.from_numpy(i).long()]
    if reduction in ("sum", "mean"):
        ref = torch.zeros(len(out_c), ch).scatter_reduce(0, idx, src, reduction, include_self=False)
    else:
        ref = torch.zeros(len(out_c), ch).scatter_reduce(0, idx, src, "a" + reduction, include_self=False)
    ref.backward(go)
    xg = x.clone().to(DEV).requires_grad_(True)
    vox = Voxels(torch.from_numpy(coords[:, 1:].copy()).to(DEV), xg, offsets=torch.tensor([0, n]))
    pooled = sparse_reduce(vox, 2, 2, reduction=reduction)
    assert pooled.feature_tensor.requires_grad
    assert rel_l2(pooled.feature_tensor.detach().cpu().numpy(), ref.detach().numpy()) < 1e-6
    pooled.feature_tensor.backward(go.to(DEV))
    assert rel_l2(xg.grad.cpu().numpy(), xr.grad.numpy()) < 1e-6
    check_device_status(DEV)


def test_unpool_and_reduce_and_stride_train():
    n, ch = 3000, 8
    coords = room(n, 17)
    g = torch.Generator().manual_seed(5)
    x = torch.randn(n, ch, generator=g)
    xg = x.clone().to(DEV).requires_grad_(True)
    vox = Voxels(torch.from_numpy(coords[:, 1:].copy()).to(DEV), xg, offsets=torch.tensor([0, n]))
    pooled = sparse_avg_pool(vox, 2, 2)
    back = sparse_unpool(pooled, vox, 2, 2)
    gu = torch.randn(n, ch, generator=g)
    back.feature_tensor.backward(gu.to(DEV))
    # reference: mean over each 2x2x2 cell, copied back to its members
    out_c, _ = km.stride_coords(coords, (2, 2, 2))
    i, o, f, _ = km.generate_kernel_map(coords, out_c, (2, 2, 2), (2, 2, 2))
    xr = x.clone().requires_grad_(True)
    idx = torch.from_numpy(o).long()
    mean = torch.zeros(len(out_c), ch).index_add(0, idx, xr[torch.from_numpy(i).long()]) / torch.bincount(idx).unsqueeze(1)
    rep = torch.zeros(n, ch).index_add(0, torch.from_numpy(i).long(), mean[idx])
    rep.backward(gu)
    assert rel_l2(back.feature_tensor.detach().cpu().numpy(), rep.detach().numpy()) < 1e-6
    assert rel_l2(xg.grad.cpu().numpy(), xr.grad.numpy()) < 1e-5
    # the other stride mode of the convolution now trains as well
    xg2 = x.clone().to(DEV).requires_grad_(True)
    vox2 = Voxels(torch.from_numpy(coords[:, 1:].copy()).to(DEV), xg2, offsets=torch.tensor([0, n]))
    w = (torch.randn(27, ch, 5, generator=g) * 0.2).to(DEV).requires_grad_(True)
    y = spatially_sparse_conv(vox2, w, 3, stride=2, stride_mode=STRIDED_CONV_MODE.REDUCE_AND_STRIDE, stride_reduce="max",
                              fwd_algo=ALGO.IMPLICIT_GEMM, bwd_algo=BWD.IMPLICIT_GEMM)
    y.feature_tensor.sum().backward()
    assert xg2.grad is not None and w.grad is not None and float(xg2.grad.abs().sum()) > 0
    check_device_status(DEV)
