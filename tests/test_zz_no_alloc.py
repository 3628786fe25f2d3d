"""The allocation-free kernel-map entry point (collected last on purpose: if it fails, a run
that stops at the first failure has already run everything else).

``wcn_kmap_search_static`` is for hosts that cannot allocate device memory around the call
(plugins with a fixed arena, serving loops that forbid allocator calls, exhausted pools): its scratch is an array inside the library.
It must give exactly what ``wcn_kmap_search`` + ``wcn_kmap_scan`` give with a caller-owned
workspace — bit for bit, these are integers — on two calls in a row that reuse the array.
"""
import ctypes

import numpy as np
import pytest
import torch

from warpconvnet_b200 import _native
from warpconvnet_b200.datasets import synthetic

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _i3(v):
    arr = (ctypes.c_int32 * 3)(*v)
    return arr, ctypes.addressof(arr)


def _build_table(coords):
    n = coords.shape[0]
    cap = max(16, 2 * n)
    table = torch.empty(_native.query_bytes("wcn_hash_table_bytes", cap), dtype=torch.uint8, device=DEV)
    _native.check(_native.lib().wcn_hash_build(coords.data_ptr(), n, None, table.data_ptr(), cap, 1, None,
                                               _native.device_status(DEV).data_ptr(), _native.stream_ptr(torch.device(DEV))))
    return table, cap


def _existing(table, cap, queries, stride, ksize, K):
    m = queries.shape[0]
    st = _native.stream_ptr(torch.device(DEV))
    nbr = torch.empty((K, m), dtype=torch.int32, device=DEV)
    ws = torch.empty(_native.query_bytes("wcn_kmap_workspace_bytes", m, K), dtype=torch.uint8, device=DEV)
    offsets = torch.empty(K + 1, dtype=torch.int32, device=DEV)
    sk, sp = _i3(stride)
    kk, kp = _i3(ksize)
    _native.check(_native.lib().wcn_kmap_search(table.data_ptr(), cap, 1, queries.data_ptr(), m, sp, kp, K,
                                                nbr.data_ptr(), ws.data_ptr(), st))
    _native.check(_native.lib().wcn_kmap_scan(ws.data_ptr(), m, K, offsets.data_ptr(), st))
    return nbr, offsets


def _static(table, cap, queries, stride, ksize, K, nbr, offsets):
    sk, sp = _i3(stride)
    kk, kp = _i3(ksize)
    return _native.lib().wcn_kmap_search_static(table.data_ptr(), cap, 1, queries.data_ptr(), queries.shape[0], sp, kp,
                                                K, nbr.data_ptr(), offsets.data_ptr(),
                                                _native.stream_ptr(torch.device(DEV)))


def test_static_scratch_matches_workspace_variant_twice_in_a_row():
    cases = []
    for seed, n, stride, ksize in ((11, 90000, (1, 1, 1), (3, 3, 3)), (12, 30000, (1, 1, 1), (3, 3, 3)),
                                   (13, 50000, (1, 1, 1), (2, 2, 2))):
        xyz = synthetic.room_scene(n, 0.05, seed, "sample")
        coords = torch.from_numpy(np.concatenate([np.zeros((n, 1), np.int32), xyz], 1)).to(DEV)
        table, cap = _build_table(coords)
        K = ksize[0] * ksize[1] * ksize[2]
        # outputs are allocated here, before the calls under test
        cases.append((table, cap, coords, stride, ksize, K, torch.empty((K, n), dtype=torch.int32, device=DEV),
                      torch.empty(K + 1, dtype=torch.int32, device=DEV)))
    # back-to-back calls on the shared array: a larger problem first, so stale counts remain behind the smaller one
    for table, cap, coords, stride, ksize, K, nbr, offsets in cases:
        _native.check(_static(table, cap, coords, stride, ksize, K, nbr, offsets), "wcn_kmap_search_static")
        ref_nbr, ref_offsets = _existing(table, cap, coords, stride, ksize, K)
        assert torch.equal(nbr, ref_nbr)
        assert torch.equal(offsets, ref_offsets)
        assert int(offsets[-1]) == int((nbr >= 0).sum())
    _native.check_device_status(DEV)


def test_static_scratch_rejects_oversized_problems():
    # the size check comes first and launches nothing, so dummy pointers are never touched
    dummy = torch.zeros(64, dtype=torch.int32, device=DEV)
    too_many = 11_000_000  # 27 * ceil(11e6 / 256) exceeds the built-in array
    sk, sp = _i3((1, 1, 1))
    kk, kp = _i3((3, 3, 3))
    rc = _native.lib().wcn_kmap_search_static(dummy.data_ptr(), 16, 1, dummy.data_ptr(), too_many, sp, kp, 27,
                                              dummy.data_ptr(), dummy.data_ptr(), _native.stream_ptr(torch.device(DEV)))
    assert rc == -9 and "scratch" in _native.status_string(rc)
    torch.cuda.synchronize()
