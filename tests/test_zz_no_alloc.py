"""The matvec entry point that allocates nothing (tg_dev_qmatvec_static).

Callers such as a serving process that has given all of HBM to its own memory
pools, or code that runs while a stream is being captured, cannot let a library
call cudaMalloc behind their back. This entry point keeps its split-K scratch in
a fixed array inside the library. The test calls it through the C ABI twice in a
row and compares with the allocating entry point; it also checks that the free
device memory does not move and that sizes beyond the array are refused.

Collected last (file name) so that a run that stops at the first failure has
already run every other test.
"""

import ctypes as C

import numpy as np
import pytest

import cases
from conftest import rel_l2

pytestmark = pytest.mark.gpu


def _ptr(t):
    return C.c_void_p(t.data_ptr())


@pytest.mark.parametrize("K,N", [(6912, 1152), (1152, 6912), (640, 1024), (1152, 262144)])
def test_static_scratch_matvec_matches_allocating_entry_point(capi, port, K, N):
    import torch

    lib = capi.load()
    x, w, s = cases.linear_case(K, N, 1)
    dx = torch.from_numpy(x[0].copy()).cuda()
    dw = torch.from_numpy(w).cuda()
    ds = torch.from_numpy(s).cuda()
    y_ref, y1, y2 = (torch.full((N,), float("nan"), device="cuda") for _ in range(3))
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.tg_dev_qmatvec(_ptr(y_ref), _ptr(dx), _ptr(dw), _ptr(ds), K, N, stream) == 0, lib.tg_last_error()
    # first call on this device does the one-time address look-up
    assert lib.tg_dev_qmatvec_static(_ptr(y1), _ptr(dx), _ptr(dw), _ptr(ds), K, N, stream) == 0, lib.tg_last_error()
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    # two calls in a row share the scratch: the second finds the first one's contents in it
    assert lib.tg_dev_qmatvec_static(_ptr(y1), _ptr(dx), _ptr(dw), _ptr(ds), K, N, stream) == 0, lib.tg_last_error()
    assert lib.tg_dev_qmatvec_static(_ptr(y2), _ptr(dx), _ptr(dw), _ptr(ds), K, N, stream) == 0, lib.tg_last_error()
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before  # nothing was allocated or freed
    ref = y_ref.cpu().numpy()
    # the two entry points may split K differently, hence the matvec tolerance rather than equality
    assert rel_l2(y1.cpu().numpy(), ref) <= 5e-6
    assert rel_l2(y2.cpu().numpy(), ref) <= 5e-6
    assert torch.equal(y1, y2)
    # and against the oracle's restatement of the reference operator (linalg.hpp:41-204)
    want = port.lm_head_decode(x[0], w, s) if N == 262144 else port.linear_decode(x[0], w, s)
    assert rel_l2(y1.cpu().numpy(), want) <= 5e-6


def test_static_scratch_rejects_sizes_beyond_its_maximum(capi):
    import torch

    lib = capi.load()
    d = torch.zeros(16, device="cuda")
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = lib.tg_dev_qmatvec_static(_ptr(d), _ptr(d), _ptr(d), _ptr(d), 1152, 524288, stream)
    assert rc == capi.TG_EINVAL and b"maximum" in lib.tg_last_error()
