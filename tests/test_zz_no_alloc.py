"""The router entry point that allocates nothing.

glmrt_b200_router_topk_bf16_f32w_static_async is for callers that may not call cudaMalloc
and have no scratch buffer of their own to pass: its logits scratch is an array compiled into
the library.  It must give exactly what the entry point with caller-provided scratch gives,
also on a second call that finds the first call's values still in the shared array, and it
must refuse problems larger than the array.

Collected last on purpose: a failure here cannot hide the result of any other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import glmrt_oracle as O

pytestmark = pytest.mark.gpu


def _ptr(t):
    return C.c_void_p(t.data_ptr())


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _run_both(lib, T, H, E, K, seed):
    rng = np.random.default_rng(seed)
    rw = torch.from_numpy((rng.standard_normal((E, H), np.float32) * np.float32(0.02)).astype(np.float32)).cuda()
    bias = torch.from_numpy((rng.standard_normal(E, np.float32) * np.float32(0.01)).astype(np.float32)).cuda()
    hid = O.make_hidden(seed + 1, T, H)
    x = torch.from_numpy(hid.view(np.int16)).view(torch.bfloat16).cuda()
    outs = []
    for static in (False, True):
        idx = torch.full((T, K), -1, dtype=torch.int32, device="cuda")
        sc = torch.zeros((T, K), dtype=torch.float32, device="cuda")
        wt = torch.zeros((T, K), dtype=torch.float32, device="cuda")
        if static:
            lib.call("glmrt_b200_router_topk_bf16_f32w_static_async", _ptr(x), _ptr(rw), _ptr(bias), _ptr(idx),
                     _ptr(sc), _ptr(wt), C.c_size_t(T), C.c_size_t(H), C.c_size_t(E), C.c_size_t(K), _stream())
        else:
            scratch = torch.empty(T * E, dtype=torch.float32, device="cuda")
            lib.call("glmrt_b200_router_topk_bf16_f32w_async", _ptr(x), _ptr(rw), _ptr(bias), _ptr(scratch),
                     _ptr(idx), _ptr(sc), _ptr(wt), C.c_size_t(T), C.c_size_t(H), C.c_size_t(E), C.c_size_t(K),
                     _stream())
        torch.cuda.synchronize()
        outs.append((idx.cpu().numpy(), sc.cpu().numpy(), wt.cpu().numpy()))
    return outs


def test_static_scratch_router_matches_the_scratch_taking_entry_point_twice(pkg):
    from glmrt_b200 import native as N
    lib = N.library()
    # two calls in a row with different shapes: the second one finds the first one's logits
    # in the shared array and must not be affected by them
    for T, H, E, K, seed in ((64, 6144, 256, 8, 3), (9, 512, 64, 4, 4)):
        (i0, s0, w0), (i1, s1, w1) = _run_both(lib, T, H, E, K, seed)
        np.testing.assert_array_equal(i1, i0)      # indices: exact
        np.testing.assert_array_equal(s1, s0)      # same kernels, same order of operations:
        np.testing.assert_array_equal(w1, w0)      # bit-identical scores and weights
        assert (i1 >= 0).all() and np.allclose(w1.sum(axis=1), 2.5, atol=1e-5)


def test_static_scratch_router_rejects_oversized_problems(pkg):
    from glmrt_b200 import native as N
    lib = N.library()
    one = torch.zeros(16, dtype=torch.float32, device="cuda")
    st = lib.call_status("glmrt_b200_router_topk_bf16_f32w_static_async", _ptr(one), _ptr(one), _ptr(one),
                         _ptr(one), _ptr(one), _ptr(one), C.c_size_t(2048), C.c_size_t(256), C.c_size_t(256),
                         C.c_size_t(8), _stream())
    assert st == 2  # GLMRT_STATUS_BUFFER_TOO_SMALL, nothing launched
    assert "262144" in lib.last_error()
