"""ember_gemm_tc_noalloc, the entry point for callers that cannot allocate device memory (a host
that gave its whole memory budget away at start-up, a loop that cannot afford the device
synchronisation of cudaMalloc, a plug-in without an allocator): called through its exported C
symbol, twice in a row, and compared with the regular entry point.

This file sorts last on purpose: a run that stops at the first failure has then already run
every other test.  It passes alone in a fresh process and after the others."""
import ctypes
from ctypes import c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu


def rel(a, b):
    a, b = a.double().flatten(), b.double().flatten()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def call_noalloc(lib, a, w, out, M, epilogue, err):
    N, K = w.shape
    ldc = out.shape[-1]
    fn = lib.ember_gemm_tc_noalloc            # the exported C symbol itself, not a Python wrapper
    fn.restype = c_int
    rc = fn(c_void_p(a.data_ptr()), c_void_p(w.data_ptr()), c_void_p(out.data_ptr()), c_int(ldc), c_int(M), c_int(N),
            c_int(K), c_int(epilogue), c_void_p(err.data_ptr()), c_void_p(torch.cuda.current_stream().cuda_stream))
    return rc, lib.ember_last_error().decode()


def test_noalloc_matches_the_regular_entry_point_twice_in_a_row():
    from ember_b200 import ops
    from ember_b200.csrc import build
    lib = build.load("no_alloc")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    torch.manual_seed(3)
    # two calls in a row that share the built-in scratch: the second is smaller and uses another
    # epilogue, so anything the first left behind would show; then the first shape once more
    cases = [(8, 4096, 2048, 0), (5, 1024, 1536, 3), (8, 4096, 2048, 1), (64, 2048, 6144, 2)]
    free_after_setup = None
    for M, N, K, epilogue in cases:
        a = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
        w = (torch.randn(N, K, device="cuda") * 0.5).bfloat16()
        n_out = N // 2 if epilogue == 3 else N
        prev = torch.randn(M, n_out, device="cuda")
        odt = torch.bfloat16 if epilogue in (0, 3) else torch.float32
        want = prev.clone().to(odt)
        got = prev.clone().to(odt)
        ops.gemm_tc(a, w, want, M, epilogue, err=err)                      # the existing entry point
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        rc, msg = call_noalloc(lib, a, w, got, M, epilogue, err)
        assert rc == 0, msg
        torch.cuda.synchronize()
        # the first call loads the library's device code (its 4 MiB array with it); after that set-up
        # no call changes the free device memory: nothing is allocated
        if free_after_setup is None:
            free_after_setup = torch.cuda.mem_get_info()[0]
            free_before = None
        else:
            assert torch.cuda.mem_get_info()[0] == free_before
        assert int(err.item()) == 0
        tol = 5e-3 if epilogue in (0, 3) else 1e-5                         # the tolerances of the kernel tests
        assert rel(got.float(), want.float()) < tol
        ref = a.float() @ w.float().t()
        if epilogue == 3:
            ref = ref[:, 0::2] / (1 + torch.exp(-ref[:, 0::2])) * ref[:, 1::2]
        elif epilogue == 2:
            ref = prev + ref
        assert rel(got.float(), ref) < tol


def test_noalloc_refuses_what_does_not_fit():
    from ember_b200.csrc import build
    lib = build.load("no_alloc")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    a = torch.zeros(128, 64, device="cuda", dtype=torch.bfloat16)
    w = torch.zeros(16384, 64, device="cuda", dtype=torch.bfloat16)
    out = torch.zeros(128, 16384, device="cuda", dtype=torch.bfloat16)
    rc, msg = call_noalloc(lib, a, w, out, 128, 0, err)                    # 128 * 16384 floats > 4 MiB of scratch
    assert rc != 0 and "exceeds the built-in scratch" in msg
    big = torch.zeros(200, 64, device="cuda", dtype=torch.bfloat16)
    rc, msg = call_noalloc(lib, big, w[:64].contiguous(), out, 200, 0, err)
    assert rc != 0 and "up to 128 rows" in msg
    # a row stride shorter than the output's width would write past the caller's rows: refused, like a null output
    from ctypes import c_int, c_void_p
    small_w = w[:256].contiguous()
    narrow = torch.zeros(8, 128, device="cuda", dtype=torch.bfloat16)
    fn = lib.ember_gemm_tc_noalloc
    rc = fn(c_void_p(a.data_ptr()), c_void_p(small_w.data_ptr()), c_void_p(narrow.data_ptr()), c_int(128), c_int(8),
            c_int(256), c_int(64), c_int(0), c_void_p(err.data_ptr()), c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc != 0 and "shorter than" in lib.ember_last_error().decode()
    rc = fn(c_void_p(a.data_ptr()), c_void_p(small_w.data_ptr()), c_void_p(0), c_int(256), c_int(8), c_int(256), c_int(64),
            c_int(0), c_void_p(err.data_ptr()), c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc != 0 and "must not be null" in lib.ember_last_error().decode()
