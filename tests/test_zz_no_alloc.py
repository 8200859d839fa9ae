"""The allocation-free GEMM entry point (``onecat_gemm_bf16_splitk_noalloc``) called through its exported C symbol.

It serves callers that cannot allocate device memory at the call site (code inside another framework's memory-planned
region, latency-critical loops where cudaMalloc's implicit synchronisation is unacceptable, C programs that link the library
without PyTorch's caching allocator). Its split-K scratch is a fixed array inside the library, so the test checks that (a) the
result equals the regular entry point's, which takes its workspace from the caller, (b) a second call right after the first one
is still right although both share the scratch, and (c) oversized problems are refused instead of overrunning the array."""
import ctypes
import gc

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from onecat_vllm.ops import _C  # loads the shared object that exports the symbol
    lib = ctypes.CDLL(_C.__file__)
    fn = lib.onecat_gemm_bf16_splitk_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_int] * 7 + [ctypes.c_void_p]
    return fn


def _call(fn, x, w, out, splits):
    T, K = x.shape
    N = w.shape[0]
    return fn(x.data_ptr(), w.data_ptr(), out.data_ptr(), T, N, K, x.stride(0), w.stride(0), out.stride(0), splits,
              torch.cuda.current_stream().cuda_stream)


def test_noalloc_gemm_matches_regular_entry_point_twice_in_a_row():
    from onecat_vllm.ops import cuda as K
    fn = _lib()
    g = torch.Generator(device="cuda").manual_seed(11)
    # decode-sized and prefill-sized token tiles, a ragged last weight tile (N = 200), and the one-split path
    for (T, N, Kd, splits) in [(48, 640, 1280, 4), (5, 1024, 2048, 8), (300, 200, 1280, 1), (300, 640, 1280, 2), (130, 200, 2048, 4)]:
        x = torch.randn(T, Kd, device="cuda", generator=g).bfloat16()
        w = (torch.randn(N, Kd, device="cuda", generator=g) * 0.05).bfloat16()
        expect = K.gemm_bf16(x, w, force_splits=splits)
        ref32 = x.float() @ w.float().t()
        for attempt in range(2):  # the second call reuses the scratch the first one left behind
            out = torch.full((T, N), float("nan"), device="cuda", dtype=torch.bfloat16)
            # the collector may free tensors that earlier tests left in reference cycles at any Python allocation: run it now and
            # keep it off while the allocator's counter is compared
            gc.collect()
            gc.disable()
            try:
                before = torch.cuda.memory_allocated()
                rc = _call(fn, x, w, out, splits)
                assert rc == 0, f"entry point returned {rc}"
                torch.cuda.synchronize()
                assert torch.cuda.memory_allocated() == before, "the entry point must not allocate through the caching allocator"
            finally:
                gc.enable()
            err = (out.float() - expect.float()).abs()
            tol = 2e-2 + 2e-2 * expect.float().abs()
            assert bool((err <= tol).all()), f"call {attempt}: max deviation {float(err.max())} from the regular entry point"
            assert bool(((out.float() - ref32).abs() <= 5e-2 + 2e-2 * ref32.abs()).all())
    assert K.check_status() == 0


def test_noalloc_gemm_rejects_what_does_not_fit():
    fn = _lib()
    x = torch.zeros(4096, 1024, device="cuda", dtype=torch.bfloat16)
    w = torch.zeros(8192, 1024, device="cuda", dtype=torch.bfloat16)
    out = torch.zeros(4096, 8192, device="cuda", dtype=torch.bfloat16)
    assert _call(fn, x, w, out, 4) == -2  # ONECAT_NOALLOC_TOO_LARGE: more tiles / partial bytes than the fixed scratch holds
    assert _call(fn, x[:8], w[:256], out[:8, :256], 64) == -1  # more splits than k tiles: bad argument
    assert _call(fn, x[:8, :1000], w[:256], out[:8, :256], 1) == -1  # K not a multiple of 64
