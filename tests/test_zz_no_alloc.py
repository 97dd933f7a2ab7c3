"""The allocation-free Hyena-LI forward entry point (`sb_li_fwd_noalloc`, csrc/li_scan_noalloc.h).

Some embedders of the library may not allocate device memory at call time (all memory already belongs to
their own pool, or an allocation's device-wide synchronisation is not acceptable in their loop).  For them
the library offers one entry point whose scratch lives in a fixed 16 MiB array inside the library.  This
test calls it through its exported C symbol, twice in a row, and checks both results against the regular
entry point (`sb_li_fwd`, which takes a caller-allocated scratch buffer); it also checks that a problem
beyond the built-in buffer is refused.  The file name sorts last so that a stop-at-first-failure run has
already executed every other test.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from savanna_b200.ops import cuda_ops
    lib = cuda_ops.require()
    P, I = ctypes.c_void_p, ctypes.c_int
    lib.sb_li_fwd_noalloc.restype = I
    lib.sb_li_fwd_noalloc.argtypes = [P, P, P, P, P, P, P, I, I, I, I, P]
    return lib


def _inputs(B, L, D, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    feat = (torch.randn(B, L, 3 * D, device="cuda", generator=g) * 0.7).to(torch.bfloat16)
    gamma = (torch.rand(D, 16, device="cuda", generator=g) * 0.09 + 0.01).log()
    loglam = (-torch.exp(-torch.ones(D, 16, device="cuda")) * torch.exp(gamma)).contiguous()
    R = (0.1 * torch.randn(D, 16, device="cuda", generator=g) / 4).contiguous()
    bias = torch.randn(D, device="cuda", generator=g)
    return feat, loglam, R, bias


def _run_regular(lib, feat, loglam, R, bias, TC):
    B, L, C3 = feat.shape
    D = C3 // 3
    NC = (L + TC - 1) // TC
    S = torch.empty(B * NC * D * 16, dtype=torch.float32, device="cuda")
    z = torch.empty(B, L, D, dtype=torch.bfloat16, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    rc = lib.sb_li_fwd(feat.data_ptr(), loglam.data_ptr(), R.data_ptr(), bias.data_ptr(), None, None, S.data_ptr(),
                       z.data_ptr(), B, L, D, TC, st)
    assert rc == 0
    return z


def _run_noalloc(lib, feat, loglam, R, bias, TC):
    B, L, C3 = feat.shape
    D = C3 // 3
    z = torch.empty(B, L, D, dtype=torch.bfloat16, device="cuda")      # output only: the caller provides no scratch
    st = torch.cuda.current_stream().cuda_stream
    rc = lib.sb_li_fwd_noalloc(feat.data_ptr(), loglam.data_ptr(), R.data_ptr(), bias.data_ptr(), None, None, z.data_ptr(),
                               B, L, D, TC, st)
    assert rc == 0, f"sb_li_fwd_noalloc returned {rc}"
    return z


def _close(a, b):
    a, b = a.float(), b.float()
    scale = b.abs().max().clamp(min=1e-6)
    assert (a - b).abs().max() <= 4e-2 * scale


def test_noalloc_matches_regular_entry_point_twice():
    lib = _lib()
    TC = 128
    # call 1 and call 2 use different shapes and data, so stale scratch contents from call 1 would show in call 2
    for seed, (B, L, D) in enumerate([(2, 1000, 256), (1, 2048, 512)]):
        feat, loglam, R, bias = _inputs(B, L, D, seed)
        want = _run_regular(lib, feat, loglam, R, bias, TC)
        got = _run_noalloc(lib, feat, loglam, R, bias, TC)
        torch.cuda.synchronize()
        _close(got, want)
        assert torch.equal(got, want), "same kernels, same inputs: results should be bit-identical"


def test_noalloc_rejects_oversized_problem():
    lib = _lib()
    B, L, D, TC = 1, 8192, 8192, 128          # needs 32 MiB of chunk states: twice the built-in buffer
    feat = torch.empty(1, dtype=torch.bfloat16, device="cuda")
    rc = lib.sb_li_fwd_noalloc(feat.data_ptr(), None, None, None, None, None, None, B, L, D, TC,
                               torch.cuda.current_stream().cuda_stream)
    assert rc == -20
