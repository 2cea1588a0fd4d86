"""The allocation-free GEMM entry point, called through its exported C symbol.

Who needs it: callers that may not allocate device memory where they run the GEMM (inside a stream
capture, in a loop that must stay off the allocator's lock, or beside a framework that owns all of
the device's memory).  The library keeps the split-K scratch in a fixed array of its own, so the
call takes only inputs and outputs.  This test checks it against the ordinary entry point, twice in
a row (the second call meets whatever the first left in the shared array), and checks the refusal
of a problem that does not fit the array.  It is collected last on purpose.
"""
import ctypes as C

import pytest
import torch

from saber_engine_b200.ops import functional as F
from saber_engine_b200.ops import layouts as L
from saber_engine_b200.ops import native as N

pytestmark = pytest.mark.gpu


def _noalloc():
    fn = N.lib().saber_gemm_i8_noalloc
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p] * 6 + [C.c_int] * 9 + [C.c_void_p]
    return fn


def _operands(M, Nn, K, bits, seed):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(Nn, K, generator=g) * 0.02
    x = torch.randn(M, K, generator=g)
    qw = F.QuantWeight.from_float(w, bits, "cuda")
    qa = F.plain_quant(x.to(torch.bfloat16).cuda())
    return qw, qa


@pytest.mark.parametrize("M,Nn,K,bits,splits", [(9, 512, 2048, 4, 4), (40, 768, 1024, 8, 2), (5, 256, 512, 4, 1)])
def test_matches_the_allocating_entry_point_on_two_calls_in_a_row(M, Nn, K, bits, splits):
    fn = _noalloc()
    for call in range(2):
        qw, qa = _operands(M, Nn, K, bits, seed=10 * call + M)
        want = F.gemm_i8(qw, qa, splits=splits)
        got = torch.full((M, Nn), float("nan"), dtype=torch.bfloat16, device="cuda")
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        rc = fn(qw.tiles.data_ptr(), qw.scale.data_ptr(), qa.q.data_ptr(), qa.scale.data_ptr(), got.data_ptr(),
                status.data_ptr(), M, qa.M_pad, Nn, qw.N_pad, K, L.token_tile(M), splits, int(qw.w4), got.stride(0),
                N.stream_handle())
        assert rc == 0
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        F.scratch("cuda").check()
        # same kernel, same operands: the tolerance of the GEMM tests holds with room to spare
        err = (got.float() - want.float()).abs().max().item()
        assert err <= 1e-2 * want.float().abs().max().item() + 1e-6
        assert torch.equal(got, want)


def test_refuses_a_problem_larger_than_its_array():
    fn = _noalloc()
    z = torch.zeros(16, dtype=torch.uint8, device="cuda")
    # 16 splits x 128 rows x 262144 columns of int32 partials: far beyond the 4 Mi ints it holds
    rc = fn(z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(), None, 128, 128, 262144, 262144,
            2048, 128, 16, 1, 262144, N.stream_handle())
    assert rc == -2
    torch.cuda.synchronize()
