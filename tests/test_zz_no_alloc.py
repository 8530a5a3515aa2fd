"""The allocation-free argmax entry point (for callers that cannot use the CUDA allocator: host
callbacks, real-time threads, processes without a memory pool of their own) against the ordinary
one, through the C ABI.  Collected last on purpose."""
import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def test_argmax_noalloc_matches_argmax_twice_in_a_row(cuda_lib):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from wick_b200 import ops
    rng = np.random.default_rng(21)
    out = torch.empty(1, dtype=torch.int32, device="cuda")       # the caller's buffer: nothing is allocated inside
    for rnd, n in enumerate((65536, 70001)):                     # two calls in a row share the fixed scratch
        x = rng.standard_normal(n, dtype=np.float32)
        x[[7, n // 2, n - 3]] = x.max() + 1.0                    # equal maxima: the last index wins
        if rnd == 1:
            x[n - 3] = np.nan                                    # NaN never wins
        t = torch.from_numpy(x).cuda()
        want = int(ops.argmax(t).cpu()[0])
        got = int(ops.argmax_noalloc(t, out).cpu()[0])
        assert got == want == (n - 3 if rnd == 0 else n // 2)
    # small and ragged sizes, straight after a large one (stale partials must not leak in)
    for n in (1, 5, 1023, 1024, 1025, 4097):
        x = torch.from_numpy(rng.standard_normal(n, dtype=np.float32)).cuda()
        assert int(ops.argmax_noalloc(x, out).cpu()[0]) == int(ops.argmax(x).cpu()[0])


def test_argmax_noalloc_rejects_oversize(cuda_lib):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from wick_b200 import ops, _lib
    x = torch.zeros(8, dtype=torch.float32, device="cuda")
    out = torch.empty(1, dtype=torch.int32, device="cuda")
    code = cuda_lib.wick_cuda_argmax_noalloc(x.data_ptr(), ops.ARGMAX_NOALLOC_MAX + 1, out.data_ptr(), None)
    assert code == _lib.ERR_BAD_ARG
    assert b"exceed the fixed scratch" in cuda_lib.wick_cuda_argmax_noalloc_last_error()
    assert cuda_lib.wick_cuda_argmax_noalloc(None, 8, out.data_ptr(), None) == _lib.ERR_BAD_ARG
