"""The allocation-free W8A16 entry point against the workspace-taking one.

``tybok_w8a16_linear_noalloc`` is for hosts that cannot give the library a workspace (no device
allocator of their own, or a rule against allocating once running): its scratch is a fixed
array inside the library.  It must produce exactly what ``tybok_w8a16_linear`` produces, also on
a second call that reuses the array with a different problem, and refuse problems that do not
fit.  Collected last so that a first-failure stop has already run every other test."""

import pytest
import torch

from oracle import w8_ref

pytestmark = pytest.mark.gpu


def _problem(seed, m, n, k):
    g = torch.Generator().manual_seed(seed)
    w8, scale = w8_ref.quantize_w8(torch.empty(n, k).normal_(0, 0.02, generator=g))
    x = torch.empty(m, k).normal_(0, 1, generator=g).to(torch.bfloat16)
    res = torch.empty(m, n).normal_(0, 1, generator=g).to(torch.bfloat16)
    return x.cuda(), w8.cuda(), scale.cuda(), res.cuda(), (x, w8, scale, res)


def test_noalloc_matches_workspace_entry_point_twice():
    from tybok_b200 import _lib

    lib = _lib.load()
    stream = torch.cuda.current_stream().cuda_stream
    for seed, (m, n, k) in enumerate([(50, 1024, 2048), (128, 256, 4096)]):  # second call reuses the array
        x, w8, scale, res, cpu = _problem(seed, m, n, k)
        y_ws = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
        y_na = torch.empty_like(y_ws)
        need = lib.tybok_w8a16_workspace_bytes(m, n, k, 0)
        ws = torch.empty(need, dtype=torch.uint8, device="cuda")
        rc = lib.tybok_w8a16_linear(x.data_ptr(), w8.data_ptr(), scale.data_ptr(), None, y_ws.data_ptr(), m, n, k, k, n,
                                    2, res.data_ptr(), n, None, 0, 1, 0, 0, 0, ws.data_ptr(), need, None, stream)
        assert rc == 0, lib.tybok_last_error()
        rc = lib.tybok_w8a16_linear_noalloc(x.data_ptr(), w8.data_ptr(), scale.data_ptr(), None, y_na.data_ptr(), m, n,
                                            k, k, n, 2, res.data_ptr(), n, None, 0, 1, 0, None, stream)
        assert rc == 0, lib.tybok_last_error()
        torch.cuda.synchronize()
        ref = cpu[3] + w8_ref.w8_linear(cpu[0], cpu[1], cpu[2])
        assert w8_ref.rel_l2(y_na.cpu(), ref) <= 1e-2  # the tolerance of every W8 linear test
        assert torch.equal(y_na, y_ws)  # same kernels, same planes: identical bits


@pytest.mark.parametrize("pdl", [1, 0])
def test_noalloc_calls_back_to_back_on_one_stream(pdl):
    """Two calls with different inputs queued on one stream with nothing between them: the second
    call's split kernel may not overwrite the shared array while the first call's GEMM still reads
    it.  Stream order guarantees that without programmatic dependent launch; with it, the split
    kernel's own wait for its predecessor does.  Both outputs equal the workspace entry point's."""
    from tybok_b200 import _lib

    lib = _lib.load()
    stream = torch.cuda.current_stream().cuda_stream
    m, n, k = 96, 512, 4096
    probs = [_problem(10 + i, m, n, k) for i in range(2)]
    want = []
    for x, w8, scale, res, _ in probs:
        y = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
        need = lib.tybok_w8a16_workspace_bytes(m, n, k, 0)
        ws = torch.empty(need, dtype=torch.uint8, device="cuda")
        rc = lib.tybok_w8a16_linear(x.data_ptr(), w8.data_ptr(), scale.data_ptr(), None, y.data_ptr(), m, n, k, k, n,
                                    2, res.data_ptr(), n, None, 0, 1, 0, 0, 0, ws.data_ptr(), need, None, stream)
        assert rc == 0, lib.tybok_last_error()
        want.append(y)
    torch.cuda.synchronize()
    got = [torch.empty(m, n, dtype=torch.bfloat16, device="cuda") for _ in probs]
    lib.tybok_set_pdl(pdl)
    try:
        for _ in range(3):  # several rounds, so that a race would have more than one chance to show
            for (x, w8, scale, res, _), y in zip(probs, got):
                rc = lib.tybok_w8a16_linear_noalloc(x.data_ptr(), w8.data_ptr(), scale.data_ptr(), None, y.data_ptr(), m,
                                                    n, k, k, n, 2, res.data_ptr(), n, None, 0, 1, 0, None, stream)
                assert rc == 0, lib.tybok_last_error()
        torch.cuda.synchronize()
    finally:
        lib.tybok_set_pdl(1)
    for y, ref in zip(got, want):
        assert torch.equal(y, ref)


def test_noalloc_refused_call_leaves_the_array_alone():
    """A call whose GEMM arguments are bad is refused before the split kernel runs."""
    from tybok_b200 import _lib

    lib = _lib.load()
    x, w8, scale, _, _ = _problem(7, 16, 128, 128)
    y = torch.empty(16, 128, dtype=torch.bfloat16, device="cuda")
    n0 = lib.tybok_launch_count()
    rc = lib.tybok_w8a16_linear_noalloc(x.data_ptr(), w8.data_ptr(), scale.data_ptr(), None, y.data_ptr(), 16, 126,
                                        128, 128, 128, 0, None, 0, None, 0, 1, 0, None, None)  # N % 4 != 0
    assert rc == 1 and lib.tybok_launch_count() == n0


def test_noalloc_refuses_what_does_not_fit():
    from tybok_b200 import _lib

    lib = _lib.load()
    x, w8, scale, _, _ = _problem(5, 16, 128, 128)
    y = torch.empty(16, 128, dtype=torch.bfloat16, device="cuda")
    rc = lib.tybok_w8a16_linear_noalloc(x.data_ptr(), w8.data_ptr(), scale.data_ptr(), None, y.data_ptr(), 129, 128,
                                        4096, 4096, 128, 0, None, 0, None, 0, 1, 0, None, None)
    assert rc == 3 and b"TYBOK_STATIC_PLANES_BYTES" in lib.tybok_last_error()
