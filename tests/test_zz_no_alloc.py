"""The sampler's entry point for callers that cannot allocate device memory.

Some users of the kernel library have no allocator at hand when they sample: a C host
that links the library by its symbols without PyTorch, a server that gave all free device
memory to its cache pool at start-up, a latency-critical loop that cannot afford the
device-wide synchronisation of cudaMalloc.  For them ``cj_sample_static`` runs the sampler
with its scratch in a fixed 4 MiB array inside the library instead of a caller's buffer.

This test calls it through its exported C symbol (ctypes, raw device pointers), twice in
a row with different inputs - the shared array keeps the first call's contents, which must
not leak into the second - and compares the drawn tokens with the regular entry point's,
which must be identical.  It also checks that a request larger than the array is refused.
The file sorts last so that, if it fails, every other test has already run.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _lib():
    from cajeta_llm_b200.csrc import build
    lib = ctypes.CDLL(build.build("sampling"))
    lib.cj_sample_static_capacity.restype = ctypes.c_longlong
    return lib


def _p(t):
    return ctypes.c_void_p(t.data_ptr() if t is not None else 0)


def _inputs(rows, V, seed):
    g = torch.Generator().manual_seed(seed)
    logits = (torch.randn(rows, V, generator=g) * 2.0).to(DEV)
    temperature = torch.tensor([0.0, 0.7, 1.0, 1.3][:rows] + [0.9] * max(0, rows - 4), dtype=torch.float32, device=DEV)
    top_k = torch.tensor([0, 0, 50, 7][:rows] + [0] * max(0, rows - 4), dtype=torch.int32, device=DEV)
    top_p = torch.tensor([0.0, 0.9, 0.0, 0.8][:rows] + [0.0] * max(0, rows - 4), dtype=torch.float32, device=DEV)
    penalty = torch.tensor([1.0, 1.0, 1.2, 1.0][:rows] + [1.0] * max(0, rows - 4), dtype=torch.float32, device=DEV)
    uniform = torch.rand(rows, generator=g).to(DEV)
    history = torch.randint(0, V, (3 * rows,), generator=g).to(torch.int32).to(DEV)
    offsets = torch.arange(0, 3 * rows + 1, 3, dtype=torch.int32, device=DEV)
    return logits, temperature, top_k, top_p, penalty, uniform, history, offsets


def test_static_scratch_sampler_matches_the_regular_one_on_two_calls_in_a_row():
    lib = _lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    capacity = lib.cj_sample_static_capacity()
    assert capacity == 1 << 20
    for rows, V, seed in ((4, 5003, 1), (6, 151936, 2)):          # the second call is larger and overwrites the first
        assert rows * V <= capacity
        logits, temperature, top_k, top_p, penalty, uniform, history, offsets = _inputs(rows, V, seed)
        want = torch.empty(rows, dtype=torch.int32, device=DEV)
        scratch = torch.empty(rows * V, dtype=torch.float32, device=DEV)
        st = lib.cj_sample(_p(logits), rows, V, _p(temperature), _p(top_k), _p(top_p), _p(penalty), _p(uniform),
                           _p(history), _p(offsets), _p(scratch), _p(want), stream)
        assert st == 0
        got = torch.full((rows,), -1, dtype=torch.int32, device=DEV)
        st = lib.cj_sample_static(_p(logits), rows, V, _p(temperature), _p(top_k), _p(top_p), _p(penalty), _p(uniform),
                                  _p(history), _p(offsets), _p(got), stream)
        assert st == 0
        torch.cuda.synchronize()
        assert got.cpu().tolist() == want.cpu().tolist()
        assert all(0 <= t < V for t in got.cpu().tolist())


def test_static_scratch_sampler_refuses_what_does_not_fit():
    lib = _lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rows, V = 8, 151936                                           # 1.2 M floats: more than the array holds
    logits, temperature, top_k, top_p, penalty, uniform, history, offsets = _inputs(rows, V, 3)
    out = torch.full((rows,), -1, dtype=torch.int32, device=DEV)
    st = lib.cj_sample_static(_p(logits), rows, V, _p(temperature), _p(top_k), _p(top_p), _p(penalty), _p(uniform),
                              _p(history), _p(offsets), _p(out), stream)
    torch.cuda.synchronize()
    assert st == -6                                               # CJ_SAMPLE_STATIC_TOO_LARGE
    assert out.cpu().tolist() == [-1] * rows                      # nothing was launched
