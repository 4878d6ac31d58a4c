"""The entry point that allocates nothing (csrc/no_alloc.h), called through its exported C symbol
as a foreign caller would, against the ordinary entry point: two calls in a row on the library's
one fixed array, the second after NaN marks were left in it as by a call that broke off halfway.

For users of the library: `vob_pick_tokens_static` is for callers that cannot obtain scratch
buffers because they may not allocate device memory at all (all memory already handed to another
owner, or a context in which allocating CUDA calls are not allowed). This file is collected last
on purpose, so that a run that stops at the first failure has already run every other test."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _static_fn():
    from vllm_oxide_b200.csrc.build import cuda_library_path
    lib = ctypes.CDLL(cuda_library_path("sampling"))
    f = lib.vob_pick_tokens_static
    P, I, L = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
    f.argtypes = [P, L, I, I, P, P, P, P, P]
    f.restype = I
    return f


def _call_static(f, logits, temps, seeds, steps, out):
    p = lambda t: ctypes.c_void_p(t.data_ptr() if t is not None else 0)
    return f(p(logits), logits.stride(0), logits.shape[0], logits.shape[1], p(temps), p(seeds), p(steps), p(out),
             ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


def _reference(logits, temps, seeds, steps):
    from vllm_oxide_b200 import kernels
    R, V = logits.shape
    sp = kernels.pick_splits(V)
    out = torch.zeros(R, dtype=torch.int32, device=DEV)
    kernels.pick_tokens(logits, out, torch.zeros(R, dtype=torch.int32, device=DEV), torch.empty(R * sp, device=DEV),
                        torch.empty(R * sp, dtype=torch.int32, device=DEV), temps, seeds, steps)
    return out


def test_static_pick_matches_the_ordinary_entry_point_twice_in_a_row():
    f = _static_fn()
    from vllm_oxide_b200.csrc.build import cuda_library_path
    leave_marks = ctypes.CDLL(cuda_library_path("sampling")).vob_pick_static_test_leave_marks
    leave_marks.argtypes, leave_marks.restype = [ctypes.c_int, ctypes.c_void_p], ctypes.c_int
    g = torch.Generator().manual_seed(17)
    V = 128256
    for call in range(2):
        R = 8 if call == 0 else 5
        logits = (torch.randn(R, V, generator=g) * 3).to(DEV)
        if call == 0:
            logits[3, 77777] = float("nan")
        else:
            # what a call that failed between its two kernels would leave: marks on every row
            stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
            assert leave_marks(64, stream) == 0
        temps = torch.tensor([0.0, 0.7, 0.0, 0.0, 1.3, 0.7, 0.0, 0.2][:R], device=DEV)
        seeds = torch.tensor([[i + 1, 3 * i] for i in range(R)], dtype=torch.int32, device=DEV)
        steps = torch.arange(call * 10, call * 10 + R, dtype=torch.int32, device=DEV)
        out = torch.full((R,), -7, dtype=torch.int32, device=DEV)
        assert _call_static(f, logits, temps, seeds, steps, out) == 0
        torch.cuda.synchronize()
        want = _reference(logits, temps, seeds, steps)
        assert out.tolist() == want.tolist()          # token ids: exact, as in the tests of the ordinary entry point
        assert (out[3].item() == -1) == (call == 0)
    # greedy without sampling parameters, a small vocabulary that is no power of two
    small = torch.randn(3, 301, generator=g).to(DEV)
    out = torch.zeros(3, dtype=torch.int32, device=DEV)
    assert _call_static(f, small, None, None, None, out) == 0
    torch.cuda.synchronize()
    assert out.tolist() == small.argmax(dim=1).tolist()


def test_static_pick_refuses_what_does_not_fit():
    f = _static_fn()
    too_many = torch.zeros(65, 100, device=DEV)
    out = torch.zeros(65, dtype=torch.int32, device=DEV)
    assert _call_static(f, too_many, None, None, None, out) == 2003      # VOB_ERR_STATIC_TOO_LARGE
    ok = torch.zeros(64, 100, device=DEV)
    assert _call_static(f, ok, None, None, None, out[:64]) == 0
    temps = torch.ones(2, device=DEV)
    assert _call_static(f, ok[:2], temps, None, None, out[:2]) == 2001   # sampling without seeds: bad argument
    torch.cuda.synchronize()
