"""The argmax entry point that allocates nothing, called through its exported C symbol.

Some hosts of these kernels cannot call cudaMalloc (all device memory went to a pool of
their own at start-up, or their loop cannot take the synchronisation an allocation implies),
so ``einf_argmax_no_alloc`` keeps its scratch in a device array inside the library.  Here it
runs twice in a row on different inputs, as a caller's loop would, and must agree exactly
with the ordinary entry point both times; more rows than its fixed scratch holds are refused.
This file sorts last on purpose: a run that stops at the first failure has then already
run every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_ROWS = 256


def load_library():
    from einf_b200.ops import build

    library = ctypes.CDLL(str(build.build_kernel_library("sampling")))
    function = library.einf_argmax_no_alloc
    function.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    function.restype = ctypes.c_int
    library.einf_argmax_no_alloc_strerror.argtypes = [ctypes.c_int]
    library.einf_argmax_no_alloc_strerror.restype = ctypes.c_char_p
    return library


def test_no_alloc_argmax_twice_in_a_row():
    from einf_b200 import ops

    library = load_library()
    device = torch.device("cuda:0")
    torch.cuda.set_device(device)
    stream = torch.cuda.current_stream().cuda_stream
    # the third call follows one that used every row of the scratch: what that call left there
    # (partial pairs of 256 rows, counters that were counted up) must not reach this one
    for call, (rows, vocab, seed) in enumerate([(7, 151936, 0), (MAX_ROWS, 331, 1), (5, 4099, 2)]):
        generator = torch.Generator(device=device).manual_seed(seed)
        logits = torch.randn((rows, vocab), generator=generator, device=device)
        logits[0, vocab - 1] = logits[0, 3] = 99.0          # a tie: the first index wins
        got = torch.full((rows,), -1, dtype=torch.int32, device=device)
        want = torch.full((rows,), -2, dtype=torch.int32, device=device)
        code = library.einf_argmax_no_alloc(logits.data_ptr(), got.data_ptr(), rows, vocab, stream)
        assert code == 0, library.einf_argmax_no_alloc_strerror(code).decode()
        ops.argmax(logits, want)
        torch.cuda.synchronize()
        assert torch.equal(got, want), f"call {call}"
        assert int(got[0]) == 3
        # row 0 holds the tie, on which torch.argmax promises nothing: it is checked above
        assert torch.equal(got[1:].long(), torch.argmax(logits[1:], dim=-1))


def test_no_alloc_argmax_refuses_what_its_scratch_cannot_hold():
    library = load_library()
    device = torch.device("cuda:0")
    torch.cuda.set_device(device)
    rows = MAX_ROWS + 1
    logits = torch.zeros((rows, 8), device=device)
    tokens = torch.full((rows,), -5, dtype=torch.int32, device=device)
    stream = torch.cuda.current_stream().cuda_stream
    code = library.einf_argmax_no_alloc(logits.data_ptr(), tokens.data_ptr(), rows, 8, stream)
    assert code == -1
    assert b"256" in library.einf_argmax_no_alloc_strerror(code)
    assert library.einf_argmax_no_alloc(None, None, 4, 8, stream) == -2
    torch.cuda.synchronize()
    assert int((tokens != -5).sum()) == 0     # nothing was launched
    assert library.einf_argmax_no_alloc(logits.data_ptr(), tokens.data_ptr(), 0, 8, stream) == 0
