"""The argmax entry point that allocates nothing, called through its exported C symbol.

Some callers hold a CUDA context but cannot allocate device memory where they run (a plug-in
whose host owns all device memory, a loop that must stay clear of the allocator, code running
beside a stream capture).  For them the library exports `tau_argmax_static`, which keeps its
scratch in a fixed array inside the library (see tau.rs_b200/csrc/sampling_static.h).  This test
calls the symbol directly with raw device pointers, twice in a row, and compares each result with
the ordinary entry point's, which must agree exactly: both choose one token id per row.
The file sorts last so that a run that stops at the first failure has run every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
STATIC_WORDS = 24576


def exported():
    from tau_rs_b200.csrc import build

    library = build.load_library("sampling.cu")
    function = library.tau_argmax_static
    function.restype = ctypes.c_int
    function.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    library.tau_argmax_static_error.restype = ctypes.c_char_p
    library.tau_argmax_static_error.argtypes = [ctypes.c_int]
    library.tau_argmax_static_words_needed.restype = ctypes.c_longlong
    library.tau_argmax_static_words_needed.argtypes = [ctypes.c_int, ctypes.c_int]
    return library, function


def logits_for(rows, vocab, seed):
    generator = torch.Generator().manual_seed(seed)
    logits = torch.randn(rows, vocab, generator=generator) * 3.0
    logits[0, vocab // 3] = float("nan")
    if rows > 1:
        logits[1, :] = float("nan")                 # a row of NaN only is reported, not chosen from
        logits[rows - 1, -1] = logits[rows - 1].max() if rows > 2 else logits[rows - 1, -1]   # a tie: the highest id wins
    return logits.cuda()


def test_static_argmax_agrees_with_the_ordinary_entry_point_twice_in_a_row():
    from tau_rs_b200.csrc import kernels

    library, function = exported()
    stream = torch.cuda.current_stream().cuda_stream
    # The second call is smaller than the first, so it meets scratch words that the first call left behind.
    for rows, vocab, seed in ((8, 151936, 1), (3, 5000, 2)):
        assert library.tau_argmax_static_words_needed(rows, vocab) <= STATIC_WORDS
        logits = logits_for(rows, vocab, seed)
        wanted_tokens = torch.empty(rows, dtype=torch.int32, device="cuda")
        wanted_valid = torch.empty(rows, dtype=torch.int32, device="cuda")
        kernels.argmax(logits, wanted_tokens, wanted_valid)
        tokens = torch.full((rows,), -5, dtype=torch.int32, device="cuda")
        valid = torch.full((rows,), -5, dtype=torch.int32, device="cuda")
        code = function(logits.data_ptr(), rows, vocab, tokens.data_ptr(), valid.data_ptr(), stream)
        assert code == 0, library.tau_argmax_static_error(code).decode()
        torch.cuda.synchronize()
        assert torch.equal(valid, wanted_valid)
        live = wanted_valid.bool()
        assert torch.equal(tokens[live], wanted_tokens[live])
        assert int(valid[1]) == 0 and int(valid[0]) == 1


def test_static_argmax_refuses_what_does_not_fit():
    library, function = exported()
    rows, vocab = 65, 262144          # 65 * 128 * 3 words: one row too many
    assert library.tau_argmax_static_words_needed(rows, vocab) > STATIC_WORDS
    logits = torch.zeros(1, 16, device="cuda")       # never read: the call is refused before any launch
    tokens = torch.full((1,), -5, dtype=torch.int32, device="cuda")
    code = function(logits.data_ptr(), rows, vocab, tokens.data_ptr(), tokens.data_ptr(), 0)
    assert code == -1 and b"exceeds" in library.tau_argmax_static_error(code)
    assert function(None, 1, 16, tokens.data_ptr(), tokens.data_ptr(), 0) == -2
    torch.cuda.synchronize()
    assert int(tokens[0]) == -5
