"""The entry point that allocates no device memory (quench6k_b200/csrc/no_alloc.h), called the way
its users call it: through the exported C symbol, with raw pointers and a stream.  Its result must
equal the regular argmax's (same kernels, other scratch), on two calls in a row that share the
built-in scratch array.  The file sorts last so that a run that stops at the first failure has
already run every other test."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _entry():
    from quench6k_b200.ops.build import library
    lib = library()
    fn = lib.q6k_argmax_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
    lib.q6k_last_error.restype = ctypes.c_char_p
    return lib, fn


def test_no_alloc_argmax_matches_the_regular_one_twice_in_a_row():
    from quench6k_b200 import ops
    lib, fn = _entry()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    g = torch.Generator().manual_seed(5)
    calls = 0
    # two calls of different shapes back to back: the second reuses the scratch the first left
    for rows, vocab in ((8, 151936), (3, 50000), (64, 9000), (1, 17)):
        logits = (torch.randn(rows, vocab, generator=g) * 4).mul(8).round().div(8).cuda()     # coarse values: many ties
        out = torch.full((rows,), -1, dtype=torch.int32, device="cuda")
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]           # what the driver says is free: sees every allocation, whoever makes it
        rc = fn(logits.data_ptr(), rows, vocab, out.data_ptr(), stream)
        assert rc == 0, lib.q6k_last_error().decode()
        torch.cuda.synchronize()
        if calls:                                            # the first call on a device may load the library's device image
            assert torch.cuda.mem_get_info()[0] == free_before, "the entry point took device memory"
        calls += 1
        want = ops.argmax(logits)
        assert torch.equal(out, want)
        cpu = logits.cpu()
        for r in range(rows):
            assert int(out[r]) == int((cpu[r] == cpu[r].max()).nonzero()[0])


def test_no_alloc_argmax_refuses_what_its_scratch_cannot_hold():
    lib, fn = _entry()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    x = torch.zeros(4, device="cuda")
    out = torch.zeros(4, dtype=torch.int32, device="cuda")
    assert fn(x.data_ptr(), 65, 10, out.data_ptr(), stream) != 0
    assert b"65 rows exceed" in lib.q6k_last_error()
    assert fn(x.data_ptr(), 1, (1 << 20) + 1, out.data_ptr(), stream) != 0
    assert b"exceeds the built-in scratch" in lib.q6k_last_error()
