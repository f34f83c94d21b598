"""The allocation-free argmax entry point, called through its exported C symbol.

Some users of the kernel library cannot allocate device memory when they need a token: a serving
loop that froze its allocator after start-up, or code running inside another runtime that owns all
device memory.  ``cb_argmax_static`` serves them with scratch memory built into the library.  This
test drives it exactly as such a caller would (ctypes, raw pointers, no wrapper) and checks it
against the ordinary ``cb_argmax`` entry point on two consecutive calls, since the built-in scratch
is reused from call to call.  It is collected last so that a failure here cannot hide others.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_static_argmax_matches_regular_entry_point_twice():
    from coffin_b200.ops import _lib, kernels as K
    lib = _lib.lib()
    fn = lib.cb_argmax_static
    fn.restype = ctypes.c_int
    lib.cb_argmax_static_max_rows.restype = ctypes.c_int64
    max_rows = int(lib.cb_argmax_static_max_rows())
    assert max_rows == 64
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def static_argmax(logits):
        out = torch.full((logits.shape[0],), -1, dtype=torch.int64, device="cuda")
        rc = fn(ctypes.c_void_p(logits.data_ptr()), ctypes.c_void_p(out.data_ptr()), ctypes.c_int64(logits.shape[0]),
                ctypes.c_int64(logits.shape[1]), ctypes.c_int64(logits.stride(0)), stream)
        assert rc == 0, f"cb_argmax_static returned {rc}"
        return out

    g = torch.Generator().manual_seed(7)
    for call, (rows, vocab) in enumerate([(5, 151936), (64, 4099)]):      # two calls in a row, different shapes
        logits = torch.randn(rows, vocab, generator=g).cuda()
        logits[0, 17] = logits[0, vocab - 1] = 99.0                       # a tie: lowest index wins
        got = static_argmax(logits)
        ref = K.argmax(logits)                                            # the existing entry point
        torch.cuda.synchronize()
        assert torch.equal(got, ref), f"call {call}: static and regular entry points disagree"
        assert torch.equal(got.cpu(), logits.cpu().argmax(-1)) and int(got[0]) == 17
    # sizes beyond the built-in scratch are refused with the shape error, nothing is launched
    big = torch.zeros(max_rows + 1, 8, device="cuda")
    out = torch.zeros(max_rows + 1, dtype=torch.int64, device="cuda")
    rc = fn(ctypes.c_void_p(big.data_ptr()), ctypes.c_void_p(out.data_ptr()), ctypes.c_int64(max_rows + 1),
            ctypes.c_int64(8), ctypes.c_int64(8), stream)
    assert rc == 10001
