"""`fz_argmax_no_alloc`: the argmax entry point for callers that may not allocate device memory (a host program that owns
all device memory through a pool of its own, a loop that cannot afford an allocation's synchronisation, a sandbox that
bans allocating calls after start-up). It is called here through its exported C symbol, twice in a row, and must give what
the ordinary entry point (`fz_argmax`, with caller-allocated scratch) gives; a call beyond its fixed scratch is refused.
This file is named so that pytest collects it last."""
import ctypes
from ctypes import c_int, c_void_p

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_argmax_without_allocation_matches_the_ordinary_entry_point():
    from fusezap_core_b200.kernels import cuda_ops
    from fusezap_core_b200.kernels.build import load
    lib = load("fzb200_core")
    lib.fz_no_alloc_last_error.restype = ctypes.c_char_p
    ops = cuda_ops("float32")
    side = torch.cuda.Stream()
    g = torch.Generator().manual_seed(12)
    cases = []
    for rows, vocab in ((37, 50021), (200, 1511)):
        logits = (torch.randn(rows, vocab, generator=g) * 4).cuda()
        logits[1, 7] = logits[1, vocab - 3] = 99.0              # a tie: the first index wins
        logits[2, 100] = float("nan")                           # a NaN is the maximum
        want = torch.empty(rows, dtype=torch.int32, device="cuda")
        ops.argmax(logits, want)
        cases.append((logits, want, torch.full((rows,), -1, dtype=torch.int32, device="cuda")))
    torch.cuda.synchronize()
    free_before = None
    for call, (logits, want, got) in enumerate(cases):         # two calls in a row share the scratch
        rows, vocab = logits.shape
        if call == 0:
            stream = torch.cuda.current_stream()
        else:
            # The second call goes to another stream. Calls that overlap on the GPU would race on the shared scratch, so
            # it is ordered behind the first with an event, as the header asks. By now the first call has looked the
            # scratch's address up, so from here on the driver's count of free device memory must not move: that count,
            # unlike torch's own, would show a cudaMalloc made inside the library.
            done = torch.cuda.Event()
            done.record(torch.cuda.current_stream())
            side.wait_event(done)
            stream = side
            torch.cuda.synchronize()
            free_before = torch.cuda.mem_get_info()[0]
        status = lib.fz_argmax_no_alloc(c_void_p(logits.data_ptr()), c_void_p(got.data_ptr()), c_int(rows), c_int(vocab),
                                        c_void_p(stream.cuda_stream))
        assert status == 0, lib.fz_no_alloc_last_error().decode()
        stream.synchronize()
        if free_before is not None:
            assert torch.cuda.mem_get_info()[0] == free_before, "the call changed the device's free memory"
        assert torch.equal(got, want), f"call {call}: rows {torch.where(got != want)[0].tolist()[:8]} differ"
        assert got.cpu().tolist() == np.argmax(logits.cpu().numpy(), -1).tolist()
    too_many = torch.zeros(257, 16, device="cuda")
    out = torch.zeros(257, dtype=torch.int32, device="cuda")
    status = lib.fz_argmax_no_alloc(c_void_p(too_many.data_ptr()), c_void_p(out.data_ptr()), c_int(257), c_int(16),
                                    c_void_p(torch.cuda.current_stream().cuda_stream))
    assert status == 1004 and b"at most 256 rows" in lib.fz_no_alloc_last_error()
