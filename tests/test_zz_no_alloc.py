"""cobalt_gemv_static(): the GEMV for callers that may not allocate device memory (plug-ins
in a serving process whose memory pool is frozen after start-up, real-time loops that cannot
take the synchronisation an allocation implies, processes at their memory limit).  Its split-K scratch is a fixed array inside the library instead of a buffer
the caller sizes and owns.  The test calls it through the C ABI twice in a row -- the second
call inherits whatever the first one left in the shared array -- and requires the same bits
as the ordinary entry point, then checks that an oversized request is refused cleanly.

Collected last on purpose (file name), so a stop-at-first-failure run has already run
everything else.
"""
import ctypes

import pytest
import torch

from cobalt_b200 import CobaltSparseLinear, _lib
from oracle import cobalt_oracle as O

pytestmark = pytest.mark.gpu


def _module(K, N, bits, seed):
    raw = O.synth_raw(K, N, 0.5, bits, seed=seed)
    return CobaltSparseLinear(raw["q"].cuda(), raw["scale"].cuda(), raw["zero"].cuda(), raw["keep"].cuda(), None, None,
                              {"nbits": bits})


def _static_call(lib, mod, x):
    y = torch.empty(x.shape[0], mod.out_features, dtype=torch.bfloat16, device="cuda")
    rc = lib.cobalt_gemv_static(ctypes.byref(mod._descriptor()), x.data_ptr(), x.stride(0), y.data_ptr(), y.stride(0),
                                None, x.shape[0], torch.cuda.current_stream().cuda_stream)
    return rc, y


def test_static_scratch_gemv_matches_regular_entry_point_twice():
    lib = _lib.load()
    mod = _module(640, 2048, 4, 21)          # 40 row blocks x 4 column tiles: row blocks are split over warps
    other = _module(192, 1536, 3, 22)        # a different matrix in between dirties the shared array
    free_after_first = None
    for call, M in enumerate((1, 8)):
        x = O.seeded_activation(M, 2048, 300 + call).cuda()
        want = mod(x)                                         # cobalt_gemv with a caller-owned scratch buffer
        xo = O.seeded_activation(4, 1536, 400 + call).cuda()
        want_o = other(xo)
        torch.cuda.synchronize()
        if call == 1:                                         # the first call has resolved the array's address
            free_after_first = torch.cuda.mem_get_info()[0]
        rc, got = _static_call(lib, mod, x)
        assert rc == 0, lib.cobalt_strerror(rc)
        rc, got_o = _static_call(lib, other, xo)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.equal(got, want), f"call {call}: static-scratch result differs"
        assert torch.equal(got_o, want_o)
        if call == 1:
            # the property in the name: the calls themselves take no device memory (the outputs come from the
            # caching allocator's pool, which this test warmed with the same shapes in the first round)
            assert torch.cuda.mem_get_info()[0] == free_after_first
    status = ctypes.c_uint32(7)
    assert lib.cobalt_device_status(None, torch.cuda.current_stream().cuda_stream, ctypes.byref(status)) == 0
    assert status.value == 0                                  # the private array's status word is readable and clean
    # oracle check of the last result as well (rel-L2 bar of the other GEMV tests)
    raw = O.synth_raw(640, 2048, 0.5, 4, seed=21)
    Wb = O.dequantize(raw["q"], raw["scale"], raw["zero"], raw["keep"]).to(torch.bfloat16)
    ref = torch.matmul(x.cpu(), Wb.t())
    rel = float((got.cpu().double() - ref.double()).norm() / ref.double().norm())
    assert rel <= 1e-3


def test_static_scratch_rejects_oversized_request():
    lib = _lib.load()
    mod = _module(64, 512, 4, 23)
    d = _lib.CobaltMat()
    ctypes.memmove(ctypes.byref(d), ctypes.byref(mod._descriptor()), ctypes.sizeof(d))
    d.K = 16 * 3_000_000                       # pretend: far more row blocks than the array has counters for
    d.n_row_blocks = 3_000_000                 # (12 MB of arrival counters; the partition arithmetic still fits 32 bits)
    need = lib.cobalt_gemv_scratch_bytes(ctypes.byref(d), 1)
    assert need > 8 << 20                      # a caller-owned buffer could serve it, the 8 MiB array cannot
    x = torch.zeros(1, 512, dtype=torch.bfloat16, device="cuda")
    y = torch.zeros(1, 16, dtype=torch.bfloat16, device="cuda")
    rc = lib.cobalt_gemv_static(ctypes.byref(d), x.data_ptr(), 512, y.data_ptr(), d.K, None, 1,
                                torch.cuda.current_stream().cuda_stream)
    assert rc == -6 and b"maximum" in lib.cobalt_strerror(rc)
