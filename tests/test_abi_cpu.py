"""The C-ABI library loads without a GPU, exports every symbol the header declares, and the
lane-level decoder passes its host-side check (compiled with g++ from the same .cuh file)."""
import ctypes
import os
import re
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from cobalt_b200 import build, _lib
    build.build()
    return _lib.load()


def test_header_symbols_exported(lib):
    hdr = open(os.path.join(ROOT, "include", "cobalt_b200.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    names = set(re.findall(r"\b(cobalt_[a-z_0-9]+)\s*\(", hdr))
    assert {"cobalt_gemv", "cobalt_gemm", "cobalt_dequant", "cobalt_unpack", "cobalt_linear_host"} <= names
    from cobalt_b200 import _lib
    assert names == set(_lib.EXPORTS), (names ^ set(_lib.EXPORTS))
    for n in names:
        assert hasattr(lib, n), n


def test_struct_layout_and_strerror(lib):
    from cobalt_b200 import _lib
    assert ctypes.sizeof(_lib.CobaltMat) == 64
    assert lib.cobalt_version() >> 16 == 1
    assert lib.cobalt_strerror(0) == b"ok"
    assert b"invalid" in lib.cobalt_strerror(-1)


def test_ctypes_mirrors_match_the_header(tmp_path):
    """Sizes and field offsets of the ctypes mirrors against the C compiler's view of include/cobalt_b200.h."""
    from cobalt_b200 import _lib
    structs = {"CobaltMat": _lib.CobaltMat, "CobaltStagedInput": _lib.CobaltStagedInput, "CobaltPeerSlots": _lib.CobaltPeerSlots}
    lines = []
    for name, cls in structs.items():
        lines.append(f'printf("{name} %zu\\n", sizeof({name}));')
        for field, _ in cls._fields_:
            lines.append(f'printf("{name}.{field} %zu\\n", offsetof({name}, {field}));')
    src = tmp_path / "layout.c"
    src.write_text('#include <stdio.h>\n#include <stddef.h>\n#include "cobalt_b200.h"\nint main(void) {\n' + "\n".join(lines) + "\nreturn 0; }\n")
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-I", os.path.join(ROOT, "include"), "-o", str(exe), str(src)], check=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout
    seen = dict(line.split() for line in out.strip().splitlines())
    for name, cls in structs.items():
        assert int(seen[name]) == ctypes.sizeof(cls), name
        for field, _ in cls._fields_:
            assert int(seen[f"{name}.{field}"]) == getattr(cls, field).offset, f"{name}.{field}"


def test_argument_validation_without_gpu(lib):
    """Host-side validation rejects bad descriptors before any CUDA call."""
    from cobalt_b200 import _lib
    m = _lib.CobaltMat()
    assert lib.cobalt_gemv(ctypes.byref(m), None, 0, None, 0, None, 1, None, 0, None) == -1
    assert lib.cobalt_unpack(None, None, None, None) == -1
    m.tiles, m.tile_off, m.K, m.N, m.bits, m.group = 4096, 4096, 16, 100, 4, 128
    assert lib.cobalt_dequant(ctypes.byref(m), None, None) == -1      # N not a multiple of 128


def test_decoder_core_host_build(tmp_path):
    exe = tmp_path / "test_decode_core"
    src = os.path.join(ROOT, "tests", "cpp", "test_decode_core.cpp")
    subprocess.run(["g++", "-O2", "-std=c++17", "-o", str(exe), src], check=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True)
    assert out.returncode == 0 and "OK" in out.stdout, out.stdout + out.stderr


def test_forward_refuses_cpu_tensor():
    import torch
    from cobalt_b200 import CobaltSparseLinear
    keep = torch.ones(16, 128, dtype=torch.bool)
    q = torch.zeros(16, 128, dtype=torch.uint8)
    sc = torch.ones(16, 1).half()
    mod = CobaltSparseLinear(q, sc, sc, keep, None, None, {"nbits": 4, "group_size": 128})
    with pytest.raises(RuntimeError):
        mod(torch.zeros(1, 128, dtype=torch.bfloat16))


def test_decoder_refuses_more_tokens_than_cache_slots():
    """The captured decode step advances the position on the device, so running past the KV cache is refused on the
    host before anything is launched."""
    from types import SimpleNamespace
    from cobalt_b200.decoder import CobaltDecoder
    d = SimpleNamespace(max_ctx=32)
    CobaltDecoder._check_room(d, 32)
    with pytest.raises(ValueError):
        CobaltDecoder._check_room(d, 33)
    with pytest.raises(ValueError):
        CobaltDecoder._check_room(d, 8, start=30)
