"""CPU checks of the C ABI: the library loads, exports every symbol that
include/fa_b200.h declares, the ctypes mirror of fa_fwd_params has the C layout,
and the pure-host entry points behave (no compute call needs a GPU here)."""
import ctypes
import json
import os
import re
import subprocess
import tempfile

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "fa_b200.h")


@pytest.fixture(scope="module")
def lib():
    from flash_attn_b200 import _lib, build
    build.build()
    return _lib.load()


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fa_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    from flash_attn_b200 import _lib
    names = declared_functions()
    assert "fa_fwd" in names and "fa_fwd_host" in names and len(names) >= 10
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in fa_b200.h but not exported"
    assert sorted(_lib.EXPORTS) == names


def test_struct_layout_matches_the_header():
    from flash_attn_b200 import _lib
    fields = [f[0] for f in _lib.FwdParams._fields_]
    src = '#include <stdio.h>\n#include <stddef.h>\n#include "fa_b200.h"\nint main(void){printf("%zu", sizeof(fa_fwd_params));\n'
    for f in fields:
        src += f'printf(" %zu", offsetof(fa_fwd_params, {f}));\n'
    src += "return 0;}\n"
    with tempfile.TemporaryDirectory() as tmp:
        c = os.path.join(tmp, "layout.c")
        open(c, "w").write(src)
        exe = os.path.join(tmp, "layout")
        subprocess.check_call(["/usr/bin/gcc" if os.path.exists("/usr/bin/gcc") else "gcc", "-std=c99", "-I",
                               os.path.join(ROOT, "include"), c, "-o", exe])
        out = subprocess.check_output([exe]).decode().split()
    assert int(out[0]) == ctypes.sizeof(_lib.FwdParams)
    for f, off in zip(fields, out[1:]):
        assert getattr(_lib.FwdParams, f).offset == int(off), f


def test_ring_struct_layout_matches_the_header():
    from flash_attn_b200 import _lib
    fields = [f[0] for f in _lib.RingParams._fields_]
    src = '#include <stdio.h>\n#include <stddef.h>\n#include "fa_b200.h"\nint main(void){printf("%zu", sizeof(fa_ring_params));\n'
    for f in fields:
        src += f'printf(" %zu", offsetof(fa_ring_params, {f}));\n'
    src += "return 0;}\n"
    with tempfile.TemporaryDirectory() as tmp:
        c = os.path.join(tmp, "layout.c")
        open(c, "w").write(src)
        exe = os.path.join(tmp, "layout")
        subprocess.check_call(["/usr/bin/gcc" if os.path.exists("/usr/bin/gcc") else "gcc", "-std=c99", "-I",
                               os.path.join(ROOT, "include"), c, "-o", exe])
        out = subprocess.check_output([exe]).decode().split()
    assert int(out[0]) == ctypes.sizeof(_lib.RingParams)
    for f, off in zip(fields, out[1:]):
        assert getattr(_lib.RingParams, f).offset == int(off), f


def test_ring_entry_points_reject_bad_arguments(lib):
    from flash_attn_b200 import _lib
    p = _lib.RingParams()
    assert lib.fa_ring_message_bytes(ctypes.byref(p)) == 0
    assert lib.fa_ring_fwd(ctypes.byref(p)) == -1  # world = 0
    p.world, p.rank = 2, 0
    assert lib.fa_ring_fwd(ctypes.byref(p)) == -1  # no communicator, no buffers
    p.batch, p.heads, p.chunk_rows, p.head_dim, p.dtype = 1, 32, 8192, 128, _lib.FA_DTYPE_BF16
    assert lib.fa_ring_message_bytes(ctypes.byref(p)) == 4 * 32 * 8192 * 128 * 2  # 268 MB per ring step at 8 GPUs


def test_split_policy_matches_reference_table(lib, golden_dir):
    t = json.load(open(os.path.join(golden_dir, "num_splits_heuristic.json")))
    for a, b, c, d, e, want in t["rows"]:
        assert lib.fa_num_splits_heuristic(a, b, c, d, e) == want, (a, b, c, d, e)


def test_error_paths_without_a_gpu(lib):
    from flash_attn_b200 import _lib
    assert lib.fa_version() == 100
    assert lib.fa_fwd(None) == -1
    assert lib.fa_fwd_host(None) == -1
    assert lib.fa_fwd_static_scratch(None) == -1
    p = _lib.FwdParams()
    assert lib.fa_fwd(ctypes.byref(p)) == -1           # NULL tensors
    p.q = p.k = p.v = p.o = 4096
    p.batch = p.heads = 1
    p.seqlen_q = p.seqlen_k = 128
    p.head_dim = 136
    p.softmax_scale = 1.0
    p.window_left = p.window_right = -1
    assert lib.fa_fwd(ctypes.byref(p)) == -2           # head_dim > 128
    p.head_dim = 60                                     # not a multiple of 8: served through a padded copy
    p.num_splits = 1
    assert lib.fa_fwd_workspace_bytes(ctypes.byref(p)) == 4 * ((128 * 64 * 2 + 255) // 256) * 256
    p.head_dim = 64
    p.num_splits = 0
    p.dtype = 2
    assert lib.fa_fwd(ctypes.byref(p)) == -2           # fp32 inputs
    p.dtype = p.o_dtype = 0
    p.softmax_scale = 0.0
    assert lib.fa_fwd(ctypes.byref(p)) == -1
    p.softmax_scale = 1.0
    p.q = 4100                                          # misaligned
    assert lib.fa_fwd(ctypes.byref(p)) == -1
    p.q = 4096
    p.num_splits = 4
    p.seqlen_k = 1024
    assert lib.fa_fwd_resolve_splits(ctypes.byref(p)) == 4
    assert lib.fa_fwd_workspace_bytes(ctypes.byref(p)) == ((4 * 128 * 64 * 4 + 255) // 256 + (4 * 128 * 4 + 255) // 256) * 256
    p.num_splits = 100                                  # clamped to the number of KV tiles
    assert lib.fa_fwd_resolve_splits(ctypes.byref(p)) == 8
    p.heads, p.heads_k = 6, 4                           # query heads must be a multiple of K/V heads
    assert lib.fa_fwd_resolve_splits(ctypes.byref(p)) == -1
    p.heads_k = 3
    assert lib.fa_fwd_resolve_splits(ctypes.byref(p)) == 8
    p.head_dim, p.num_splits = 60, 1                    # padded copy: Q and O for 6 heads, K and V for 3
    assert lib.fa_fwd_workspace_bytes(ctypes.byref(p)) == 2 * 6 * 128 * 64 * 2 + 2 * 3 * 1024 * 64 * 2
    for code in range(-7, 1):
        assert lib.fa_strerror(code)
    assert _lib.strerror(-3).startswith("workspace")


def test_missing_library_fails_loudly(monkeypatch):
    from flash_attn_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", "/nonexistent/libfa_b200.so")
    with pytest.raises(ImportError):
        _lib.load()
