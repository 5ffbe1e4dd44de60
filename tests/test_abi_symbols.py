"""The C-ABI library loads on a machine without a GPU and exports every symbol the header declares."""
import ctypes
import os
import re

import pytest

from singe_b200 import kernel_sys as ks

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "singe_kernel_sys.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(singe_[a-z0-9_]+)\s*\(", text)))


def test_library_is_built_and_exports_every_declared_symbol():
    if not os.path.exists(ks.LIB_PATH):
        from singe_b200 import build

        build.build()
    handle = ctypes.CDLL(ks.LIB_PATH)
    declared = _declared()
    assert len(declared) >= 20
    missing = [name for name in declared if not hasattr(handle, name)]
    assert not missing, f"declared in include/singe_kernel_sys.h but not exported: {missing}"


def test_python_binding_covers_the_header():
    declared = set(_declared())
    bound = set(ks.SIGNATURES)
    assert declared - bound == set(), f"unbound symbols: {sorted(declared - bound)}"
    assert bound - declared == set()


def test_status_strings_and_host_only_helpers_need_no_gpu():
    lib = ks.lib()
    assert lib.singe_kernel_sys_version() >= 1000
    assert ks.status_string(ks.OK) == "ok"
    assert ks.status_string(ks.ERR_INVALID_LENGTH) == "invalid length"
    # split sizing is host arithmetic: ceil(bound / splits) rounded up to whole pages
    assert lib.singe_paged_kv_decode_split_tokens(4096, 8, 16) == 512
    assert lib.singe_paged_kv_decode_split_tokens(4096, 6, 16) == 688
    assert lib.singe_paged_kv_decode_split_tokens(100, 64, 16) == 16
    # the drop-in decode's own split count: 512-key pieces, larger ones where a wave model of the grid (148 SMs when no
    # device is present, three CTAs each) prefers them and 2.5 waves of CTAs remain
    assert lib.singe_paged_kv_decode_default_splits(32, 8, 4096, 16) == 5      # five 832-key pieces
    assert lib.singe_paged_kv_decode_default_splits(16, 8, 4096, 16) == 8      # too few CTAs for larger pieces
    assert lib.singe_paged_kv_decode_default_splits(64, 8, 4096, 16) == 4      # 1024-key pieces
    assert lib.singe_paged_kv_decode_default_splits(128, 8, 1024, 16) == 2     # 512-key pieces of a short bound
    assert lib.singe_paged_kv_decode_default_splits(1, 1, 2048, 16) == 16      # one row: the finest split


def test_validation_runs_before_any_device_work():
    lib = ks.lib()
    # heads not a multiple of kv_heads -> InvalidLength; checked before the (absent) device is touched
    assert lib.singe_paged_kv_decode_attention_f32(None, None, None, None, None, None, None, 1, 3, 2, 8, 4, 2, 2,
                                                   1.0) == ks.ERR_INVALID_LENGTH
    assert lib.singe_kv_cache_write_bf16(None, None, None, None, None, None, None, 8, 0, 1, 1, 1, 1,
                                         None) == ks.ERR_INVALID_LENGTH
    assert lib.singe_matmul_bf16_f32(None, None, None, None, 0, 1, 1, 1, 1, 1, 0, 1) == ks.ERR_INVALID_LENGTH


def test_missing_library_fails_loudly(monkeypatch):
    monkeypatch.setattr(ks, "_lib", None)
    monkeypatch.setattr(ks, "LIB_PATH", os.path.join(ROOT, "no_such_dir", "libsinge_kernel_sys.so"))
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        ks.lib()


def test_the_rust_binding_block_in_the_integration_notes_is_the_generator_output():
    # include/rust_bindings.py prints the extern "C" block from the header; the integration notes carry that output
    sys_path = os.path.join(ROOT, "include")
    import importlib.util

    spec = importlib.util.spec_from_file_location("rust_bindings", os.path.join(sys_path, "rust_bindings.py"))
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    block = module.render()
    with open(os.path.join(ROOT, "include", "singe_kernel_sys.h")) as handle:
        declared = list(module.declarations(handle.read()))
    assert sorted(name for name, _, _ in declared) == _declared()
    for name, fields, _ in declared:
        assert len(fields) == len(ks.SIGNATURES[name]), name
    with open(os.path.join(ROOT, "INTEGRATION.md")) as handle:
        assert block in handle.read(), "run `python include/rust_bindings.py` and paste its output into appendix A"
