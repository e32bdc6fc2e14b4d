"""The C-ABI library loads on a machine without a GPU and exports every symbol
that include/kvcache_b200.h declares (no compute calls here)."""
import ctypes
import os
import re

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "kvcache_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"\b(kvc_[a-z0-9_]+)\s*\(", text)
    return sorted(set(names))


def test_header_declares_the_expected_surface():
    names = declared_functions()
    for must in ("kvc_create", "kvc_free", "kvc_update", "kvc_update_quantized", "kvc_attention",
                 "kvc_attention_host", "kvc_trim", "kvc_is_trimmable_after", "kvc_state_get", "kvc_state_set",
                 "kvc_meta_state", "kvc_set_meta_state", "kvc_copy", "kvc_logical_view", "kvc_round_begin",
                 "kvc_round_commit", "kvc_round_rollback", "kvc_rewind_last_round", "kvc_quantized_sdpa",
                 "kvc_sdpa", "kvc_turbo_encode", "kvc_comm_init", "kvc_attention_sharded",
                 "kvc_last_error_message", "kvc_version"):
        assert must in names, must


def test_library_exports_every_declared_symbol(kvc):
    lib = ctypes.CDLL(kvc.LIB_PATH)
    missing = [n for n in declared_functions() if not hasattr(lib, n)]
    assert not missing, f"declared in the header but not exported: {missing}"


def test_version_and_error_channel(kvc):
    assert "sm_100a" in kvc.version()
    # a null handle is rejected with a discriminated status and a message
    st = kvc.lib().kvc_trim(None, 1, None)
    assert st == kvc.ERR_INVALID_ARG
    assert b"null handle" in kvc.lib().kvc_last_error_message()


def test_modulemap_names_the_header():
    mm = open(os.path.join(ROOT, "include", "module.modulemap")).read()
    assert 'header "kvcache_b200.h"' in mm


def test_cpp_host_mirror_compiles_and_runs_without_a_device(kvc, tmp_path):
    """host/KVCache.hpp (the C++ mirror of the KVCache protocol surface) compiles against the C header,
    links the shared library and passes its host-only checks."""
    import subprocess
    here = os.path.dirname(os.path.abspath(__file__))
    lib_dir = os.path.dirname(kvc.LIB_PATH)
    exe = str(tmp_path / "host_mirror")
    subprocess.run(["g++", "-std=c++17", "-O1", "-Wall", "-Werror", os.path.join(here, "host_mirror_main.cpp"), "-o", exe,
                    "-L" + lib_dir, "-lkvcache_b200", "-Wl,-rpath," + lib_dir], check=True)
    out = subprocess.run([exe, str(tmp_path / "mirror.safetensors")], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0 and out.stdout.strip().endswith("ok"), out.stdout + out.stderr
