"""The build helper: hash-named libraries, the host-only library with the host compiler (no GPU)."""
import ctypes
import os

from cajeta_llm_b200.csrc import build


def test_host_library_compiles_with_the_host_compiler_into_a_given_folder(tmp_path, monkeypatch):
    monkeypatch.setenv("CAJETA_B200_BUILD_DIR", str(tmp_path))
    assert build._build_dirs()[0] == str(tmp_path)
    build._compile_unlocked("host_books", verbose=False)
    name = build._file_name("host_books")
    path = os.path.join(str(tmp_path), name)
    assert os.path.isfile(path) and build.find_built("host_books") == path
    lib = ctypes.CDLL(path)
    lib.cj_pages_create.restype = ctypes.c_void_p
    lib.cj_pages_free_count.argtypes = [ctypes.c_void_p]
    lib.cj_pages_destroy.argtypes = [ctypes.c_void_p]
    h = lib.cj_pages_create(5)
    assert lib.cj_pages_free_count(h) == 5
    lib.cj_pages_destroy(h)


def test_a_library_name_carries_the_hash_of_its_sources_and_flags(monkeypatch):
    a = build._file_name("host_books")
    monkeypatch.setattr(build, "CXX_FLAGS", build.CXX_FLAGS + ["-DOTHER"])
    assert build._file_name("host_books") != a
    assert a.startswith("libcj_host_books-") and a.endswith(".so")
    for name in build.LIBRARIES:
        assert os.path.isfile(os.path.join(build.HERE, build.LIBRARIES[name]))


def test_unknown_library_is_an_error():
    import pytest
    with pytest.raises(build.BuildError, match="unknown kernel library"):
        build.build("no_such_library")
