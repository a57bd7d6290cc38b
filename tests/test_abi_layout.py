"""The ctypes mirrors in ``ops/_lib.py`` against the C header: same size, same field names in the same order,
same offsets.  A tiny program that includes the header is compiled with the host compiler and prints
``offsetof`` for every field; no GPU and no CUDA toolkit are needed."""

import ctypes
import json
import re
import shutil
import subprocess
from pathlib import Path

import pytest

from moeflow_b200.ops import _lib

HEADER = Path(_lib.__file__).resolve().parent.parent / "csrc" / "moeflow_b200.h"
MIRRORS = {
    "mf_gemm_args": _lib.GemmArgs,
    "mf_dispatch_args": _lib.DispatchArgs,
    "mf_meta_args": _lib.MetaArgs,
    "mf_reduce_push_args": _lib.ReducePushArgs,
    "mf_combine_args": _lib.CombineArgs,
}


def _fields_in_header(struct: str) -> list[str]:
    """Field names of ``typedef struct { ... } <struct>;`` in declaration order."""
    text = HEADER.read_text()
    end = text.index("} " + struct + ";")
    body = text[text.rindex("typedef struct {", 0, end) + len("typedef struct {"):end]
    body = re.sub(r"//[^\n]*", "", body)
    names = []
    for declaration in body.split(";"):
        declaration = declaration.strip()
        if not declaration:
            continue
        # "const unsigned long long* peer_recv" or "int R, C, H, K, rank"
        first, *more = [part.strip() for part in declaration.split(",")]
        names.append(re.search(r"(\w+)\s*$", first).group(1))
        names.extend(re.search(r"(\w+)\s*$", part).group(1) for part in more)
    return names


@pytest.fixture(scope="module")
def c_layout(tmp_path_factory):
    compiler = shutil.which("g++") or shutil.which("c++")
    if compiler is None:
        pytest.skip("no host C++ compiler")
    lines = ["#include <cstddef>", "#include <cstdio>", f'#include "{HEADER}"', "int main() {", '  std::printf("{");']
    for i, struct in enumerate(MIRRORS):
        fields = _fields_in_header(struct)
        sep = "" if i == 0 else ","
        lines.append(f'  std::printf("{sep}\\"{struct}\\": {{\\"size\\": %zu", sizeof({struct}));')
        for name in fields:
            lines.append(f'  std::printf(", \\"{name}\\": %zu", offsetof({struct}, {name}));')
        lines.append('  std::printf("}");')
    lines += ['  std::printf("}\\n");', "  return 0;", "}"]
    work = tmp_path_factory.mktemp("abi")
    (work / "layout.cpp").write_text("\n".join(lines))
    subprocess.run([compiler, "-std=c++17", "-o", str(work / "layout"), str(work / "layout.cpp")], check=True,
                   capture_output=True, text=True)
    return json.loads(subprocess.run([str(work / "layout")], check=True, capture_output=True, text=True).stdout)


@pytest.mark.parametrize("struct", list(MIRRORS))
def test_ctypes_mirror_matches_the_header(c_layout, struct):
    mirror = MIRRORS[struct]
    in_c = c_layout[struct]
    assert [name for name, _ in mirror._fields_] == _fields_in_header(struct)
    assert ctypes.sizeof(mirror) == in_c["size"]
    for name, _ in mirror._fields_:
        assert getattr(mirror, name).offset == in_c[name], name


def test_plan_word_indices_match_the_header():
    text = HEADER.read_text()
    for name in ("N_TILES", "SPLIT1", "SPLIT2", "N_ENTRIES", "SLOT_COLS", "VALID_ROWS", "WORDS"):
        value = int(re.search(rf"MF_PLAN_{name}\s*=\s*(\d+)", text).group(1))
        assert getattr(_lib, f"PLAN_{name}") == value


def test_every_bound_function_is_declared_with_the_same_number_of_parameters():
    """``ops/_lib.py`` sets ``argtypes`` per function; the header declares them.  Both lists must name the same
    functions with the same arity, and the built library must export every one of them."""
    text = re.sub(r"//[^\n]*", "", HEADER.read_text())
    declared = {}
    for match in re.finditer(r"\b(?:int|void|const char\*)\s+(mf_\w+)\s*\(([^;{]*)\)\s*;", text):
        params = match.group(2).strip()
        declared[match.group(1)] = 0 if params in ("", "void") else params.count(",") + 1
    if not _lib.LIB_PATH.exists() and shutil.which("nvcc") is None:
        pytest.skip("native library not built and no nvcc")
    handle = _lib.lib()
    bound = {name: len(getattr(handle, name).argtypes) for name in declared if getattr(getattr(handle, name, None), "argtypes", None) is not None}
    assert bound, "no bound functions found"
    for name, arity in bound.items():
        assert declared[name] == arity, f"{name}: header declares {declared[name]} parameters, ctypes binds {arity}"
    for name in declared:
        assert hasattr(handle, name), f"{name} is declared but not exported by the library"
