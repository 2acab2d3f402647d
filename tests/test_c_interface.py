"""The C header of the kernel library: it is plain C, and it declares every exported entry
point of the library the package builds, no more and no less."""
from __future__ import annotations

import os
import re
import subprocess
import tempfile

from conftest import ROOT

HEADER = os.path.join(ROOT, "include", "helix_b200", "kernels.h")
CSRC = os.path.join(ROOT, "helix_runtime_b200", "csrc")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(hx_[a-z0-9_]+)\s*\(", text)))


def exported_functions():
    names = set()
    for name in os.listdir(CSRC):
        if name.endswith(".cu"):
            names.update(re.findall(r"^HX_API\s+[\w\s\*]+?\b(hx_[a-z0-9_]+)\s*\(",
                                    open(os.path.join(CSRC, name)).read(), flags=re.M))
    return sorted(names)


def test_header_declares_exactly_the_exported_entry_points():
    assert declared_functions() == exported_functions()


def test_header_is_plain_c_and_matches_the_library():
    with tempfile.TemporaryDirectory() as scratch:
        source = os.path.join(scratch, "use.c")
        with open(source, "w") as out:
            out.write('#include "helix_b200/kernels.h"\n'
                      "int use(void) { return hx_abi_version() + (hx_last_error() != 0); }\n")
        subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-pedantic", "-fsyntax-only",
                        "-I", os.path.join(ROOT, "include"), source], check=True)
    from helix_runtime_b200.ops import library as ops
    library = ops.lib()
    for name in declared_functions():
        assert hasattr(library, name), f"{name} is declared but the library does not export it"
    assert library.hx_abi_version() >= 3


def test_declarations_agree_with_the_definitions():
    """Every source compiles with the header forced in front of it: a declaration whose
    parameters differ from the definition's is a compile error for a C function."""
    from concurrent.futures import ThreadPoolExecutor

    from helix_runtime_b200.csrc import build

    nvcc = build.find_nvcc()

    def compile_one(name):
        with tempfile.TemporaryDirectory() as scratch:
            return subprocess.run(
                [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17",
                 "--expt-relaxed-constexpr", "-I", CSRC, "-include", HEADER, "-c",
                 os.path.join(CSRC, name), "-o", os.path.join(scratch, "out.o")],
                stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)

    with ThreadPoolExecutor(max_workers=len(build.SOURCES)) as pool:
        for name, result in zip(build.SOURCES, pool.map(compile_one, build.SOURCES)):
            assert result.returncode == 0, f"{name}:\n{result.stdout[-2000:]}"
