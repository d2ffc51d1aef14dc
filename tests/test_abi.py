"""CPU-only checks of the drop-in boundary: the shared library loads, exports every C symbol
that include/nd4j_b200.h declares and the mangled NativeOps members nd4j's JavaCPP layer binds,
and its pure-host entry points (shape / TAD helpers, argument validation) behave. No compute
entry point is called here."""
import ctypes
import os
import re
import subprocess

import numpy as np
import pytest

from libnd4j_b200 import native_ops, shape as S

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "nd4j_b200.h")
CLASS_HEADER = os.path.join(ROOT, "include", "NativeOps.h")


@pytest.fixture(scope="module")
def lib():
    if not os.path.exists(native_ops.LIB_PATH):
        import __graft_entry__
        __graft_entry__.build()
    return native_ops.load_library()


def exported_symbols():
    out = subprocess.run(["nm", "-D", "--defined-only", native_ops.LIB_PATH], capture_output=True, text=True, check=True)
    return {line.split()[-1] for line in out.stdout.splitlines() if line.strip()}


def test_every_declared_c_symbol_is_exported(lib):
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    declared = set(re.findall(r"\b(nd4jb200_[a-z0-9_]+)\s*\(", text))
    assert len(declared) >= 50
    missing = declared - exported_symbols()
    assert not missing, "declared but not exported: %s" % sorted(missing)
    for name in declared:
        assert hasattr(lib, name)


# Manglings of the reference's members as produced by gcc for blas/NativeOps.h.
MANGLED = [
    "_ZN9NativeOps19execReduce3AllFloatEPPviPfPxS2_S2_S3_S2_S3_PiiS3_S3_S3_S3_",
    "_ZN9NativeOps18execReduce3AllHalfEPPviP7float16PxS3_S3_S4_S3_S4_PiiS4_S4_S4_S4_",
    "_ZN9NativeOps15execReduceFloatEPPviPfPxS2_S2_S3_Pii",
    "_ZN9NativeOps15execReduceFloatEPPviPfPxS2_S2_S3_",
    "_ZN9NativeOps21execReduceScalarFloatEPPviPfPxS2_",
    "_ZN9NativeOps18execBroadcastFloatEPPviPfPxS2_S3_S2_S3_Pii",
    "_ZN9NativeOps18execTransformFloatEPPviPfPxS2_S3_S2_",
    "_ZN9NativeOps18execTransformFloatEPPviPfxS2_xS2_x",
    "_ZN9NativeOps26execPairwiseTransformFloatEPPviPfPxS2_S3_S2_S3_S2_",
    "_ZN9NativeOps26execPairwiseTransformFloatEPPviPfxS2_xS2_xS2_x",
    "_ZN9NativeOps20execIndexReduceFloatEPPviPfPxS2_S2_S3_Pii",
    "_ZN9NativeOps21execSummaryStatsFloatEPPviPfPxS2_S2_S3_Piib",
    "_ZN9NativeOps16execReduce3FloatEPPviPfPxS2_S2_S3_S2_S3_Pii",
    "_ZN9NativeOps15execReduce3HalfEPPviP7float16PxS3_S3_S4_S3_S4_Pii",
    "_ZN9NativeOps15execScalarFloatEPPviPfPxS2_S3_fS2_",
    "_ZN9NativeOps15execRandomFloatEPPviS0_PfPxS2_",
    "_ZN9NativeOps15execRandomFloatEPPviS0_PfPxS2_S3_S2_",
    "_ZN9NativeOps15execRandomFloatEPPviS0_PfPxS2_S3_S2_S3_S2_",
    "_ZN9NativeOps10initRandomEPPvllS0_",
    "_ZN9NativeOps13refreshBufferEPPvlS0_",
    "_ZN9NativeOps12reSeedBufferEPPvlS0_",
    "_ZN9NativeOps13destroyRandomEPv",
    "_ZN9NativeOps16tadOnlyShapeInfoEPxPiiS0_S0_",
    "_ZN9NativeOps16execReduceDoubleEPPviPdPxS2_S2_S3_Pii",
    "_ZN9NativeOps14execReduceHalfEPPviP7float16PxS3_S3_S4_Pii",
]


def test_mangled_nativeops_members_are_exported(lib):
    syms = exported_symbols()
    missing = [m for m in MANGLED if m not in syms]
    assert not missing, missing
    members = [s for s in syms if s.startswith("_ZN9NativeOps")]
    assert len(members) >= 100


REFERENCE = os.environ.get("ND4J_REFERENCE", "/root/reference")
REF_INCLUDES = ["blas", "include", "include/helpers", "include/loops", "include/graph", "include/ops", "include/types",
                "include/array", "include/cnpy", "include/memory", "include/indexing"]


def reference_member_declarations(ref_root):
    """(return type, name, [parameter types]) of every member function the reference's class declares
    (blas/NativeOps.h), read from the header text."""
    text = open(os.path.join(ref_root, "blas", "NativeOps.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = re.sub(r"//[^\n]*", "", text)
    body = text[text.index("class ND4J_EXPORT NativeOps"):]
    body = body[body.index("{") + 1:]
    decls = []
    for stmt in body.split(";"):
        m = re.match(r"^\s*(?:public:\s*)?([\w\s\*:]+?)\s*\b(\w+)\s*\((.*)\)\s*$", stmt, flags=re.S)
        if not m:
            continue
        types = []
        for prm in [q.strip() for q in m.group(3).split(",") if q.strip()]:
            prm = prm.split("=")[0].strip()
            named = re.match(r"^(.*?[\s\*&])(\w+)$", prm, flags=re.S)
            types.append(named.group(1).strip() if named else prm)
        decls.append((m.group(1).strip(), m.group(2), types))
    return decls


def test_exports_equal_the_reference_headers_manglings(lib, tmp_path):
    """With the reference checkout present: a translation unit that takes the address of every member the
    reference's own blas/NativeOps.h declares is compiled against that header; its undefined symbols are the
    manglings nd4j's JNI layer binds. Every overload of every member name this library serves must be exported
    under exactly that mangling, and the library must export no NativeOps member the reference does not have."""
    if not os.path.isfile(os.path.join(REFERENCE, "blas", "NativeOps.h")):
        pytest.skip("reference checkout not present")
    decls = reference_member_declarations(REFERENCE)
    assert len(decls) >= 200
    lines = ["#include <NativeOps.h>", "void *sink[%d];" % len(decls), "void take() {"]
    for i, (ret, name, types) in enumerate(decls):
        lines.append("  { %s (NativeOps::*p)(%s) = &NativeOps::%s; sink[%d] = *reinterpret_cast<void **>(&p); }"
                     % (ret, ", ".join(types), name, i))
    lines.append("}")
    src = tmp_path / "members.cpp"
    src.write_text("\n".join(lines))
    obj = str(tmp_path / "members.o")
    cmd = ["g++", "-std=c++11", "-w", "-include", "limits", "-include", "cstdint", "-D__CPUBLAS__=true"]
    for d in REF_INCLUDES:
        cmd += ["-I", os.path.join(REFERENCE, d)]
    env = dict(os.environ, PATH="/usr/bin:" + os.environ.get("PATH", ""))
    subprocess.run(cmd + ["-c", str(src), "-o", obj], check=True, env=env)
    out = subprocess.run(["nm", "-u", obj], capture_output=True, text=True, check=True).stdout
    wanted = {l.split()[-1] for l in out.splitlines() if "_ZN9NativeOps" in l}
    assert len(wanted) == len(decls)
    ours = {sym for sym in exported_symbols() if sym.startswith("_ZN9NativeOps")}
    strays = ours - wanted
    assert not strays, "exported but not declared by the reference: %s" % sorted(strays)
    # member names served here = the names our class header declares
    mine = open(CLASS_HEADER).read()
    served = {name for _, name, _ in decls if re.search(r"\b%s\b|\b%s##S" % (name, re.sub(r"(Float|Double|Half)$", "", name)), mine)}

    def member_name(sym):
        m = re.match(r"_ZN9NativeOps(\d+)", sym)
        n = int(m.group(1))
        return sym[len(m.group(0)):len(m.group(0)) + n]
    missing = sorted(sym for sym in wanted if member_name(sym) in served and sym not in ours)
    assert not missing, "overloads of served members that are not exported: %s" % missing
    assert len(ours) >= 140


def test_class_header_and_c_header_compile_as_c_and_cpp(tmp_path):
    c = tmp_path / "t.c"
    c.write_text('#include "nd4j_b200.h"\nint main(void) { return nd4jb200_get_device == 0; }\n')
    subprocess.run(["gcc", "-I", os.path.join(ROOT, "include"), "-c", str(c), "-o", str(tmp_path / "t.o")], check=True)
    cpp = tmp_path / "t.cpp"
    cpp.write_text('#include "NativeOps.h"\nint main() { NativeOps *ops = nullptr; (void) ops; return sizeof(float16) == 2 ? 0 : 1; }\n')
    subprocess.run(["g++", "-std=c++11", "-I", os.path.join(ROOT, "include"), "-c", str(cpp), "-o", str(tmp_path / "u.o")], check=True)


def test_host_side_validation_reports_errors(lib):
    info = S.shape_info([4, 5])
    bad = info.copy()
    bad[0] = 77
    lp = ctypes.POINTER(ctypes.c_longlong)
    ip = ctypes.POINTER(ctypes.c_int)
    dims = np.array([1], dtype=np.int32)
    assert lib.nd4jb200_tad_count(bad.ctypes.data_as(lp), dims.ctypes.data_as(ip), 1) == -1
    assert b"rank" in lib.nd4jb200_last_error()
    dims = np.array([5], dtype=np.int32)
    assert lib.nd4jb200_tad_count(info.ctypes.data_as(lp), dims.ctypes.data_as(ip), 1) == -1
    assert b"not an axis" in lib.nd4jb200_last_error()
    # null data pointers are rejected before anything touches the GPU
    rc = lib.nd4jb200_exec_transform(None, 0, 0, None, info.ctypes.data_as(lp), None, info.ctypes.data_as(lp), None)
    assert rc == 1 and b"null" in lib.nd4jb200_last_error()
    rc = lib.nd4jb200_exec_transform(None, 9, 0, ctypes.c_void_p(16), info.ctypes.data_as(lp), ctypes.c_void_p(16),
                                     info.ctypes.data_as(lp), None)
    assert rc == 1 and b"dtype" in lib.nd4jb200_last_error()


def test_product_package_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "libnd4j_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp")):
                text = open(os.path.join(dirpath, f), errors="ignore").read()
                assert "oracle" not in text, "%s mentions the oracle" % f
