"""Builds the DAPHNE-facing adapter library from a DAPHNE source tree.

    python daphne_b200/csrc/daphne_abi/build_adapter.py [DAPHNE_SRC]

Steps:
  1. the tree's own kernels.json is filtered to the kernel templates this library implements for the CUDA backend
     (the DNN operators are left to DAPHNE's own library);
  2. the tree's own generator (src/runtime/local/kernels/genKernelInst.py) emits the extern "C" wrappers and the
     catalog JSON for backend "CUDA" -- names, argument order and the kId/ctx tail are therefore exactly DAPHNE's;
  3. the wrappers are compiled against the tree's data-structure headers and the headers in include/ here, which carry
     the reference's header names (runtime/local/kernels/CUDA/AggRow.h, ...) and forward to libdaphne_b200.so.
  4. the same generator, with API "CPP", emits wrappers for operators that DAPHNE's compiler never tags for the CUDA
     backend (ewUnaryMat, ctable, and the aggregation opcodes beyond SUM/MIN/MAX): they carry the CPU kernels' names
     (leading "_") and go into an EXTENSION catalog (daphne --kernel-ext B200ExtCatalog.json:1) so that they are
     preferred over the built-in CPU kernels and keep device-resident operands on the device.
Nothing of the tree is copied; generated sources and the outputs live in daphne_b200/_abi_build/ (git-ignored):
    libCUDAKernels.so   CUDAcatalog.json   libB200ExtKernels.so   B200ExtCatalog.json
    (+ libabi_driver.so, the JIT stand-in used by the tests)
Outside a DAPHNE build tree (as here) DaphneContext.h / ErrorHandler.h / KernelInstrumentation.h come from shim/."""
from __future__ import annotations

import json
import subprocess
import sys
import sysconfig
from pathlib import Path

HERE = Path(__file__).resolve().parent
PKG = HERE.parents[1]
OUT = PKG / "_abi_build"
SUPPORTED_HEADERS = {"AggAll.h", "AggCol.h", "AggRow.h", "EwBinaryMat.h", "EwBinaryObjSca.h", "MatMul.h", "Syrk.h",
                     "Gemv.h", "Solve.h", "Transpose.h", "Fill.h", "CreateCUDAContext.h", "ColBind.h", "ExtractCol.h"}


# backend-"CPP" extension: header -> opcodes to register (None: all of the entry's opcodes / no opcode)
EXT_HEADERS = {"EwUnaryMat.h": None, "CTable.h": None, "OuterBinary.h": None, "AggCum.h": None, "OneHot.h": None, "CondMatMatMat.h": None,
               "CondMatMatSca.h": None, "CondMatScaMat.h": None, "CondMatScaSca.h": None,
               "AggRow.h": {"IDXMIN", "IDXMAX", "MEAN", "VAR", "STDDEV", "PROD"},
               "AggCol.h": {"IDXMIN", "IDXMAX", "MEAN", "VAR", "STDDEV", "PROD"},
               "AggAll.h": {"MEAN", "VAR", "STDDEV", "PROD"},
               # CSRMatrix operands (double): the sparse-times-dense product, its row aggregation, CSR @ dense
               "EwBinaryMat.h": {"MUL"}, "MatMul.h": None, "Gemv.h": None}
CSR_HEADERS = {"EwBinaryMat.h": [["CSRMatrix", "double"], ["CSRMatrix", "double"], ["DenseMatrix", "double"]],
               "MatMul.h": [["DenseMatrix", "double"], ["CSRMatrix", "double"], ["DenseMatrix", "double"]],
               "Gemv.h": [["DenseMatrix", "double"], ["CSRMatrix", "double"], ["DenseMatrix", "double"]],
               "AggRow.h": [["DenseMatrix", "double"], ["CSRMatrix", "double"]]}
CSR_AGG_OPS = ["SUM", "MIN", "MAX"]
DEVICE_VTS = {"double", "float", "int64_t"}


def default_source() -> Path:
    """$DAPHNE_ROOT, else a directory `reference` beside the repository."""
    import os
    return Path(os.environ.get("DAPHNE_ROOT") or PKG.parents[1] / "reference")


def _ext_instantiation_ok(header: str, inst) -> bool:
    """Dense matrices of the value types the device kernels implement; index results are size_t."""
    if header == "MatMul.h" and all(list(t) in (["DenseMatrix", "int64_t"], ["DenseMatrix", "int32_t"]) for t in inst):
        return len({t[1] for t in inst}) == 1  # dense integer products (the reference's Eigen path)
    if header in ("EwBinaryMat.h", "MatMul.h", "Gemv.h"):
        return [list(t) for t in inst] == CSR_HEADERS[header]
    vts, scalars = [], []
    for tv in inst:
        if isinstance(tv, list):
            if tv[0] != "DenseMatrix":
                return False
            vts.append(tv[1])
        else:
            scalars.append(tv)
    if header == "CTable.h":  # DTRes, DTLhs, DTRhs, VTWeight
        return vts == ["double", "int64_t", "int64_t"]
    if header.startswith("CondMat"):  # DTRes, DTCond, then, else: values double / float / int64, cond double / int64
        if len(vts) < 2 or vts[0] not in DEVICE_VTS or vts[1] not in ("double", "int64_t"):
            return False
        return all(v == vts[0] for v in vts[2:]) and all(sc == vts[0] for sc in scalars)
    if header == "OneHot.h":  # DTRes, DTArg: double or int64
        return len(vts) == 2 and vts[0] == vts[1] and vts[0] in ("double", "int64_t")
    if header == "OuterBinary.h":  # DTRes, DTLhs, DTRhs of one value type
        return len(vts) == 3 and len(set(vts)) == 1 and vts[0] in DEVICE_VTS
    if header == "AggAll.h":  # VTRes, DTArg
        return len(vts) == 1 and vts[0] in ("double", "float") and scalars == vts
    res, arg = vts[0], vts[-1]
    if arg not in DEVICE_VTS:
        return False
    return res == arg or (header in ("AggRow.h", "AggCol.h") and res == "size_t")


def ext_spec(daphne_src: Path) -> list:
    spec = json.loads((daphne_src / "src/runtime/local/kernels/kernels.json").read_text())
    keep = []
    for k in spec:
        header = k["kernelTemplate"]["header"]
        if header not in EXT_HEADERS:
            continue
        apis = k["api"] if "api" in k else [{"name": ["CPP"], "instantiations": k["instantiations"],
                                             **({"opCodes": k["opCodes"]} if "opCodes" in k else {})}]
        out = []
        for a in apis:
            names = a["name"] if isinstance(a["name"], list) else [a["name"]]
            if "CPP" not in names:
                continue
            inst = [i for i in a["instantiations"] if _ext_instantiation_ok(header, i)]
            b = {"name": ["CPP"], "instantiations": inst}
            if "opCodes" in a:
                want = EXT_HEADERS[header]
                b["opCodes"] = [o for o in a["opCodes"] if want is None or o in want]
                if not b["opCodes"]:
                    continue
            if inst:
                out.append(b)
            if header == "AggRow.h" and CSR_HEADERS[header] in [[list(t) for t in i] for i in a["instantiations"]]:
                out.append({"name": ["CPP"], "instantiations": [CSR_HEADERS[header]], "opCodes": CSR_AGG_OPS})
        if out:
            keep.append({"kernelTemplate": k["kernelTemplate"], "api": out})
    return keep


def _is_cuda(api) -> bool:
    names = api["name"] if isinstance(api["name"], list) else [api["name"]]
    return "CUDA" in names


def filtered_spec(daphne_src: Path) -> list:
    spec = json.loads((daphne_src / "src/runtime/local/kernels/kernels.json").read_text())
    keep = []
    for k in spec:
        t = k["kernelTemplate"]
        if t["header"] not in SUPPORTED_HEADERS:
            continue
        apis = [a for a in k.get("api", []) if _is_cuda(a)]
        if not apis:
            continue
        k = dict(k)
        k["api"] = [dict(a, name=["CUDA"]) for a in apis]
        keep.append(k)
    return keep


def build(daphne_src: str | Path | None = None) -> Path:
    daphne_src = Path(daphne_src or default_source())
    if not (daphne_src / "src/runtime/local/kernels/genKernelInst.py").exists():
        raise RuntimeError(f"no DAPHNE source tree at {daphne_src}")
    from daphne_b200 import build as core
    core.build()
    OUT.mkdir(exist_ok=True)
    for old in OUT.glob("CUDAkernels*.cpp"):
        old.unlink()
    spec_path = OUT / "kernels_b200.json"
    spec_path.write_text(json.dumps(filtered_spec(daphne_src)))
    r = subprocess.run([sys.executable, str(daphne_src / "src/runtime/local/kernels/genKernelInst.py"), str(spec_path),
                        str(OUT / "CUDAkernels"), str(OUT / "CUDAcatalog.json"), "CUDA"],
                       capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("genKernelInst.py failed:\n" + r.stdout + r.stderr)
    site = Path(sysconfig.get_paths()["purelib"])
    ds = daphne_src / "src/runtime/local/datastructures"
    inc = ["-I", str(HERE / "include"), "-I", str(HERE), "-I", str(HERE / "shim"), "-I", str(daphne_src / "src"),
           "-I", str(site / "flashinfer/data/spdlog/include"), "-I", str(PKG.parent / "include")]
    flags = ["-std=c++20", "-O2", "-fPIC", "-pthread", "-DFMT_HEADER_ONLY", "-w"]
    gen = sorted(OUT.glob("CUDAkernels*.cpp"))
    ref_srcs = [ds / n for n in ("Structure.cpp", "MetaDataObject.cpp", "DenseMatrix.cpp", "CSRMatrix.cpp",
                                 "DataPlacement.cpp", "ValueTypeUtils.cpp")]
    lib = OUT / "libCUDAKernels.so"
    cmd = ["g++", *flags, "-shared", "-o", str(lib), *inc, *map(str, gen), str(HERE / "adapter.cpp"),
           *map(str, ref_srcs), "-L", str(PKG), "-ldaphne_b200", f"-Wl,-rpath,{PKG}", "-Wl,-rpath,$ORIGIN/.."]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("compiling the adapter failed:\n" + r.stdout[-4000:] + r.stderr[-8000:])
    # ---- backend-"CPP" extension catalog ----
    for old in OUT.glob("B200Extkernels*.cpp"):
        old.unlink()
    ext_path = OUT / "kernels_b200_ext.json"
    ext_path.write_text(json.dumps(ext_spec(daphne_src)))
    r = subprocess.run([sys.executable, str(daphne_src / "src/runtime/local/kernels/genKernelInst.py"), str(ext_path),
                        str(OUT / "B200Extkernels"), str(OUT / "B200ExtCatalog.json"), "CPP"],
                       capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("genKernelInst.py (extension) failed:\n" + r.stdout + r.stderr)
    cat = json.loads((OUT / "B200ExtCatalog.json").read_text())
    for e in cat:
        e["libPath"] = "libB200ExtKernels.so"  # the generator assumes libAllKernels.so for backend "CPP"
    (OUT / "B200ExtCatalog.json").write_text(json.dumps(cat, indent=1))
    ext_lib = OUT / "libB200ExtKernels.so"
    ext_inc = ["-I", str(HERE / "include_cpp")] + inc  # the CPU kernels' header names resolve to the adapter's
    # ... plus the scheduler entry point under DAPHNE's name (vectorized_pipeline.cpp)
    cmd = ["g++", *flags, "-shared", "-o", str(ext_lib), *ext_inc, *map(str, sorted(OUT.glob("B200Extkernels*.cpp"))),
           str(HERE / "vectorized_pipeline.cpp"), "-L", str(OUT), "-lCUDAKernels", "-L", str(PKG), "-ldaphne_b200", f"-Wl,-rpath,{OUT}", f"-Wl,-rpath,{PKG}",
           "-Wl,-rpath,$ORIGIN", "-Wl,-rpath,$ORIGIN/.."]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("compiling the extension kernels failed:\n" + r.stdout[-4000:] + r.stderr[-8000:])
    drv = OUT / "libabi_driver.so"
    cmd = ["g++", *flags, "-shared", "-o", str(drv), *inc, str(HERE / "abi_driver.cpp"), "-L", str(OUT),
           "-lCUDAKernels", "-L", str(PKG), "-ldaphne_b200", "-ldl", f"-Wl,-rpath,{OUT}", f"-Wl,-rpath,{PKG}",
           "-Wl,-rpath,$ORIGIN", "-Wl,-rpath,$ORIGIN/.."]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("compiling the ABI driver failed:\n" + r.stdout[-4000:] + r.stderr[-8000:])
    return lib


if __name__ == "__main__":
    sys.path.insert(0, str(PKG.parent))
    print(build(sys.argv[1] if len(sys.argv) > 1 else None))
