"""In-tree build of the native code for sm_100a.

`python -m pocketllm_b200.build` compiles every `.cu` / `.cpp` under `csrc/` with nvcc
(`-gencode arch=compute_100a,code=sm_100a -lineinfo`) into

* `pocketllm_b200/_C/libpocket_kernels.so`  -- the CUDA kernels behind `pocketllm_b200.ops`
* `pocketllm_b200/_C/libpocket_kernels_debug.so` -- the same kernels compiled with `-DPK_DEBUG_BOUNDS=1`: bad KV positions and
  route ids are recorded in a status word and the access is skipped (`POCKET_KERNELS_DEBUG=1` makes `ops` load it)
* `pocketllm_b200/_C/libpocket_engine.so`   -- the native engine (links the kernels)
* `pocketllm_b200/_C/pocket_engine`         -- the engine CLI
* `pocketllm_b200/_C/libpocket_cpu.so`      -- host-only code (CPU MoE oracle, GGUF block codecs)

Objects are cached by source hash under `build/`, compiled in parallel, and nothing here
needs a GPU (nvcc cross-compiles).
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "csrc"
OUT = ROOT / "pocketllm_b200" / "_C"
OBJ = ROOT / "build" / "obj"

NVCC = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
          "-Xcompiler", "-Wall", "-Xcudafe", "--diag_suppress=177"]


def _headers_digest() -> str:
    h = hashlib.sha256()
    for p in sorted(list(CSRC.rglob("*.cuh")) + list(CSRC.rglob("*.h")) + list(CSRC.rglob("*.hpp")) + list(CSRC.rglob("*.inc"))):
        h.update(p.read_bytes())
    return h.hexdigest()


def _compile_one(src: Path, hdr_digest: str, extra: list[str], verbose: bool) -> Path:
    key = hashlib.sha256(src.read_bytes() + hdr_digest.encode() + " ".join(extra).encode()).hexdigest()[:16]
    obj = OBJ / f"{src.stem}.{key}.o"
    if obj.exists():
        return obj
    OBJ.mkdir(parents=True, exist_ok=True)
    if src.suffix == ".cu":
        cmd = [NVCC, *ARCH, *COMMON, *extra, "-c", str(src), "-o", str(obj)]
    else:
        cmd = [NVCC, *COMMON, *extra, "-c", str(src), "-o", str(obj)]
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"compile failed: {src}\n{r.stdout}\n{r.stderr}")
    if verbose and r.stderr.strip():
        print(r.stderr)
    return obj


def _link(objs: list[Path], out: Path, shared: bool, extra: list[str], verbose: bool) -> None:
    cmd = [NVCC, *ARCH, "-o", str(out)] + (["-shared"] if shared else []) + [str(o) for o in objs] + extra
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed: {out}\n{r.stdout}\n{r.stderr}")


def build(verbose: bool = False, jobs: int | None = None) -> dict[str, Path]:
    """Compile everything; returns the produced artefacts."""
    OUT.mkdir(parents=True, exist_ok=True)
    hdr = _headers_digest()
    kernel_srcs = sorted((CSRC / "kernels").glob("*.cu")) + sorted((CSRC / "comm").glob("*.cu")) + [CSRC / "common" / "pk_status.cu"]
    engine_srcs = sorted(p for p in (CSRC / "engine").iterdir() if p.suffix in (".cu", ".cpp") and p.name != "main.cpp")
    cpu_srcs = sorted((CSRC / "cpu").glob("*.cpp")) if (CSRC / "cpu").exists() else []
    main_src = CSRC / "engine" / "main.cpp"
    tool_srcs = sorted((CSRC / "tools").glob("*.cpp")) if (CSRC / "tools").exists() else []
    cpu_flags = ["-Xcompiler", "-fopenmp", "-Xcompiler", "-mavx2", "-Xcompiler", "-mfma"]

    work: list[tuple[Path, list[str]]] = [(s, []) for s in kernel_srcs + engine_srcs]
    debug_flags = ["-DPK_DEBUG_BOUNDS=1"]
    work += [(s, debug_flags) for s in kernel_srcs]          # the same kernels with recording index checks
    work += [(s, cpu_flags) for s in cpu_srcs]
    if main_src.exists():
        work.append((main_src, []))
    work += [(s, []) for s in tool_srcs]

    jobs = jobs or max(1, (os.cpu_count() or 4))
    objs: dict[Path, Path] = {}
    dbg_objs: dict[Path, Path] = {}
    with cf.ThreadPoolExecutor(max_workers=jobs) as ex:
        futs = {ex.submit(_compile_one, s, hdr, extra, verbose): (s, extra) for s, extra in work}
        for f in cf.as_completed(futs):
            s, extra = futs[f]
            (dbg_objs if extra == debug_flags else objs)[s] = f.result()

    arts: dict[str, Path] = {}
    kern_so = OUT / "libpocket_kernels.so"
    _link([objs[s] for s in kernel_srcs], kern_so, True, ["-lcudart"], verbose)
    arts["kernels"] = kern_so
    dbg_so = OUT / "libpocket_kernels_debug.so"
    _link([dbg_objs[s] for s in kernel_srcs], dbg_so, True, ["-lcudart"], verbose)
    arts["kernels_debug"] = dbg_so
    rpath = ["-Xlinker", "-rpath", "-Xlinker", "$ORIGIN"]
    eng_so = OUT / "libpocket_engine.so"
    _link([objs[s] for s in engine_srcs], eng_so, True, ["-L" + str(OUT), "-lpocket_kernels", "-lcudart", "-ldl", *rpath], verbose)
    arts["engine"] = eng_so
    if cpu_srcs:
        cpu_so = OUT / "libpocket_cpu.so"
        _link([objs[s] for s in cpu_srcs], cpu_so, True, ["-Xcompiler", "-fopenmp"], verbose)
        arts["cpu"] = cpu_so
    if main_src.exists():
        exe = OUT / "pocket_engine"
        # The engine's C++ classes are not exported from the shared library (only its C ABI
        # is), so the CLI links the engine objects themselves.
        _link([objs[main_src]] + [objs[s] for s in engine_srcs], exe, False,
              ["-L" + str(OUT), "-lpocket_kernels", "-lcudart", "-lpthread", "-ldl", *rpath], verbose)
        arts["cli"] = exe
    for s in tool_srcs:
        exe = OUT / s.stem
        _link([objs[s]] + [objs[e] for e in engine_srcs], exe, False,
              ["-L" + str(OUT), "-lpocket_kernels", "-lcudart", "-lpthread", "-ldl", *rpath], verbose)
        arts[s.stem] = exe
    return arts


def main() -> int:
    verbose = "-v" in sys.argv
    arts = build(verbose=verbose)
    for k, v in arts.items():
        print(f"{k}: {v}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
