"""Build libb200decode.so in-tree with nvcc for sm_100a (no torch headers, no JIT cache).

    python -m llm_decode_kernels_b200.build [--force] [--verbose]

Each csrc/*.cu is compiled to an object next to the sources (csrc/_obj/) in parallel and linked into
llm_decode_kernels_b200/libb200decode.so. A source is recompiled when it, or any header in csrc/ or include/,
is newer than its object. nvcc cross-compiles without a GPU, so this runs on a CPU-only machine.
"""
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
INCLUDE = PKG.parent / "include"
LIB = PKG / "libb200decode.so"

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
              "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]


def nvcc():
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(exe).exists():
        raise RuntimeError("nvcc not found: libb200decode.so cannot be built on this machine")
    return exe


def sources():
    return sorted(CSRC.glob("*.cu"))


def _newest_header():
    hs = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list(INCLUDE.glob("*.h"))
    return max((h.stat().st_mtime for h in hs), default=0.0)


def build(force=False, verbose=False, defines=(), lib=LIB):
    """Compile what is stale and link. Returns the path of the shared library. `defines` (macro names) and `lib`
    make a variant of the library next to the normal one, with its own object directory: step_trace.py builds
    libb200decode_trace.so with B200_STEP_TRACE this way."""
    lib = Path(lib)
    OBJ = CSRC / ("_obj" if not defines else "_obj_" + "_".join(sorted(defines)).lower())
    OBJ.mkdir(exist_ok=True)
    hdr = _newest_header()
    jobs = []
    for src in sources():
        obj = OBJ / (src.stem + ".o")
        if force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr):
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        cmd = [nvcc(), *NVCC_FLAGS, *[f"-D{d}" for d in defines], "-I", str(INCLUDE), "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        r = subprocess.run(cmd, capture_output=True, text=True)
        return src, r

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        for src, r in ex.map(compile_one, jobs):
            if verbose or r.returncode:
                sys.stderr.write(f"--- {src.name}\n{r.stdout}{r.stderr}")
            if r.returncode:
                raise RuntimeError(f"nvcc failed on {src.name}")
    objs = [OBJ / (s.stem + ".o") for s in sources()]
    if jobs or not lib.exists():
        cmd = [nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(lib), *map(str, objs)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError(f"link of {lib.name} failed")
    return lib


if __name__ == "__main__":
    p = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(p)
