"""In-tree build of the runner-utils shared libraries for sm_100a.

`python hands-on-mlir_b200/build.py` compiles every `.cu`/`.cpp` under `csrc/` with nvcc
(`-gencode arch=compute_100a,code=sm_100a`) and links

  lib/libhands_on_mlir_nvgpu_runner_utils.so   the kernel layer (same file name as the
                                               library the reference builds in
                                               lib/CMakeLists.txt:40-55)
  lib/libhom_bert_replay.so                    the BERT call-sequence replay program

nvcc cross-compiles without a GPU, so this also runs on a CPU-only machine.

`python hands-on-mlir_b200/build.py --diagnostics` builds a second copy of both libraries
under lib/diagnostics/ with -DHOM_DIAGNOSTICS (role cycle counters, launch timelines and the
experiment knobs read from the environment); set HOM_LIB_DIR to that directory to load it.
The product build contains none of that code.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
REPO_DIR = PKG_DIR.parent
CSRC = PKG_DIR / "csrc"
LIB_DIR = PKG_DIR / "lib"
OBJ_DIR = PKG_DIR / "build"
INCLUDE = REPO_DIR / "include"

RUNNER_LIB = LIB_DIR / "libhands_on_mlir_nvgpu_runner_utils.so"
REPLAY_LIB = LIB_DIR / "libhom_bert_replay.so"

RUNNER_SOURCES = [
    "context.cu",
    "gemm_sm100.cu",
    "gemm_pair_sm100.cu",
    "attention_sm100.cu",
    "attention_pingpong_sm100.cu",
    "bandwidth_kernels.cu",
    "runner_utils.cu",
    "no_alloc_entry.cu",
]
REPLAY_SOURCES = ["bert_replay.cpp", "model_loader.cpp"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
    f"-I{INCLUDE}", f"-I{CSRC}",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; set NVCC or put it on PATH")


def _newest_header_mtime() -> float:
    files = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list(INCLUDE.glob("*.h"))
    files.append(Path(__file__))
    return max(f.stat().st_mtime for f in files)


def _compile(src: Path, obj: Path, verbose: bool, extra: tuple[str, ...] = ()) -> None:
    cmd = [_nvcc(), *NVCC_FLAGS, *extra, "-c", str(src), "-o", str(obj)]
    if src.suffix == ".cpp":
        cmd[1:1] = ["-x", "cu"]
    if verbose:
        print(" ".join(cmd), flush=True)
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{proc.stdout}\n{proc.stderr}")


def _link(objs: list[Path], out: Path, extra: list[str], verbose: bool) -> None:
    cmd = [_nvcc(), "-shared", "-o", str(out), *map(str, objs), *extra]
    if verbose:
        print(" ".join(cmd), flush=True)
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"link failed for {out.name}:\n{proc.stdout}\n{proc.stderr}")


def build(force: bool = False, verbose: bool = False, diagnostics: bool = False) -> dict[str, Path]:
    """Compile what is out of date and return the paths of the two libraries."""
    lib_dir = LIB_DIR / "diagnostics" if diagnostics else LIB_DIR
    obj_dir = OBJ_DIR / "diagnostics" if diagnostics else OBJ_DIR
    runner_lib, replay_lib = lib_dir / RUNNER_LIB.name, lib_dir / REPLAY_LIB.name
    # The diagnostics build also brackets every launch in an NVTX range named after its op family
    # (hom.gemm, hom.attention, ...), for timelines taken with an external profiler.
    extra = ("-DHOM_DIAGNOSTICS", "-DHOM_NVTX") if diagnostics else ()
    lib_dir.mkdir(parents=True, exist_ok=True)
    obj_dir.mkdir(parents=True, exist_ok=True)
    hdr_mtime = _newest_header_mtime()
    jobs = []
    objs: dict[str, Path] = {}
    for name in RUNNER_SOURCES + REPLAY_SOURCES:
        src = CSRC / name
        if not src.exists():
            continue
        obj = obj_dir / (src.stem + ".o")
        objs[name] = obj
        stale = force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_mtime)
        if stale:
            jobs.append((src, obj))
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
        for fut in [pool.submit(_compile, s, o, verbose, extra) for s, o in jobs]:
            fut.result()

    runner_objs = [objs[n] for n in RUNNER_SOURCES if n in objs]
    if force or jobs or not runner_lib.exists():
        _link(runner_objs, runner_lib, [], verbose)
    replay_objs = [objs[n] for n in REPLAY_SOURCES if n in objs]
    if replay_objs and (force or jobs or not replay_lib.exists()):
        _link(replay_objs, replay_lib,
              [f"-L{lib_dir}", "-lhands_on_mlir_nvgpu_runner_utils", "-ldl", "-Xlinker",
               "-rpath=$ORIGIN"],
              verbose)
    return {"runner": runner_lib, "replay": replay_lib}


if __name__ == "__main__":
    out = build(force="--force" in sys.argv, verbose=True, diagnostics="--diagnostics" in sys.argv)
    for k, v in out.items():
        print(f"{k}: {v} ({'ok' if v.exists() else 'missing'})")
