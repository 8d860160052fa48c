"""In-tree build of the native extension (``astrai_b200/ops/_C.so``).

Kernels are plain ``.cu`` files compiled by nvcc for sm_100a only; a single C++ file binds them to
``torch.ops.astrai_b200``.  Object files are cached by source hash under ``ops/build/``.  Run as
``python -m astrai_b200.ops.build`` or call :func:`build`.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
SRC = HERE / "csrc"
OUT = HERE / "build"
LIB = HERE / "_C.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "--use_fast_math",
]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; the sm_100a extension cannot be built")
    return cand


def _digest(path: Path, extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    h.update(path.read_bytes())
    for header in sorted(SRC.glob("*.h")) + sorted(SRC.glob("*.cuh")):
        h.update(header.read_bytes())
    return h.hexdigest()[:16]


def _run(cmd):
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("command failed: " + " ".join(map(str, cmd)) + "\n" + proc.stdout + proc.stderr)
    return proc.stdout + proc.stderr


def _compile_one(src: Path, verbose: bool) -> Path:
    import torch
    from torch.utils import cpp_extension as ce

    if src.suffix == ".cu":
        cmd = [_nvcc(), *NVCC_FLAGS, "-I", str(SRC), "-c", str(src)]
        if verbose:
            cmd += ["-Xptxas", "-v"]
    else:
        incs = [p for p in ce.include_paths(device_type="cuda")] + [sysconfig.get_path("include"), str(SRC)]
        cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI),
               "-DTORCH_API_INCLUDE_EXTENSION_H", "-w"]
        for i in incs:
            cmd += ["-isystem", i]
        cmd += ["-c", str(src)]
    obj = OUT / f"{src.stem}.{_digest(src, ' '.join(cmd))}.o"
    if not obj.exists():
        for stale in OUT.glob(f"{src.stem}.*.o"):
            stale.unlink()
        log = _run(cmd + ["-o", str(obj)])
        if verbose and log.strip():
            print(log)
    return obj


def sources():
    return sorted(SRC.glob("*.cu")) + sorted(SRC.glob("*.cpp"))


def build(verbose: bool = False, force: bool = False) -> Path:
    """Compile every source for sm_100a and link ``_C.so``.  Returns the library path."""
    import torch
    from torch.utils import cpp_extension as ce

    OUT.mkdir(exist_ok=True)
    if force:
        for o in OUT.glob("*.o"):
            o.unlink()
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        objs = list(pool.map(lambda s: _compile_one(s, verbose), sources()))
    stamp = OUT / "link.stamp"
    key = " ".join(o.name for o in objs)
    if LIB.exists() and stamp.exists() and stamp.read_text() == key:
        return LIB
    torch_lib = Path(torch.__file__).parent / "lib"
    cuda_lib = Path(_nvcc()).resolve().parent.parent / "lib64"
    cmd = ["g++", "-shared", "-o", str(LIB), *map(str, objs), f"-L{torch_lib}", f"-L{cuda_lib}",
           "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-lcudart",
           f"-Wl,-rpath,{torch_lib}", f"-Wl,-rpath,{cuda_lib}"]
    _run(cmd)
    stamp.write_text(key)
    return LIB


STANDALONE = {
    # torch-free check binaries: main source -> the kernel sources it links
    "attn_check": ("flash_fwd.cu", "paged_attention.cu"),
    "quant_paged_check": ("gemm_tcgen05.cu", "gemm_tcgen05_2cta.cu", "gemm_fp8.cu", "gemm_fp8_block.cu", "flash_fwd.cu"),
}


def build_standalone(which: str = "attn_check") -> Path:
    """Link one of the torch-free check programs (``csrc/standalone/<which>.cu`` + the objects of the kernels it calls)."""
    OUT.mkdir(exist_ok=True)
    objs = [_compile_one(SRC / name, False) for name in STANDALONE[which]]
    main_src = SRC / "standalone" / f"{which}.cu"
    exe = OUT / which
    _run([_nvcc(), *NVCC_FLAGS, "-I", str(SRC), str(main_src), *map(str, objs), "-o", str(exe), "-lcudart"])
    return exe


def main(argv=None) -> int:
    """``python -m astrai_b200.ops.build [-v] [--force] [--standalone]``: build the extension (or the torch-free test
    programs) in the source tree and print what was written."""
    argv = sys.argv[1:] if argv is None else list(argv)
    unknown = [a for a in argv if a not in ("-v", "--force", "--standalone")]
    if unknown:
        print(f"unknown option(s): {' '.join(unknown)}\nusage: python -m astrai_b200.ops.build [-v] [--force] [--standalone]", file=sys.stderr)
        return 2
    if "--standalone" in argv:
        for name in STANDALONE:
            print(build_standalone(name))
    else:
        print(build(verbose="-v" in argv, force="--force" in argv))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
