"""Build libcnb200.so in-tree with nvcc for sm_100a.

    python -m charmnumeric_b200.build [--force] [--verbose]

The device header and the exp table are embedded into the library as text, because every
kernel generated at run time includes them through NVRTC.
"""
import hashlib
import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OUT = HERE / "libcnb200.so"
BUILD = HERE / "_build"
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
HOST_SOURCES = ["wire.cpp", "lower.cpp", "fuse.cpp", "regions.cpp", "decomp.cpp", "codegen.cpp", "jit.cpp", "comm.cpp", "context.cpp",
                "executor.cpp", "capi.cpp"]
CUDA_SOURCES = ["kernels.cu", "noalloc.cu"]


def _embed():
    """Write embedded_headers.cpp holding the texts NVRTC needs."""
    dev = (CSRC / "cn_device.cuh").read_text()
    tab = (CSRC / "cn_exp_table.inc").read_text()
    aot = hashlib.sha256((CSRC / "kernels.cu").read_bytes() + (CSRC / "kernels.hpp").read_bytes()).hexdigest()[:8]
    def lit(text):
        # split into chunks: one raw string literal must stay below compiler limits
        parts = [text[i:i + 8000] for i in range(0, len(text), 8000)]
        return "\n".join('R"CNB200(' + p + ')CNB200"' for p in parts)
    body = ('#include "jit.hpp"\nnamespace cn {\n'
            "const char* const kDeviceHeaderText =\n" + lit(dev) + ";\n"
            "const char* const kExpTableText =\n" + lit(tab) + ";\n"
            # the kernels built ahead of time (matvec, dot, halo copies) are identified in
            # profile labels by a digest of their source
            'const char* const kAotSourceDigest = "' + aot + '";\n}\n')
    path = BUILD / "embedded_headers.cpp"
    if not path.exists() or path.read_text() != body:
        path.write_text(body)
    return path


def _digest(paths):
    h = hashlib.sha256()
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def build(force=False, verbose=False):
    BUILD.mkdir(exist_ok=True)
    cuda_sources = [s for s in CUDA_SOURCES if (CSRC / s).exists()]
    inputs = [CSRC / s for s in HOST_SOURCES + cuda_sources]
    inputs += list(CSRC.glob("*.hpp")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.inc"))
    inputs += [HERE.parent / "include" / "cnb200.h", Path(__file__)]
    stamp = BUILD / "stamp"
    digest = _digest(inputs)
    if not force and OUT.exists() and stamp.exists() and stamp.read_text() == digest:
        return OUT
    emb = _embed()
    common = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-Wall,-Wno-unused-function",
              "-I", str(CSRC), "-I", str(BUILD)]
    objs = []
    for src in [CSRC / s for s in HOST_SOURCES] + [emb]:
        obj = BUILD / (src.stem + ".o")
        cmd = [NVCC, "-x", "cu"] + ARCH + common + ["-c", str(src), "-o", str(obj)]
        if verbose:
            print(" ".join(cmd))
        subprocess.run(cmd, check=True)
        objs.append(obj)
    for s in cuda_sources:
        src = CSRC / s
        obj = BUILD / (src.stem + ".o")
        cmd = [NVCC] + ARCH + common + ["-Xptxas", "-v", "-c", str(src), "-o", str(obj)]
        if verbose:
            print(" ".join(cmd))
        res = subprocess.run(cmd, check=True, capture_output=True, text=True)
        (BUILD / (src.stem + ".ptxas.txt")).write_text(res.stderr)
        if verbose:
            print(res.stderr)
        objs.append(obj)
    cmd = [NVCC, "-shared"] + ARCH + ["-o", str(OUT)] + [str(o) for o in objs] + ["-ldl", "-lpthread"]
    if verbose:
        print(" ".join(cmd))
    subprocess.run(cmd, check=True)
    stamp.write_text(digest)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
