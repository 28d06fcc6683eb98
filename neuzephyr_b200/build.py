"""Builds libnzb.so (the sm_100a kernel library) in-tree with nvcc.

    python -m neuzephyr_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU. The shared object is written next to this file so it
travels with a snapshot of the repository.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libnzb.so")
SOURCES = ["nzb_api.cu", "nzb_cast.cu", "nzb_gemm.cu", "nzb_static.cu", "nzb_selftest.cu", "nzb_matmul32.cu", "nzb_host_gemm.cu", "nzb_ops.cu", "nzb_train_ops.cu", "nzb_conv.cu", "nzb_conv_nhwc.cu", "nzb_linear.cu"]
HEADERS = ["nzb_internal.h", "nzb_ptx.cuh", os.path.join("..", "..", "include", "nzb.h")]
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
         "-Xcompiler", "-fPIC,-fvisibility=hidden", "-shared"] + os.environ.get("NZB_EXTRA_NVCC_FLAGS", "").split()


OBJ_DIR = os.path.join(HERE, "build")  # per-source objects, so that editing one file recompiles one file


def _obj(src):
    return os.path.join(OBJ_DIR, src[:-3] + ".o")


def _headers_mtime():
    return max(os.path.getmtime(os.path.join(CSRC, h)) for h in HEADERS)


def _stale_sources():
    hm = _headers_mtime()
    out = []
    for f in SOURCES:
        o = _obj(f)
        if not os.path.exists(o) or os.path.getmtime(o) < max(os.path.getmtime(os.path.join(CSRC, f)), hm):
            out.append(f)
    return out


def _stale():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(os.path.join(CSRC, f)) > t for f in SOURCES + HEADERS)


HOST = os.path.join(HERE, "host")
HOST_LIB = os.path.join(HERE, "libneuzephyr_host.so")
HOST_SOURCES = ["Runtime.cpp", "Ops.cpp", "Nodes.cpp", "Graph.cpp", "DataParallel.cpp"]
CXX = "/usr/bin/g++"
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")


def _host_stale():
    if not os.path.exists(HOST_LIB):
        return True
    t = os.path.getmtime(HOST_LIB)
    files = [os.path.join(HOST, "src", f) for f in HOST_SOURCES]
    inc = os.path.join(HOST, "include", "NeuZephyr")
    files += [os.path.join(inc, f) for f in os.listdir(inc)] + [os.path.join(HERE, "..", "include", "nzb.h")]
    return any(os.path.getmtime(f) > t for f in files)


def host_flags():
    """Compiler flags a program needs to use the C++ host layer (nz:: API) and libnzb."""
    return ["-std=c++17", "-O2", "-I" + os.path.join(HOST, "include"), "-I" + os.path.join(HERE, "..", "include"),
            "-I" + os.path.join(CUDA_HOME, "include")]


def host_link_flags(origin_relative=None):
    """Linker flags for a program using the host layer. origin_relative: path from the program's
    directory to this package, embedded as an $ORIGIN rpath so the program finds the libraries
    wherever the tree is copied."""
    flags = ["-L" + HERE, "-lneuzephyr_host", "-lnzb", "-L" + os.path.join(CUDA_HOME, "lib64"), "-lcudart", "-lnccl",
             "-Wl,-rpath," + os.path.join(CUDA_HOME, "lib64"), "-lpthread"]
    flags.append("-Wl,-rpath," + ("$ORIGIN/" + origin_relative if origin_relative else HERE))
    return flags


def build_program(source, output, origin_relative):
    """Compiles one C++ program against the host layer (used for the C++ tests and tools)."""
    os.makedirs(os.path.dirname(output), exist_ok=True)
    if os.path.exists(output) and os.path.getmtime(output) > max(os.path.getmtime(source), os.path.getmtime(HOST_LIB)):
        return output
    subprocess.check_call([CXX] + host_flags() + [source, "-o", output] + host_link_flags(origin_relative))
    return output


def build_host(force=False):
    """Compiles the C++ host layer (nz:: mirror of NeuZephyr's API) into libneuzephyr_host.so."""
    if not force and not _host_stale():
        return HOST_LIB
    cmd = [CXX] + host_flags() + ["-fPIC", "-shared", "-o", HOST_LIB] + \
        [os.path.join(HOST, "src", f) for f in HOST_SOURCES] + \
        ["-L" + HERE, "-lnzb", "-L" + os.path.join(CUDA_HOME, "lib64"), "-lcudart", "-lnccl",
         "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + os.path.join(CUDA_HOME, "lib64")]
    subprocess.check_call(cmd)
    return HOST_LIB


def build_tools():
    """Compiles the C++ tools shipped with the host layer into neuzephyr_b200/bin/."""
    tools = os.path.join(HOST, "tools")
    out = []
    for name in sorted(os.listdir(tools)):
        if name.endswith(".cpp"):
            out.append(build_program(os.path.join(tools, name), os.path.join(HERE, "bin", name[:-4]), ".."))
    return out


def build(force=False, verbose=False):
    if force or _stale():
        os.makedirs(OBJ_DIR, exist_ok=True)
        todo = SOURCES if force else _stale_sources()
        compile_flags = [f for f in FLAGS if f != "-shared"] + (["-Xptxas", "-v"] if verbose else [])
        procs = [(f, subprocess.Popen([NVCC] + compile_flags + ["-c", f, "-o", _obj(f)], cwd=CSRC)) for f in todo]
        failed = [f for f, p in procs if p.wait() != 0]
        if failed:
            raise subprocess.CalledProcessError(1, "nvcc -c " + " ".join(failed))
        # link to a temporary name and rename: the library in place is always a complete file
        tmp = LIB + ".tmp"
        subprocess.check_call([NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", tmp] +
                              [_obj(f) for f in SOURCES], cwd=CSRC)
        os.replace(tmp, LIB)
    build_host(force)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
