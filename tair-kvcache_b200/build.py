"""Builds libkvcm_b200.so in-tree with nvcc for sm_100a.  No torch, no JIT cache."""
import os
import shutil
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libkvcm_b200.so")

SOURCES = ["runtime.cu", "move_rows.cu", "copy_segments.cu", "hash_blocks.cu", "block_index.cu", "replay.cu",
           "replay_lru.cu", "replay_leaf_lru.cu", "replay_random_lru.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall", "-shared",
]


def nvcc():
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the CUDA library cannot be built")
    return exe


def sources():
    return [os.path.join(CSRC, s) for s in SOURCES]


HEADERS = [os.path.join(CSRC, "kvcm_common.cuh"), os.path.join(CSRC, "replay_ids.cuh"),
           os.path.join(CSRC, "replay_sampling.cuh"), os.path.join(CSRC, "id_table.cuh"),
           os.path.join(ROOT, "include", "kvcm_b200.h")]
OBJ_DIR = os.path.join(HERE, "build")


def _newer(path, than):
    return not os.path.exists(than) or os.path.getmtime(path) > os.path.getmtime(than)


def is_stale():
    return any(_newer(d, LIB) for d in sources() + HEADERS)


def build_library(force=False, verbose=False):
    """Compile every kernel for sm_100a into tair-kvcache_b200/libkvcm_b200.so: one object per source file
    (compiled side by side, only the ones whose source or a shared header changed), then one link."""
    from concurrent.futures import ThreadPoolExecutor
    if not force and not is_stale():
        return LIB
    os.makedirs(OBJ_DIR, exist_ok=True)
    flags = [f for f in NVCC_FLAGS if f != "-shared"] + ["-I", os.path.join(ROOT, "include"), "-I", CSRC]
    if verbose:
        flags += ["-Xptxas", "-v"]

    def compile_one(src):
        obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o")
        if not force and not verbose and not _newer(src, obj) and not any(_newer(h, obj) for h in HEADERS):
            return obj, 0, ""
        proc = subprocess.run([nvcc()] + flags + ["-c", "-o", obj, src], stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True)
        return obj, proc.returncode, proc.stdout

    with ThreadPoolExecutor(max_workers=min(len(SOURCES), os.cpu_count() or 1)) as pool:
        results = list(pool.map(compile_one, sources()))
    for obj, rc, out in results:
        if verbose or rc != 0:
            print(out)
        if rc != 0:
            raise RuntimeError("nvcc failed on %s (exit %d)" % (os.path.basename(obj), rc))
    cmd = [nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB] + [o for o, _, _ in results]
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        print(proc.stdout)
        raise RuntimeError("linking libkvcm_b200.so failed (exit %d)" % proc.returncode)
    return LIB


HOST_TEST_SRC = os.path.join(ROOT, "tests", "cpp", "host_adapter_test.cc")
HOST_TEST_BIN = os.path.join(ROOT, "tests", "cpp", "host_adapter_test.bin")


def build_host_adapter_test():
    """Compile the C++ test of the host adapters against the built library (host code only; nvcc is used as the
    compiler driver so that the CUDA runtime headers and library are found)."""
    cmd = [nvcc(), "-O2", "-std=c++17", "-I", os.path.join(ROOT, "include"), "-I", os.path.join(HERE, "host"),
           "-o", HOST_TEST_BIN, HOST_TEST_SRC, "-L", HERE, "-lkvcm_b200", "-Xlinker", "-rpath=" + HERE]
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        print(proc.stdout)
        raise RuntimeError("building the host adapter test failed (exit %d)" % proc.returncode)
    return HOST_TEST_BIN


def pybind_path():
    import sysconfig
    return os.path.join(HERE, "kvcm_b200_py" + sysconfig.get_config_var("EXT_SUFFIX"))


def build_pybind_shim():
    """Compile the pybind11 shim for py_connector (plain g++: it only forwards to the C ABI)."""
    import sysconfig

    import pybind11
    out = pybind_path()
    src = os.path.join(HERE, "pybind", "kvcm_b200_py.cc")
    cxx = shutil.which("g++") or "g++"
    cmd = [cxx, "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden", "-I", pybind11.get_include(),
           "-I", sysconfig.get_paths()["include"], "-I", os.path.join(ROOT, "include"), "-o", out, src,
           "-L", HERE, "-lkvcm_b200", "-Wl,-rpath,$ORIGIN"]
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        print(proc.stdout)
        raise RuntimeError("building the pybind shim failed (exit %d)" % proc.returncode)
    return out


if __name__ == "__main__":
    import sys
    print(build_library(force=True, verbose="-v" in sys.argv))
    print(build_host_adapter_test())
    print(build_pybind_shim())
