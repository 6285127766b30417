"""Builds libSpMM_API.so in-tree with nvcc for sm_100a (cross-compiles without a GPU)."""
import os
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(_HERE, "csrc")
LIB_PATH = os.path.join(_HERE, "libSpMM_API.so")
SOURCES = ["spmm_api.cu", "encode_tiled_csl.cu", "encode_structured.cu", "pack_a1_tcgen05.cu", "allreduce_peer.cu", "host_utils.cu",
           "validate.cu", "model_files.cu"]
NVCC_FLAGS = [
    "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "-Xcompiler", "-fPIC", "-shared",
]


def _newest_source_mtime():
    newest = 0.0
    for root in (CSRC, os.path.join(_HERE, "..", "include")):
        for name in os.listdir(root):
            if name.endswith((".cu", ".cuh", ".h")):
                newest = max(newest, os.path.getmtime(os.path.join(root, name)))
    return newest


def build(force=False, verbose=False):
    """Compile the library if it is missing or older than any source. Returns its path.

    Safe when several processes (the ranks of one job) find the library stale at once: one compiles, into a
    temporary file that is renamed into place, the others wait on a lock file and then find it fresh."""
    def fresh():
        return os.path.exists(LIB_PATH) and os.path.getmtime(LIB_PATH) >= _newest_source_mtime()

    if not force and fresh():
        return LIB_PATH
    import fcntl
    with open(LIB_PATH + ".lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and fresh():
                return LIB_PATH
            nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
            tmp = "%s.%d.tmp" % (LIB_PATH, os.getpid())
            cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-o", tmp] + SOURCES
            proc = subprocess.run(cmd, cwd=CSRC, capture_output=True, text=True)
            if proc.returncode != 0:
                if os.path.exists(tmp):
                    os.remove(tmp)
                raise RuntimeError("nvcc failed:\n" + proc.stdout + proc.stderr)
            os.replace(tmp, LIB_PATH)
            if verbose:
                print(proc.stderr)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force=True, verbose=True))
