"""Builds and loads the sm_100a kernel libraries.

Each library is one or more `.cu` files of this folder compiled by nvcc into a
shared object of plain C entry points, loaded with ctypes.  A library is built
the first time something needs it (so a run compiles what its model uses) and
is found again by a hash of its sources and flags; a progress line is printed
while nvcc runs.  There is no fallback: without nvcc or without the sources
the call fails with the reason.
"""
import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time

HERE = os.path.dirname(os.path.abspath(__file__))

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC"]

# library name -> (sources, extra nvcc flags, libraries to link)
LIBRARIES = {
    "core": (["core.cu"], [], []),
    "gemm_simt": (["gemm_simt.cu"], [], []),
    "attention_generic": (["attention_generic.cu"], [], []),
    "sampling": (["sampling.cu"], [], []),
    "gemm_tc": (["gemm_tc.cu"], [], []),
    "attention_bf16": (["attention_bf16.cu"], [], []),
    "attention_tc": (["attention_tc.cu"], [], []),
}
HEADERS = ["common.cuh", "attn_decode_noalloc.h"]

_loaded = {}
_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 shutil.which("nvcc")):
        if cand and os.path.isfile(cand):
            return cand
    raise BuildError("nvcc was not found (looked at $NVCC, $CUDA_HOME/bin, /usr/local/cuda/bin and PATH); "
                     "the kernels of this library cannot be built")


def build_dir() -> str:
    """In-tree `_build/` when it can be written, else a per-user folder under
    the system's temporary directory ($GPT_FAST_B200_BUILD_DIR overrides)."""
    cands = [os.environ.get("GPT_FAST_B200_BUILD_DIR"), os.path.join(HERE, "_build"),
             os.path.join(tempfile.gettempdir(), f"gpt_fast_b200-build-{os.getuid()}")]
    for d in cands:
        if not d:
            continue
        try:
            os.makedirs(d, exist_ok=True)
            probe = os.path.join(d, f".probe-{os.getpid()}")
            with open(probe, "w"):
                pass
            os.remove(probe)
            return d
        except OSError:
            continue
    raise BuildError(f"no writable build folder among {cands}")


def _digest(name: str) -> str:
    sources, flags, libs = LIBRARIES[name]
    h = hashlib.sha256()
    for fn in list(sources) + HEADERS:
        path = os.path.join(HERE, fn)
        if not os.path.isfile(path):
            raise BuildError(f"kernel source {path} is missing")
        with open(path, "rb") as f:
            h.update(fn.encode() + b"\0" + f.read())
    h.update(" ".join(ARCH_FLAGS + COMMON_FLAGS + flags + libs).encode())
    return h.hexdigest()[:16]


def library_path(name: str, must_exist=False):
    """Path of the built library for the current sources (searched in the
    in-tree folder first, so that a library built beforehand is used even when
    the tree is read-only)."""
    fn = f"libgfb_{name}-{_digest(name)}.so"
    in_tree = os.path.join(HERE, "_build", fn)
    if os.path.isfile(in_tree):
        return in_tree
    if must_exist:
        return None
    return os.path.join(build_dir(), fn)


def build(name: str, verbose=True) -> str:
    """Compile library `name` if its current build is absent; return its path."""
    if name not in LIBRARIES:
        raise BuildError(f"unknown kernel library '{name}'")
    path = library_path(name)
    if os.path.isfile(path):
        return path
    sources, flags, libs = LIBRARIES[name]
    tmp = f"{path}.{os.getpid()}.tmp"
    cmd = [_nvcc()] + ARCH_FLAGS + COMMON_FLAGS + flags + ["-I", HERE, "-o", tmp] + \
          [os.path.join(HERE, s) for s in sources] + [f"-l{l}" for l in libs]
    t0 = time.time()
    if verbose:
        print(f"[gpt_fast_b200] compiling kernel library '{name}' for sm_100a ...", file=sys.stderr, flush=True)
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    done = threading.Event()

    def ticker():
        while not done.wait(10.0):
            if verbose:
                print(f"[gpt_fast_b200]   still compiling '{name}' ({time.time() - t0:.0f} s)", file=sys.stderr, flush=True)
    th = threading.Thread(target=ticker, daemon=True)
    th.start()
    out, _ = proc.communicate()
    done.set()
    if proc.returncode != 0:
        if os.path.exists(tmp):
            os.remove(tmp)
        raise BuildError(f"nvcc failed for kernel library '{name}':\n{' '.join(cmd)}\n{out}")
    os.replace(tmp, path)
    if verbose:
        print(f"[gpt_fast_b200]   built '{name}' in {time.time() - t0:.1f} s -> {path}", file=sys.stderr, flush=True)
    return path


def library(name: str) -> ctypes.CDLL:
    """The loaded library `name` (built first if needed)."""
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            lib = ctypes.CDLL(build(name))
            lib.gfb_last_error.restype = ctypes.c_char_p
            _loaded[name] = lib
        return lib


def build_all(names=None, verbose=True, prune=True):
    """Build every library (or `names`); with prune, builds of earlier source states are removed from the
    folder the current ones went to, so that it holds one file per library."""
    built = {n: build(n, verbose) for n in (names or LIBRARIES) if _sources_exist(n)}
    if prune:
        keep = {os.path.basename(p) for p in built.values()}
        for folder in {os.path.dirname(p) for p in built.values()}:
            for fn in os.listdir(folder):
                stem = fn.split("-")[0]
                if fn.endswith(".so") and stem in {f"libgfb_{n}" for n in built} and fn not in keep:
                    try:
                        os.remove(os.path.join(folder, fn))
                    except OSError:
                        pass
    return built


def _sources_exist(name):
    return all(os.path.isfile(os.path.join(HERE, s)) for s in LIBRARIES[name][0])
