"""Builds gradcraft_b200/libgradc_b200.so from csrc/*.cu with nvcc for sm_100a (in-tree, incremental)."""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libgradc_b200.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC", 
         "--expt-relaxed-constexpr", "-Xptxas", "-v"]


def _newer(src, dst, extra=()):
    if not os.path.exists(dst):
        return True
    t = os.path.getmtime(dst)
    return any(os.path.getmtime(p) > t for p in (src,) + tuple(extra))


def build(verbose=False, force=False):
    os.makedirs(OBJ, exist_ok=True)
    headers = tuple(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))) + (os.path.join(HERE, "..", "include", "gradc_b200.h"),)
    srcs = sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))
    jobs = []
    for f in srcs:
        src, obj = os.path.join(CSRC, f), os.path.join(OBJ, f[:-3] + ".o")
        if force or _newer(src, obj, headers):
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        r = subprocess.run([NVCC] + FLAGS + ["-c", src, "-o", obj], capture_output=True, text=True)
        with open(obj[:-2] + ".ptxas.log", "w") as fh:
            fh.write(r.stderr)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed for %s:\n%s" % (src, r.stderr[-6000:]))
        if verbose:
            print("compiled", os.path.basename(src))
        return obj

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        list(ex.map(compile_one, jobs))
    objs = [os.path.join(OBJ, f[:-3] + ".o") for f in srcs]
    if jobs or not os.path.exists(LIB):
        r = subprocess.run([NVCC, "-shared", "-o", LIB] + objs + ["-lcudart", "-ldl", "-Xlinker", "-rpath", "-Xlinker", "/usr/local/cuda/lib64"], capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n" + r.stderr[-4000:])
        if verbose:
            print("linked", LIB)
    build_trainer(verbose, force or bool(jobs))
    return LIB


TRAINER_SRC = os.path.join(CSRC, "host", "trainer.cpp")
TRAINER_LIB = os.path.join(HERE, "libgradc_trainer.so")


def build_trainer(verbose=False, force=False):
    """Host-side C++ (the gradc API mirror + the training step) into libgradc_trainer.so, linked against the kernel library."""
    hdrs = tuple(os.path.join(HERE, "gradc", f) for f in os.listdir(os.path.join(HERE, "gradc"))) + (os.path.join(HERE, "..", "include", "gradc_trainer.h"), os.path.join(HERE, "..", "include", "gradc_b200.h"))
    if not (force or _newer(TRAINER_SRC, TRAINER_LIB, hdrs)):
        return TRAINER_LIB
    cmd = ["g++", "-std=c++20", "-O2", "-fPIC", "-shared", "-fvisibility=hidden", "-I/usr/local/cuda/include", TRAINER_SRC, "-o", TRAINER_LIB,
           "-L" + HERE, "-lgradc_b200", "-L/usr/local/cuda/lib64", "-lcudart", "-Wl,-rpath,$ORIGIN", "-Wl,-rpath,/usr/local/cuda/lib64"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("g++ failed for trainer.cpp:\n" + r.stderr[-6000:])
    if verbose:
        print("linked", TRAINER_LIB)
    return TRAINER_LIB


TRAIN_BIN = os.path.join(OBJ, "train_ref")


def reference_root():
    """Where the reference project's source tree is: the GRADC_REFERENCE_ROOT environment variable, else a directory named
    `reference` beside this repository.  Returns None when neither holds a GradCraft tree (prebuilt checker binaries are then used as they are)."""
    cands = [os.environ.get("GRADC_REFERENCE_ROOT"), os.path.join(HERE, "..", "..", "reference")]
    for c in cands:
        if c and os.path.isdir(os.path.join(c, "gradc")):
            return os.path.abspath(c)
    return None


def build_reference_train(reference_root=None, verbose=False):
    """Compiles the reference's own train.cpp, unchanged, against gradcraft_b200/gradc and links it with the sm_100a backend.
    The source is read where it lies (a scratch copy is needed only because a quoted include searches the including file's
    directory first); nothing of it is stored in this repository.  Returns the binary's path, or None without the reference."""
    import shutil
    import tempfile

    if reference_root is None:
        reference_root = globals()["reference_root"]()
    src = os.path.join(reference_root or "", "train.cpp")
    if not os.path.exists(src):
        return TRAIN_BIN if os.path.exists(TRAIN_BIN) else None
    hdrs = tuple(os.path.join(HERE, "gradc", f) for f in os.listdir(os.path.join(HERE, "gradc")))
    if not _newer(src, TRAIN_BIN, hdrs + (LIB,)):
        return TRAIN_BIN
    os.makedirs(OBJ, exist_ok=True)
    with tempfile.TemporaryDirectory() as tmp:
        shutil.copy(src, os.path.join(tmp, "train.cpp"))
        cmd = ["g++", "-std=c++23", "-O2", "-I", HERE, "-I/usr/local/cuda/include", os.path.join(tmp, "train.cpp"), "-o", TRAIN_BIN,
               "-L" + HERE, "-lgradc_b200", "-L/usr/local/cuda/lib64", "-lcudart", "-Wl,-rpath,$ORIGIN/..", "-Wl,-rpath,/usr/local/cuda/lib64"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("train.cpp did not build against the host API:\n" + r.stderr[-6000:])
    if verbose:
        print("built", TRAIN_BIN)
    return TRAIN_BIN


if __name__ == "__main__":
    build(verbose=True, force="--force" in sys.argv)
    build_reference_train(verbose=True)
