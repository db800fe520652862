"""Build libfa_b200.so for sm_100a with nvcc (cross-compiles without a GPU).

    python flash-attention-npu_b200/build.py [--force]

One object per .cu file, compiled in parallel, linked into lib/libfa_b200.so."""
import concurrent.futures as cf
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "lib")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
         "-Xcompiler", "-fPIC", "-DFA_B200", "-Xptxas", "-v"]


def _newer(a, b):
    return not os.path.exists(b) or os.path.getmtime(a) > os.path.getmtime(b)


def build(force=False, verbose=False):
    os.makedirs(OUT, exist_ok=True)
    os.makedirs(os.path.join(HERE, "build"), exist_ok=True)
    sources = sorted(glob.glob(os.path.join(SRC, "*.cu")))
    headers = glob.glob(os.path.join(SRC, "*.h")) + glob.glob(os.path.join(SRC, "*.cuh")) + \
        glob.glob(os.path.join(HERE, "..", "include", "*.h"))
    newest_header = max(os.path.getmtime(h) for h in headers)
    jobs = []
    objs = []
    for s in sources:
        o = os.path.join(HERE, "build", os.path.basename(s)[:-3] + ".o")
        objs.append(o)
        if force or _newer(s, o) or os.path.getmtime(o) < newest_header:
            jobs.append((s, o))

    def compile_one(job):
        s, o = job
        r = subprocess.run([NVCC] + FLAGS + ["-c", s, "-o", o], capture_output=True, text=True)
        with open(o[:-2] + ".log", "w") as f:
            f.write(r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {s}:\n{r.stdout}\n{r.stderr}")
        return s

    with cf.ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for s in ex.map(compile_one, jobs):
            if verbose:
                print("compiled", os.path.basename(s))
    lib = os.path.join(OUT, "libfa_b200.so")
    if jobs or not os.path.exists(lib):
        r = subprocess.run([NVCC, "-shared", "-o", lib] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"],
                           capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n" + r.stdout + r.stderr)
    return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
