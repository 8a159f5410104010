"""Builds libllmp_b200.so in-tree with nvcc for sm_100a (llmp_b200/csrc/Makefile).  The
tensor-core microbenchmark is a separate target: make -C llmp_b200/csrc probe."""
import os
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))


def build(jobs: int | None = None, verbose: bool = False) -> str:
    jobs = jobs or min(16, os.cpu_count() or 4)
    r = subprocess.run(["make", "-C", os.path.join(_HERE, "csrc"), f"-j{jobs}", "all"],
                       capture_output=not verbose, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc build failed:\n" + (r.stdout or "")[-4000:] + (r.stderr or "")[-4000:])
    return os.path.join(_HERE, "_lib", "libllmp_b200.so")


if __name__ == "__main__":
    print(build(verbose=True))
