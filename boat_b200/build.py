"""Build ``libboat_b200.so`` in-tree with make (gcc for the C host layer, nvcc for sm_100a)."""
import os
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))


def build(jobs=None, verbose=False):
    """Compile every CUDA and C source under ``csrc/`` into ``boat_b200/libboat_b200.so``.

    nvcc cross-compiles for sm_100a, so this works on a machine without a GPU.  Raises
    ``RuntimeError`` with the compiler output when the build fails.
    """
    jobs = jobs or os.cpu_count() or 4
    cmd = ["make", "-C", os.path.join(_HERE, "csrc"), "-j%d" % jobs]
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if verbose:
        print(proc.stdout)
    if proc.returncode != 0:
        raise RuntimeError("building libboat_b200.so failed:\n" + proc.stdout[-8000:])
    return os.path.join(_HERE, "libboat_b200.so")
