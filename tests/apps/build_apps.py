"""Builds the compat-layer test applications (tests/apps/compat_apps.cu) against include/nextdoor/
and libnextdoor_b200.so.  Where the reference tree is present its application files are compiled
in as well, from where they lie (output under tests/apps/_ref/, not tracked by git)."""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
REF = os.environ.get("NEXTDOOR_REFERENCE", "/root/reference")
OWN = os.path.join(HERE, "libnd_compat_apps.so")
WITH_REF = os.path.join(HERE, "_ref", "libnd_compat_ref.so")


def _build(out, extra):
    src = os.path.join(HERE, "compat_apps.cu")
    deps = [src] + [os.path.join(ROOT, "include", "nextdoor", f) for f in os.listdir(os.path.join(ROOT, "include", "nextdoor"))]
    if os.path.exists(out) and os.path.getmtime(out) >= max(os.path.getmtime(d) for d in deps):
        return out
    os.makedirs(os.path.dirname(out), exist_ok=True)
    cmd = [NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-fmad=false", "-w",
           "-Xcompiler", "-fPIC", "-shared", "-I", os.path.join(ROOT, "include", "nextdoor"), "-I", os.path.join(ROOT, "include")] + extra + \
          [src, "-o", out, "-L", os.path.join(ROOT, "nextdoor_b200"), "-lnextdoor_b200",
           "-Xlinker", "-rpath," + os.path.join("$ORIGIN", os.path.relpath(os.path.join(ROOT, "nextdoor_b200"), os.path.dirname(out)))]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        raise RuntimeError("nvcc failed for the compat apps")
    return out


def _build_module(src, out, extra):
    """A CPython extension module from an application file that ends with
    #include "nextDoorPythonModule.cu" -- the build line of the reference's example/Makefile:9-11
    (py3module) with this repository's include/nextdoor/ in place of the reference's src/."""
    import sysconfig
    deps = [src] + [os.path.join(ROOT, "include", "nextdoor", f) for f in os.listdir(os.path.join(ROOT, "include", "nextdoor"))]
    if os.path.exists(out) and os.path.getmtime(out) >= max(os.path.getmtime(d) for d in deps):
        return out
    os.makedirs(os.path.dirname(out), exist_ok=True)
    cmd = [NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-fmad=false", "-w", "-DPYTHON_3",
           "-Xcompiler", "-fPIC", "-shared", "-I", sysconfig.get_paths()["include"],
           "-I", os.path.join(ROOT, "include", "nextdoor"), "-I", os.path.join(ROOT, "include")] + extra + \
          [src, "-o", out, "-L", os.path.join(ROOT, "nextdoor_b200"), "-lnextdoor_b200",
           "-Xlinker", "-rpath," + os.path.join("$ORIGIN", os.path.relpath(os.path.join(ROOT, "nextdoor_b200"), os.path.dirname(out)))]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        raise RuntimeError("nvcc failed for the Python module " + out)
    return out


OWN_MODULE = os.path.join(HERE, "NdOwnWalkPy3.so")
REF_MODULE = os.path.join(HERE, "_ref", "UniformRandomWalkPy3.so")   # the name the reference's example builds


def build():
    outs = [_build(OWN, []), _build_module(os.path.join(HERE, "own_walk_module.cu"), OWN_MODULE, [])]
    if os.path.isdir(os.path.join(REF, "src")):
        outs.append(_build(WITH_REF, ["-DNDC_WITH_REFERENCE", "-I", os.path.join(REF, "src"), "-I", os.path.join(REF, "example")]))
        # the reference's own example application, unchanged, as its README builds it
        outs.append(_build_module(os.path.join(REF, "example", "uniformRandWalk.cu"), REF_MODULE, []))
    return outs


if __name__ == "__main__":
    print(build())
