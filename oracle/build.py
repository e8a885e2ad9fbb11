"""TEST INFRASTRUCTURE ONLY: builds the CPU oracle.

  liboracle.so            the restatement (surfel_oracle.cpp: the tracer; prep_oracle.cpp: quad
                          expansion and ray generation), always
  _ref/libref_{fwd,bwd}{1,2}.so   the reference's own shader sources compiled for the host
                          (ref_driver.cpp), only where the reference tree is present

Run as `python oracle/build.py`. The reference tree is taken from $DST_REFERENCE_DIR, else from a
directory `reference` next to this repository; it is read in place, never copied.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.environ.get("DST_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
CUDA_INC = os.environ.get("CUDA_HOME", "/usr/local/cuda") + "/include"
COMMON = ["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-fopenmp", "-ffp-contract=off", "-mfma", "-fno-fast-math"]


def _stale(out, srcs):
    if not os.path.exists(out):
        return True
    t = os.path.getmtime(out)
    return any(os.path.exists(s) and os.path.getmtime(s) > t for s in srcs)


def build_restatement(force=False):
    out = os.path.join(HERE, "liboracle.so")
    srcs = [os.path.join(HERE, f) for f in ("surfel_oracle.cpp", "prep_oracle.cpp", "quad_enum.h", "orc_args.h")]
    if force or _stale(out, srcs):
        subprocess.check_call(COMMON + ["-Wall", "-Wno-unused", "-o", out, srcs[0], srcs[1]])
    return out


def reference_available():
    return os.path.exists(os.path.join(REF, "optix_tracer", "forward.cu"))


def build_reference(force=False):
    """Returns the list of built libraries, or [] when the reference tree is absent."""
    if not reference_available():
        return []
    outdir = os.path.join(HERE, "_ref")
    os.makedirs(outdir, exist_ok=True)
    srcs = [os.path.join(HERE, f) for f in ("ref_driver.cpp", "quad_enum.h", "orc_args.h", "optix.h")]
    srcs += [os.path.join(REF, "optix_tracer", f) for f in ("forward.cu", "backward.cu", "auxiliary.h", "params.h", "config.h")]
    outs = []
    for which, flag in (("fwd", []), ("bwd", ["-DREF_BACKWARD"])):
        for mtd in (1, 2):
            out = os.path.join(outdir, f"libref_{which}{mtd}.so")
            if force or _stale(out, srcs):
                subprocess.check_call(COMMON + ["-w", "-Wno-narrowing", "-x", "c++", f"-DREF_MTD={mtd}"] + flag +
                                      ["-I", HERE, "-I", os.path.join(REF, "optix_tracer"), "-I", CUDA_INC,
                                       "-o", out, srcs[0]])
            outs.append(out)
    return outs


if __name__ == "__main__":
    force = "--force" in sys.argv
    print(build_restatement(force))
    for o in build_reference(force):
        print(o)
