"""Build the reference (JiangkuoWang/PlanMoE) offline into ``baseline/_ref``.

The reference does not install as shipped: its ``setup.py`` compiles sources under ``./schemoe/custom/`` while
the tree on disk is ``PlanMoE/`` (setup.py:130-143), and it links a privately patched libzfp from the authors'
home directory (setup.py:127,146; zfpc.cpp:35).  This script copies the reference to a scratch directory, makes
the BUILD-ONLY edits listed in ``PATCHES`` (nothing on the timed path of the naive/no MoE layer changes) and
installs the result with pip, offline, into ``baseline/_ref``.

    python baseline/build_reference.py --src <reference checkout> [--keep]

Every edit asserts that its pattern was found, so a reference that differs from the one surveyed fails loudly.
``bench.py --impl reference`` only ever imports from ``baseline/_ref``.
"""
import argparse
import os
import re
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")

# (file, what, why) -- printed into baseline/_ref/BUILD_PATCHES.txt
PATCHES = [
    ("PlanMoE/ -> schemoe/", "directory renamed",
     "setup.py:130-143 names ./schemoe/custom/*.cpp and every Python file imports `schemoe`"),
    ("setup.py", "dropped library `zfp`, source zfpc.cpp and the /home/xinglinpan include/library dirs; "
     "CUDA stubs dir points at this image's CUDA",
     "the patched libzfp the authors linked is not part of the repository (zfpc.cpp:35 uses a member stock zfp lacks)"),
    ("schemoe/custom/custom_kernel.cpp", "removed `#include \"zfp.h\"`, `#include \"compressor/zfpc.h\"` and the "
     "`name == \"zfp\"` factory branch", "same: no libzfp; codec 'zfp' is not part of the measured config"),
]


def _sub(path, pattern, repl, count=1, flags=0):
    with open(path) as f:
        src = f.read()
    new, n = re.subn(pattern, repl, src, count=count, flags=flags)
    assert n >= 1, f"pattern {pattern!r} not found in {path}"
    with open(path, "w") as f:
        f.write(new)


def prepare(src, work):
    tree = os.path.join(work, "reference")
    shutil.copytree(src, tree, ignore=shutil.ignore_patterns(".git"))
    os.rename(os.path.join(tree, "PlanMoE"), os.path.join(tree, "schemoe"))
    setup_py = os.path.join(tree, "setup.py")
    _sub(setup_py, r'ext_libs, ext_args = \[\s*"zfp",\s*\]', "ext_libs, ext_args = []")
    _sub(setup_py, r'\s*"\./schemoe/custom/compressor/zfpc\.cpp",', "")
    _sub(setup_py, r'include_dirs=\[\s*"/home/xinglinpan/zfp/include/",\s*\]', "include_dirs=[]")
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    _sub(setup_py, r'library_dirs=\[\s*"/home/xinglinpan/zfp/build/lib",\s*"/usr/local/cuda-10\.2/lib64/stubs",\s*\]',
         f'library_dirs=["{cuda_home}/lib64/stubs", "{cuda_home}/lib64"]')
    ck = os.path.join(tree, "schemoe", "custom", "custom_kernel.cpp")
    _sub(ck, r'#include "zfp\.h"\n', "")
    _sub(ck, r'#include "compressor/zfpc\.h"\n', "")
    _sub(ck, r'  if \(name == "zfp"\) \{\n    return new ZfpCompressor\(comm_ptr\);\n  \}\n', "")
    os.remove(os.path.join(tree, "schemoe", "custom", "compressor", "zfpc.cpp"))
    os.remove(os.path.join(tree, "schemoe", "custom", "compressor", "zfpc.h"))
    return tree


def build(src, keep=False):
    work = tempfile.mkdtemp(prefix="planmoe_refbuild_")
    try:
        tree = prepare(src, work)
        if os.path.isdir(DEST):
            shutil.rmtree(DEST)
        env = dict(os.environ)
        env.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")   # the reference passes no arch flags; build for B200 only
        env.setdefault("MAX_JOBS", "8")
        cmd = [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps",
               "--find-links", "/opt/wheelhouse", "--target", DEST, tree]
        proc = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        log = proc.stdout
        if proc.returncode != 0:
            errs = [l for l in log.splitlines() if "error" in l.lower()]
            sys.stderr.write(log[-6000:])
            raise SystemExit("reference build failed: " + (errs[-1] if errs else log.splitlines()[-1]))
        with open(os.path.join(DEST, "BUILD_PATCHES.txt"), "w") as f:
            f.write("Build-only edits applied to a scratch copy of the reference before `pip install`:\n")
            for where, what, why in PATCHES:
                f.write(f"- {where}: {what}.  Reason: {why}.\n")
        print("installed into", DEST)
        print(sorted(os.listdir(DEST)))
    finally:
        if keep:
            print("scratch tree kept at", work)
        else:
            shutil.rmtree(work, ignore_errors=True)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--src", required=True, help="checkout of the reference repository (read-only is fine)")
    ap.add_argument("--keep", action="store_true")
    a = ap.parse_args()
    build(a.src, a.keep)
