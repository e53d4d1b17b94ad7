"""In-tree build of the native extension ``planmoe_b200/_C.so`` for sm_100a.

    python -m planmoe_b200.utils.build [--force] [--verbose]

Every ``csrc/**/*.cu`` is compiled with
``nvcc -gencode arch=compute_100a,code=sm_100a -lineinfo -O3`` (nvcc cross-compiles without a
GPU), ``csrc/bindings.cpp`` and the other ``.cpp`` files with g++, and everything is linked
against libtorch into one shared object next to the Python sources.  Object files are cached
in ``csrc/build/`` and rebuilt when the source or any header is newer.  This takes the place
of the reference's ``setup.py`` CUDAExtension (``setup.py:57-163``), which passes no arch flags.
"""

import concurrent.futures as cf
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
CSRC = os.path.join(PKG, 'csrc')
OBJ = os.path.join(CSRC, 'build')
TARGET = os.path.join(PKG, '_C.so')

ARCH = ['-gencode', 'arch=compute_100a,code=sm_100a']


def _cuda_home():
    for c in (os.environ.get('CUDA_HOME'), os.environ.get('CUDA_PATH'), '/usr/local/cuda'):
        if c and os.path.exists(os.path.join(c, 'bin', 'nvcc')):
            return c
    raise RuntimeError('nvcc not found (set CUDA_HOME)')


def _sources():
    cu, cpp = [], []
    for root, dirs, files in os.walk(CSRC):
        dirs[:] = [d for d in dirs if d != 'build']
        for f in sorted(files):
            p = os.path.join(root, f)
            if f.endswith('.cu'):
                cu.append(p)
            elif f.endswith('.cpp'):
                cpp.append(p)
    return cu, cpp


def _headers_mtime():
    newest = 0.0
    for root, dirs, files in os.walk(CSRC):
        dirs[:] = [d for d in dirs if d != 'build']
        for f in files:
            if f.endswith(('.h', '.cuh', '.hpp')):
                newest = max(newest, os.path.getmtime(os.path.join(root, f)))
    return newest


def _obj_path(src):
    rel = os.path.relpath(src, CSRC).replace(os.sep, '__')
    return os.path.join(OBJ, rel + '.o')


def _run(cmd, verbose):
    if verbose:
        print(' '.join(cmd), flush=True)
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        raise RuntimeError('build command failed:\n%s\n%s' % (' '.join(cmd), res.stdout))
    if verbose and res.stdout.strip():
        print(res.stdout)
    return res.stdout


def build(force=False, verbose=False, ptxas_info=False):
    import torch
    from torch.utils import cpp_extension as ce

    cuda = _cuda_home()
    nvcc = os.path.join(cuda, 'bin', 'nvcc')
    os.makedirs(OBJ, exist_ok=True)
    cu, cpp = _sources()
    hdr_m = _headers_mtime()

    abi = '-D_GLIBCXX_USE_CXX11_ABI=%d' % int(torch._C._GLIBCXX_USE_CXX11_ABI)
    inc = ['-I' + CSRC, '-I' + os.path.join(cuda, 'include')]
    torch_inc = ['-isystem' + p for p in ce.include_paths()] + \
                ['-isystem' + sysconfig.get_paths()['include']]
    common_cxx = ['-O2', '-fPIC', '-std=c++17', abi]

    jobs = []
    for s in cu:
        o = _obj_path(s)
        cmd = [nvcc] + ARCH + ['-lineinfo', '-O3', '-std=c++17', '--expt-relaxed-constexpr',
                               '-Xcompiler', '-fPIC', abi] + inc
        if ptxas_info:
            cmd += ['-Xptxas', '-v']
        cmd += ['-c', s, '-o', o]
        jobs.append((s, o, cmd))
    for s in cpp:
        o = _obj_path(s)
        needs_torch = any(w in open(s).read(8192) for w in ('torch', 'pybind11'))
        cmd = ['g++'] + common_cxx + inc + (torch_inc if needs_torch else []) + \
              ['-DTORCH_EXTENSION_NAME=_C', '-DTORCH_API_INCLUDE_EXTENSION_H', '-c', s, '-o', o]
        jobs.append((s, o, cmd))

    todo = []
    for s, o, cmd in jobs:
        stale = (force or not os.path.exists(o) or
                 os.path.getmtime(o) < max(os.path.getmtime(s), hdr_m))
        if stale:
            todo.append(cmd)
    if todo:
        with cf.ThreadPoolExecutor(max_workers=min(len(todo), os.cpu_count() or 4)) as ex:
            outs = list(ex.map(lambda c: _run(c, verbose), todo))
        if ptxas_info:
            print('\n'.join(outs))

    objs = [o for _, o, _ in jobs]
    relink = bool(todo) or not os.path.exists(TARGET) or \
        any(os.path.getmtime(o) > os.path.getmtime(TARGET) for o in objs)
    if relink:
        libs = ['-L' + p for p in ce.library_paths()] + \
               ['-L' + os.path.join(cuda, 'lib64'),
                '-lc10', '-ltorch_cpu', '-ltorch', '-ltorch_python', '-lc10_cuda', '-ltorch_cuda',
                '-lcudart', '-ldl', '-lpthread']
        rpath = ['-Wl,-rpath,' + p for p in ce.library_paths()]
        # link beside the target and rename: a reader (an importing process, a snapshot of the tree) sees the old
        # or the new library, never a partly written one
        tmp = TARGET + '.linking'
        _run(['g++', '-shared', '-o', tmp] + objs + libs + rpath +
             ['-Wl,--no-as-needed'], verbose)
        os.replace(tmp, TARGET)
    return TARGET


def main(argv=None):
    argv = sys.argv[1:] if argv is None else argv
    path = build(force='--force' in argv, verbose='--verbose' in argv,
                 ptxas_info='--ptxas-info' in argv)
    print('built', path)


if __name__ == '__main__':
    main()
