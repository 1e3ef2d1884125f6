"""Build ``libfwp.so`` (the C-ABI library) in-tree with nvcc for sm_100a.

    python recurrent_fwp_b200/build.py [--force] [--verbose]

Each ``csrc/*.cu`` is compiled to an object file (in parallel) and linked into
``recurrent_fwp_b200/libfwp.so`` with the CUDA runtime linked statically, so the
library has no dependency beyond the driver.  Objects are rebuilt only when a
source or header is newer.  nvcc cross-compiles without a GPU.
"""
import concurrent.futures
import glob
import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, 'csrc')
OBJ = os.path.join(PKG, 'build')
LIB = os.path.join(PKG, 'libfwp.so')
NVCC = os.environ.get('NVCC', '/usr/local/cuda/bin/nvcc')
FLAGS = ['-gencode', 'arch=compute_100a,code=sm_100a', '-lineinfo', '-O3', '-std=c++17',
         '-Xcompiler', '-fPIC', '-Xcompiler', '-fvisibility=hidden']


def _newer(src_list, target):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in src_list)


def _compile(args):
    src, obj, verbose = args
    cmd = [NVCC] + FLAGS + (['-Xptxas', '-v'] if verbose else []) + ['-c', src, '-o', obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    return src, r.returncode, r.stdout + r.stderr


def build(force=False, verbose=False):
    os.makedirs(OBJ, exist_ok=True)
    sources = sorted(glob.glob(os.path.join(CSRC, '*.cu')))
    headers = glob.glob(os.path.join(CSRC, '*.cuh')) + glob.glob(os.path.join(PKG, '..', 'include', '*.h'))
    jobs, objs = [], []
    for src in sources:
        obj = os.path.join(OBJ, os.path.basename(src)[:-3] + '.o')
        objs.append(obj)
        if force or _newer([src] + headers, obj):
            jobs.append((src, obj, verbose))
    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for src, rc, log in ex.map(_compile, jobs):
                if verbose or rc:
                    sys.stderr.write(log)
                if rc:
                    raise RuntimeError('nvcc failed on %s' % src)
    if jobs or _newer(objs, LIB):
        cmd = [NVCC, '-shared', '-o', LIB] + objs + ['-cudart', 'static',
               '-gencode', 'arch=compute_100a,code=sm_100a', '-Xcompiler', '-fPIC']
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError('link failed')
    return LIB


if __name__ == '__main__':
    print(build(force='--force' in sys.argv, verbose='--verbose' in sys.argv))
