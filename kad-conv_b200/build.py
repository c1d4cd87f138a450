"""Build libkadconv_b200.so (hand-written sm_100a CUDA behind a C ABI) in-tree.

    python kad-conv_b200/build.py [--force]

nvcc cross-compiles for sm_100a without a GPU. The library lands in kadconv/_lib/ next to the
Python package that loads it with ctypes; it is a build artefact and is not committed.
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / 'csrc'
OUT_DIR = HERE / 'kadconv' / '_lib'
LIB = OUT_DIR / 'libkadconv_b200.so'
SOURCES = ['kad_api.cu', 'kad_simt.cu', 'kad_px.cu', 'kad_elementwise.cu', 'kad_dsc_tc.cu', 'kad_dsc_mma.cu', 'kad_stem.cu', 'kad_pyramid.cu', 'kad_gemm_tc.cu', 'kad_conv3x3_tc.cu', 'kad_postprocess.cu', 'kad_preprocess.cu', 'kad_layer.cu']
NVCC_FLAGS = ['-gencode', 'arch=compute_100a,code=sm_100a', '-lineinfo', '-O3', '-std=c++17', '-Xcompiler', '-fPIC']


def _nvcc():
    cand = os.environ.get('NVCC') or '/usr/local/cuda/bin/nvcc'
    return cand if Path(cand).exists() else 'nvcc'


def _stale(target, deps):
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def build(force=False, verbose=False):
    OUT_DIR.mkdir(parents=True, exist_ok=True)
    obj_dir = HERE / 'build'
    obj_dir.mkdir(exist_ok=True)
    headers = list(CSRC.glob('*.cuh')) + [HERE.parent / 'include' / 'kadconv_b200.h']
    srcs = [CSRC / s for s in SOURCES if (CSRC / s).exists()]
    nvcc = _nvcc()

    def compile_one(src):
        obj = obj_dir / (src.stem + '.o')
        if force or _stale(obj, [src] + headers):
            cmd = [nvcc, *NVCC_FLAGS, '-c', str(src), '-o', str(obj)]
            if verbose:
                cmd.insert(1, '-Xptxas'); cmd.insert(2, '-v')
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError(f'nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}')
            if verbose:
                print(r.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(compile_one, srcs))
    if force or _stale(LIB, objs):
        cmd = [nvcc, '-shared', '-o', str(LIB), *map(str, objs)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f'link failed:\n{r.stdout}\n{r.stderr}')
    return LIB


if __name__ == '__main__':
    print(build(force='--force' in sys.argv, verbose='-v' in sys.argv))
