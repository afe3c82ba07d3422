"""Builds libqmm_b200.so (CUDA kernels + C ABI) in-tree with nvcc, for sm_100a only."""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libqmm_b200.so")
SOURCES = ["abi.cu", "generic.cu", "gemv.cu", "act_quant.cu", "pack.cu", "w8a8_gemm.cu", "mixed_gemm.cu", "limb_gemm.cu", "decode_mma.cu",
           "static_scratch.cu", "peer_reduce.cu", "host_pipeline.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--use_fast_math=false",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "-cudart", "static",
]


def _nvcc():
  for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
    if cand and os.path.exists(cand):
      return cand
  raise RuntimeError("nvcc not found; set NVCC")


def _stale(target, deps):
  if not os.path.exists(target):
    return True
  t = os.path.getmtime(target)
  return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
  """Compiles every .cu under csrc/ into one shared library. Returns its path."""
  os.makedirs(LIB_DIR, exist_ok=True)
  obj_dir = os.path.join(LIB_DIR, "obj")
  os.makedirs(obj_dir, exist_ok=True)
  headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h", ".inc"))]
  headers.append(os.path.join(os.path.dirname(HERE), "include", "qmm_b200.h"))
  nvcc = _nvcc()
  objs, procs = [], []
  for src in SOURCES:
    s = os.path.join(CSRC, src)
    o = os.path.join(obj_dir, src.replace(".cu", ".o"))
    objs.append(o)
    if force or _stale(o, [s] + headers):
      cmd = [nvcc] + [f for f in NVCC_FLAGS if f != "--use_fast_math=false"] + os.environ.get("QMM_NVCC_EXTRA", "").split() + ["-c", s, "-o", o]
      if verbose:
        cmd.insert(1, "-Xptxas=-v")
      procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
  failed = False
  for src, p in procs:
    out, _ = p.communicate()
    if p.returncode != 0 or verbose:
      sys.stderr.write(f"--- nvcc {src} ---\n{out}\n")
    failed |= p.returncode != 0
  if failed:
    raise RuntimeError("nvcc failed")
  if force or procs or _stale(LIB_PATH, objs):
    cmd = [nvcc, "-shared", "-cudart", "static", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB_PATH] + objs
    subprocess.check_call(cmd)
  return LIB_PATH


if __name__ == "__main__":
  print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
