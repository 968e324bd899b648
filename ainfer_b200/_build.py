"""In-tree build of the native libraries.

  ainfer_b200/lib/libainfer_cuda.so     CUDA kernels + the device C ABI (nvcc, sm_100a)
  ainfer_b200/lib/libainfer_runtime.so  C++ decode runtime over that ABI (g++)
  ainfer_b200/lib/ainfer_decode         the decode CLI

nvcc cross-compiles without a GPU. Objects are cached under ainfer_b200/lib/obj
and rebuilt when a source or header is newer.
"""
import concurrent.futures as cf
import glob
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "lib")
OBJ = os.path.join(LIB, "obj")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-fmad=false",  # fused multiply-add only where fmaf is written (bit-exact contract)
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fno-fast-math"]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-ffp-contract=off", "-fno-fast-math", "-pthread", "-Wall"]


def _nvcc():
    return shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"


def _cxx():
    for c in ("/usr/bin/g++", shutil.which("g++")):
        if c and os.path.exists(c):
            return c
    raise RuntimeError("g++ not found")


def _newest(paths):
    return max(os.path.getmtime(p) for p in paths)


def _headers():
    hs = glob.glob(os.path.join(CSRC, "**", "*.h"), recursive=True)
    hs += glob.glob(os.path.join(CSRC, "**", "*.cuh"), recursive=True)
    hs += glob.glob(os.path.join(ROOT, "include", "*.h"))
    return hs


def _compile(cmd, out, src, hdr_time, verbose):
    if os.path.exists(out) and os.path.getmtime(out) >= max(os.path.getmtime(src), hdr_time):
        return out
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"build failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    return out


def build_cuda(verbose=False, ptxas_v=False):
    # AINFER_TIMELINE=1 in the environment builds the profiling variant (every kernel stamps the
    # global timer around its dependency wait); its objects are cached apart from the product's.
    timeline = os.environ.get("AINFER_TIMELINE") == "1"
    OBJ = os.path.join(LIB, "obj_timeline" if timeline else "obj")
    os.makedirs(OBJ, exist_ok=True)
    srcs = sorted(glob.glob(os.path.join(CSRC, "kernels", "*.cu")) +
                  glob.glob(os.path.join(CSRC, "abi", "*.cu")))
    ht = _newest(_headers() + [os.path.abspath(__file__)])
    jobs = []
    with cf.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        for s in srcs:
            o = os.path.join(OBJ, os.path.basename(s) + ".o")
            cmd = ([_nvcc()] + NVCC_FLAGS + (["-DAINFER_TIMELINE"] if timeline else []) +
                   (["-Xptxas", "-v"] if ptxas_v else []) + ["-c", s, "-o", o])
            jobs.append(ex.submit(_compile, cmd, o, s, ht, verbose))
        objs = [j.result() for j in jobs]
    out = os.path.join(LIB, "libainfer_cuda.so")
    marker = os.path.join(LIB, "variant.txt")
    want = "timeline" if timeline else "product"
    have = open(marker).read().strip() if os.path.exists(marker) else ""
    if not os.path.exists(out) or os.path.getmtime(out) < _newest(objs) or have != want:
        cmd = [_nvcc(), "-shared", "-o", out] + objs + ["-cudart", "static", "-Xcompiler", "-fPIC"]
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.run(cmd, check=True)
        with open(marker, "w") as f:
            f.write(want + "\n")
    return out


def build_runtime(verbose=False):
    os.makedirs(OBJ, exist_ok=True)
    srcs = sorted(glob.glob(os.path.join(CSRC, "runtime", "*.cpp")))
    if not srcs:
        return None
    ht = _newest(_headers() + [os.path.abspath(__file__)])
    lib_srcs = [s for s in srcs if not s.endswith("_main.cpp")]
    objs = []
    with cf.ThreadPoolExecutor(max_workers=8) as ex:
        jobs = []
        for s in srcs:
            o = os.path.join(OBJ, os.path.basename(s) + ".o")
            cmd = [_cxx()] + CXX_FLAGS + ["-I", os.path.join(ROOT, "include"), "-c", s, "-o", o]
            jobs.append((s, ex.submit(_compile, cmd, o, s, ht, verbose)))
        objmap = {s: j.result() for s, j in jobs}
    objs = [objmap[s] for s in lib_srcs]
    out = os.path.join(LIB, "libainfer_runtime.so")
    cuda_so = os.path.join(LIB, "libainfer_cuda.so")
    if not os.path.exists(out) or os.path.getmtime(out) < max(_newest(objs), os.path.getmtime(cuda_so)):
        cmd = [_cxx(), "-shared", "-o", out] + objs + ["-L", LIB, "-lainfer_cuda", "-Wl,-rpath,$ORIGIN",
                                                       "-pthread"]
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.run(cmd, check=True)
    for s in srcs:
        if s.endswith("_main.cpp"):
            exe = os.path.join(LIB, os.path.basename(s)[:-len("_main.cpp")])
            if not os.path.exists(exe) or os.path.getmtime(exe) < max(os.path.getmtime(objmap[s]),
                                                                      os.path.getmtime(out)):
                cmd = [_cxx(), "-o", exe, objmap[s], "-L", LIB, "-lainfer_runtime", "-lainfer_cuda",
                       "-Wl,-rpath,$ORIGIN", "-pthread"]
                if verbose:
                    print(" ".join(cmd), flush=True)
                subprocess.run(cmd, check=True)
    return out


def build_all(verbose=False):
    a = build_cuda(verbose)
    b = build_runtime(verbose)
    return a, b


if __name__ == "__main__":
    build_all(verbose="-q" not in sys.argv)
    print("built:", os.listdir(LIB))
