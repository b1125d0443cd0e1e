"""Build libqlm_b200.so in-tree with nvcc for sm_100a.

    python -m cudalm_c_b200.build [--force] [--verbose]

Every translation unit is compiled with
`-gencode arch=compute_100a,code=sm_100a -lineinfo`; the ones that hold the
bit-exact integer-state and router arithmetic add `--fmad=false` (a fused
multiply-add changes the rounding the reference's CPU build produces).  The CUDA
runtime is linked statically and the driver API is reached through
cudaGetDriverEntryPoint, so the library loads on a machine without a GPU.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libqlm_b200.so")
OBJ = os.path.join(HERE, "build")

# translation unit -> extra flags
UNITS = {
    "qlmb_runtime.cu": [],
    "qlmb_state.cu": ["--fmad=false"],
    "qlmb_route.cu": ["--fmad=false"],
    "qlmb_dispatch.cu": [],
    "qlmb_gemm.cu": [],
    "qlmb_linear.cu": [],
    "qlmb_gemv.cu": [],
    "qlmb_moe.cu": [],
    "qlmb_statefile.cu": [],
    "qlmb_q4n.cu": ["--fmad=false"],
    "qlmb_comm.cu": [],
    "qlmb_attn.cu": [],
    "qlmb_block.cu": [],
}
COMMON = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
          "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]


def _newer(src, dst, deps):
    if not os.path.exists(dst):
        return True
    t = os.path.getmtime(dst)
    return any(os.path.getmtime(p) > t for p in [src] + deps)


def build(force=False, verbose=False):
    nvcc = os.environ.get("NVCC", "nvcc")
    os.makedirs(OBJ, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    headers.append(os.path.join(os.path.dirname(HERE), "include", "qlm_b200.h"))
    objs, procs = [], []
    for unit, extra in UNITS.items():
        src = os.path.join(CSRC, unit)
        if not os.path.exists(src):
            continue
        obj = os.path.join(OBJ, unit.replace(".cu", ".o"))
        objs.append(obj)
        if force or _newer(src, obj, headers):
            cmd = [nvcc] + COMMON + extra + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
            procs.append((unit, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for unit, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            sys.stderr.write("---- %s ----\n%s\n" % (unit, out))
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    if force or procs or not os.path.exists(OUT):
        cmd = [nvcc, "-shared", "-cudart", "static", "-o", OUT] + objs + ["-Xlinker", "--no-undefined", "-lpthread", "-ldl", "-lrt"]
        subprocess.check_call(cmd)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
