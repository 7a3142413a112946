"""Builds oracle/_ref/libref_vllm.so: the reference's OWN paged-attention and KV-cache CUDA
kernels (and rotary embedding), compiled unmodified for sm_100a from where they lie in the reference tree, plus a small
plain-pointer shim (oracle/ref_shim.cpp).  TEST INFRASTRUCTURE: a GPU-side comparator for the
parity tests, never part of the product.

    python oracle/build_ref.py [--force]

Needs the reference checkout (the directory named by AICI_REFERENCE_DIR, default `reference` next to
the repository's parent) and the
installed PyTorch headers/libraries (the kernels are written against libtorch).  Takes about ten
minutes.  Where the reference tree is absent the script does nothing; the prebuilt library in
oracle/_ref/ (git-ignored) is what travels to a GPU machine.  The reference's flash-attention
sources are not built: they need a CUTLASS checkout the reference tree does not carry, and their
host code refuses compute capability 10.x (kernels/flash_attn/flash_api.cpp:467-471).
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
OUT = os.path.join(OUT_DIR, "libref_vllm.so")


def build(force: bool = False):
    ref = os.environ.get("AICI_REFERENCE_DIR",
                         os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"))
    kdir = os.path.join(ref, "rllm", "tch-cuda", "kernels")
    srcs = [os.path.join(kdir, "vllm", "cache_kernels.cu"),
            os.path.join(kdir, "vllm", "pos_encoding_kernels.cu"),
            os.path.join(kdir, "vllm", "attention", "attention_kernels.cu")]
    if not all(os.path.exists(s) for s in srcs):
        return None
    shim = os.path.join(HERE, "ref_shim.cpp")
    if os.path.exists(OUT) and not force and os.path.getmtime(OUT) >= os.path.getmtime(shim):
        return OUT
    import torch
    from torch.utils import cpp_extension
    os.makedirs(OUT_DIR, exist_ok=True)
    inc = cpp_extension.include_paths("cuda")
    libdir = os.path.join(os.path.dirname(torch.__file__), "lib")
    objs = []
    common = ["-O2", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC",
              "--expt-relaxed-constexpr", "-DTORCH_API_INCLUDE_EXTENSION_H",
              "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch.compiled_with_cxx11_abi()),
              "-I" + kdir, "-I" + os.path.join(kdir, "vllm")] + ["-I" + i for i in inc]
    procs = []
    for s in srcs + [os.path.join(HERE, "ref_shim.cpp")]:
        o = os.path.join(OUT_DIR, os.path.basename(s).rsplit(".", 1)[0] + ".o")
        objs.append(o)
        if os.path.exists(o) and os.path.getmtime(o) >= os.path.getmtime(s):
            continue  # left over from an interrupted build of the same source
        cmd = ["nvcc", *common, "-x", "cu", "-c", s, "-o", o]
        procs.append((s, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for s, pr in procs:
        out, _ = pr.communicate()
        if pr.returncode != 0:
            raise RuntimeError("nvcc failed for %s:\n%s" % (s, out[-4000:]))
    link = ["nvcc", "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", OUT, *objs, "-L" + libdir,
            "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda", "-Xlinker", "-rpath," + libdir]
    res = subprocess.run(link, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("link failed:\n%s\n%s" % (res.stdout, res.stderr))
    for o in objs:
        os.remove(o)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
