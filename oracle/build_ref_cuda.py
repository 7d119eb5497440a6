"""Compile the reference project's own CUDA extension (`CG_cuda_ops`, CGNet/cudaCG) for sm_100a, from the sources where
they lie in a reference checkout, into oracle/_ref/ (git-ignored; travels to the GPU box with the tree).

    python oracle/build_ref_cuda.py [--ref /path/to/CGNet-checkout]

TEST INFRASTRUCTURE: the resulting module is the GPU-side parity oracle (the reference's kernels on the same inputs
as ours).  Nothing under cgnet_b200/ loads it.  The reference's own setup.py passes no architecture flags and
installs into site-packages; here the four translation units are handed to torch's extension builder with an explicit
-gencode for sm_100a and an in-tree build directory.  No reference source is copied or modified.
"""
import argparse
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def build(ref):
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    os.environ.setdefault("MAX_JOBS", "4")
    from torch.utils.cpp_extension import load
    src_dir = os.path.join(ref, "CGNet", "cudaCG")
    out = os.path.join(HERE, "_ref", "cuda_build")
    os.makedirs(out, exist_ok=True)
    return load(name="CG_cuda_ops",
                sources=[os.path.join(src_dir, f) for f in ("cudaCG_all.cpp", "cudaCG_utils.cu", "cudaCG_sparse.cu", "cudaCG_FNWMM.cu")],
                extra_include_paths=[src_dir], build_directory=out,
                extra_cuda_cflags=["-gencode", "arch=compute_100a,code=sm_100a", "-w"], extra_cflags=["-w"], verbose=False)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("CGNET_REFERENCE"), required=os.environ.get("CGNET_REFERENCE") is None,
                    help="path of a zlin7/CGNet checkout (or set CGNET_REFERENCE)")
    args = ap.parse_args()
    mod = build(args.ref)
    print("built", mod.__file__, "sparse_maxL =", mod.sparse_maxL())
