#!/usr/bin/env python
"""Builds the reference's own TokenWeave kernels, unchanged, as a stand-alone torch extension.

The reference (a vLLM fork) cannot be installed offline as a whole; its TokenWeave kernels can be compiled
on their own: ``csrc/tokenweave_fused_kernels.cu`` and ``csrc/tokenweave_artifact_kernels.cu`` with the four
headers they include are copied byte for byte into ``baseline/_ref/tw_ref_kernels/src`` and compiled for
sm_100a together with a registration file written here (the reference registers the same functions with the
same schemas in ``csrc/torch_bindings.cpp:146-196`` next to hundreds of unrelated ops). The library lands in
``baseline/_ref/tw_ref_kernels/tw_ref_kernels.so``; ``artifact/fused_microbench.py --impl reference`` loads it
and times ``torch.ops.tw_ref.fused_rs_ln_ag_cta`` and friends the way the reference's own
``artifact/figure_4_10/bench.py`` does.

Usage: ``python baseline/build_ref_kernels.py [--reference /path/to/tokenweave]``. The outcome (or the
compiler's answer when it fails) is appended to ``baseline/REFERENCE_INSTALL.txt``.
"""
from __future__ import annotations

import argparse
import os
import shutil
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref", "tw_ref_kernels")
FILES = ["tokenweave_fused_kernels.cu", "tokenweave_artifact_kernels.cu", "tokenweave_multimem_utils.cuh",
         "type_convert.cuh", "dispatch_utils.h", "cuda_compat.h"]

BINDING = r'''
// Registration of the reference's TokenWeave kernels under the namespace "tw_ref"; the declarations and
// schemas are those of the reference's csrc/ops.h:69-134 and csrc/torch_bindings.cpp:146-196.
#include <torch/all.h>
#include <torch/library.h>

void rms_norm_inplace(torch::Tensor& out, torch::Tensor& input, torch::Tensor& weight, double epsilon);
void fused_rs_ln_ag_cta(torch::Tensor& input, torch::Tensor& residual, torch::Tensor& weight, int64_t mcptr,
                        int64_t signal_pads, int64_t rank, int64_t world_size, int64_t MAX_CTAS, double epsilon);
void fused_add_rms_norm_cta(torch::Tensor& input, torch::Tensor& residual, torch::Tensor& weight, int64_t MAX_CTAS,
                            double epsilon);
void fused_rs_ln_cta(torch::Tensor& input, torch::Tensor& residual, torch::Tensor& weight, int64_t mcptr,
                     int64_t signal_pads, int64_t rank, int64_t world_size, int64_t MAX_CTAS, double epsilon);
void multimem_ar_cta(torch::Tensor& input, int64_t mcptr, int64_t signal_pads, int64_t rank, int64_t world_size,
                     int64_t MAX_CTAS);
void multimem_rs_cta(torch::Tensor& input, int64_t mcptr, int64_t signal_pads, int64_t rank, int64_t world_size,
                     int64_t MAX_CTAS);
void multimem_ag_cta(torch::Tensor& input, int64_t mcptr, int64_t signal_pads, int64_t rank, int64_t world_size,
                     int64_t MAX_CTAS);
void simple_fusion_rs_ln_ag_cta(torch::Tensor& input, torch::Tensor& residual, torch::Tensor& weight, int64_t mcptr,
                                int64_t signal_pads, int64_t rank, int64_t world_size, int64_t MAX_CTAS,
                                double epsilon);

TORCH_LIBRARY(tw_ref, ops) {
  ops.def("rms_norm_inplace(Tensor! result, Tensor! input, Tensor weight, float epsilon) -> ()");
  ops.impl("rms_norm_inplace", torch::kCUDA, &rms_norm_inplace);
  ops.def("fused_rs_ln_ag_cta(Tensor! input, Tensor! residual, Tensor weight, int mcptr, int signal_pads, int rank, "
          "int world_size, int MAX_CTAS, float epsilon) -> ()");
  ops.impl("fused_rs_ln_ag_cta", torch::kCUDA, &fused_rs_ln_ag_cta);
  ops.def("fused_add_rms_norm_cta(Tensor! input, Tensor! residual, Tensor weight, int MAX_CTAS, float epsilon) -> ()");
  ops.impl("fused_add_rms_norm_cta", torch::kCUDA, &fused_add_rms_norm_cta);
  ops.def("fused_rs_ln_cta(Tensor! input, Tensor! residual, Tensor weight, int mcptr, int signal_pads, int rank, "
          "int world_size, int MAX_CTAS, float epsilon) -> ()");
  ops.impl("fused_rs_ln_cta", torch::kCUDA, &fused_rs_ln_cta);
  ops.def("multimem_ar_cta(Tensor input, int mcptr, int signal_pads, int rank, int world_size, int MAX_CTAS) -> ()");
  ops.impl("multimem_ar_cta", torch::kCUDA, &multimem_ar_cta);
  ops.def("multimem_rs_cta(Tensor input, int mcptr, int signal_pads, int rank, int world_size, int MAX_CTAS) -> ()");
  ops.impl("multimem_rs_cta", torch::kCUDA, &multimem_rs_cta);
  ops.def("multimem_ag_cta(Tensor input, int mcptr, int signal_pads, int rank, int world_size, int MAX_CTAS) -> ()");
  ops.impl("multimem_ag_cta", torch::kCUDA, &multimem_ag_cta);
  ops.def("simple_fusion_rs_ln_ag_cta(Tensor! input, Tensor! residual, Tensor weight, int mcptr, int signal_pads, "
          "int rank, int world_size, int MAX_CTAS, float epsilon) -> ()");
  ops.impl("simple_fusion_rs_ln_ag_cta", torch::kCUDA, &simple_fusion_rs_ln_ag_cta);
}
'''


def note(line: str) -> None:
    with open(os.path.join(HERE, "REFERENCE_INSTALL.txt"), "a") as f:
        f.write(line.rstrip() + "\n")


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("TW_REFERENCE_DIR"),
                    help="checkout of microsoft/tokenweave (or set TW_REFERENCE_DIR)")
    args = ap.parse_args()
    if not args.reference or not os.path.isdir(os.path.join(args.reference, "csrc")):
        ap.error("give the reference checkout with --reference DIR (it must contain csrc/)")
    src = os.path.join(OUT, "src")
    os.makedirs(src, exist_ok=True)
    for name in FILES:
        shutil.copyfile(os.path.join(args.reference, "csrc", name), os.path.join(src, name))
    with open(os.path.join(src, "tw_ref_binding.cpp"), "w") as f:
        f.write(BINDING)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    from torch.utils import cpp_extension
    build_dir = os.path.join(OUT, "build")
    os.makedirs(build_dir, exist_ok=True)
    t0 = time.time()
    stamp = time.strftime("%Y-%m-%d")
    try:
        cpp_extension.load(
            name="tw_ref_kernels",
            sources=[os.path.join(src, n) for n in ("tw_ref_binding.cpp", "tokenweave_fused_kernels.cu",
                                                    "tokenweave_artifact_kernels.cu")],
            extra_include_paths=[src],
            # torch's extension builder defines __CUDA_NO_HALF_OPERATORS__ and friends; the reference's own
            # build strips them (cmake/utils.cmake, "Remove -D__CUDA_NO_..."), and its kernels use the
            # bf16x2 operators, so they are undefined again here
            extra_cuda_cflags=["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "--expt-relaxed-constexpr",
                               "-lineinfo", "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__",
                               "-U__CUDA_NO_BFLOAT16_CONVERSIONS__", "-U__CUDA_NO_HALF2_OPERATORS__",
                               "-U__CUDA_NO_BFLOAT162_OPERATORS__", "-U__CUDA_NO_BFLOAT16_OPERATORS__"],
            extra_cflags=["-O2"], build_directory=build_dir, is_python_module=False, verbose=True)
    except Exception as e:       # the compiler's answer goes on record
        msg = str(e).strip().splitlines()
        note(f"[{stamp}] reference TokenWeave kernels (stand-alone extension): build FAILED: {msg[-1] if msg else e!r}")
        print(e, file=sys.stderr)
        return 1
    shutil.copyfile(os.path.join(build_dir, "tw_ref_kernels.so"), os.path.join(OUT, "tw_ref_kernels.so"))
    note(f"[{stamp}] reference TokenWeave kernels (csrc/tokenweave_fused_kernels.cu, tokenweave_artifact_kernels.cu, "
         f"unchanged) built stand-alone for sm_100a in {time.time() - t0:.0f} s: baseline/_ref/tw_ref_kernels/tw_ref_kernels.so")
    print(os.path.join(OUT, "tw_ref_kernels.so"))
    return 0


if __name__ == "__main__":
    sys.exit(main())
