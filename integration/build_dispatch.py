"""Builds Bolt's own dispatchers with a CUDA_B200 branch, against libbolt_b200.so.

    python integration/build_dispatch.py [BOLT_ROOT]

What a Bolt maintainer would commit is a handful of `else if (IS_CUDA_B200(arch))` branches in the files that
switch on `Arch` (INTEGRATION.md lists them).  This script applies exactly those edits to copies of the
reference's files -- read from the mounted tree, written under integration/_build/src (git-ignored, never
committed) -- and compiles the copies with only -D_USE_CUDA_B200, so that the resulting library,
integration/_build/libbolt_dispatch_b200.so, contains Bolt's public entry points

    matrix_matrix_multiply*, matrix_vector_multiply*                  (compute/blas_enhance/src/mmm.cpp, mvm.cpp)
    quantize, dequantize, convolution*, matmul*                       (compute/tensor/src/*.cpp)

with the new architecture as their only back end.  bolt_api_shim.cpp adds C-callable wrappers around the C++
(Tensor-based) ones for the tests.  The edits are anchored on lines of the reference; if the reference
changes, an anchor fails loudly.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
OUT = os.path.join(HERE, "_build")
LIB = os.path.join(OUT, "libbolt_dispatch_b200.so")


def _edit(text, anchor, new, where="before", count=1):
    assert text.count(anchor) >= count, "anchor not found: %r" % anchor[:60]
    if where == "before":
        return text.replace(anchor, new + anchor, count)
    if where == "after":
        return text.replace(anchor, anchor + new, count)
    return text.replace(anchor, new, count)


def patch_sys_h(t):
    t = _edit(t, "    X86_AVXVNNI = 10\n} Arch;", "    X86_AVXVNNI = 10,\n    CUDA_B200 = 11\n} Arch;", "replace")
    t = _edit(t, "#define IS_MALI_GPU(arch)", "#define IS_CUDA_B200(arch) (arch == CUDA_B200)\n")
    t = _edit(t, '"QUALCOMM", "X86_AVX2", "X86_AVX512"};', '"QUALCOMM", "X86_AVX2", "X86_AVX512", "X86_AVXVNNI", "CUDA_B200"};', "replace")
    return t


B200_INCLUDE = '#ifdef _USE_CUDA_B200\n#define BOLT_B200_WITH_BOLT_HEADERS\n#include "bolt_b200.h"\n#endif\n'


def patch_mmm(t):
    t = _edit(t, '#include "uni.h"\n', B200_INCLUDE, "after")
    t = _edit(t, "#ifdef _USE_NEON\n    } else if (IS_ARM(arch)) {\n        ret = matrix_matrix_multiply_tmp_bytes_arm(",
              "#ifdef _USE_CUDA_B200\n    } else if (IS_CUDA_B200(arch)) {\n"
              "        ret = matrix_matrix_multiply_tmp_bytes_cuda_b200(matrixB_N, matrixA_M, matrixB_K, matrixADataType,\n"
              "            matrixADataFormat, matrixBDataType, matrixBDataFormat, bytes);\n#endif\n")
    t = _edit(t, "#ifdef _USE_NEON\n    } else if (IS_ARM(arch)) {\n        ret = matrix_matrix_multiply_transform_rhs_bytes_arm(",
              "#ifdef _USE_CUDA_B200\n    } else if (IS_CUDA_B200(arch)) {\n"
              "        ret = matrix_matrix_multiply_transform_rhs_bytes_cuda_b200(\n"
              "            matrixB_N, matrixB_K, matrixBDataType, matrixBDataFormat, bytes, rhsBytes);\n#endif\n")
    t = _edit(t, "#ifdef _USE_X86\n    } else if (IS_X86(arch)) {\n        ret = matrix_matrix_multiply_transform_rhs_x86(",
              "#ifdef _USE_CUDA_B200\n    } else if (IS_CUDA_B200(arch)) {\n"
              "        ret = matrix_matrix_multiply_transform_rhs_cuda_b200(&desc, src, descTran, dst);\n#endif\n")
    t = _edit(t, "    if (IS_CPU(arch)) {\n        if (IS_GENERAL(arch)) {", "    if (IS_CPU(arch) || IS_CUDA_B200(arch)) {\n        if (IS_GENERAL(arch)) {", "replace")
    t = _edit(t, "#ifdef _USE_NEON\n            if (IS_ARM(arch)) {\n                ret = mmm_arm(",
              "#ifdef _USE_CUDA_B200\n            if (IS_CUDA_B200(arch)) {\n"
              "                if (matrixCDataType == DT_I32) {\n                    scale = nullptr;\n                }\n"
              "                ret = mmm_cuda_b200(matrixC_N, matrixC_M, matrixA_K, matrixBDataType, matrixADataFormat,\n"
              "                    matrixAData, transB, tmp, matrixCData, scale);\n            }\n#endif\n")
    return t


def patch_mvm(t):
    t = _edit(t, '#include "uni.h"\n', B200_INCLUDE, "after")
    # tmp bytes: `if (IS_X86(arch)) {...} else {*bytes = 0}` gains a branch in front of the else
    t = _edit(t, "    } else {\n        *bytes = 0;\n        ret = SUCCESS;\n    }",
              "#ifdef _USE_CUDA_B200\n    } else if (IS_CUDA_B200(arch)) {\n"
              "        ret = matrix_vector_multiply_tmp_bytes_cuda_b200(\n"
              "            matrixRow, matrixColumn, matrixDataType, matrixDataFormat, bytes);\n#endif\n")
    t = _edit(t, "#ifdef _USE_X86\n    } else if (IS_X86(arch)) {\n        ret = matrix_vector_multiply_transform_weight_bytes_x86(",
              "#ifdef _USE_CUDA_B200\n    } else if (IS_CUDA_B200(arch)) {\n"
              "        ret = matrix_vector_multiply_transform_weight_bytes_cuda_b200(\n"
              "            matrixRow, matrixColumn, matrixDataType, matrixDataFormat, bytes);\n#endif\n")
    t = _edit(t, "#ifdef _USE_X86\n    } else if (IS_X86(arch)) {\n        ret = matrix_vector_multiply_transform_weight_x86(",
              "#ifdef _USE_CUDA_B200\n    } else if (IS_CUDA_B200(arch)) {\n"
              "        ret = matrix_vector_multiply_transform_weight_cuda_b200(&desc, src, descTran, dst, nullptr);\n#endif\n")
    # the compute entry: same protocol as the x86 branch (on-the-fly packing into tmp, offsetC first)
    t = _edit(t, "#ifdef _USE_NEON\n    } else if (IS_ARM(arch)) {\n        ret = mvm_arm(",
              "#ifdef _USE_CUDA_B200\n    } else if (IS_CUDA_B200(arch)) {\n"
              "        U8 *dataB = (U8 *)matrix;\n"
              "        if (matrixDataType == DT_U8_Q &&\n"
              "            matrixDataFormat == matrix_vector_multiply_weight_format(matrixDataType)) {\n"
              "            return NOT_SUPPORTED;\n        }\n"
              "        if (matrixDataType == DT_I8 &&\n"
              "            matrixDataFormat != matrix_vector_multiply_weight_format(matrixDataType)) {\n"
              "            dataB = ((U8 *)tmp);\n            TensorDesc tranDescB;\n"
              "            CHECK_STATUS(matrix_vector_multiply_transform_weight_cuda_b200(\n"
              "                &matrixDesc, matrix, &tranDescB, dataB + resultColumn * bytesOf(DT_I32), dataB));\n        }\n"
              "        ret = mvm_cuda_b200(matrixRow, matrixColumn, matrixDataType, matrixDataFormat, dataB, vector,\n"
              "            result, tmp, scale);\n#endif\n")
    return t


def patch_quantize(t):
    t = _edit(t, '#include "tensor_computing.h"\n', B200_INCLUDE, "after")
    t = _edit(t, "    }\n    output->resize(qDesc);",
              "#ifdef _USE_CUDA_B200\n    } else if (IS_CUDA_B200(arch)) {\n"
              "        ret = quantize_cuda_b200(&dDesc, data, &qDesc, qData, scale, 0);\n#endif\n")
    return t


def patch_dequantize(t):
    t = _edit(t, '#include "tensor_computing.h"\n', B200_INCLUDE, "after")
    t = _edit(t, "    }\n    return ret;\n}",
              "#ifdef _USE_CUDA_B200\n    } else if (IS_CUDA_B200(arch)) {\n"
              "        ret = dequantize_cuda_b200(&qDesc, qData, scale, &bDesc, bData, &dDesc, data);\n#endif\n")
    return t


def patch_convolution(t):
    t = _edit(t, '#include "tensor_computing.h"\n', B200_INCLUDE, "after")
    # output size: the CPU rule with the AVX512 int8 output format
    t = _edit(t, "    } else if (IS_CPU(arch)) {\n        if (fn % 8 != 0) {", "    } else if (IS_CPU(arch) || IS_CUDA_B200(arch)) {\n        if (fn % 8 != 0) {", "replace")
    t = _edit(t, "#ifdef _USE_INT8\n        if (IS_X86_AVX512(arch) && (targetDataType == DT_U8_Q) && (fn != 8)) {",
              "#if defined(_USE_INT8) || defined(_USE_CUDA_B200)\n        if ((IS_X86_AVX512(arch) || IS_CUDA_B200(arch)) && (targetDataType == DT_U8_Q) && (fn != 8)) {", "replace")
    t = _edit(t, "#ifdef _USE_NEON\n    } else if (IS_ARM(arch)) {\n        ret = convolution_infer_forward_algorithm_arm(",
              "#ifdef _USE_CUDA_B200\n    } else if (IS_CUDA_B200(arch)) {\n"
              "        ret = convolution_infer_forward_algorithm_cuda_b200(\n"
              "            &inputDesc, &filterDesc, &outputDesc, &convParamSpec, policy, algorithm, targetDataType);\n#endif\n")
    t = _edit(t, "#ifdef _USE_NEON\n    } else if (IS_ARM(arch)) {\n        ret = convolution_transform_filter_bytes_arm(",
              "#ifdef _USE_CUDA_B200\n    } else if (IS_CUDA_B200(arch)) {\n"
              "        ret = convolution_transform_filter_bytes_cuda_b200(\n"
              "            &filterDesc, &convParamSpec, algorithm, (U32 *)bytes);\n#endif\n")
    t = _edit(t, "#ifdef _USE_NEON\n    } else if (IS_ARM(arch)) {\n        ret = convolution_transform_filter_arm(",
              "#ifdef _USE_CUDA_B200\n    } else if (IS_CUDA_B200(arch)) {\n"
              "        ret = convolution_transform_filter_cuda_b200(\n"
              "            &filterDesc, filter, &convParamSpec, algorithm, &ftmDesc, filterTransformed);\n#endif\n")
    t = _edit(t, "#ifdef _USE_NEON\n    } else if (IS_ARM(arch)) {\n        ret = convolution_infer_forward_tmp_bytes_arm(",
              "#ifdef _USE_CUDA_B200\n    } else if (IS_CUDA_B200(arch)) {\n"
              "        ret = convolution_infer_forward_tmp_bytes_cuda_b200(\n"
              "            &inputDesc, &filterDesc, &outputDesc, &convParamSpec, algorithm, bytes);\n#endif\n")
    # the residual input is fused as on x86
    t = _edit(t, "#if defined(_USE_GENERAL) || defined(_USE_X86)\n    if (tensorNumElements(eltwiseInputDesc)",
              "#if defined(_USE_GENERAL) || defined(_USE_X86) || defined(_USE_CUDA_B200)\n    if (tensorNumElements(eltwiseInputDesc)", "replace")
    t = _edit(t, "#ifdef _USE_NEON\n    } else if (IS_ARM(arch)) {\n        ret = convolution_arm(",
              "#ifdef _USE_CUDA_B200\n    } else if (IS_CUDA_B200(arch)) {\n"
              "        ret = convolution_cuda_b200(&inputDesc, input, eltwiseInput, &filterDesc, filter, &convParamSpec,\n"
              "            algorithm, &scaleDesc, scale, &biasDesc, bias, tmpBytes, tmp, &outputDesc, output, &activationDesc);\n#endif\n")
    return t


def patch_matmul(t):
    t = _edit(t, '#include "blas_enhance.h"\n', B200_INCLUDE, "after")
    # tmp bytes
    t = _edit(t, "    bool quantA = false;\n    bool quantB = false;\n    bool quantC = false;\n",
              "#ifdef _USE_CUDA_B200\n    if (IS_CUDA_B200(archInfo->arch)) {\n"
              "        return matmul_infer_forward_tmp_bytes_cuda_b200(&matrixADesc, transposeA, &matrixBDesc, transposeB,\n"
              "            &matrixCDesc, matrixCTensor.get_scale(), bytes);\n    }\n#endif\n")
    # the operator: scales travel in the tensors
    t = _edit(t, "    if (!isSameDataFormat(matrixADesc.df, DF_NCHW)) {\n        TensorDesc desc = matrixADesc;",
              "#ifdef _USE_CUDA_B200\n    if (IS_CUDA_B200(arch)) {\n"
              "        F32 cScale = matrixCTensor.get_scale();\n"
              "        TensorDesc biasDesc = biasTensor.get_desc();\n"
              "        void *bias = biasTensor.bytes() > 0 ? get_ptr_from_tensor(biasTensor, arch) : nullptr;\n"
              "        EE ret = matmul_cuda_b200(&matrixADesc, transposeA, matrixA, matrixATensor.get_scale(), &matrixBDesc,\n"
              "            transposeB, matrixB, matrixBTensor.get_scale(), &biasDesc, bias, tmpBytes, tmp, &matrixCDesc, matrixC,\n"
              "            &cScale);\n"
              "        matrixCTensor.set_scale(cScale);\n        return ret;\n    }\n#endif\n")
    return t


FILES = [
    ("common/uni/include/sys.h", "include/sys.h", patch_sys_h),
    ("compute/blas_enhance/src/mmm.cpp", "mmm.cpp", patch_mmm),
    ("compute/blas_enhance/src/mvm.cpp", "mvm.cpp", patch_mvm),
    ("compute/tensor/src/quantize.cpp", "quantize.cpp", patch_quantize),
    ("compute/tensor/src/dequantize.cpp", "dequantize.cpp", patch_dequantize),
    ("compute/tensor/src/convolution.cpp", "convolution.cpp", patch_convolution),
    ("compute/tensor/src/matmul.cpp", "matmul.cpp", patch_matmul),
]


def build(bolt_root):
    src = os.path.join(OUT, "src")
    os.makedirs(os.path.join(src, "include"), exist_ok=True)
    for rel, dst, fn in FILES:
        with open(os.path.join(bolt_root, rel)) as f:
            text = fn(f.read())
        with open(os.path.join(src, dst), "w") as f:
            f.write(text)
    inc = [os.path.join(src, "include")] + [os.path.join(bolt_root, d) for d in (
        "common/uni/include", "common/memory/include", "compute/blas_enhance/include", "compute/blas_enhance/src",
        "compute/tensor/include", "compute/tensor/src")] + [os.path.join(ROOT, "include")]
    cmd = ["g++", "-O2", "-fPIC", "-std=c++11", "-include", "cstdint", "-w", "-D_USE_CUDA_B200", "-shared", "-o", LIB]
    for d in inc:
        cmd += ["-I", d]
    cmd += [os.path.join(src, f) for f in ("mmm.cpp", "mvm.cpp", "quantize.cpp", "dequantize.cpp", "convolution.cpp", "matmul.cpp")]
    cmd += [os.path.join(HERE, "bolt_api_shim.cpp"), os.path.join(bolt_root, "common/uni/src/profiling.cpp"),
            os.path.join(bolt_root, "common/uni/src/tensor_transpose.cpp")]
    cmd += ["-L", os.path.join(ROOT, "bolt_b200", "lib"), "-lbolt_b200", "-Wl,-rpath,$ORIGIN/../../bolt_b200/lib", "-Wl,--no-undefined"]
    subprocess.check_call(cmd)
    return LIB


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("BOLT_ROOT")
    if not root:
        raise SystemExit("usage: build_dispatch.py BOLT_ROOT (the huawei-noah/bolt source tree)")
    print(build(root))
