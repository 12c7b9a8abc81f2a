"""The Java side of the boundary, checked as text (the image has no JDK): `CudaBackend.java` implements every
method of the reference's `TensorBackend` interface (tensor/TensorBackend.java:3-112) over a `ComputeGraph` on
`CudaGpuRuntime`, and the `OP_METADATA` patch for `ComputeGraph.java` carries the same op codes, strides and
buffer-id slots as the Python mirror the GPU tests run on (`deepj_b200/compute_graph.py`)."""
import os
import re

from deepj_b200 import compute_graph as cg

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
JAVA = os.path.join(ROOT, "java", "io", "github", "kirstenali", "deepj", "tensor", "cuda")

# tensor/TensorBackend.java:3-112 — every abstract method and the two defaults a GPU backend overrides
TENSOR_BACKEND_METHODS = """matmul add subtract multiply divide addRowVector addBroadcastCols divideBroadcastCols subtractBroadcastCols
multiplyBroadcastCols addBroadcastRows multiplyBroadcastRows multiplyScalar addScalar divideScalar sumRows sumAlongRows sumAlongCols
meanAlongRows varianceAlongRows maxAlongRows sum sumAbs transpose clamp sqrt pow neg exp log tanh sigmoid relu reluBackward gelu
geluBackward softmaxRows softmaxBackward crossEntropyLoss crossEntropyGradient adamWUpdate layerNormBackward scatterAddRows addInPlace
subtractInPlace multiplyInPlace divideInPlace multiplyScalarInPlace addScalarInPlace divideScalarInPlace sqrtInPlace negInPlace
expInPlace logInPlace reluInPlace geluInPlace tanhInPlace sigmoidInPlace materializeTensor releaseResources""".split()


def test_cuda_backend_implements_the_whole_tensor_backend_interface():
    src = open(os.path.join(JAVA, "CudaBackend.java")).read()
    assert "public final class CudaBackend implements TensorBackend" in src
    assert "new ComputeGraph(runtime)" in src and "new CudaGpuRuntime(device)" in src
    overridden = re.findall(r"@Override\s+public\s+[\w\[\]<>]+\s+(\w+)\(", src)
    assert sorted(overridden) == sorted(TENSOR_BACKEND_METHODS), sorted(set(TENSOR_BACKEND_METHODS) ^ set(overridden))
    # every op code it records exists in the stream format with the code the Python mirror uses
    for name in set(re.findall(r"ComputeGraph\.(OP_\w+)", src)):
        assert hasattr(cg, name), name
    # the Python twin exposes the same surface (snake_case aside, it keeps the Java names)
    from deepj_b200.tensor import CudaBackend
    for m in TENSOR_BACKEND_METHODS:
        assert hasattr(CudaBackend, m), m


def test_op_metadata_patch_matches_the_stream_format_the_gpu_tests_use():
    patch = open(os.path.join(ROOT, "java", "patches", "ComputeGraph-fused-op-metadata.patch")).read()
    consts = {name: int(v) for name, v in re.findall(r"^\+\s+public static final int (OP_\w+) = (\d+);", patch, flags=re.M)}
    metas = {}
    for name, args in re.findall(r"^\+\s+registerMeta\(meta, (OP_\w+), ([\d, ]+)\);", patch, flags=re.M):
        nums = [int(x) for x in args.split(",")]
        metas[name] = (nums[0], tuple(nums[1:]))
    fused = {n: getattr(cg, n) for n in dir(cg) if n.startswith("OP_") and isinstance(getattr(cg, n), int) and getattr(cg, n) >= 64}
    assert consts == fused                                   # same names, same codes, none missing
    assert set(metas) == set(fused)
    for name, code in fused.items():
        assert cg.OP_METADATA[code] == metas[name], name
    assert f"new OpMeta[{max(fused, key=fused.get)} + 1]" in patch      # the table is sized for the highest code


def test_header_lists_every_fused_op_code():
    hdr = open(os.path.join(ROOT, "include", "deepj_cuda.h")).read()
    defined = {name: int(v) for name, v in re.findall(r"#define DEEPJ_(OP_\w+)\s+(\d+)", hdr)}
    fused = {n: getattr(cg, n) for n in dir(cg) if n.startswith("OP_") and isinstance(getattr(cg, n), int) and getattr(cg, n) >= 64}
    assert defined == fused
