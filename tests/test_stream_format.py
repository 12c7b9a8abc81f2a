"""The ComputeGraph mirror emits the reference's command stream: these cases restate
ComputeGraphTest (recording fake runtime, call order, stream growth, AdamW encoding,
op-code table, id restart, orphan release, materialise-once) without a GPU."""
import gc
import struct

import numpy as np
import pytest

from deepj_b200 import compute_graph as cg
from deepj_b200.compute_graph import ComputeGraph, GpuBuffer, float_bits
from deepj_b200.tensor import GraphBackend, Tensor


class RecordingRuntime:
    """Port of the reference's test double (ComputeGraphTest.java:546-591)."""

    def __init__(self):
        self.calls, self.allocs, self.uploads, self.released, self.streams = [], [], [], [], []
        self.download_result = None

    def alloc_buffers(self, ids, sizes, count):
        self.calls.append("alloc"); self.allocs.append((list(ids[:count]), list(sizes[:count])))

    def upload_buffer(self, buf_id, data):
        self.calls.append("upload"); self.uploads.append((buf_id, np.array(data, copy=True)))

    def download_buffer(self, buf_id, out):
        self.calls.append("download")
        if self.download_result is not None:
            out[...] = np.asarray(self.download_result, dtype=np.float32).ravel()[: out.size]

    def release_buffers(self, ids, count):
        self.calls.append("release"); self.released.extend(ids[:count])

    def flush_ops(self, cmd, length):
        self.calls.append("flush"); self.streams.append(np.array(cmd[:length], copy=True))


@pytest.fixture()
def rt():
    r = RecordingRuntime()
    Tensor.setBackend(GraphBackend(r))
    return r


def test_op_code_table_has_42_distinct_reference_codes():      # ComputeGraphTest.java:362-390
    codes = {v for k, v in vars(cg).items() if k.startswith("OP_") and isinstance(v, int) and v <= 42}
    assert codes == set(range(1, 43))
    assert cg.OP_MATMUL == 5 and cg.OP_SOFTMAX_ROWS == 17 and cg.OP_ADAMW_UPDATE == 20 and cg.OP_SCATTER_ADD_ROWS_ATOMIC == 42
    for op in range(1, 43):
        assert op in cg.OP_METADATA
    assert cg.OP_METADATA[cg.OP_MATMUL] == (7, (1, 2, 3)) and cg.OP_METADATA[cg.OP_ADAMW_UPDATE] == (13, (1, 2, 3, 4))
    assert cg.OP_METADATA[cg.OP_CLAMP][0] == 6 and cg.OP_METADATA[cg.OP_SQRT] == (4, (1, 2))


def test_flush_order_is_alloc_then_upload_then_flush(rt):      # ComputeGraphTest.java:190-210
    a, b = Tensor.from2D([[1, 2], [3, 4]]), Tensor.from2D([[5, 6], [7, 8]])
    c = a.add(b)
    assert rt.calls == []                                      # nothing runs until a materialise
    c.materialize()
    assert rt.calls == ["alloc", "upload", "upload", "flush", "download"]
    assert rt.allocs[0] == ([0, 1, 2], [4, 4, 4])
    assert list(rt.streams[0]) == [cg.OP_ADD, 0, 1, 2, 4]
    assert np.array_equal(rt.uploads[0][1], [1, 2, 3, 4])


def test_matmul_encodes_m_n_k(rt):                             # ComputeGraph.java:272-282
    a, b = Tensor(2, 3), Tensor(3, 5)
    a.matmul(b).materialize()
    assert list(rt.streams[0]) == [cg.OP_MATMUL, 0, 1, 2, 2, 5, 3]


def test_scalar_travels_as_raw_float_bits(rt):
    Tensor(1, 3).multiplyScalar(0.125).addScalar(1e-6).materialize()
    s = list(rt.streams[0])
    assert s[:5] == [cg.OP_MULTIPLY_SCALAR, 0, 1, struct.unpack("<i", struct.pack("<f", 0.125))[0], 3]
    assert s[5:] == [cg.OP_ADD_SCALAR, 1, 2, float_bits(1e-6), 3]
    assert float_bits(-0.0) == -2147483648 and float_bits(1.0) == 0x3F800000


def test_adamw_encodes_exactly_13_ints(rt):                    # ComputeGraphTest.java:423-450
    w, g, m, v = (Tensor(2, 2) for _ in range(4))
    Tensor.backend().adamWUpdate(w, g, m, v, 1e-3, 0.9, 0.999, 1e-8, 0.01, 0.1, 0.001)
    Tensor.backend().graph.flush()
    s = list(rt.streams[0])
    assert len(s) == 13 and s[0] == cg.OP_ADAMW_UPDATE and s[1:5] == [0, 1, 2, 3] and s[12] == 4
    assert s[5:12] == [float_bits(x) for x in (1e-3, 0.9, 0.999, 1e-8, 0.01, 0.1, 0.001)]


def test_rmsnorm_records_the_six_reference_ops(rt):
    from deepj_b200.layers import RMSNorm1D
    RMSNorm1D(4).forward(Tensor(2, 4)).materialize()
    s = rt.streams[0]
    ops, pos = [], 0
    while pos < len(s):
        ops.append(int(s[pos])); pos += cg.OP_METADATA[int(s[pos])][0]
    assert ops == [cg.OP_MULTIPLY, cg.OP_MEAN_ALONG_ROWS, cg.OP_ADD_SCALAR, cg.OP_SQRT, cg.OP_DIVIDE_BROADCAST_COLS,
                   cg.OP_MULTIPLY_BROADCAST_ROWS]


def test_stream_grows_past_4096_ints(rt):                      # ComputeGraphTest.java:255-270
    t = Tensor(1, 1)
    for _ in range(1200):
        t = t.neg()
    t.materialize()
    assert len(rt.streams[0]) == 1200 * 4 and Tensor.backend().graph.cmd.size >= 4800


def test_materialize_downloads_once(rt):                       # ComputeGraphTest.java:319-333
    rt.download_result = [7.0]
    t = Tensor(1, 1).neg()
    assert t.numpy()[0, 0] == 7.0
    t.materialize()
    assert rt.calls.count("download") == 1


def test_ids_restart_at_zero_after_release_all(rt):            # ComputeGraphTest.java:338-352
    x = Tensor(1, 2)
    y = x.neg()
    y.materialize()
    Tensor.backend().releaseResources()
    assert set(rt.released) == {0, 1} and x.gpu_tag is None and y.gpu_tag is None
    z = Tensor(1, 2).neg()
    z.materialize()
    assert rt.allocs[-1][0] == [0, 1]


def test_orphaned_buffers_are_released_on_flush(rt):           # ComputeGraphTest.java:488-527
    keep = Tensor(1, 2)
    out = keep.neg().neg()          # the intermediate tensor dies immediately
    out.materialize()
    gc.collect()
    Tensor.backend().graph.flush()
    assert 1 in rt.released and 0 not in rt.released and 2 not in rt.released


def test_in_place_rebinds_to_a_fresh_buffer(rt):               # MetalBackend.java:400-526
    a, b = Tensor(1, 2), Tensor(1, 2)
    a.addInPlace(b)
    assert isinstance(a.gpu_tag, GpuBuffer) and a.gpu_tag.id == 2
    a.materialize()
    assert list(rt.streams[0]) == [cg.OP_ADD, 0, 1, 2, 2]


def test_shape_errors_raise_before_recording(rt):
    with pytest.raises(ValueError):
        Tensor(2, 3).matmul(Tensor(2, 3))
    with pytest.raises(ValueError):
        Tensor.backend().layerNormBackward(Tensor(2, 3), Tensor(2, 3), Tensor(2, 2), 3)
    with pytest.raises(ValueError):
        Tensor.backend().scatterAddRows(Tensor(4, 3), [0, 1], Tensor(3, 3))
    assert Tensor.backend().graph.is_empty() and rt.calls == []


def test_fused_op_metadata_matches_header():
    """Strides of the fused decode ops in the recorder equal the header's documentation."""
    import os, re
    hdr = open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include", "deepj_cuda.h")).read()
    for m in re.finditer(r"\*\s+(\d+)\s+(\w+)\s*\[([^\]]+)\]", hdr):
        code, fields = int(m.group(1)), [f.strip() for f in m.group(3).split(",")]
        assert cg.OP_METADATA[code][0] == len(fields), m.group(2)
