"""The JNI natives (deepj_b200/csrc/jni_shim.cpp), compiled against the stand-in jni.h of
tests/fake_jni and driven through ctypes.

What the reference's natives promise (native/deepj_metal_jni.mm:1480-1560) and these must too:
input arrays are released without write-back, the download array is committed, every pin is
released on every path, and a failed call leaves a pending java.lang.RuntimeException with the
library's message instead of crashing the VM.
"""
import ctypes
import os
import subprocess

import numpy as np
import pytest

from deepj_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
FAKE = os.path.join(ROOT, "tests", "fake_jni")
PREFIX = "Java_io_github_kirstenali_deepj_tensor_cuda_CudaNative_"
JNI_ABORT = 2
NATIVES = ["nativeAllocBuffers", "nativeUploadBuffer", "nativeDownloadBuffer", "nativeReleaseBuffers", "nativeFlushOps",
           "nativeFlushOpsAsync", "nativeSynchronize", "nativeInit", "nativeShutdown", "nativeQ8Alloc",
           "nativeQ8QuantizeInto", "nativeKvAlloc", "nativeKvAllocF16", "nativeDecodePlan", "nativeStats", "nativeTpCreate", "nativeTpConnect", "nativeTpDestroy"]


@pytest.fixture(scope="module")
def shim(tmp_path_factory):
    out = str(tmp_path_factory.mktemp("jni") / "libdeepj_jni_under_test.so")
    lib_dir = os.path.dirname(_lib.LIB_PATH)
    cmd = ["g++", "-shared", "-fPIC", "-std=c++17", "-Wall", "-Werror", "-I", FAKE, "-I", os.path.join(ROOT, "include"),
           os.path.join(ROOT, "deepj_b200", "csrc", "jni_shim.cpp"), os.path.join(FAKE, "harness.cpp"), "-o", out,
           "-L", lib_dir, "-ldeepj_cuda_jni", f"-Wl,-rpath,{lib_dir}"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    lib = ctypes.CDLL(out)
    lib.fj_bytes_new.restype = ctypes.c_void_p
    lib.fj_bytes_new.argtypes = [ctypes.c_void_p, ctypes.c_int]
    lib.fj_array_length.argtypes = [ctypes.c_void_p]
    for name, restype in (("fj_env_new", ctypes.c_void_p), ("fj_ints_new", ctypes.c_void_p), ("fj_floats_new", ctypes.c_void_p),
                          ("fj_longs_new", ctypes.c_void_p), ("fj_thrown_class", ctypes.c_char_p),
                          ("fj_thrown_message", ctypes.c_char_p), ("fj_release_array", ctypes.c_void_p)):
        getattr(lib, name).restype = restype
    for name in ("fj_env_free", "fj_pending", "fj_thrown_class", "fj_thrown_message", "fj_clear", "fj_release_count",
                 "fj_calls_in_critical", "fj_array_pins", "fj_array_free"):
        getattr(lib, name).argtypes = [ctypes.c_void_p]
    lib.fj_release_mode.argtypes = [ctypes.c_void_p, ctypes.c_int]
    lib.fj_release_array.argtypes = [ctypes.c_void_p, ctypes.c_int]
    lib.fj_array_read.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    lib.fj_ints_new.argtypes = [ctypes.c_void_p, ctypes.c_int]
    lib.fj_floats_new.argtypes = [ctypes.c_void_p, ctypes.c_int]
    lib.fj_longs_new.argtypes = [ctypes.c_int]
    return lib


class Jvm:
    """One stand-in JNIEnv plus helpers that build Java arrays and call a native."""

    def __init__(self, lib):
        self.lib = lib
        self.env = ctypes.c_void_p(lib.fj_env_new())
        self.arrays = []

    def ints(self, values):
        a = np.ascontiguousarray(values, dtype=np.int32)
        h = ctypes.c_void_p(self.lib.fj_ints_new(a.ctypes.data, a.size))
        self.arrays.append(h)
        return h

    def floats(self, values):
        a = np.ascontiguousarray(values, dtype=np.float32)
        h = ctypes.c_void_p(self.lib.fj_floats_new(a.ctypes.data, a.size))
        self.arrays.append(h)
        return h

    def bytes_(self, values):
        a = np.ascontiguousarray(values, dtype=np.int8)
        h = ctypes.c_void_p(self.lib.fj_bytes_new(a.ctypes.data, a.size))
        self.arrays.append(h)
        return h

    def longs(self, n):
        h = ctypes.c_void_p(self.lib.fj_longs_new(n))
        self.arrays.append(h)
        return h

    def read(self, handle, dtype, n):
        out = np.empty(n, dtype=dtype)
        self.lib.fj_array_read(handle, out.ctypes.data)
        return out

    def call(self, name, *args, restype=None):
        fn = getattr(self.lib, PREFIX + name)
        fn.restype = restype
        conv = [a if isinstance(a, (ctypes.c_void_p, ctypes.c_int64)) else ctypes.c_int32(a) for a in args]
        return fn(self.env, None, *conv)

    def exception(self):
        if not self.lib.fj_pending(self.env):
            return None
        return self.lib.fj_thrown_class(self.env).decode(), self.lib.fj_thrown_message(self.env).decode()

    def releases(self):
        return [(self.lib.fj_release_array(self.env, i), self.lib.fj_release_mode(self.env, i))
                for i in range(self.lib.fj_release_count(self.env))]

    def check_unpinned(self):
        for h in self.arrays:
            assert self.lib.fj_array_pins(h) == 0
        assert self.lib.fj_calls_in_critical(self.env) == 0

    def clear(self):
        self.lib.fj_clear(self.env)

    def close(self):
        for h in self.arrays:
            self.lib.fj_array_free(h)
        self.lib.fj_env_free(self.env)


@pytest.fixture
def jvm(shim):
    j = Jvm(shim)
    yield j
    j.close()


def test_every_native_of_cuda_native_is_exported(shim):
    for n in NATIVES:
        assert hasattr(shim, PREFIX + n), n


def test_natives_match_the_java_declarations():
    """java/…/CudaNative.java declares exactly the natives the shim defines."""
    import re
    src = open(os.path.join(ROOT, "java", "io", "github", "kirstenali", "deepj", "tensor", "cuda", "CudaNative.java")).read()
    declared = re.findall(r"static native [\w\[\]]+ (\w+)\(", src)
    assert sorted(declared) == sorted(NATIVES)


def test_count_beyond_the_array_raises_instead_of_reading_past_it(jvm):
    ids, sizes = jvm.ints([1, 2]), jvm.ints([4, 4])
    jvm.call("nativeAllocBuffers", ids, sizes, 3)
    cls, msg = jvm.exception()
    assert cls == "java/lang/RuntimeException" and "count exceeds" in msg
    assert sorted(m for _, m in jvm.releases()) == [JNI_ABORT, JNI_ABORT]
    jvm.check_unpinned()
    jvm.clear()
    cmd = jvm.ints([1, 1, 2, 3])
    jvm.call("nativeFlushOps", cmd, 5)
    assert "cmdStreamLength exceeds" in jvm.exception()[1]
    jvm.call("nativeFlushOps", cmd, -1)
    jvm.check_unpinned()


def test_null_arrays_raise(jvm):
    null = ctypes.c_void_p(None)
    for name, args in (("nativeUploadBuffer", (7, null)), ("nativeDownloadBuffer", (7, null)), ("nativeStats", (null,)),
                       ("nativeFlushOps", (null, 0)), ("nativeReleaseBuffers", (null, 1))):
        jvm.clear()
        jvm.call(name, *args)
        assert jvm.exception() is not None, name


def test_tp_connect_checks_the_handle_array_before_touching_the_library(jvm):
    jvm.call("nativeTpConnect", jvm.bytes_(np.zeros(100)), 2)
    assert "world x 64" in jvm.exception()[1]
    jvm.clear()
    jvm.call("nativeTpConnect", ctypes.c_void_p(None), 2)
    assert jvm.exception() is not None
    jvm.check_unpinned()


def _no_cuda_device():
    import torch
    return not torch.cuda.is_available()


@pytest.mark.skipif(not _no_cuda_device(), reason="needs a machine without a CUDA device")
def test_library_failure_becomes_a_runtime_exception_and_releases_the_arrays(jvm):
    """With no device every compute call fails inside the library; the shim must surface that."""
    cmd = jvm.ints([1, 1, 2, 3, 4])
    jvm.call("nativeFlushOps", cmd, 5)
    cls, msg = jvm.exception()
    assert cls == "java/lang/RuntimeException" and "CUDA" in msg
    assert jvm.releases() == [(cmd.value, JNI_ABORT)]
    jvm.clear()
    got = jvm.call("nativeTpCreate", 0, 2, ctypes.c_int64(1024), restype=ctypes.c_void_p)
    assert got is None and jvm.exception() is not None               # no handle, an exception instead
    jvm.clear()
    out = jvm.floats(np.full(4, 5.0))
    jvm.call("nativeDownloadBuffer", 1, out)
    assert jvm.exception() is not None
    assert jvm.releases() == []                                      # the wait for the device comes before the array is pinned: never pinned, nothing committed
    np.testing.assert_array_equal(jvm.read(out, np.float32, 4), 5.0)
    jvm.check_unpinned()


@pytest.mark.gpu
def test_graph_natives_round_trip_on_the_device(jvm):
    """alloc → upload → flush(OP_ADD, OP_MATMUL) → download → release, as ComputeGraph drives them."""
    base = 7 << 20
    a, b, c, m = base, base + 1, base + 2, base + 3
    jvm.call("nativeInit", 0)
    assert jvm.exception() is None
    ids, sizes = jvm.ints([a, b, c, m]), jvm.ints([6, 6, 6, 4])
    jvm.call("nativeAllocBuffers", ids, sizes, 4)
    assert jvm.exception() is None
    assert sorted(md for _, md in jvm.releases()) == [JNI_ABORT, JNI_ABORT]
    rng = np.random.default_rng(5)
    xa, xb = rng.standard_normal(6).astype(np.float32), rng.standard_normal(6).astype(np.float32)
    ja, jb = jvm.floats(xa), jvm.floats(xb)
    jvm.call("nativeUploadBuffer", a, ja)
    jvm.call("nativeUploadBuffer", b, jb)
    assert jvm.exception() is None
    # [OP_ADD a b c n] then [OP_MATMUL a(2×3) b(3×2) → m(2×2)] (tensor/ComputeGraph.java:19-60)
    from deepj_b200 import compute_graph as cg
    stream = [cg.OP_ADD, a, b, c, 6, cg.OP_MATMUL, a, b, m, 2, 2, 3]
    cmd = jvm.ints(stream)
    jvm.clear()
    jvm.call("nativeFlushOps", cmd, len(stream))
    assert jvm.exception() is None
    assert jvm.releases() == [(cmd.value, JNI_ABORT)]
    jc, jm = jvm.floats(np.zeros(6)), jvm.floats(np.zeros(4))
    jvm.clear()
    jvm.call("nativeDownloadBuffer", c, jc)
    jvm.call("nativeDownloadBuffer", m, jm)
    assert jvm.exception() is None
    assert [md for _, md in jvm.releases()] == [0, 0]               # committed
    np.testing.assert_array_equal(jvm.read(jc, np.float32, 6), xa + xb)
    np.testing.assert_allclose(jvm.read(jm, np.float32, 4).reshape(2, 2), xa.reshape(2, 3) @ xb.reshape(3, 2), rtol=1e-6, atol=1e-6)
    # an id nobody allocated: the reference's message, as an exception
    jvm.clear()
    jvm.call("nativeUploadBuffer", base + 99, ja)
    assert "Buffer not found for upload" in jvm.exception()[1]
    jvm.clear()
    stats = jvm.longs(8)
    jvm.call("nativeStats", stats)
    assert jvm.exception() is None and jvm.read(stats, np.int64, 8)[0] > 0
    jvm.call("nativeReleaseBuffers", ids, 4)
    assert jvm.exception() is None
    jvm.call("nativeDownloadBuffer", c, jc)
    assert "Buffer not found for download" in jvm.exception()[1]
    jvm.check_unpinned()


@pytest.mark.gpu
def test_q8_and_kv_natives_build_a_projection(jvm):
    """nativeQ8Alloc + nativeQ8QuantizeInto + a Q8_LINEAR op give the oracle's Q8 product."""
    import oracle
    from deepj_b200 import compute_graph as cg
    base = (7 << 20) + 1000
    K, N = 64, 48
    w_id, x_id, y_id, q_id, kv_id = base, base + 1, base + 2, base + 3, base + 4
    jvm.call("nativeInit", 0)
    jvm.call("nativeAllocBuffers", jvm.ints([w_id, x_id, y_id]), jvm.ints([K * N, K, N]), 3)
    rng = np.random.default_rng(11)
    W = (rng.standard_normal((K, N)) * 0.05).astype(np.float32)
    x = rng.standard_normal(K).astype(np.float32)
    jvm.call("nativeUploadBuffer", w_id, jvm.floats(W))
    jvm.call("nativeUploadBuffer", x_id, jvm.floats(x))
    jvm.call("nativeQ8Alloc", q_id, K, N)
    jvm.call("nativeQ8QuantizeInto", q_id, 0, w_id, 0, 0, N, N)
    jvm.call("nativeKvAlloc", kv_id, 1, 1, 2, 16, 8)
    assert jvm.exception() is None
    stream = [cg.OP_Q8_LINEAR, x_id, 0, K, -1, 0, q_id, -1, -1, 0, 0, y_id, 0, N, 1]
    cmd = jvm.ints(stream)
    jvm.call("nativeFlushOps", cmd, len(stream))
    assert jvm.exception() is None
    out = jvm.floats(np.zeros(N))
    jvm.call("nativeDownloadBuffer", y_id, out)
    want = oracle.matmul(x.reshape(1, K), oracle.q8_dequantize(*oracle.q8_quantize(W))).reshape(-1)
    got = jvm.read(out, np.float32, N)
    assert np.all(np.abs(got - want) <= 1e-4 + 1e-4 * np.abs(want))
    jvm.call("nativeReleaseBuffers", jvm.ints([w_id, x_id, y_id, q_id, kv_id]), 5)
    assert jvm.exception() is None
    jvm.check_unpinned()


@pytest.mark.gpu
def test_tp_natives_create_connect_destroy_on_one_rank(jvm):
    """A world of one: the handle comes back as a 64-byte array, connecting it maps no peer, destroy frees the buffer."""
    jvm.call("nativeInit", 0)
    handle = jvm.call("nativeTpCreate", 0, 1, ctypes.c_int64(1024), restype=ctypes.c_void_p)
    assert jvm.exception() is None and handle
    handle = ctypes.c_void_p(handle)
    assert jvm.lib.fj_array_length(handle) == 64
    try:
        jvm.call("nativeTpConnect", handle, 1)
        assert jvm.exception() is None
        assert [m for _, m in jvm.releases()][-1] == JNI_ABORT
        jvm.clear()
        jvm.call("nativeTpCreate", 0, 1, ctypes.c_int64(1024), restype=ctypes.c_void_p)      # a second buffer is refused
        assert "already created" in jvm.exception()[1]
        jvm.clear()
    finally:
        jvm.call("nativeTpDestroy")
    assert jvm.exception() is None
