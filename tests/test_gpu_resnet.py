"""GPU parity of the whole INT8 ResNet-50 module (the benchmark workload): every tensor of a
batch-1 run equals the CPU oracle bit for bit; larger batches are checked through the
size-independent property that images do not interact (a batch equals its images run alone)."""
import numpy as np
import pytest

from oracle import graph_runner
from tpu_compiler_b200 import graphs

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def model_b1():
    return graphs.resnet50_int8(batch=1, seed=1001)


def test_resnet50_b1_every_tensor(model_b1):
    from tpu_compiler_b200 import module
    img = np.random.default_rng(123).uniform(-1, 1, (1, 3, 224, 224)).astype(np.float32)
    ref = graph_runner.run(model_b1.text, model_b1.weights, {"data": img})
    m = module(0)
    m.load_text(model_b1.text, model_b1.weights)
    m.set_tensor("data", img)
    m.invoke()
    first_bad = None
    for name in m.get_all_tensor_names():
        got = m.get_tensor(name)
        if not np.array_equal(got.reshape(-1), ref[name].reshape(-1)):
            first_bad = (name, int((got.reshape(-1) != ref[name].reshape(-1)).sum()), got.size)
            break
    assert first_bad is None, "first mismatching op: %s (%d of %d values)" % first_bad
    assert m.get_data_type("res2a") == "INT8" and m.get_data_type("fc1000_dequant") == "FP32"
    assert m.get_output_details() == ["fc1000_dequant"] and m.get_input_details() == ["data"]
    m.close()


def test_resnet50_batch_equals_single_images_and_graph_equals_eager(model_b1):
    from tpu_compiler_b200 import module
    B = 5
    imgs = np.random.default_rng(321).uniform(-1, 1, (B, 3, 224, 224)).astype(np.float32)
    mb = graphs.resnet50_int8(batch=B, seed=1001)
    m = module(0)
    m.load_text(mb.text, mb.weights)
    m.set_tensor("data", imgs)
    m.invoke()          # first invoke captures the CUDA graph
    m.invoke()          # replay
    names = ["conv1", "pool1", "res2c", "res3a_branch1", "res4f", "res5c", "pool5", "fc1000", "fc1000_dequant"]
    batch = {n: m.get_tensor(n) for n in names}
    m.set_option("cuda_graph", 0)
    m.invoke()
    for n in names:
        assert np.array_equal(batch[n], m.get_tensor(n)), "graph replay differs from eager at " + n
    m.close()
    s = module(0)
    s.load_text(model_b1.text, model_b1.weights)
    for i in (0, B - 1):
        s.set_tensor("data", imgs[i:i + 1])
        s.invoke()
        for n in names:
            assert np.array_equal(batch[n][i:i + 1], s.get_tensor(n)), "image %d differs at %s" % (i, n)
    s.close()


def test_run_api_and_errors():
    from tpu_compiler_b200 import TpucbError, module
    model = graphs.single_conv_i8(1, 32, 32, 8, 3, 1, 1, seed=5)
    m = module(0)
    m.load_text(model.text, model.weights)
    out = m.run(model.meta["x"])
    assert list(out) == ["conv"] and out["conv"].shape == (1, 32, 8, 8)
    with pytest.raises(TpucbError):
        m.set_tensor("x", np.zeros(7, np.float32))
    with pytest.raises(TpucbError):
        m.get_tensor("nope")
    with pytest.raises(TpucbError):
        m.load_text("frobnicate name=a shape=1,1,1,1 dtype=INT8\n", {})
    m.close()


def test_set_tensor_async_pipeline_matches_synchronous_path():
    """The pipelined upload (copy stream + double-buffered staging) feeds each launch the right batch."""
    import ctypes as C
    from tpu_compiler_b200 import module
    from tpu_compiler_b200._lib import check, lib
    model = graphs.single_conv_i8(4, 64, 64, 28, 3, 1, 1, seed=909)
    m = module(0)
    m.load_text(model.text, model.weights)
    rng = np.random.default_rng(5)
    xs = [rng.integers(-128, 128, (4, 64, 28, 28)).astype(np.float32) for _ in range(5)]
    expect = []
    for x in xs:
        m.set_tensor("x", x)
        m.invoke()
        expect.append(m.get_tensor("conv"))
    L = lib()
    numel = xs[0].size
    bufs = []
    for _ in range(2):
        p = C.c_void_p()
        check(L.tpucb_host_alloc(C.byref(p), numel * 4))
        bufs.append(p)
    views = [np.ctypeslib.as_array(C.cast(b, C.POINTER(C.c_float)), shape=(numel,)) for b in bufs]
    views[0][:] = xs[0].reshape(-1)
    m.set_tensor_async("x", bufs[0], numel)
    for i in range(len(xs)):
        m.launch()
        if i + 1 < len(xs):
            views[(i + 1) & 1][:] = xs[i + 1].reshape(-1)   # the other buffer: not in flight
            m.set_tensor_async("x", bufs[(i + 1) & 1], numel)
        got = m.get_tensor("conv")                           # syncs: both buffers are free again
        assert np.array_equal(got, expect[i]), "step %d" % i
    for b in bufs:
        check(L.tpucb_host_free(b))
    m.close()


def test_resnet50_with_residual_adds_in_the_convolution_epilogue(model_b1):
    """Option fuse_residual_add: the 16 eltwise adds run inside the epilogue of the convolution that produces their
    second operand. Every tensor (the convolution results and the sums) still equals the oracle, at a batch whose
    pixel count leaves ragged tiles, and 16 kernels fewer are launched."""
    from tpu_compiler_b200 import module
    B = 3
    imgs = np.random.default_rng(99).uniform(-1, 1, (B, 3, 224, 224)).astype(np.float32)
    mb = graphs.resnet50_int8(batch=B, seed=1001)
    plain = module(0)
    plain.load_text(mb.text, mb.weights)
    m = module(0)
    m.set_option("fuse_residual_add", 1)
    m.load_text(mb.text, mb.weights)
    assert plain.kernel_count() - m.kernel_count() == 16
    plain.close()
    m.set_tensor("data", imgs)
    m.invoke()
    ref = graph_runner.run(mb.text, mb.weights, {"data": imgs})
    for name in m.get_all_tensor_names():
        assert np.array_equal(m.get_tensor(name).reshape(-1), ref[name].reshape(-1)), name
    m.close()


def test_programmatic_dependent_launch_on_and_off(model_b1):
    """Option pdl: kernels (1: the convolution kernels, 2: every kernel of the op list) are launched so that they may
    start while their predecessor finishes and order themselves behind it on the device. Off and both on forms must
    give the same tensors, launch after launch (a kernel that read its input too early would show as a difference
    between replays)."""
    from tpu_compiler_b200 import module
    B = 2
    imgs = np.random.default_rng(7).uniform(-1, 1, (B, 3, 224, 224)).astype(np.float32)
    mb = graphs.resnet50_int8(batch=B, seed=1001)
    names = ["conv1", "pool1", "res2a", "res3d", "res4f", "res5c", "pool5", "fc1000_dequant"]
    got = {}
    for pdl in (0, 1, 2):
        m = module(0)
        m.set_option("pdl", pdl)
        m.load_text(mb.text, mb.weights)
        for rep in range(6):
            m.set_tensor("data", imgs if rep % 2 == 0 else imgs[::-1].copy())
            m.invoke()
            cur = {n: m.get_tensor(n) for n in names}
            if rep >= 2:
                for n in names:
                    assert np.array_equal(cur[n], got[(pdl, rep % 2)][n]), (pdl, rep, n)
            else:
                got[(pdl, rep)] = cur
        m.close()
    for n in names:
        for pdl in (1, 2):
            assert np.array_equal(got[(0, 0)][n], got[(pdl, 0)][n]) and np.array_equal(got[(0, 1)][n], got[(pdl, 1)][n]), n
        assert np.array_equal(got[(0, 0)][n][0], got[(0, 1)][n][1]), n


def test_int8_input_upload_replaces_the_quant_op():
    """tpucb_interp_set_tensor_async_i8: the caller quantises the image on the host and uploads one byte per value into
    the result of the input quant op, which is then skipped; setting the fp32 input again brings the op back."""
    import ctypes as C
    from tpu_compiler_b200 import TpucbError, module
    from tpu_compiler_b200._lib import check, lib
    B = 2
    rng = np.random.default_rng(17)
    x = rng.uniform(-1, 1, (B, 3, 224, 224)).astype(np.float32)
    x2 = rng.uniform(-1, 1, (B, 3, 224, 224)).astype(np.float32)
    mb = graphs.resnet50_int8(batch=B, seed=1001)
    names = ["data_quant", "conv1", "res2c", "res5c", "fc1000_dequant"]
    m = module(0)
    m.load_text(mb.text, mb.weights)
    m.set_tensor("data", x)
    m.invoke()
    ref = {n: m.get_tensor(n) for n in names}
    m.set_tensor("data", x2)
    m.invoke()
    ref2 = {n: m.get_tensor(n) for n in names}
    full = m.kernel_count()
    # QuantOpKernel at the graph input (core/quant.cpp:22-30): sat8(std::round(x * scale)), half away from zero
    v = x * np.float32(128.0)
    q = np.clip(np.where(v >= 0, np.floor(v + np.float32(0.5)), np.ceil(v - np.float32(0.5))), -128, 127).astype(np.int8)
    L = lib()
    buf = C.c_void_p()
    check(L.tpucb_host_alloc_write_combined(C.byref(buf), q.size))
    C.memmove(buf, q.ctypes.data, q.size)
    m.set_tensor_async_i8("data_quant", buf, q.size)
    m.launch()
    m.sync()
    assert m.kernel_count() == full - 1
    for n in names:
        assert np.array_equal(m.get_tensor(n), ref[n]), n
    m.set_tensor_async_i8("data_quant", buf, q.size)   # again, through the second staging buffer and the replayed graph
    m.launch()
    m.sync()
    assert np.array_equal(m.get_tensor("fc1000_dequant"), ref["fc1000_dequant"])
    with pytest.raises(TpucbError):
        m.set_tensor_async_i8("conv1", buf, q.size)     # not an input
    with pytest.raises(TpucbError):
        m.set_tensor_async_i8("data", buf, q.size)      # not INT8
    m.set_tensor("data", x2)                            # the fp32 way again: the quant op is back
    m.invoke()
    assert m.kernel_count() == full
    for n in names:
        assert np.array_equal(m.get_tensor(n), ref2[n]), n
    m.sync()
    check(L.tpucb_host_free(buf))
    m.close()
