"""Error paths, exercised without faulting, trapping or hanging anything: a bounded device wait that runs out (a
barrier that nothing arrives at; no copy in flight) comes back as an error status and leaves the interpreter usable;
malformed modules are refused at load with a status."""
import numpy as np
import pytest

from oracle import graph_runner
from tpu_compiler_b200 import graphs

pytestmark = pytest.mark.gpu


def test_bounded_wait_runs_out_and_the_interpreter_stays_usable():
    from tpu_compiler_b200 import TpucbError, module
    # 784 pixel tiles on 296 persistent CTAs: some CTAs own three tiles, and the third needs an accumulator buffer
    # back from the epilogue. With the self-test option the epilogue never hands it back.
    model = graphs.single_conv_i8(64, 64, 64, 56, 3, 1, 1, seed=31)
    m = module(0)
    m.set_option("selftest_lost_arrival", 4)       # every wait: 4 rounds of 1024 polls
    m.load_text(model.text, model.weights)
    m.set_tensor("x", model.meta["x"])
    with pytest.raises(TpucbError, match="bounded wait"):
        m.invoke()
    with pytest.raises(TpucbError, match="bounded wait"):
        m.invoke()                                  # the same module fails the same way again: nothing is left wedged
    # the same interpreter, the same module without the self-test: correct results
    m.set_option("selftest_lost_arrival", 0)
    m.load_text(model.text, model.weights)
    m.set_tensor("x", model.meta["x"])
    m.invoke()
    ref = graph_runner.run(model.text, model.weights, {"x": model.meta["x"]})["conv"]
    assert np.array_equal(m.get_tensor("conv"), ref)
    m.close()
    # and a fresh interpreter on the same device works too (the context survived)
    small = graphs.single_conv_i8(1, 32, 32, 8, 3, 1, 1, seed=5)
    s = module(0)
    s.load_text(small.text, small.weights)
    out = s.run(small.meta["x"])["conv"]
    assert np.array_equal(out, graph_runner.run(small.text, small.weights, {"x": small.meta["x"]})["conv"])
    s.close()


def test_malformed_modules_are_refused_with_a_status():
    from tpu_compiler_b200 import TpucbError, module
    model = graphs.single_conv_i8(1, 32, 32, 8, 3, 1, 1, seed=6)
    m = module(0)
    # a filter of the wrong size
    w = dict(model.weights)
    w["conv_filter"] = w["conv_filter"][:, :, :, :2]
    with pytest.raises(TpucbError, match="filter has"):
        m.load_text(model.text, w)
    # a multiplier outside [0, 2^31): the reference's quantiser emits none, the epilogue could not represent it
    w = dict(model.weights)
    mult = w["conv_multiplier"].copy()
    mult[3] = np.float32(2 ** 31)
    w["conv_multiplier"] = mult
    with pytest.raises(TpucbError, match="outside"):
        m.load_text(model.text, w)
    w["conv_multiplier"] = -model.weights["conv_multiplier"]
    with pytest.raises(TpucbError, match="outside"):
        m.load_text(model.text, w)
    # an operand that does not exist, an INT8 convolution without its requantisation operands
    with pytest.raises(TpucbError):
        m.load_text(model.text.replace("in=x,", "in=y,"), model.weights)
    with pytest.raises(TpucbError, match="rshift and multiplier"):
        m.load_text(model.text.replace("conv_rshift,conv_multiplier", "-,-"), model.weights)
    # after all that the interpreter still loads and runs the good module
    m.load_text(model.text, model.weights)
    out = m.run(model.meta["x"])["conv"]
    assert np.array_equal(out, graph_runner.run(model.text, model.weights, {"x": model.meta["x"]})["conv"])
    m.close()
