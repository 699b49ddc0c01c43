"""GPU tests of the drop-in boundary beyond the whole-module calls: batch slots (the bidx arguments and
fastInvokeAllBatch of MlirModuleInterpreter), the per-op create / invoke surface of CPUOpKernel, dump, the
``pytuner.tuner`` method set driven by the reference's tuning loop, and the tpuc-interpreter command line. Every
call goes through the C ABI; expected values come from the CPU oracle."""
import ctypes as C
import os

import numpy as np
import pytest

from oracle import graph_runner
from tpu_compiler_b200 import graphs
from tpu_compiler_b200 import quantize as Q

from .test_gpu_tuner import N, small_fp32_net
from .test_mlir_text import MLIR, tiny_weights

pytestmark = pytest.mark.gpu


def small_int8_net():
    b = graphs.GraphBuilder(21, simulate=True)
    img = np.random.default_rng(5).uniform(-1, 1, (1, 3, 20, 20))
    b.input("data", (1, 3, 20, 20), sample=img)
    x = b.quant_in("q", "data", 1.0)
    x = b.conv_i8("c1", x, 32, 3, stride=2, pad=1)
    x = b.pool_max("p1", x, 3, 2, pad=(0, 1, 0, 1))
    y = b.conv_i8("c2", x, 16, 1, pad=0)
    y = b.conv_i8("c3", y, 32, 3, pad=1, relu=False)
    x = b.eltwise_add_i8("add", [x, y])
    x = b.pool_avg_i8("gap", x)
    x = b.fc_i8("fc", x, 10)
    b.dequant("out", x, 100.0)
    return graphs.Model(b.text(), b.weights, ["data"], ["out"])


def test_batch_slots_and_fast_invoke_all_batch():
    """max_batch_size 3: slot b of every tensor is what the batch-1 module computes for image b."""
    from tpu_compiler_b200 import TpucbError, module
    model = small_int8_net()
    imgs = np.random.default_rng(6).uniform(-1, 1, (3, 1, 3, 20, 20)).astype(np.float32)
    refs = [graph_runner.run(model.text, model.weights, {"data": imgs[b]}) for b in range(3)]
    m = module(0, max_batch_size=3)
    m.load_text(model.text, model.weights)
    assert m.get_tensor_shape("c1") == [1, 32, 10, 10] and m.input_sizes() == [("data", 3 * 20 * 20)]
    assert [o["shape"] for o in m.op_info if o["name"] == "c1"] == [[1, 32, 10, 10]]
    for b in range(3):
        m.set_tensor("data", imgs[b], b)
    assert "dirty: 1" in m.dump("c2") and "op_type: conv_2d" in m.dump("c2") and "max_batch_size: 3" in m.dump("c2")
    m.fast_invoke_all_batch("c3", 3)            # one launch per op over all three slots, up to c3
    assert "dirty: 0" in m.dump("c2") and "dirty: 1" in m.dump("add")
    for b in range(3):
        assert np.array_equal(m.get_tensor("c3", b), refs[b]["c3"])
    m.fast_invoke_all_batch("", 3)              # the remaining (still dirty) ops
    for b in range(3):
        for n in ("q", "c1", "p1", "add", "gap", "fc", "out"):
            assert np.array_equal(m.get_tensor(n, b), refs[b][n]), (n, b)
    # setTensor(bidx) + invoke(bidx): the slot's results follow its input
    new = np.random.default_rng(7).uniform(-1, 1, (1, 3, 20, 20)).astype(np.float32)
    m.set_tensor("data", new, 1)
    m.invoke(1)
    ref_new = graph_runner.run(model.text, model.weights, {"data": new})
    assert np.array_equal(m.get_tensor("out", 1), ref_new["out"])
    assert np.array_equal(m.get_tensor("out", 0), refs[0]["out"]) and np.array_equal(m.get_tensor("out", 2), refs[2]["out"])
    whole = m.get_tensor("fc")                  # no slot: all slots, slot-major
    assert whole.shape == (3, 10) and np.array_equal(whole[2:3], refs[2]["fc"])
    with pytest.raises(TpucbError):
        m.get_tensor("fc", 3)
    with pytest.raises(TpucbError):
        m.set_tensor("data", np.zeros(5, np.float32), 0)
    m.close()
    # an op that may mix the leading dimension with the others is refused on a slotted interpreter
    bad = module(0, max_batch_size=2)
    with pytest.raises(TpucbError, match="max_batch_size"):
        bad.load_text("input name=x shape=1,4,4,4 dtype=FP32\npermute name=p in=x shape=4,1,4,4 dtype=FP32 order=1,0,2,3\n", {})
    bad.close()


def test_per_op_create_invoke():
    """One op at a time, as a CPUOpKernel-shaped adapter would own them: operands looked up in the context,
    results visible to later ops, invoke() per op."""
    from tpu_compiler_b200 import TpucbError, module
    model = small_int8_net()
    img = np.random.default_rng(9).uniform(-1, 1, (1, 3, 20, 20)).astype(np.float32)
    ref = graph_runner.run(model.text, model.weights, {"data": img})
    ctx = module(0)
    ctx.set_weights(model.weights)
    ops = {}
    for line in model.text.splitlines():
        k = ctx.create_op(line)
        ops[k.name] = k
    assert ops["c1"].op_type == "conv_2d" and ops["c1"].datatype == "INT8" and ops["c1"].shape == [1, 32, 10, 10]
    assert ops["c1"].dirty and ops["out"].datatype == "FP32"
    ops["data"].set_tensor(img)
    with pytest.raises(TpucbError, match="not an input op"):
        ops["c1"].set_tensor(np.zeros((1, 32, 10, 10), np.float32))
    for name in ("q", "c1", "p1", "c2", "c3"):
        ops[name].invoke()
        assert np.array_equal(ops[name].get_tensor(), ref[name]), name
    assert not ops["c3"].dirty and ops["add"].dirty
    assert ctx.get_output_details() == ["out"] and ctx.get_input_details() == ["data"]
    ctx.invoke()                                 # the context still runs as a whole module
    for name in ("add", "gap", "fc", "out"):
        assert np.array_equal(ops[name].get_tensor(), ref[name]), name
    with pytest.raises(TpucbError):
        ctx.create_op("conv_2d name=zz in=nope,w,-,-,-,r,m shape=1,8,4,4 dtype=INT8 kh=1 kw=1")
    ctx.load_text("input name=x shape=1,4,4,4 dtype=FP32\n", {})
    with pytest.raises(TpucbError, match="stale"):
        ops["c1"].invoke()
    ctx.close()


def drive_like_the_reference_loop(t, text_file, cands, images, ref_act, tmp_table):
    """The call sequence of SimpleTuner.run (kld_calibrator.py:156-201) against a ``pytuner.tuner``-shaped object:
    per op and candidate a table file, load, quantize, build(op), invoke(op), get_tensor_type, get_tensor(op, i)."""
    table = {k: v[0] for k, v in cands.items()}
    dists = {}
    for op in t.op_info():
        name = op["name"]
        if op["type"] == "tpu.input":
            continue
        best, minimum = cands[name][0], float("inf")
        dists[name] = {}
        for threshold in cands[name]:
            if threshold <= 1e-6:
                continue
            trial = dict(table)
            trial[name] = threshold
            with open(tmp_table, "w") as f:
                for k, v in trial.items():
                    f.write("{} {:.7f} {:.7f} {:.7f}\n".format(k, v, 0.0, 0.0))
            t.load(text_file)
            t.quantize(tmp_table)
            t.build(name)
            t.invoke(name)
            is_int8 = t.get_tensor_type(name) == "INT8"
            distance = 0.0
            for i in range(len(images)):
                target = t.get_tensor(name, i)
                if is_int8:
                    target = target * (threshold / 127.0)
                ref = ref_act[i][name]
                diff = ref.flatten() - target.flatten()
                distance += np.linalg.norm(diff) / np.linalg.norm(ref.flatten(), ord=1)
            dists[name][threshold] = float(distance)
            if distance < minimum:
                best, minimum = threshold, distance
        table[name] = best
    return table, dists


def test_pytuner_class_under_the_reference_loop(tmp_path):
    """pytuner.tuner over this backend gives the thresholds and distances of the incremental device tuner
    (tests/test_gpu_tuner.py checks that one against the whole-module loop on the CPU oracle)."""
    from tpu_compiler_b200.pytuner import tuner
    from tpu_compiler_b200.tuner import SimpleTuner
    rng = np.random.default_rng(77)
    text, weights = small_fp32_net(rng)
    one = text.replace("shape=%d," % N, "shape=1,")      # the module the reference tunes is batch 1, one slot per image
    images = rng.normal(0, 1, (N, 3, 16, 16)).clip(-3, 3).astype(np.float32)
    f = tmp_path / "net.txt"
    f.write_text(one)
    np.savez(str(f) + ".npz", **weights)
    t = tuner(N)
    t.load(str(f))
    t.build()
    for i in range(N):
        t.set_data(images[i:i + 1], i)
    t.invoke()
    ref_act = {i: t.get_all_tensors(i) for i in range(N)}
    fp32 = graph_runner.run(text, weights, {"data": images})
    names = [o["name"] for o in Q.parse_text(text)]
    for n in names:
        assert np.abs(ref_act[2][n] - fp32[n][2].reshape(-1)).max() <= 1e-4 * max(np.abs(fp32[n]).max(), 1e-6), n
    assert [o["type"] for o in t.op_info()][:2] == ["tpu.input", "tpu.conv_2d"] and t.get_output_details() == ["fc"]
    absmax = {k: float(np.abs(v).max()) for k, v in fp32.items()}
    factors = [(1.0, 0.6, 0.35), (0.6, 1.0, 0.35), (0.35, 0.6, 1.0)]
    cand_map = {"t%d" % k: {n: absmax[n] * factors[i % 3][k] for i, n in enumerate(names)} for k in range(3)}
    cands = {}
    for _, mm in cand_map.items():
        for op, thr in mm.items():
            cands.setdefault(op, []).append(thr)
    got_table, got_d = drive_like_the_reference_loop(t, str(f), cands, images, ref_act, str(tmp_path / "tmp_table.txt"))
    t.close()
    dev = SimpleTuner(text, weights, cand_map, None, images)
    exp_table = dev.run()
    for n in names[1:]:
        assert got_table[n] == exp_table[n], n
        for thr, d in dev.distances[n].items():
            assert abs(got_d[n][thr] - d) <= 1e-5 * abs(d) + 1e-12, (n, thr)
    dev.close()


def test_command_line_round_trip(tmp_path):
    """<mlir> --tensor-in npz --tensor-out npz --dump-all-tensor npz on a generic-form TPU-dialect file."""
    from tpu_compiler_b200 import cli, mlir_text
    (tmp_path / "tiny.mlir").write_text(MLIR)
    np.savez(str(tmp_path / "tiny_net_1a2b3c4d.npz"), **tiny_weights())
    x = np.random.default_rng(3).normal(0, 1, (2, 3, 16, 16)).astype(np.float32)
    np.savez(str(tmp_path / "in.npz"), whatever=x)
    rc = cli.main([str(tmp_path / "tiny.mlir"), "--tensor-in", str(tmp_path / "in.npz"), "--tensor-out",
                   str(tmp_path / "out.npz"), "--dump-all-tensor", str(tmp_path / "all.npz")])
    assert rc == 0
    text, _ = mlir_text.convert(MLIR)
    ref = graph_runner.run(text, tiny_weights(), {"image": x})
    out, allt = dict(np.load(str(tmp_path / "out.npz"))), dict(np.load(str(tmp_path / "all.npz")))
    assert list(out) == ["prob"] and set(allt) == set(ref)
    for n, v in allt.items():
        assert v.shape == ref[n].shape and np.abs(v - ref[n]).max() <= 1e-4 * max(np.abs(ref[n]).max(), 1e-6), n
