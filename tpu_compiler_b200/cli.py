"""Command line of the interpreter, with the flags of the reference's ``tpuc-interpreter`` tool
(tools/tpuc-interpreter/tpuc-interpreter.cpp:50-65, 123-176):

    python -m tpu_compiler_b200.cli <module> --tensor-in in.npz [--tensor-out out.npz] [--dump-all-tensor all.npz]

``<module>`` is a generic-form TPU-dialect ``.mlir`` (weights from the ``.npz`` its ``tpu.weight_file`` op names, looked
up next to it) or this package's one-op-per-line module text (weights from ``<module>.npz``). The input ``.npz`` holds
one fp32 array per module input; with one input its name is free, with several a name matches an input when one is
a prefix of the other (the reference's rule). The outputs (``--tensor-out``) and every activation
(``--dump-all-tensor``) are written as fp32 arrays in the module's shapes.
"""
import argparse
import sys

import numpy as np

from .interpreter import module


def _name_match(a, b):
    return a == b[:len(a)] if len(a) <= len(b) else a[:len(b)] == b


def main(argv=None):
    ap = argparse.ArgumentParser(prog="tpuc-interpreter (B200)", description="TPU-dialect interpreter on a B200")
    ap.add_argument("module", help="module file (.mlir in generic form, or module text)")
    ap.add_argument("--tensor-in", required=True, help="Input Tensor Filename (npz)")
    ap.add_argument("--tensor-out", default="-", help="Output Tensor Filename (npz)")
    ap.add_argument("--dump-all-tensor", default="-", help="dump all tensor into a npz file")
    ap.add_argument("--device", type=int, default=0, help="CUDA device ordinal")
    args = ap.parse_args(argv)

    m = module(args.device)
    with open(args.module) as f:
        generic = '"tpu.' in f.read()
    (m.load_mlir if generic else m.load)(args.module)
    inputs = dict(np.load(args.tensor_in))
    details = m.input_sizes()
    if len(details) != len(inputs):
        sys.exit("Input number not same, needed is %d, get %d" % (len(details), len(inputs)))
    if len(inputs) == 1:
        pairs = [(details[0], next(iter(inputs.values())))]
    else:
        pairs = []
        for name, arr in inputs.items():
            hit = [d for d in details if _name_match(name, d[0])]
            if not hit:
                sys.exit("not find target tensor in input npz: %s" % name)
            pairs.append((hit[0], arr))
    for (name, size), arr in pairs:
        if arr.size != size:
            sys.exit("input tensor size not same, needed is %d, get %d" % (size, arr.size))
        m.set_tensor(name, np.asarray(arr, np.float32))
    m.invoke()
    if args.tensor_out != "-":
        np.savez(args.tensor_out, **{n: m.get_tensor(n) for n in m.get_output_details()})
    if args.dump_all_tensor != "-":
        np.savez(args.dump_all_tensor, **m.get_all_tensor())
    m.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
