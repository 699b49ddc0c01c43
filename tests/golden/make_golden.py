"""Generate the golden vectors under tests/golden/ from the reference's own
arithmetic sources, compiled unmodified into oracle/_ref (needs the reference
checkout; run once, commit the .npz files).

    python tests/golden/make_golden.py
"""
import ctypes as C
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
import oracle  # noqa: E402

_f = C.POINTER(C.c_float)


def p(a):
    return a.ctypes.data_as(_f)


def main():
    ref = oracle.ref()
    assert ref is not None, "reference checkout not available"
    rng = np.random.default_rng(20240607)

    # ---- QDM requant (int32 and float overloads) --------------------------------
    edge_v = [0, 1, -1, 2, -2, 127, -128, 255, -255, 2 ** 15, -2 ** 15, 2 ** 24 - 1, -2 ** 24,
              2 ** 30, -2 ** 30, 2 ** 31 - 1, -2 ** 31]
    edge_m = [2 ** 30, 2 ** 30 + 128, 2 ** 31 - 128, 1518500224]
    vs, rs, ms = [], [], []
    for v in edge_v:
        for r in [0, 1, 2, 7, 15, 30, 31]:
            for m in edge_m:
                vs.append(v), rs.append(r), ms.append(m)
    nrand = 20000
    vs += list(rng.integers(-2 ** 25, 2 ** 25, nrand)) + list(rng.integers(-2 ** 31, 2 ** 31, nrand))
    rs += list(rng.integers(0, 32, 2 * nrand))
    ms += list((rng.integers(2 ** 30, 2 ** 31 - 128, 2 * nrand) // 128) * 128)
    vs, rs, ms = np.array(vs, np.int64), np.array(rs, np.uint32), np.array(ms, np.uint32)
    q_i32 = np.array([ref.ref_qdm_i32(int(v), int(r), int(m)) for v, r, m in zip(vs, rs, ms)], np.int32)
    fv = vs.astype(np.float32)
    ok = np.abs(fv.astype(np.float64)) < 2 ** 31 - 200  # float->int32 cast defined
    q_f32 = np.array([ref.ref_qdm_f32(float(v), int(r), int(m)) if o else 0
                      for v, r, m, o in zip(fv, rs, ms, ok)], np.int32)
    np.savez_compressed(os.path.join(HERE, "qdm.npz"), v=vs.astype(np.int32), rshift=rs, multiplier=ms,
                        out_i32=q_i32, v_f32=fv, f32_valid=ok, out_f32=q_f32)

    # ---- non-QDM requant and plain rshift ---------------------------------------
    v2 = np.concatenate([np.arange(-300, 301), rng.integers(-2 ** 15, 2 ** 15, 20000)]).astype(np.float32)
    r2 = rng.integers(0, 16, v2.size).astype(np.uint32)
    m2 = rng.integers(0, 128, v2.size).astype(np.uint32)
    o_mr = np.array([ref.ref_mul_rshift_f32(float(v), int(r), int(m)) for v, r, m in zip(v2, r2, m2)], np.int32)
    o_r = np.array([ref.ref_rshift_f32(float(v), int(r)) for v, r in zip(v2, r2)], np.int32)
    np.savez_compressed(os.path.join(HERE, "nonqdm.npz"), v=v2, rshift=r2, multiplier=m2, out_mul_rshift=o_mr,
                        out_rshift=o_r)

    # ---- BF16 rounding and F32->int8 --------------------------------------------
    bits = np.concatenate([
        np.array([0x00000000, 0x80000000, 0x3f800000, 0x3f808000, 0x3f818000, 0x3f80ffff, 0x7f800000,
                  0xff800000, 0x7f7fffff, 0x7f7f8000, 0x00000001, 0x00800000, 0x7fc00000], np.uint32),
        rng.integers(0, 2 ** 32, 30000, dtype=np.uint64).astype(np.uint32)])
    x = bits.view(np.float32)
    b_r = np.array([ref.ref_f32_to_bf16(float(v), 1) for v in x], np.uint16)
    b_t = np.array([ref.ref_f32_to_bf16(float(v), 0) for v in x], np.uint16)
    y = np.concatenate([np.arange(-260, 260, 0.25), rng.uniform(-200, 200, 5000)]).astype(np.float32)
    i_e = np.array([ref.ref_f32_to_int8(float(v), 0) for v in y], np.int32)
    i_z = np.array([ref.ref_f32_to_int8(float(v), 1) for v in y], np.int32)
    np.savez_compressed(os.path.join(HERE, "bf16_int8.npz"), bits=bits, bf16_round=b_r, bf16_trunc=b_t, y=y,
                        int8_even=i_e, int8_zero=i_z)

    # ---- per-channel conv requant (the tensor-level entry conv.cpp calls) --------
    on, oc, isz = 2, 24, 50
    acc = rng.integers(-2 ** 22, 2 ** 22, (on, oc, isz)).astype(np.float32)
    bias = rng.integers(-2 ** 16, 2 ** 16, oc).astype(np.float32)
    rsh = rng.integers(0, 32, oc).astype(np.float32)
    rsh[:8] = rng.integers(12, 18, 8)
    mul = ((rng.integers(2 ** 30, 2 ** 31 - 128, oc) // 128) * 128).astype(np.float32)
    outs = {}
    for relu in (0, 1):
        o = np.empty_like(acc)
        a = acc.copy()
        ref.ref_requant_per_channel(p(o), p(a), p(bias), relu, C.c_int64(on), C.c_int64(oc), C.c_int64(isz),
                                    p(rsh), p(mul))
        outs[relu] = o
    np.savez_compressed(os.path.join(HERE, "requant_per_channel.npz"), acc=acc, bias=bias, rshift=rsh,
                        multiplier=mul, out=outs[0], out_relu=outs[1])

    # ---- BF16 LUT tables + interpolation -----------------------------------------
    lut = {}
    xs = np.concatenate([np.linspace(-20, 20, 4001), rng.normal(0, 4, 8000),
                         np.array([0.0, -0.0, 1e-8, 127.9, -128.5, 1e9, -1e9])]).astype(np.float32)
    xs = np.array([ref.ref_bf16(float(v), 1) for v in xs], np.float32)
    lut["x"] = xs
    for name in ("sigmoid", "mish", "exp", "tanh"):
        base, slope = np.zeros(256, np.float32), np.zeros(256, np.float32)
        ref.ref_lut_gen_slope_tables(name.encode(), C.c_float(1.0), C.c_float(0.0), p(base), p(slope))
        out = np.empty_like(xs)
        xin = xs.copy()
        ref.ref_lut_bf16_slope(name.encode(), p(xin), p(out), xs.size, p(base), p(slope))
        lut[name + "_base"], lut[name + "_slope"], lut[name + "_out"] = base, slope, out
    e, m = np.zeros(256, np.float32), np.zeros(256, np.float32)
    ref.ref_lut_gen_expmant_tables(b"pow", C.c_float(-1.0), p(e), p(m))
    xm = np.concatenate([rng.uniform(1e-3, 1e3, 6000), -rng.uniform(1e-3, 1e3, 2000), np.array([0.0, 1.0, 2.0, 0.5])]
                        ).astype(np.float32)
    xm = np.array([ref.ref_bf16(float(v), 1) for v in xm], np.float32)
    om = np.empty_like(xm)
    xmi = xm.copy()
    ref.ref_lut_bf16_mantissa(p(xmi), p(om), xm.size, p(e), p(m))
    lut.update(recip_exp=e, recip_mant=m, recip_x=xm, recip_out=om)
    np.savez_compressed(os.path.join(HERE, "lut_bf16.npz"), **lut)

    # ---- KLD threshold search ----------------------------------------------------
    hists, widths, thr = [], [], []
    for k in range(12):
        n = int(rng.integers(10 ** 4, 10 ** 6))
        if k % 3 == 0:
            data = np.abs(rng.normal(0, 1, n))
        elif k % 3 == 1:
            data = np.abs(rng.laplace(0, 1, n))
        else:
            data = np.maximum(rng.normal(0, 1, n), 0)
        data = data.astype(np.float32)
        amax = np.float32(data.max())
        width = np.float32(amax / np.float32(2047))
        t = data[data != 0]
        h, _ = np.histogram(np.floor(t / width + np.float32(0.5)), bins=2048, range=(0, 2047))
        h = h.astype(np.int32)
        hc = h.copy()
        thr.append(ref.kl_diversity_hist(hc.ctypes.data_as(C.c_void_p), C.c_float(float(width)), 2048))
        hists.append(h), widths.append(width)
    np.savez_compressed(os.path.join(HERE, "kld.npz"), hist=np.stack(hists), width=np.array(widths, np.float32),
                        threshold=np.array(thr, np.float32))
    make_softmax_bf16(ref)
    make_weight_quant(ref)
    print("golden vectors written to", HERE)


def make_softmax_bf16(ref):
    """BF16 softmax cases. softmax.cpp itself needs the MLIR headers and cannot be compiled alone, so the sequence
    of core/softmax.cpp:88-151 is stepped here in numpy fp32 over the reference's own compiled primitives
    (BF16 rounding, bf16_lut_slope "exp", bf16_lut_mantissa "mantissa" / "log" and their table generators)."""
    rng = np.random.default_rng(77)
    bf = lambda a: np.array([ref.ref_bf16(float(v), 1) for v in np.asarray(a, np.float32).ravel()], np.float32).reshape(np.shape(a))  # noqa: E731
    eb, es = np.zeros(256, np.float32), np.zeros(256, np.float32)
    ref.ref_lut_gen_slope_tables(b"exp", C.c_float(1.0), C.c_float(0.0), p(eb), p(es))
    tabs = {}
    for nm, coeff in (("pow", -1.0), ("log", 0.0)):
        e, m = np.zeros(256, np.float32), np.zeros(256, np.float32)
        ref.ref_lut_gen_expmant_tables(nm.encode(), C.c_float(coeff), p(e), p(m))
        tabs[nm] = (e, m)
    out = dict(exp_base=eb, exp_slope=es, rec_exp=tabs["pow"][0], rec_mant=tabs["pow"][1], log_exp=tabs["log"][0],
               log_mant=tabs["log"][1])
    for ci, (outer, ch, inner, sd) in enumerate([(3, 21, 4, 3.0), (2, 1000, 1, 2.0), (1, 80, 9, 8.0)]):
        x = bf(rng.normal(0, sd, (outer, ch, inner)))
        out["x%d" % ci] = x
        for do_log in (0, 1):
            y = np.empty_like(x)
            for i in range(outer):
                mx = x[i].max(axis=0)
                sub = bf(x[i] - mx[None, :])
                ex = np.empty_like(sub)
                si = np.ascontiguousarray(sub)
                ref.ref_lut_bf16_slope(b"exp", p(si), p(ex), sub.size, p(eb), p(es))
                const_val = np.float32(ref.ref_bf16(float(np.float32(ref.ref_bf16(float(ch), 1)) / np.float32(ch)), 1))
                sm = np.zeros(inner, np.float32)
                for j in range(ch):
                    sm = (sm + ex[j] * const_val).astype(np.float32)
                sm = bf(sm)
                r = np.empty_like(sm)
                e, m = tabs["log" if do_log else "pow"]
                (ref.ref_lut_bf16_mantissa_log if do_log else ref.ref_lut_bf16_mantissa)(p(sm), p(r), sm.size, p(e), p(m))
                y[i] = bf(sub - r[None, :]) if do_log else bf(ex * r[None, :])
            out["y%d_log%d" % (ci, do_log)] = y
    np.savez_compressed(os.path.join(HERE, "softmax_bf16.npz"), **out)


def make_weight_quant(ref):
    """Weight quantisers and the no-weight rescale of the INT8 quantisation pass, as the reference's
    own code computes them, on seeded inputs (also run alone: make_golden.py weight_quant)."""
    rng = np.random.default_rng(20240611)
    out = {}
    cases = [(8, 27, 2.5, 1.0, 0.05), (16, 64, 0.8, 3.1, 0.3), (5, 9, 6.0, 6.0, 0.0), (12, 144, 0.02, 4.0, 2.0),
             (6, 32, 30.0, 0.1, 0.01), (4, 16, 1.0, 1.0, 1e4)]
    for ci, (oc, isz, ty, tx, bstd) in enumerate(cases):
        w = rng.normal(0, 0.2, (oc, isz)).astype(np.float32)
        w[0] *= 40.0  # a channel whose qscale passes 1
        b = rng.normal(0, bstd, oc).astype(np.float32) if bstd else None
        nf, nb = np.zeros_like(w), np.zeros(oc, np.float32)
        r, m = np.zeros(oc, np.float32), np.zeros(oc, np.float32)
        ref.ref_quantize_weight_int8_multiplier(p(w), p(b) if b is not None else None, oc, isz, C.c_float(ty),
                                                C.c_float(tx), p(nf), p(nb) if b is not None else None, p(r), p(m))
        out.update({"conv%d_w" % ci: w, "conv%d_b" % ci: b if b is not None else np.zeros(0, np.float32),
                    "conv%d_t" % ci: np.array([ty, tx], np.float32), "conv%d_nf" % ci: nf, "conv%d_nb" % ci: nb,
                    "conv%d_r" % ci: r, "conv%d_m" % ci: m})
    for ci, (n, k, ty, tx, bstd) in enumerate([(10, 64, 9.0, 4.0, 0.05), (7, 33, 0.5, 2.0, 0.0), (12, 20, 3.0, 3.0, 50.0)]):
        w = rng.normal(0, 0.1, (n, k)).astype(np.float32)
        b = rng.normal(0, bstd, n).astype(np.float32) if bstd else None
        nf, nb = np.zeros_like(w), np.zeros(n, np.float32)
        r, m = np.zeros(1, np.float32), np.zeros(1, np.float32)
        ref.ref_quantize_weight_int8_fc(p(w), p(b) if b is not None else None, n, k, C.c_float(ty), C.c_float(tx),
                                        p(nf), p(nb) if b is not None else None, p(r), p(m))
        out.update({"fc%d_w" % ci: w, "fc%d_b" % ci: b if b is not None else np.zeros(0, np.float32),
                    "fc%d_t" % ci: np.array([ty, tx], np.float32), "fc%d_nf" % ci: nf, "fc%d_nb" % ci: nb,
                    "fc%d_r" % ci: r, "fc%d_m" % ci: m})
    qs, rr, mm = [], [], []
    for _ in range(400):
        n = int(rng.integers(1, 4))
        q = np.zeros(3, np.float32)
        q[:n] = np.exp(rng.uniform(np.log(1e-4), np.log(60.0), n)).astype(np.float32)
        mult = np.zeros(3, np.float32)
        r = ref.ref_rescale_no_weight(p(q), n, p(mult))
        qs.append(q), rr.append(r), mm.append(mult)
    out.update({"rescale_qscale": np.stack(qs), "rescale_rshift": np.array(rr, np.int32), "rescale_mult": np.stack(mm)})
    np.savez_compressed(os.path.join(HERE, "weight_quant.npz"), **out)


if __name__ == "__main__":
    if len(sys.argv) > 1 and sys.argv[1] == "weight_quant":
        make_weight_quant(oracle.ref())
    else:
        main()
