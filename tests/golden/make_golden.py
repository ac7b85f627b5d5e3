"""Generates tests/golden/reference_cpu.npz from the reference's OWN compiled CPU code
(oracle/_ref/libpxref_cpu.so, built by `make -C oracle ref_cpu` where a checkout of trieck/pixienn is
present).  Inputs are seeded; outputs are whatever the reference computes.  The fixtures let the C
restatement be pinned bit for bit on machines that have no checkout of the reference.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import pxoracle as po  # noqa: E402
from pixienn_b200 import synth  # noqa: E402

ACTS = ["leaky", "linear", "loggy", "logistic", "mish", "relu", "softplus", "swish", "tanh"]


def main():
    ref = po.ref_cpu()
    if ref is None:
        raise SystemExit("oracle/_ref/libpxref_cpu.so is missing: run `make -C oracle ref_cpu` first")
    out = {}
    x = np.concatenate([synth.normal(11, "golden/act", 3000, 0, 7), np.linspace(-24, 24, 1501, dtype=np.float32),
                        np.array([0, -0.0, 1, -2, 3, -4, 20, -20, 20.5, -20.5, 1e-40, 88, -88, 90, -104], np.float32)])
    out["act_x"] = x
    for a in ACTS:
        out[f"act_{a}"] = ref.activate(a, x)
    bx = synth.normal(12, "golden/bn_x", (2, 6, 5, 7), 0, 2)
    g, b, m, v = synth.bn_params(12, "golden/bn", 6)
    out.update(bn_x=bx, bn_gamma=g, bn_beta=b, bn_mean=m, bn_var=v, bn_y=ref.batchnorm_inference(bx, g, b, m, v))
    bias = synth.normal(13, "golden/bias", 6)
    out.update(bias=bias, bias_y=ref.add_bias(bx, bias), scale_y=ref.scale_bias(bx, bias))
    sv = synth.normal(14, "golden/softmax", 37, 0, 4)
    out.update(softmax_x=sv, softmax_t1=ref.softmax_one(sv, 1.0), softmax_t05=ref.softmax_one(sv, 0.5))
    fl = synth.normal(15, "golden/flatten", 2 * 5 * 12)
    out.update(flatten_x=fl, flatten_y=ref.flatten(fl, 12, 5, 2, True))
    img = synth.uniform(16, "golden/img", (1, 3, 7, 9))
    w = synth.normal(16, "golden/w", (4, 3, 3, 3), 0, 0.3)
    col = np.empty(3 * 3 * 3 * 4 * 5, np.float32)
    ref.L.pxref_im2col(img[0].ctypes.data_as(po._f), 3, 7, 9, 3, 3, 1, 1, 2, 2, 1, 1, col.ctypes.data_as(po._f))
    out.update(conv_img=img, conv_w=w, im2col_k3_s2_p1=col, conv_y=ref.conv_forward(img, w, 4, 3, 2, 1))
    # the training side: activation gradients, bias gradient, clip, batch norm with batch statistics both ways
    gd = synth.normal(17, "golden/grad_delta", len(x), 0, 3)
    out["grad_delta"] = gd
    for a in ACTS:
        out[f"grad_{a}"] = ref.gradient(a, x, gd)
    bd = synth.normal(18, "golden/bias_delta", (3, 5, 4, 6), 0, 2)
    bs = synth.normal(18, "golden/bias_start", 5)
    out.update(bias_delta=bd, bias_start=bs, bias_updates=ref.backward_bias(bs, bd), constrain_y=ref.constrain(gd, 2.5))
    tx = synth.normal(19, "golden/bnt_x", (3, 5, 7, 9), 0.7, 2.0)
    tg, tb, trm, trv = synth.bn_params(19, "golden/bnt", 5)
    ty, tm, tv, trm2, trv2, txn = ref.batchnorm_forward_training(tx, tg, tb, trm, trv)
    tdy = synth.normal(20, "golden/bnt_dy", tx.shape, 0, 1.5)
    su0, bu0 = synth.normal(20, "golden/bnt_su", 5), synth.normal(20, "golden/bnt_bu", 5)
    tdx, tsu, tbu = ref.batchnorm_backward(tdy, tx, txn, tm, tv, tg, su0, bu0)
    out.update(bnt_x=tx, bnt_gamma=tg, bnt_beta=tb, bnt_rm=trm, bnt_rv=trv, bnt_y=ty, bnt_mean=tm, bnt_var=tv,
               bnt_rm_out=trm2, bnt_rv_out=trv2, bnt_dy=tdy, bnt_su0=su0, bnt_bu0=bu0, bnt_dx=tdx, bnt_su=tsu, bnt_bu=tbu)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_cpu.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
