"""ctypes front end of the CPU oracle (TEST INFRASTRUCTURE ONLY).

Two libraries sit behind this module:

* ``_build/libpxoracle.so`` -- ``px_oracle.c``, the C restatement of the
  reference's CPU epilogue path.  Built on demand with gcc.
* ``_ref/libpxref_cpu.so`` -- the reference's own CPU sources compiled in place
  (see ``Makefile``).  Optional: present when it was built in a container that
  has the reference checkout.

Only tests, the smoke check and the CPU-baseline leg of the benchmark may
import this module; the shipped package never does.
"""
from __future__ import annotations

import ctypes as C
import glob
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "_build", "libpxoracle.so")
REF_CPU_SO = os.path.join(HERE, "_ref", "libpxref_cpu.so")
REF_CUDA_SO = os.path.join(HERE, "_ref", "libpxref_cuda.so")

# ActivationType, include/ActivationTypes.h:19-30
ACT = {"leaky": 0, "linear": 1, "loggy": 2, "logistic": 3, "mish": 4, "relu": 5,
       "softplus": 6, "swish": 7, "tanh": 8}

DET_DTYPE = np.dtype([("x", "f4"), ("y", "f4"), ("w", "f4"), ("h", "f4"), ("prob", "f4"),
                      ("class_id", "i4"), ("batch_id", "i4"), ("source", "i4")])

_f = C.POINTER(C.c_float)
_i = C.POINTER(C.c_int)


def _fp(a):
    return a.ctypes.data_as(_f) if a is not None else None


def _ip(a):
    return a.ctypes.data_as(_i) if a is not None else None


def reference_root():
    """Root of the trieck/pixienn checkout the ref_* libraries are compiled from: $PXE_REFERENCE_ROOT, else a
    directory ``reference`` beside this repository.  None when neither exists."""
    cand = os.environ.get("PXE_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
    return cand if os.path.isdir(os.path.join(cand, "src")) else None


def build(ref: bool = True) -> None:
    """Compile the oracle (always) and the reference libraries (when the
    reference checkout is present and ``ref`` is true)."""
    subprocess.run(["make", "-s", "-C", HERE, "oracle"], check=True)
    root = reference_root()
    if ref and root:
        subprocess.run(["make", "-s", "-C", HERE, "ref_cpu", f"REF={root}"], check=True)
        subprocess.run(["make", "-s", "-C", HERE, "ref_cuda", f"REF={root}"], check=True)
        if os.path.exists(os.path.join(os.path.dirname(HERE), "pixienn_b200", "lib", "libpxe.so")):
            subprocess.run(["make", "-s", "-C", HERE, "ref_link", f"REF={root}"], check=True)


_lib = None


def lib():
    global _lib
    if _lib is None:
        src = os.path.join(HERE, "px_oracle.c")
        if not os.path.exists(ORACLE_SO) or os.path.getmtime(ORACLE_SO) < os.path.getmtime(src):
            build(ref=False)
        L = C.CDLL(ORACLE_SO)
        L.pxo_activate_one.restype = C.c_float
        L.pxo_activate_one.argtypes = [C.c_int, C.c_float]
        L.pxo_activate.argtypes = [C.c_int, _f, C.c_size_t]
        L.pxo_add_bias.argtypes = [_f, _f, C.c_int, C.c_int, C.c_int]
        L.pxo_gradient.argtypes = [C.c_int, _f, C.c_size_t, _f]
        L.pxo_backward_bias.argtypes = [_f, _f, C.c_int, C.c_int, C.c_int]
        L.pxo_adam.argtypes = [C.c_size_t, _f, _f, _f, C.c_float, C.c_float, C.c_float, C.c_float, C.c_int]
        L.pxo_softmax_cross_entropy.argtypes = [C.c_size_t, _f, _f, _f, _f]
        L.pxo_batchnorm_forward_training.argtypes = [_f, _f, C.c_int, C.c_int, C.c_int, _f, _f, _f, _f, C.c_float, C.c_float,
                                                     C.c_int, _f, _f]
        L.pxo_batchnorm_backward.argtypes = [_f, _f, _f, C.c_int, C.c_int, C.c_int, _f, _f, _f, _f, _f, C.c_float, C.c_int]
        L.pxo_maxpool_backward.argtypes = [_f, _i, _f, C.c_size_t]
        L.pxo_upsample_backward.argtypes = [_f, _f] + [C.c_int] * 5 + [C.c_float]
        L.pxo_constrain.argtypes = [_f, C.c_size_t, C.c_float]
        _d = C.POINTER(C.c_double)
        L.pxo_yolo_loss.argtypes = [_f, _f, _f, _i, C.c_int, _i, _i, _f, _i, _f, _d, _d] + [C.c_int] * 7 + [C.c_float] * 6
        L.pxo_centernet_loss.argtypes = [_f, _f, _f, _f, _f, _f, _d] + [C.c_int] * 3 + [C.c_float] * 4
        L.pxo_scale_bias.argtypes = [_f, _f, C.c_int, C.c_int, C.c_int]
        L.pxo_normalize.argtypes = [_f, _f, _f, C.c_int, C.c_int, C.c_int, C.c_float, C.c_int]
        L.pxo_conv_epilogue.argtypes = [_f, C.c_int, C.c_int, C.c_int, _f, _f, _f, _f, C.c_float,
                                        C.c_int, _f, C.c_int]
        L.pxo_maxpool_out_dim.restype = C.c_int
        L.pxo_maxpool_out_dim.argtypes = [C.c_int] * 4
        L.pxo_maxpool.argtypes = [_f, _f, _i] + [C.c_int] * 7
        L.pxo_upsample.argtypes = [_f, _f] + [C.c_int] * 5 + [C.c_float]
        L.pxo_shortcut.argtypes = [C.c_int] * 4 + [_f] + [C.c_int] * 3 + [C.c_float, C.c_float, _f]
        L.pxo_route.argtypes = [C.c_int, C.POINTER(_f), _i, C.c_int, _f]
        L.pxo_yolo_activate.argtypes = [_f, _f] + [C.c_int] * 4
        L.pxo_yolo_decode_image.argtypes = [_f, C.c_int, C.c_int, _i, _i] + [C.c_int] * 7 + [
            C.c_float, C.c_void_p, C.c_longlong, C.POINTER(C.c_longlong)]
        L.pxo_centernet_activate.argtypes = [_f, _f, C.c_int, C.c_int, C.c_int, C.c_float]
        L.pxo_detect_decode_image.argtypes = [_f] + [C.c_int] * 8 + [C.c_float, C.c_void_p, C.c_longlong, C.POINTER(C.c_longlong)]
        L.pxo_avgpool.argtypes = [_f, _f, C.c_int, C.c_int, C.c_int]
        L.pxo_centernet_decode_image.restype = C.c_int
        L.pxo_centernet_decode_image.argtypes = [_f, _f, _f] + [C.c_int] * 6 + [
            C.c_float, C.c_int, C.c_void_p, _i]
        L.pxo_softmax_one.argtypes = [_f, C.c_int, C.c_float, _f, C.c_int]
        L.pxo_softmax.argtypes = [_f] + [C.c_int] * 6 + [C.c_float, _f]
        L.pxo_softmax_detect.restype = C.c_int
        L.pxo_softmax_detect.argtypes = [_f] + [C.c_int] * 4 + [C.c_float, C.c_void_p]
        L.pxo_flatten.argtypes = [_f] + [C.c_int] * 4
        L.pxo_region_forward.argtypes = [_f, _f] + [C.c_int] * 7
        L.pxo_region_decode_image.argtypes = [_f] + [C.c_int] * 6 + [_f, C.c_int, C.c_int, C.c_float,
                                                                    C.c_void_p, C.c_longlong,
                                                                    C.POINTER(C.c_longlong)]
        L.pxo_box_iou.restype = C.c_float
        L.pxo_box_iou.argtypes = [C.c_void_p, C.c_void_p]
        L.pxo_nms.restype = C.c_longlong
        L.pxo_nms.argtypes = [C.c_void_p, C.c_longlong, C.c_float, C.c_void_p]
        L.pxo_im2col.argtypes = [_f] + [C.c_int] * 11 + [_f]
        L.pxo_conv_forward.argtypes = [C.c_void_p, _f, _f, _f, _f] + [C.c_int] * 9
        _lib = L
    return _lib


def _c(a, dtype=np.float32):
    return np.ascontiguousarray(a, dtype=dtype)


# --------------------------------------------------------------------- ops

def activate(kind, x):
    y = _c(x).copy()
    lib().pxo_activate(ACT[kind] if isinstance(kind, str) else int(kind), _fp(y), y.size)
    return y


def gradient(kind, x, delta):
    """delta * f'(x): Activation::gradient (include/Activation.h:306-316)."""
    d = _c(delta).copy()
    xx = _c(x)
    lib().pxo_gradient(ACT[kind] if isinstance(kind, str) else int(kind), _fp(xx), xx.size, _fp(d))
    return d


def backward_bias(bias_updates, delta):
    """delta: [B, n, ...]; returns bias_updates + per-filter sums (src/CpuUtil.cpp:189-196)."""
    d = _c(delta)
    out = _c(bias_updates).copy()
    B, n = d.shape[0], d.shape[1]
    lib().pxo_backward_bias(_fp(out), _fp(d), B, n, d.size // (B * n))
    return out


def batchnorm_forward_training(x, gamma, beta, running_mean, running_var, factor=0.01, eps=1e-5, eps_mode=0):
    """Returns (y, running_mean, running_var, save_mean, save_scale); see pxo_batchnorm_forward_training."""
    x = _c(x)
    B, Cc = x.shape[:2]
    y = np.empty_like(x)
    rm, rv = _c(running_mean).copy(), _c(running_var).copy()
    sm, ss = np.empty(Cc, np.float32), np.empty(Cc, np.float32)
    lib().pxo_batchnorm_forward_training(_fp(x), _fp(y), B, Cc, x.size // (B * Cc), _fp(_c(gamma)), _fp(_c(beta)), _fp(rm),
                                         _fp(rv), C.c_float(factor), C.c_float(eps), eps_mode, _fp(sm), _fp(ss))
    return y, rm, rv, sm, ss


def batchnorm_backward(x, dy, gamma, save_mean, save_scale, dgamma, dbeta, eps=1e-5, eps_mode=0):
    """Returns (dx, dgamma, dbeta); see pxo_batchnorm_backward."""
    x, dy = _c(x), _c(dy)
    B, Cc = x.shape[:2]
    dx = np.empty_like(x)
    dg, db = _c(dgamma).copy(), _c(dbeta).copy()
    lib().pxo_batchnorm_backward(_fp(x), _fp(dy), _fp(dx), B, Cc, x.size // (B * Cc), _fp(_c(gamma)), _fp(dg), _fp(db),
                                 _fp(_c(save_mean)), _fp(_c(save_scale)), C.c_float(eps), eps_mode)
    return dx, dg, db


def adam(x, m, v, beta1, beta2, rate, eps, t):
    y = _c(x).copy()
    lib().pxo_adam(y.size, _fp(y), _fp(_c(m)), _fp(_c(v)), C.c_float(beta1), C.c_float(beta2), C.c_float(rate), C.c_float(eps), t)
    return y


def softmax_cross_entropy(pred, truth):
    """Returns (delta, error)."""
    p, t = _c(pred), _c(truth)
    delta, error = np.empty_like(p), np.empty_like(p)
    lib().pxo_softmax_cross_entropy(p.size, _fp(p), _fp(t), _fp(delta), _fp(error))
    return delta, error


def maxpool_backward(delta, indexes, grad):
    g = _c(grad).copy()
    d = _c(delta)
    idx = _c(indexes, np.int32)
    lib().pxo_maxpool_backward(_fp(d), _ip(idx), _fp(g), d.size)
    return g


def upsample_backward(acc, out, stride, scale=1.0):
    """acc: [B,C,H,W] accumulated into; out: [B,C,H*stride,W*stride]."""
    a = _c(acc).copy()
    o = _c(out)
    B, Cc, H, W = a.shape
    lib().pxo_upsample_backward(_fp(a), _fp(o), B, Cc, H, W, stride, C.c_float(scale))
    return a


def constrain(x, alpha):
    y = _c(x).copy()
    lib().pxo_constrain(_fp(y), y.size, C.c_float(alpha))
    return y


def yolo_loss(output, delta, truths, truth_counts, assigned_classes, assigned_anchors, assigned_boxes, masks, anchors,
              net_w, net_h, ignore_thr=0.5, truth_thr=1.0, coord_scale=1.0, object_scale=1.0, no_object_scale=1.0,
              class_scale=1.0):
    """yoloLossGpu as the reference's kernels compute it.  output, delta: [B, masks*(5+classes), H, W];
    truths: [B, max_truth, 5].  Returns (delta, stats[12], cost) with the sums in float64."""
    out = _c(output)
    d = _c(delta).copy()
    B, ch, H, W = out.shape
    mc = len(masks)
    classes = ch // mc - 5
    t = _c(truths)
    tc, ac, aa = _c(truth_counts, np.int32), _c(assigned_classes, np.int32), _c(assigned_anchors, np.int32)
    ab, mk, an = _c(assigned_boxes), _c(masks, np.int32), _c(anchors)
    stats, cost = np.zeros(12, np.float64), np.zeros(1, np.float64)
    dp = C.POINTER(C.c_double)
    lib().pxo_yolo_loss(_fp(out), _fp(d), _fp(t), _ip(tc), t.shape[1], _ip(ac), _ip(aa), _fp(ab), _ip(mk), _fp(an),
                        stats.ctypes.data_as(dp), cost.ctypes.data_as(dp), B, mc, classes, W, H, net_w, net_h,
                        ignore_thr, truth_thr, coord_scale, object_scale, no_object_scale, class_scale)
    return d, stats, float(cost[0])


def centernet_loss(output, delta, target_heat, target_size, target_offset, target_mask, normalizer, alpha=2.0, beta=4.0,
                   size_weight=0.1):
    """centerNetLossGpu.  output, delta: [B, classes+4, H, W].  Returns (delta, costs[3] in float64)."""
    out = _c(output)
    d = _c(delta).copy()
    B, ch, H, W = out.shape
    costs = np.zeros(3, np.float64)
    lib().pxo_centernet_loss(_fp(out), _fp(d), _fp(_c(target_heat)), _fp(_c(target_size)), _fp(_c(target_offset)),
                             _fp(_c(target_mask)), costs.ctypes.data_as(C.POINTER(C.c_double)), B, ch - 4, H * W,
                             normalizer, alpha, beta, size_weight)
    return d, costs


def conv_epilogue(x, gamma=None, beta=None, mean=None, var=None, bias=None, act="linear",
                  eps=1e-5, eps_mode=0):
    """x: [B,C,H,W] conv output.  Returns act(bn(x) + bias)."""
    y = _c(x).copy()
    B, Cc = y.shape[0], y.shape[1]
    spatial = int(np.prod(y.shape[2:])) if y.ndim > 2 else 1
    if gamma is not None:
        keep = [_c(t) for t in (gamma, beta, mean, var)]
        args = [_fp(k) for k in keep]
    else:
        args = [None, None, None, None]
    bz = _c(bias) if bias is not None else None
    lib().pxo_conv_epilogue(_fp(y), B, Cc, spatial, *args, C.c_float(eps), int(eps_mode), _fp(bz),
                            ACT[act] if isinstance(act, str) else int(act))
    return y


def maxpool_out_dim(n, kernel, stride, padding):
    return lib().pxo_maxpool_out_dim(n, kernel, stride, padding)


def maxpool(x, kernel, stride, padding=None):
    """Returns (values, int32 argmax indices into the flat input)."""
    x = _c(x)
    B, Cc, H, W = x.shape
    if padding is None:
        padding = max(0, kernel - 1)          # MaxPoolLayer.h:56
    oh, ow = maxpool_out_dim(H, kernel, stride, padding), maxpool_out_dim(W, kernel, stride, padding)
    out = np.empty((B, Cc, oh, ow), np.float32)
    idx = np.empty((B, Cc, oh, ow), np.int32)
    lib().pxo_maxpool(_fp(x), _fp(out), _ip(idx), B, Cc, H, W, kernel, stride, padding)
    return out, idx


def upsample(x, stride=2, scale=1.0):
    x = _c(x)
    B, Cc, H, W = x.shape
    out = np.empty((B, Cc, H * stride, W * stride), np.float32)
    lib().pxo_upsample(_fp(x), _fp(out), B, Cc, H, W, stride, C.c_float(scale))
    return out


def shortcut(inp, frm, alpha=1.0, beta=1.0, act="linear"):
    """ShortcutLayer::forward (ShortcutLayer.h:84-96): out = act(alpha*inp + beta*from)."""
    out = _c(inp).copy()
    frm = _c(frm)
    B, c2, h2, w2 = out.shape
    _, c1, h1, w1 = frm.shape
    # the layer passes its own input dims as (w1,h1,c1) for `from` (ShortcutLayer.h:90-91)
    lib().pxo_shortcut(B, w2, h2, c2, _fp(frm), w2, h2, c2, C.c_float(alpha), C.c_float(beta), _fp(out))
    return activate(act, out)


def shortcut_raw(batch, w1, h1, c1, add, w2, h2, c2, s1, s2, out):
    out = _c(out).copy()
    add = _c(add)
    lib().pxo_shortcut(batch, w1, h1, c1, _fp(add), w2, h2, c2, C.c_float(s1), C.c_float(s2), _fp(out))
    return out


def route(srcs):
    srcs = [_c(s) for s in srcs]
    B = srcs[0].shape[0]
    outs = np.array([int(np.prod(s.shape[1:])) for s in srcs], np.int32)
    ptrs = (_f * len(srcs))(*[_fp(s) for s in srcs])
    ch = sum(s.shape[1] for s in srcs)
    out = np.empty((B, ch) + srcs[0].shape[2:], np.float32)
    lib().pxo_route(len(srcs), ptrs, _ip(outs), B, _fp(out))
    return out


def yolo_activate(x, masks, classes):
    x = _c(x)
    B = x.shape[0]
    area = x.shape[2] * x.shape[3]
    out = np.empty_like(x)
    lib().pxo_yolo_activate(_fp(x), _fp(out), B, masks, classes, area)
    return out


def yolo_decode(pred, mask, anchors, classes, net_w, net_h, thr, img_w=0, img_h=0, cap=None):
    """All images of one activated head [B, masks*(5+classes), H, W] -> detections."""
    pred = _c(pred)
    B, _, lh, lw = pred.shape
    mask = _c(mask, np.int32)
    anchors = _c(anchors, np.int32)
    if cap is None:
        cap = B * lh * lw * len(mask) * classes
    dets = np.zeros(cap, DET_DTYPE)
    count = C.c_longlong(0)
    for b in range(B):
        lib().pxo_yolo_decode_image(_fp(pred), b, len(mask), _ip(mask), _ip(anchors), classes, lw, lh,
                                    net_w, net_h, img_w, img_h, C.c_float(thr),
                                    dets.ctypes.data, cap, C.byref(count))
    return dets[:min(count.value, cap)].copy(), count.value


def detect_decode(pred, side, num, classes, thr, coords=4, squared=False, width=1, height=1, cap=None):
    """YOLOv1 detection head: pred [B, side*side*(classes + num*(1+coords))] -> (detections, count)."""
    pred = _c(pred)
    B = pred.shape[0]
    per = pred.size // B
    if cap is None:
        cap = B * side * side * num
    dets = np.zeros(cap, DET_DTYPE)
    count = C.c_longlong(0)
    flat = pred.reshape(B, per)
    for b in range(B):
        row = np.ascontiguousarray(flat[b])
        lib().pxo_detect_decode_image(_fp(row), b, side, num, classes, coords, int(squared), int(width), int(height),
                                      C.c_float(thr), dets.ctypes.data, cap, C.byref(count))
    return dets[:min(count.value, cap)].copy(), count.value


def avgpool(x):
    x = _c(x)
    B, Cc, H, W = x.shape
    out = np.empty((B, Cc, 1, 1), np.float32)
    lib().pxo_avgpool(_fp(x), _fp(out), B, Cc, H * W)
    return out


def centernet_activate(x, classes, heatmap_bias):
    x = _c(x)
    B = x.shape[0]
    area = x.shape[2] * x.shape[3]
    out = np.empty_like(x)
    lib().pxo_centernet_activate(_fp(x), _fp(out), B, classes, area, C.c_float(heatmap_bias))
    return out


def centernet_decode(heat, size, off, thr, max_det, img_w=0, img_h=0):
    """heat [B,classes,H,W] already activated; size/off [B,2,H,W].  Returns a list of per-image
    detection arrays and the per-image candidate counts."""
    heat, size, off = _c(heat), _c(size), _c(off)
    B, classes, h, w = heat.shape
    out, ncand = [], []
    for b in range(B):
        d = np.zeros(max_det, DET_DTYPE)
        n = C.c_int(0)
        k = lib().pxo_centernet_decode_image(_fp(heat[b]), _fp(size[b]), _fp(off[b]), b, classes, w, h,
                                             img_w, img_h, C.c_float(thr), max_det, d.ctypes.data,
                                             C.byref(n))
        out.append(d[:k].copy())
        ncand.append(n.value)
    return out, ncand


def softmax(x, groups=1, temperature=1.0):
    """SoftmaxLayer::forward (SoftmaxLayer.h:86-99) over the flattened per-image inputs."""
    x = _c(x)
    B = x.shape[0]
    inputs = int(np.prod(x.shape[1:]))
    out = np.empty_like(x)
    lib().pxo_softmax(_fp(x), inputs // groups, B, inputs, groups, inputs // groups, 1,
                      C.c_float(temperature), _fp(out))
    return out


def softmax_one(x, temp=1.0):
    x = _c(x)
    out = np.empty_like(x)
    lib().pxo_softmax_one(_fp(x), x.size, C.c_float(temp), _fp(out), 1)
    return out


def region_forward(x, num, coords, classes, use_softmax=True):
    x = _c(x)
    B, _, h, w = x.shape
    out = np.empty_like(x)
    lib().pxo_region_forward(_fp(x), _fp(out), B, w, h, num, coords, classes, int(use_softmax))
    return out


def region_decode(pred, w, h, num, coords, classes, biases, thr, img_w=1, img_h=1):
    pred = _c(pred)
    B = pred.shape[0]
    biases = _c(biases)
    cap = B * w * h * num * classes
    dets = np.zeros(cap, DET_DTYPE)
    count = C.c_longlong(0)
    for b in range(B):
        lib().pxo_region_decode_image(_fp(pred), b, w, h, num, coords, classes, _fp(biases), img_w, img_h,
                                      C.c_float(thr), dets.ctypes.data, cap, C.byref(count))
    return dets[:count.value].copy()


def nms(dets, threshold):
    dets = np.ascontiguousarray(dets, DET_DTYPE)
    out = np.zeros(len(dets), DET_DTYPE)
    n = lib().pxo_nms(dets.ctypes.data, len(dets), C.c_float(threshold), out.ctypes.data)
    return out[:n].copy()


def box_iou(a, b):
    a = np.ascontiguousarray(a, DET_DTYPE)
    b = np.ascontiguousarray(b, DET_DTYPE)
    return lib().pxo_box_iou(a.ctypes.data, b.ctypes.data)


def make_det(x, y, w, h, batch, cls, prob, source=0):
    d = np.zeros(1, DET_DTYPE)
    d[0] = (x, y, w, h, prob, cls, batch, source)
    return d


# --------------------------------------------------- reference CPU library

class RefCpu:
    """The reference's own CPU code (``_ref/libpxref_cpu.so``)."""

    def __init__(self):
        if not os.path.exists(REF_CPU_SO):
            raise FileNotFoundError(REF_CPU_SO)
        L = C.CDLL(REF_CPU_SO)
        import scipy
        pat = os.path.join(os.path.dirname(os.path.dirname(scipy.__file__)), "scipy.libs",
                           "libscipy_openblas*.so")
        cands = sorted(glob.glob(pat))
        if not cands:
            raise FileNotFoundError(pat)
        L.pxref_blas_init.argtypes = [C.c_char_p]
        if L.pxref_blas_init(cands[0].encode()) != 0:
            raise OSError("pxref_blas_init failed")
        L.pxref_blas_set_threads.restype = C.c_int
        L.pxref_blas_set_threads.argtypes = [C.c_int]
        L.pxref_blas_sgemm_ptr.restype = C.c_void_p
        L.pxref_activate.argtypes = [C.c_int, _f, C.c_size_t]
        L.pxref_add_bias.argtypes = [_f, _f, C.c_int, C.c_int, C.c_int]
        L.pxref_gradient.argtypes = [C.c_int, _f, C.c_size_t, _f]
        L.pxref_backward_bias.argtypes = [_f, _f, C.c_int, C.c_int, C.c_int]
        L.pxref_constrain.argtypes = [C.c_int, C.c_float, _f]
        L.pxref_scale_bias.argtypes = [_f, _f, C.c_int, C.c_int, C.c_int]
        L.pxref_normalize.argtypes = [_f, _f, _f, C.c_int, C.c_int, C.c_int]
        L.pxref_batchnorm_inference.argtypes = [_f, _f, _f, _f, _f, C.c_int, C.c_int, C.c_int]
        L.pxref_batchnorm_forward_vec.argtypes = [_f, _f, _f, _f, _f] + [C.c_int] * 4
        L.pxref_batchnorm_forward_training.argtypes = [_f] * 8 + [C.c_int] * 4
        L.pxref_batchnorm_backward.argtypes = [_f] * 8 + [C.c_int] * 4
        L.pxref_softmax_one.argtypes = [_f, C.c_int, C.c_float, _f, C.c_int]
        L.pxref_softmax.argtypes = [_f] + [C.c_int] * 6 + [C.c_float, _f]
        L.pxref_sigmoid.restype = C.c_float
        L.pxref_sigmoid.argtypes = [C.c_float]
        L.pxref_flatten.argtypes = [_f] + [C.c_int] * 4
        L.pxref_im2col.argtypes = [_f] + [C.c_int] * 11 + [_f]
        L.pxref_conv_forward.argtypes = [_f, _f, _f, _f] + [C.c_int] * 9
        self.L = L

    def set_threads(self, n):
        return self.L.pxref_blas_set_threads(int(n))

    def sgemm_ptr(self):
        return self.L.pxref_blas_sgemm_ptr()

    def activate(self, kind, x):
        y = _c(x).copy()
        rc = self.L.pxref_activate(ACT[kind] if isinstance(kind, str) else int(kind), _fp(y), y.size)
        assert rc == 0
        return y

    def activate_inplace(self, kind, y):
        self.L.pxref_activate(ACT[kind], _fp(y), y.size)

    def gradient(self, kind, x, delta):
        d = _c(delta).copy()
        xx = _c(x)
        rc = self.L.pxref_gradient(ACT[kind] if isinstance(kind, str) else int(kind), _fp(xx), xx.size, _fp(d))
        assert rc == 0
        return d

    def backward_bias(self, bias_updates, delta):
        d = _c(delta)
        out = _c(bias_updates).copy()
        B, n = d.shape[0], d.shape[1]
        self.L.pxref_backward_bias(_fp(out), _fp(d), B, n, d.size // (B * n))
        return out

    def constrain(self, x, alpha):
        y = _c(x).copy()
        self.L.pxref_constrain(y.size, C.c_float(alpha), _fp(y))
        return y

    def batchnorm_forward_training(self, x, gamma, beta, rolling_mean, rolling_var):
        """batchNormForward(training = true): returns (y, mean, var, rolling_mean, rolling_var, xnorm)."""
        y = _c(x).copy()
        B, Cc, H, W = y.shape
        m, v = np.empty(Cc, np.float32), np.empty(Cc, np.float32)
        rm, rv = _c(rolling_mean).copy(), _c(rolling_var).copy()
        xn = np.empty_like(y)
        self.L.pxref_batchnorm_forward_training(_fp(y), _fp(_c(gamma)), _fp(_c(beta)), _fp(m), _fp(v), _fp(rm), _fp(rv),
                                                _fp(xn), B, Cc, H, W)
        return y, m, v, rm, rv, xn

    def batchnorm_backward(self, delta, x, xnorm, mean, var, gamma, scale_updates, bias_updates):
        """batchNormBackward: returns (dx, scale_updates, bias_updates)."""
        d = _c(delta).copy()
        B, Cc, H, W = d.shape
        su, bu = _c(scale_updates).copy(), _c(bias_updates).copy()
        self.L.pxref_batchnorm_backward(_fp(d), _fp(_c(x)), _fp(_c(xnorm)), _fp(_c(mean)), _fp(_c(var)), _fp(_c(gamma)),
                                        _fp(su), _fp(bu), B, Cc, H, W)
        return d, su, bu

    def batchnorm_inference(self, x, gamma, beta, mean, var, via_vector=False):
        y = _c(x).copy()
        B, Cc = y.shape[:2]
        H, W = (y.shape[2], y.shape[3]) if y.ndim == 4 else (1, 1)
        g, b, m, v = (_c(t) for t in (gamma, beta, mean, var))
        if via_vector:
            self.L.pxref_batchnorm_forward_vec(_fp(y), _fp(g), _fp(b), _fp(m), _fp(v), B, Cc, H, W)
        else:
            self.L.pxref_batchnorm_inference(_fp(y), _fp(g), _fp(b), _fp(m), _fp(v), B, Cc, H * W)
        return y

    def batchnorm_inference_inplace(self, y, g, b, m, v):
        B, Cc = y.shape[:2]
        self.L.pxref_batchnorm_inference(_fp(y), _fp(g), _fp(b), _fp(m), _fp(v), B, Cc,
                                         int(np.prod(y.shape[2:])))

    def add_bias(self, x, bias):
        y = _c(x).copy()
        B, Cc = y.shape[:2]
        bz = _c(bias)
        self.L.pxref_add_bias(_fp(y), _fp(bz), B, Cc, int(np.prod(y.shape[2:])))
        return y

    def add_bias_inplace(self, y, bz):
        B, Cc = y.shape[:2]
        self.L.pxref_add_bias(_fp(y), _fp(bz), B, Cc, int(np.prod(y.shape[2:])))

    def scale_bias(self, x, scales):
        y = _c(x).copy()
        B, Cc = y.shape[:2]
        s = _c(scales)
        self.L.pxref_scale_bias(_fp(y), _fp(s), B, Cc, int(np.prod(y.shape[2:])))
        return y

    def softmax_one(self, x, temp=1.0):
        x = _c(x)
        out = np.empty_like(x)
        self.L.pxref_softmax_one(_fp(x), x.size, C.c_float(temp), _fp(out), 1)
        return out

    def sigmoid(self, v):
        return self.L.pxref_sigmoid(C.c_float(v))

    def flatten(self, x, size, layers, batch, forward=True):
        y = _c(x).copy()
        self.L.pxref_flatten(_fp(y), size, layers, batch, int(forward))
        return y

    def conv_forward(self, x, weights, filters, kernel, stride, pad, dilation=1):
        x = _c(x)
        w = _c(weights)
        B, Cc, H, W = x.shape
        eff = dilation * (kernel - 1) + 1
        oh = (H + 2 * pad - eff) // stride + 1
        ow = (W + 2 * pad - eff) // stride + 1
        out = np.empty((B, filters, oh, ow), np.float32)
        col = np.empty(Cc * kernel * kernel * oh * ow, np.float32)
        self.L.pxref_conv_forward(_fp(x), _fp(w), _fp(out), _fp(col), B, Cc, H, W, filters, kernel,
                                  stride, pad, dilation)
        return out


_ref_cpu = None


def ref_cpu():
    """The loaded reference CPU library, or None when it was not built."""
    global _ref_cpu
    if _ref_cpu is None and os.path.exists(REF_CPU_SO):
        _ref_cpu = RefCpu()
    return _ref_cpu


def conv_forward(x, weights, filters, kernel, stride, pad, dilation=1):
    """CPU convolution by im2col + sgemm.  Uses the reference's compiled code when present,
    otherwise the restated im2col with numpy's BLAS."""
    r = ref_cpu()
    if r is not None:
        return r.conv_forward(x, weights, filters, kernel, stride, pad, dilation)
    x = _c(x)
    B, Cc, H, W = x.shape
    eff = dilation * (kernel - 1) + 1
    oh = (H + 2 * pad - eff) // stride + 1
    ow = (W + 2 * pad - eff) // stride + 1
    out = np.empty((B, filters, oh, ow), np.float32)
    col = np.empty((Cc * kernel * kernel, oh * ow), np.float32)
    wm = _c(weights).reshape(filters, -1)
    for b in range(B):
        lib().pxo_im2col(_fp(x[b]), Cc, H, W, kernel, kernel, pad, pad, stride, stride, dilation,
                         dilation, _fp(col))
        out[b] = (wm @ col).reshape(filters, oh, ow)
    return out


# -------------------------------------------------- reference CUDA library

class RefCuda:
    """The reference's own CUDA epilogue kernels compiled for sm_100a (``_ref/libpxref_cuda.so``).
    Arguments are raw device pointers (``tensor.data_ptr()``); everything runs on the legacy
    default stream, as in the reference."""

    def __init__(self, path=None):
        path = path or REF_CUDA_SO
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        L = C.CDLL(path)
        vp, i, f, sz = C.c_void_p, C.c_int, C.c_float, C.c_size_t
        protos = {
            "pxrefcu_activate": [i, vp, sz],
            "pxrefcu_add_bias": [vp, vp, i, i, i],
            "pxrefcu_maxpool": [vp, vp, vp] + [i] * 9,
            "pxrefcu_upsample": [vp, i, i, i, i, i, f, vp],
            "pxrefcu_shortcut": [i, i, i, i, vp, i, i, i, f, f, vp],
            "pxrefcu_yolo_activate": [vp, vp, i, i, i, i],
            "pxrefcu_centernet_activate": [vp, vp, i, i, i, f],
            "pxrefcu_fill": [vp, sz, f],
            "pxrefcu_batchnorm_inference": [vp, vp, vp, vp, vp, i, i, i, i],
            "pxrefcu_conv_epilogue_replay": [vp, vp, vp, vp, i, i, i, i, vp, vp, vp, vp, vp, i],
            "pxrefcu_maxpool_replay": [vp, vp, vp, vp] + [i] * 9,
            "pxrefcu_upsample_replay": [vp, vp, vp, i, i, i, i, i, f],
            "pxrefcu_shortcut_replay": [vp, vp, vp, vp, i, i, i, i, f, f, i],
            "pxrefcu_route_replay": [i, C.POINTER(vp), _i, vp, vp, i],
            "pxrefcu_yolo_replay": [vp, vp, vp, vp, i, i, i, i],
            "pxrefcu_gradient": [i, vp, sz, vp],
            "pxrefcu_backward_bias": [vp, vp, i, i, i],
            "pxrefcu_maxpool_backward": [vp, vp, vp, i],
            "pxrefcu_upsample_backward": [i, i, i, i, i, f, vp, vp],
            "pxrefcu_constrain": [i, f, vp],
            "pxrefcu_mul": [i, vp, vp],
            "pxrefcu_adam": [i, vp, vp, vp, f, f, f, f, i],
            "pxrefcu_random": [vp, sz, f, f],
            "pxrefcu_random_normal": [vp, sz, f, f],
            "pxrefcu_yolo_loss": [vp] * 12 + [i] * 9 + [f] * 6,
            "pxrefcu_centernet_loss": [vp] * 7 + [i] * 3 + [f] * 4,
        }
        L.pxrefcu_gridsize.argtypes = [C.c_uint, C.POINTER(C.c_uint)]
        L.pxrefcu_gridsize.restype = None
        for name, args in protos.items():
            fn = getattr(L, name)
            fn.argtypes = args
            fn.restype = C.c_int
        self.L = L

    def call(self, name, *args):
        rc = getattr(self.L, "pxrefcu_" + name)(*args)
        if rc != 0:
            raise RuntimeError(f"reference CUDA call {name} failed with {rc}")


_ref_cuda = None


def ref_cuda():
    """The loaded reference CUDA library, or None when it was not built."""
    global _ref_cuda
    if _ref_cuda is None and os.path.exists(REF_CUDA_SO):
        _ref_cuda = RefCuda()
    return _ref_cuda


REF_LINK_SO = os.path.join(HERE, "_ref", "libpxref_cuda_on_pxe.so")
_ref_link = None


def ref_cuda_on_pxe():
    """The same glue (the reference's call sequences, compiled against the reference's headers) linked against
    libpxe.so instead of the reference's .cu files: the link-compatible tier in use.  None when not built."""
    global _ref_link
    if _ref_link is None and os.path.exists(REF_LINK_SO):
        _ref_link = RefCuda(REF_LINK_SO)
    return _ref_link
