"""CPU forward of a PixieNN model graph, layer by layer, the way the reference's CPU path runs it
(TEST INFRASTRUCTURE / CPU BASELINE ONLY -- never imported by the shipped package).

``Model<CPU>::forward`` (include/Model.h:1740-1759) calls each layer in index order with the
previous layer's output; this walker does the same over the YAML layer list:

  conv       im2ColCpuExt + cblas_sgemm per image, then batchNormForward (CPU epsilon form) or
             addBias, then the activation                      include/ConvLayer.h:195-237
  maxpool    include/MaxPoolLayer.h:88-135          upsample   include/UpsampleLayer.h:97-121
  shortcut   include/ShortcutLayer.h:84-96          route      include/RouteLayer.h:91-113
  yolo       include/YoloLayer.h:164-196, 659-698   centernet  include/CenterNetLayer.h:85-110, 196-247
  region     include/RegionLayer.h:271-300          softmax    include/SoftmaxLayer.h:86-99

Where oracle/_ref/libpxref_cpu.so exists, convolution, batch norm, bias and activation run in the
reference's own compiled code (CpuUtil.cpp, BatchNorm.cpp, Activation.h); the remaining layer loops
are the restatements in px_oracle.c.
"""
from __future__ import annotations

import numpy as np

from . import pxoracle as po


class CpuModel:
    def __init__(self, doc: dict, weights: dict, height=None, width=None, eps_mode: int = 1,
                 use_reference_lib: bool = True, keep_outputs: bool = True):
        m = doc.get("model", doc)
        self.layers = list(m["layers"])
        self.channels = int(m["channels"])
        self.height = int(height or m["height"])
        self.width = int(width or m["width"])
        self.weights = weights
        self.eps_mode = eps_mode
        self.ref = po.ref_cpu() if use_reference_lib else None
        self.keep_outputs = keep_outputs
        self.outputs = []
        self.raw_conv = {}          # layer -> conv output before BN/bias/activation (when keep_outputs)

    # -------------------------------------------------------------- layers
    def _conv(self, i, ld, x):
        w = self.weights[i]
        k = int(ld.get("kernel", 1))
        dil = int(ld.get("dilation", 1))
        eff = dil * (k - 1) + 1
        pad = eff // 2 if ld.get("pad", False) else 0
        stride = int(ld.get("stride", 1))
        filters = int(ld.get("filters", 1))
        act = ld.get("activation", "logistic")
        out = po.conv_forward(x, w["weights"], filters, k, stride, pad, dil)
        if self.keep_outputs:
            self.raw_conv[i] = out.copy()
        if ld.get("batch_normalize", False):
            if self.ref is not None and self.eps_mode == 1:
                self.ref.batchnorm_inference_inplace(out, w["scales"], w["biases"], w["rolling_mean"], w["rolling_var"])
                self.ref.activate_inplace(act, out)
                return out
            return po.conv_epilogue(out, w["scales"], w["biases"], w["rolling_mean"], w["rolling_var"], None, act,
                                    1e-5, self.eps_mode)
        if self.ref is not None:
            self.ref.add_bias_inplace(out, w["biases"])
            self.ref.activate_inplace(act, out)
            return out
        return po.conv_epilogue(out, bias=w["biases"], act=act)

    def forward(self, x: np.ndarray):
        """x: [B, C, H, W] float32.  Returns the list of layer outputs (None where released)."""
        outs = []
        cur = np.ascontiguousarray(x, np.float32)
        n = len(self.layers)
        # last reader of each layer's output, to release memory when outputs are not kept
        last = {}
        for i, ld in enumerate(self.layers):
            srcs = [i - 1]
            if ld["type"] == "route":
                srcs = [(s if s >= 0 else i + s) for s in ld["layers"]]
            elif ld["type"] == "shortcut":
                f = int(ld["from"])
                srcs = [i - 1, f if f >= 0 else i + f]
            for s in srcs:
                last[s] = i
        for i, ld in enumerate(self.layers):
            t = ld["type"]
            if t == "conv":
                cur = self._conv(i, ld, cur)
            elif t == "maxpool":
                k = int(ld.get("kernel", 1))
                cur = po.maxpool(cur, k, int(ld.get("stride", 1)), ld.get("padding"))[0]
            elif t == "upsample":
                cur = po.upsample(cur, int(ld.get("stride", 2)), float(ld.get("scale", 1.0)))
            elif t == "route":
                srcs = [(s if s >= 0 else i + s) for s in ld["layers"]]
                cur = po.route([outs[s] for s in srcs])
            elif t == "shortcut":
                f = int(ld["from"])
                f = f if f >= 0 else i + f
                cur = po.shortcut(cur, outs[f], float(ld.get("alpha", 1.0)), float(ld.get("beta", 1.0)),
                                  ld.get("activation", "linear"))
            elif t == "yolo":
                masks = len(ld["mask"])
                cur = po.yolo_activate(cur, masks, cur.shape[1] // masks - 5)
            elif t == "centernet":
                cur = po.centernet_activate(cur, cur.shape[1] - 4, float(ld.get("heatmap_bias", -2.19)))
            elif t == "region":
                cur = po.region_forward(cur, int(ld.get("num", 1)), int(ld.get("coords", 4)),
                                        int(ld.get("classes", 20)), bool(ld.get("softmax", False)))
            elif t == "softmax":
                cur = po.softmax(cur, max(1, int(ld.get("groups", 1))), float(ld.get("temperature", 1.0)))
            elif t == "avgpool":
                cur = cur.mean(axis=(2, 3), keepdims=True).astype(np.float32)
            elif t == "dropout":
                pass
            else:
                raise NotImplementedError(t)
            outs.append(cur)
            if not self.keep_outputs:
                for s in [j for j, e in last.items() if e == i and j >= 0]:
                    if self.layers[s]["type"] not in ("yolo", "centernet", "region", "softmax"):
                        outs[s] = None
        self.outputs = outs
        return outs

    def detections(self, threshold: float):
        """Model::detections(confidence) (include/Model.h:1083-1094): detector layers in layer order,
        unscaled (normalised) boxes."""
        parts = []
        for i, ld in enumerate(self.layers):
            t = ld["type"]
            if t == "yolo":
                o = self.outputs[i]
                masks = len(ld["mask"])
                d, _ = po.yolo_decode(o, ld["mask"], ld["anchors"], o.shape[1] // masks - 5, self.width, self.height,
                                      threshold)
                parts.append(d)
            elif t == "centernet":
                o = self.outputs[i]
                cls = o.shape[1] - 4
                d, _ = po.centernet_decode(np.ascontiguousarray(o[:, :cls]), np.ascontiguousarray(o[:, cls:cls + 2]),
                                           np.ascontiguousarray(o[:, cls + 2:]), threshold,
                                           int(ld.get("max_detections", 100)))
                parts.extend(d)
        return np.concatenate(parts) if parts else np.zeros(0, po.DET_DTYPE)
