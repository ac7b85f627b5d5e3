"""Runs a planned PixieNN graph on one GPU: convolutions on cuDNN (through torch, as the reference
keeps them on its cuDNN call), everything between them on the kernels of ``libpxe.so``.

This is the host-side mirror of ``Model<Device::CUDA>::forward`` + ``Model::detections``
(include/Model.h:1740-1759, 1062-1109): layers in index order on one stream, detections gathered
from the detector layers in layer order.  Unlike the reference it holds no per-layer output /
delta / preActivation buffers: tensors live from their producer to their last reader.
"""
from __future__ import annotations

import functools
import math
from typing import Dict, List, Optional

import numpy as np
import torch
import torch.nn.functional as F

from . import graph, ops, synth


def synth_weights(model: graph.Model, seed: int = 1234, head_bias: float = 0.0, head_gain=1.0,
                  class_bias: float = 0.0) -> Dict[int, Dict[str, np.ndarray]]:
    """Seeded random-init weights: conv N(0, sqrt(2/fan_in)) with fan_in = k*k*C_in/groups
    (include/ConvLayer.h:111-115); BN gamma U(0.5,1.5), beta N(0,0.1), running mean N(0,0.1),
    running var U(0.5,1.5); non-BN conv bias 0.  ``head_bias`` is added to the objectness bias of
    convolutions feeding a YOLO layer (0 keeps the plain init), ``class_bias`` to their class biases, and
    ``head_gain`` (a number, or {conv layer index: number}) multiplies those convolutions' weights: with the
    plain init a deep residual graph feeds its heads logits of magnitude 1e6 (every box either certain or
    absent), so tests that want a realistic candidate count scale the head back to logits of order one."""
    out: Dict[int, Dict[str, np.ndarray]] = {}
    for l in model.layers:
        if l.type in ("connected", "conn"):
            # ConnLayer: weights [outputs, inputs] (row-major, include/ConnLayer.h:184-191), same init rule
            inputs = l.in_shape[0] * l.in_shape[1] * l.in_shape[2]
            d = {"weights": synth.normal(seed, f"L{l.index}/w", (l.filters, inputs), 0.0, math.sqrt(2.0 / inputs))}
            if l.batch_norm:
                g, b, m, v = synth.bn_params(seed, f"L{l.index}/bn", l.filters)
                d.update(scales=g, biases=b, rolling_mean=m, rolling_var=v)
            else:
                d["biases"] = synth.normal(seed, f"L{l.index}/b", l.filters, 0.0, 0.1)
            out[l.index] = d
            continue
        if l.type != "conv":
            continue
        cin = l.in_shape[0]
        fan_in = l.kernel * l.kernel * cin // l.groups
        w = synth.normal(seed, f"L{l.index}/w", (l.filters, cin // l.groups, l.kernel, l.kernel), 0.0,
                         math.sqrt(2.0 / fan_in))
        d = {"weights": w}
        if l.batch_norm:
            g, b, m, v = synth.bn_params(seed, f"L{l.index}/bn", l.filters)
            d.update(scales=g, biases=b, rolling_mean=m, rolling_var=v)
        else:
            bias = np.zeros(l.filters, np.float32)
            nxt = model.layers[l.index + 1] if l.index + 1 < len(model.layers) else None
            if nxt is not None and nxt.type == "yolo":
                entries = l.filters // len(nxt.params["mask"])
                if class_bias != 0.0:
                    for e in range(5, entries):
                        bias[e::entries] = class_bias
                if head_bias != 0.0:
                    bias[4::entries] = head_bias
                g = head_gain.get(l.index, 1.0) if isinstance(head_gain, dict) else head_gain
                if g != 1.0:
                    d["weights"] = (w * np.float32(g)).astype(np.float32)
            d["biases"] = bias
        out[l.index] = d
    return out


def _on_own_device(method):
    """Runs a method with the object's device current: the library launches on the current device and stream,
    whatever device the tensors live on."""
    @functools.wraps(method)
    def wrapper(self, *args, **kwargs):
        with torch.cuda.device(self._device_of()):
            return method(self, *args, **kwargs)
    return wrapper


class OpTimer:
    """Collects CUDA-event pairs around launches; resolved after a synchronise."""

    def __init__(self):
        self.records = []          # (kind, algorithmic bytes, start event, end event)
        self.enabled = False

    def begin(self):
        if not self.enabled:
            return None
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        return e

    def end(self, start, kind: str, nbytes: int):
        if start is None:
            return
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        self.records.append((kind, nbytes, start, e))

    def summary(self) -> Dict[str, Dict[str, float]]:
        out: Dict[str, Dict[str, float]] = {}
        for kind, nbytes, s, e in self.records:
            d = out.setdefault(kind, {"launches": 0, "ms": 0.0, "bytes": 0})
            d["launches"] += 1
            d["ms"] += s.elapsed_time(e)
            d["bytes"] += nbytes
        return out

    def clear(self):
        self.records = []


_HEAD_OPS = ("yolo", "centernet", "softmax", "region", "avgpool", "connected", "detection", "dropout")


class Runner:
    def __init__(self, model: graph.Model, weights: Dict[int, Dict[str, np.ndarray]], batch: int, device,
                 fuse: bool = True, raw_heads: bool = True, det_capacity: int = 1 << 20,
                 threshold: float = 0.2, batch_id_offset: int = 0, eps_mode: int = 0, layout: str = "nchw",
                 fused_stem: bool = False, conv_fusion: bool = False):
        if layout not in ("nchw", "nhwc"):
            raise ValueError("layout must be 'nchw' (the reference's) or 'nhwc' (channels-last)")
        device = torch.device(device)
        if device.type != "cuda":
            raise ValueError(f"Runner needs a CUDA device, got {device}")
        if device.index is None:
            device = torch.device("cuda", torch.cuda.current_device())
        self.model, self.batch, self.device = model, batch, device
        self._setup(weights, fuse, raw_heads, det_capacity, threshold, batch_id_offset, eps_mode, layout,
                    fused_stem, conv_fusion)

    @_on_own_device
    def _setup(self, weights, fuse, raw_heads, det_capacity, threshold, batch_id_offset, eps_mode, layout,
               fused_stem, conv_fusion):
        model, batch, device = self.model, self.batch, self.device
        # "nhwc": every activation tensor is channels-last, so cuDNN runs its tensor-core convolution kernels
        # without converting the layout around each of them; the epilogue path uses the library's NHWC tier and
        # heads are transposed to NCHW for the decoders.  Results equal the "nchw" run up to the convolutions'
        # own rounding (cuDNN picks different kernels for the two layouts).
        self.nhwc = layout == "nhwc"
        self.eps_mode = eps_mode        # 0: cuDNN form sqrt(var+eps) (the CUDA path), 1: the CPU path's sqrt(var)+eps
        self.plan = graph.plan_native(model, fuse=fuse, raw_heads=raw_heads)   # the library's C++ planner (pxe_plan.h)
        self.threshold = threshold
        self.batch_id_offset = batch_id_offset
        self.w: Dict[int, Dict[str, torch.Tensor]] = {
            i: {k: torch.from_numpy(np.ascontiguousarray(v)).to(device) for k, v in d.items()}
            for i, d in weights.items()}
        # every convolution's batch norm / bias folded once to y = a * x + b (pxe_fold_bn): the epilogue kernels then
        # read two arrays instead of building a coefficient table in every block
        for l in model.layers:
            if l.type != "conv":
                continue
            w = self.w[l.index]
            if self.nhwc:
                w["weights"] = w["weights"].contiguous(memory_format=torch.channels_last)
            if l.batch_norm:
                w["a"], w["b"] = ops.fold_bn(l.filters, device, gamma=w["scales"], beta=w["biases"],
                                             mean=w["rolling_mean"], var=w["rolling_var"], eps_mode=eps_mode)
            else:
                w["a"], w["b"] = ops.fold_bn(l.filters, device, bias=w["biases"])
        # fused_stem: the first convolution and its epilogue as one launch of the library (pxe_conv_stem) instead of
        # the cuDNN call + epilogue, where the layer and its place in the plan allow it
        self.stem = None
        if fused_stem and model.layers:
            l0, st0 = model.layers[0], self.plan.steps[0]
            others_read_input = any(-1 in l.sources for l in model.layers[1:])
            if (l0.type == "conv" and l0.kernel == 3 and l0.stride == 1 and l0.padding == 1 and l0.dilation == 1
                    and l0.groups == 1 and model.channels <= 4 and 8 <= l0.filters <= 64 and l0.filters % 8 == 0
                    and st0.op == "conv" and st0.layer == 0 and st0.fused_pool is None and st0.fused_shortcut is None
                    and not st0.head_raw and st0.dests and not others_read_input):
                w = self.w[0]
                if l0.batch_norm:
                    a, b = ops.fold_bn(l0.filters, device, gamma=w["scales"], beta=w["biases"], mean=w["rolling_mean"],
                                       var=w["rolling_var"], eps_mode=eps_mode)
                else:
                    a, b = ops.fold_bn(l0.filters, device, bias=w["biases"])
                self.stem = {"weights": w["weights"].contiguous(), "a": a, "b": b}
        # conv_fusion: a convolution and its epilogue as one cuDNN runtime-fusion launch where that measures faster
        # than the cuDNN convolution + the library's epilogue (channels-last only; see cudnn_fused.py)
        self.fused_conv = None
        if conv_fusion:
            if not self.nhwc:
                raise ValueError("conv_fusion needs layout='nhwc'")
            from . import cudnn_fused
            self.fused_conv = cudnn_fused.FusedConvPlanner(device)
        self.fused_conv_launches = 0
        self.fold_spp = fuse           # NCHW: a conv's epilogue runs inside the SPP block that reads it next
        self._spp_pending = None
        self.dets = ops.DetectionBuffer(det_capacity, device)
        self.head_marks = []           # device copies of the running detection count after each YOLO head
        self.centernet_out = []        # (dets, counts) per centernet layer of the last forward
        self.outputs: Dict[int, torch.Tensor] = {}     # softmax / region outputs of the last forward
        self.timer = OpTimer()
        self.launches = 0              # kernels of libpxe.so launched by the last forward
        self.contiguous_copies = 0     # hidden torch copies of strided conv inputs (should stay 0)
        self.region_per_image = False   # False: RegionLayer::addDetects as written (every image decodes image 0's boxes)
        self.keep: Optional[set] = None  # layer indices whose tensors to retain in self.kept
        self.kept: Dict[int, torch.Tensor] = {}
        # probe points for whole-graph comparisons with another implementation of the same model:
        #   conv_override(layer, raw) -> tensor   replaces a convolution's raw output (before its epilogue)
        #   step_hook(step_index, step, T, bufs)  runs after every step, before dead tensors are released;
        #                                         T maps layer index -> the tensor that holds its value,
        #                                         bufs maps route layer index -> its concat buffer
        self.conv_override = None
        self.step_hook = None

    # ------------------------------------------------------------------ helpers
    def _device_of(self):
        return self.device

    def _empty(self, shape) -> torch.Tensor:
        if self.nhwc:
            return ops.empty_nhwc(shape, self.device)
        return torch.empty(tuple(shape), device=self.device)

    def _nchw(self, t: torch.Tensor) -> torch.Tensor:
        """Dense NCHW tensor for the decoders and the flattening layers."""
        if self.nhwc and t.shape[1] > 1 and t.shape[2] * t.shape[3] > 1:
            self.launches += 1
            return ops.nhwc_to_nchw(t)
        return t.contiguous()

    def _view(self, bufs, route: int, offset: int, layer: graph.Layer) -> torch.Tensor:
        c, h, w = layer.out_shape
        if route not in bufs:
            bufs[route] = self._empty((self.batch, self.plan.concat_channels[route], h, w))
        return bufs[route][:, offset:offset + c]

    def _dest_tensors(self, bufs, dests: List[graph.Dest], layer: graph.Layer, dense: Optional[torch.Tensor] = None):
        out = []
        for d in dests:
            if d.kind == "dense":
                if dense is None:
                    dense = self._empty((self.batch,) + layer.out_shape)
                out.append(dense)
            else:
                out.append(self._view(bufs, d.route, d.offset, layer))
        return out

    def _extra_copies(self, src: torch.Tensor, extra: List[torch.Tensor]):
        for t in extra:
            s = self.timer.begin()
            if self.nhwc:
                ops.conv_epilogue_nhwc(src, y=t)
            else:
                ops.concat([src], out=t)
            self.launches += 1
            self.timer.end(s, "concat", 8 * src.numel())

    # ------------------------------------------------------------------ forward
    @_on_own_device
    @torch.no_grad()
    def forward(self, x: torch.Tensor) -> None:
        """Enqueues one forward pass of the whole graph for the batch ``x`` [B,C,H,W] (on the device)."""
        L = self.model.layers
        if self.nhwc and self.stem is None:
            x = x.contiguous(memory_format=torch.channels_last)
        T: Dict[int, torch.Tensor] = {-1: x}
        bufs: Dict[int, torch.Tensor] = {}
        self.dets.reset()
        self.centernet_out, self.outputs, self.kept, self.head_marks = [], {}, {}, []
        self.launches = 0
        self.fused_conv_launches = 0
        tm = self.timer
        for si, st in enumerate(self.plan.steps):
            l = L[st.layer]
            if st.op == "conv":
                nxt = self.plan.steps[si + 1] if si + 1 < len(self.plan.steps) else None
                self._conv(st, l, T, bufs, nxt)
            elif st.op == "alias":
                if st.inputs:
                    T[st.layer] = T[st.inputs[0]]
                else:
                    T[st.layer] = bufs[st.layer]
                    self._extra_copies(T[st.layer], self._dest_tensors(bufs, st.dests, l))
            elif st.op == "maxpool":
                dests = self._dest_tensors(bufs, st.dests, l)
                s = tm.begin()
                if self.nhwc:
                    ops.maxpool_nhwc(T[st.inputs[0]], l.kernel, l.stride, l.padding, out=dests[0])
                else:
                    ops.maxpool(T[st.inputs[0]], l.kernel, l.stride, l.padding, out=dests[0])
                self.launches += 1
                tm.end(s, "maxpool", 4 * (T[st.inputs[0]].numel() + dests[0].numel()))
                self._extra_copies(dests[0], dests[1:])
                T[st.layer] = dests[0]
            elif st.op == "spp":
                xin = T[st.inputs[0]]
                firsts, rest = [], []
                for g, ds in zip(st.spp_layers, st.spp_dests):
                    ts = self._dest_tensors(bufs, ds, L[g])
                    firsts.append(ts[0])
                    rest.append(ts[1:])
                    T[g] = ts[0]
                s = tm.begin()
                if self.nhwc:
                    # A (k+4)-wide stride-1 maximum is the 5-wide maximum of the k-wide one (taps outside the
                    # map are skipped, i.e. -inf): pools whose sizes step by 4 (5, 9, 13) are chained, each
                    # reading the previous result, 25 taps per output instead of 81 and 169.
                    order = sorted(range(len(firsts)), key=lambda i: L[st.spp_layers[i]].kernel)
                    prev_k, prev_t = None, None
                    for i in order:
                        k = L[st.spp_layers[i]].kernel
                        if prev_k is not None and k == prev_k + 4:
                            ops.maxpool_nhwc(prev_t, 5, 1, 4, out=firsts[i])
                        else:
                            ops.maxpool_nhwc(xin, k, 1, k - 1, out=firsts[i])
                        prev_k, prev_t = k, firsts[i]
                    self.launches += len(firsts) - 1
                elif self._spp_pending is not None:
                    raw, cd, fa, fb, act = self._spp_pending
                    self._spp_pending = None
                    ops.spp(raw, [L[g].kernel for g in st.spp_layers], firsts, a=fa, b=fb, act=act, y_identity=cd[0])
                    rest.append(cd[1:])
                    firsts.append(cd[0])
                else:
                    ops.spp(xin, [L[g].kernel for g in st.spp_layers], firsts)
                self.launches += 1
                folded = len(firsts) > len(st.spp_layers)
                tm.end(s, "epilogue+spp" if folded else "spp", 4 * xin.numel() * (1 + len(firsts)))
                for f, r in zip(firsts, rest):
                    self._extra_copies(f, r)
            elif st.op == "upsample":
                dests = self._dest_tensors(bufs, st.dests, l)
                s = tm.begin()
                if self.nhwc:
                    ops.upsample_nhwc(T[st.inputs[0]], l.stride, l.alpha, out=dests[0])
                else:
                    ops.upsample(T[st.inputs[0]], l.stride, l.alpha, out=dests[0])
                self.launches += 1
                tm.end(s, "upsample", 4 * (T[st.inputs[0]].numel() + dests[0].numel()))
                self._extra_copies(dests[0], dests[1:])
                T[st.layer] = dests[0]
            elif st.op == "shortcut" and tuple(T[st.inputs[0]].shape) != tuple(T[st.inputs[1]].shape):
                # ShortcutLayer::forward hands shortcutGpu its OWN dimensions for `from` as well
                # (include/cuda/ShortcutLayer.h:29-30): a `from` tensor of another shape (resnet18.yml adds across its
                # stride-2 stages) is read as if it had this layer's shape, image b at b*C*H*W of from's buffer.
                # Reproduced as it is, as long as those reads stay inside from's buffer.
                xin, frm = self._nchw(T[st.inputs[0]]), self._nchw(T[st.inputs[1]])
                if frm.numel() < xin.numel():
                    raise ValueError(f"layer {l.index}: shortcut from a tensor of {frm.numel()} elements into one of "
                                     f"{xin.numel()}: the reference would read past the end of `from`")
                s = tm.begin()
                out = xin.clone()
                _, c, h, w = out.shape
                ops.shortcut_general(self.batch, w, h, c, frm, w, h, c, l.alpha, l.beta, out)
                self.launches += 1
                if l.activation != "linear":
                    ops.activate(l.activation, out)
                    self.launches += 1
                tm.end(s, "shortcut", 12 * out.numel())
                if self.nhwc:
                    out = out.contiguous(memory_format=torch.channels_last)
                dests = self._dest_tensors(bufs, st.dests, l, dense=out)
                self._extra_copies(out, [d for d in dests if d is not out])
                T[st.layer] = out
            elif st.op == "shortcut":
                dests = self._dest_tensors(bufs, st.dests, l)
                s = tm.begin()
                if self.nhwc:
                    ops.conv_epilogue_nhwc(T[st.inputs[0]], y=dests[0], y2=dests[1] if len(dests) > 1 else None,
                                           residual=T[st.inputs[1]], res_alpha=l.alpha, res_beta=l.beta,
                                           res_act=l.activation)
                else:
                    ops.shortcut(T[st.inputs[0]], T[st.inputs[1]], l.alpha, l.beta, l.activation, out=dests[0],
                                 out2=dests[1] if len(dests) > 1 else None)
                self.launches += 1
                tm.end(s, "shortcut", 4 * dests[0].numel() * (2 + min(len(dests), 2)))
                self._extra_copies(dests[0], dests[2:])
                T[st.layer] = dests[0]
            elif st.op == "concat":
                s = tm.begin()
                if self.nhwc:
                    out = self._empty((self.batch,) + l.out_shape)
                    off = 0
                    for i in st.inputs:
                        ops.conv_epilogue_nhwc(T[i], y=out[:, off:off + T[i].shape[1]])
                        off += T[i].shape[1]
                    self.launches += len(st.inputs) - 1
                    T[st.layer] = out
                else:
                    T[st.layer] = ops.concat([T[i] for i in st.inputs])
                self.launches += 1
                tm.end(s, "concat", 8 * T[st.layer].numel())
            elif st.op == "yolo":
                self._yolo(st, l, T)
            elif st.op == "centernet":
                xin = self._nchw(T[st.inputs[0]]) if self.nhwc else T[st.inputs[0]]
                cls = l.in_shape[0] - 4
                s = tm.begin()
                out = ops.centernet_decode(xin[:, :cls], xin[:, cls:cls + 2], xin[:, cls + 2:], self.threshold,
                                           int(l.params.get("max_detections", 100)), logits=True,
                                           heatmap_bias=float(l.params.get("heatmap_bias", -2.19)),
                                           batch_id_offset=self.batch_id_offset)
                self.launches += 2
                tm.end(s, "centernet_decode", 4 * self.batch * cls * l.in_shape[1] * l.in_shape[2])
                self.centernet_out.append(out)
                T[st.layer] = xin
            elif st.op == "softmax":
                xin = self._nchw(T[st.inputs[0]])
                s = tm.begin()
                T[st.layer] = ops.softmax(xin, max(1, int(l.params.get("groups", 1))),
                                          float(l.params.get("temperature", 1.0)))
                self.launches += 1
                tm.end(s, "softmax", 8 * xin.numel())
                self.outputs[st.layer] = T[st.layer]
                # SoftmaxLayer::addDetects: the best class of every image, if it reaches the threshold
                ops.softmax_decode(T[st.layer], self.model.width, self.model.height, self.threshold, self.dets,
                                   batch_id_offset=self.batch_id_offset)
                self.launches += 1
                self.head_marks.append(self.dets.count.clone())
            elif st.op == "region":
                xin = self._nchw(T[st.inputs[0]])
                s = tm.begin()
                T[st.layer] = ops.region_forward(xin, int(l.params.get("num", 1)), int(l.params.get("coords", 4)),
                                                 int(l.params.get("classes", self.model.classes or 20)),
                                                 bool(l.params.get("softmax", False)))
                self.launches += 1
                tm.end(s, "region", 8 * xin.numel())
                self.outputs[st.layer] = T[st.layer]
                # RegionLayer::addDetects, with the reference's indexing unless region_per_image is set
                num = int(l.params.get("num", 1))
                anchors = [float(a) for a in l.params.get("anchors", [0.5] * (2 * num))]
                ops.region_decode(T[st.layer], l.in_shape[2], l.in_shape[1], num, int(l.params.get("coords", 4)),
                                  int(l.params.get("classes", self.model.classes or 20)), anchors, self.threshold,
                                  self.dets, per_image=self.region_per_image, batch_id_offset=self.batch_id_offset)
                self.launches += 1
                self.head_marks.append(self.dets.count.clone())
            elif st.op == "avgpool":
                xin = self._nchw(T[st.inputs[0]])
                s = tm.begin()
                T[st.layer] = ops.avgpool(xin)
                self.launches += 1
                tm.end(s, "avgpool", 4 * (xin.numel() + T[st.layer].numel()))
            elif st.op == "connected":
                # GEMM on cuBLAS as in the reference (include/cuda/ConnLayer.h:170-183), then the conv epilogue
                # kernel on [B, outputs, 1, 1]: BN inference or bias, activation (:185-217)
                w = self.w[l.index]
                xin = self._nchw(T[st.inputs[0]]).reshape(self.batch, -1)
                s = tm.begin()
                raw = F.linear(xin, w["weights"]).reshape(self.batch, l.filters, 1, 1)
                tm.end(s, "gemm(cublas)", 0)
                bn = dict(gamma=w["scales"], beta=w["biases"], mean=w["rolling_mean"], var=w["rolling_var"],
                          eps_mode=self.eps_mode) if l.batch_norm else dict(bias=w["biases"])
                s = tm.begin()
                T[st.layer] = ops.conv_epilogue(raw, act=l.activation, **bn)
                self.launches += 1
                tm.end(s, "epilogue", 8 * raw.numel())
            elif st.op == "detection":
                xin = self._nchw(T[st.inputs[0]])
                s = tm.begin()
                ops.detect_decode(xin, int(l.params.get("side", 7)), int(l.params.get("num", 1)),
                                  self.model.classes, self.threshold, self.dets,
                                  coords=int(l.params.get("coords", 4)), squared=bool(l.params.get("sqrt", False)),
                                  batch_id_offset=self.batch_id_offset)
                self.launches += 1
                tm.end(s, "detect_decode", 4 * xin.numel())
                self.head_marks.append(self.dets.count.clone())
                T[st.layer] = xin
            elif st.op == "dropout":
                T[st.layer] = T[st.inputs[0]]
            else:
                raise NotImplementedError(st.op)
            if st.op in _HEAD_OPS and len(st.dests) > 1 and st.layer in T:
                # a head-type layer that a route concatenates: its dense output is copied into the route's buffer
                self._extra_copies(T[st.layer], self._dest_tensors(bufs, st.dests[1:], l))
            if self.keep:
                for p in st.produces:
                    if p in self.keep and p in T:
                        self.kept[p] = T[p]
            if self.step_hook is not None:
                self.step_hook(si, st, T, bufs)
            # release tensors nobody reads any more
            for t in st.inputs:
                if self.plan.last_use.get(t) == si and t in T and t != -1:
                    del T[t]
                    bufs.pop(t, None)

    def _conv(self, st: graph.Step, l: graph.Layer, T, bufs, nxt: Optional[graph.Step] = None) -> None:
        w = self.w[l.index]
        self._spp_pending = None
        xin = T[st.inputs[0]]
        tm = self.timer
        if l.index == 0 and self.stem is not None:
            dests = self._dest_tensors(bufs, st.dests, l)
            s = tm.begin()
            ops.conv_stem(xin, self.stem["weights"], a=self.stem["a"], b=self.stem["b"], act=l.activation, out=dests[0],
                          nhwc=self.nhwc)
            self.launches += 1
            tm.end(s, "stem conv+epilogue", 4 * (xin.numel() + dests[0].numel()))
            self._extra_copies(dests[0], dests[1:])
            T[0] = dests[0]
            return
        if not xin.is_contiguous(memory_format=torch.channels_last if self.nhwc else torch.contiguous_format):
            self.contiguous_copies += 1
        if self.fused_conv is not None and self._conv_fused(st, l, T, bufs, xin, w):
            return
        s = tm.begin()
        raw = F.conv2d(xin, w["weights"], None, l.stride, l.padding, l.dilation, l.groups)
        tm.end(s, "conv(cudnn)", 0)
        if self.conv_override is not None:
            raw = self.conv_override(l.index, raw)
        if self.nhwc and not raw.is_contiguous(memory_format=torch.channels_last):
            raw = raw.contiguous(memory_format=torch.channels_last)      # 1-pixel or 1-channel outputs only
        if st.head_raw:
            T[l.index] = raw                 # bias + activation are applied inside the YOLO decode
            return
        n = raw.numel()
        if self.nhwc:
            return self._conv_epilogue_nhwc(st, l, T, bufs, raw, w)
        # an SPP block reads this conv next: its kernel applies the epilogue while it stages each plane, writes the
        # block's pass-through slot and the pools from one read of the raw output (pxe_spp_epilogue)
        if (self.fold_spp and nxt is not None and nxt.op == "spp" and nxt.inputs and nxt.inputs[0] == l.index
                and st.fused_pool is None and st.fused_shortcut is None and st.dests
                and 2 * raw.shape[2] * raw.shape[3] * 4 <= 48 * 1024):
            dests = self._dest_tensors(bufs, st.dests, l)
            self._spp_pending = (raw, dests, w["a"], w["b"], l.activation)
            T[l.index] = dests[0]
            return
        bn = dict(a=w["a"], b=w["b"])
        if st.fused_pool is not None:
            pl = self.model.layers[st.fused_pool]
            pd = self._dest_tensors(bufs, st.pool_dests, pl)
            full = self._dest_tensors(bufs, st.dests, l, dense=raw) if st.keep_full else []
            s = tm.begin()
            ops.conv_epilogue(raw, y=full[0] if full else False, act=l.activation, pool=(2, 2, pl.padding),
                              y_pool=pd[0], **bn)
            self.launches += 1
            tm.end(s, "epilogue+pool", 4 * n + 4 * pd[0].numel() + (4 * n if full else 0))
            self._extra_copies(pd[0], pd[1:])
            T[st.fused_pool] = pd[0]
            if full:
                self._extra_copies(full[0], full[1:])
                T[l.index] = full[0]
            return
        out_layer = self.model.layers[st.fused_shortcut] if st.fused_shortcut is not None else l
        dests = self._dest_tensors(bufs, st.dests, out_layer, dense=raw)
        kw = {}
        if st.fused_shortcut is not None:
            kw = dict(residual=T[st.inputs[1]], res_alpha=out_layer.alpha, res_beta=out_layer.beta,
                      res_act=out_layer.activation)
        s = tm.begin()
        ops.conv_epilogue(raw, y=dests[0], y2=dests[1] if len(dests) > 1 else None, act=l.activation, **bn, **kw)
        self.launches += 1
        nb = 4 * n * (1 + min(len(dests), 2) + (1 if kw else 0))
        tm.end(s, "epilogue+shortcut" if kw else "epilogue", nb)
        self._extra_copies(dests[0], dests[2:])
        T[out_layer.index] = dests[0]

    def _conv_fused(self, st: graph.Step, l: graph.Layer, T, bufs, xin, w) -> bool:
        """Convolution + epilogue (+ shortcut) of this step as one cuDNN launch, if the layer's shape has a fused
        plan that measured faster than the split form.  False: the caller runs the split form."""
        if (st.head_raw or st.fused_pool is not None or len(st.dests) != 1 or l.groups != 1 or l.dilation != 1
                or self.fused_conv is None):
            return False
        out_layer, residual, res_act = l, None, "linear"
        if st.fused_shortcut is not None:
            out_layer = self.model.layers[st.fused_shortcut]
            if out_layer.alpha != 1.0 or out_layer.beta != 1.0:
                return False
            residual, res_act = T[st.inputs[1]], out_layer.activation
        fc = self.fused_conv
        c, h, wd = out_layer.out_shape
        # the key needs the destination's strides, not its memory: probe with the dense shape first so that a
        # layer that keeps the split form allocates nothing here
        d = st.dests[0]
        if d.kind == "dense":
            probe_shape, ps = (self.batch, c, h, wd), c
        else:
            probe_shape, ps = (self.batch, c, h, wd), self.plan.concat_channels[d.route]
        probe = torch.empty_strided(probe_shape, (h * wd * ps, 1, wd * ps, ps), device="meta")
        key = fc.key(xin, w["weights"], l.stride, l.padding, l.activation, probe, residual, res_act)
        if key is None:
            return False
        capturing = torch.cuda.is_current_stream_capturing()
        if fc.known(key):
            if fc.cache[key] is None:
                return False
        elif capturing:
            return False
        dest = self._dest_tensors(bufs, st.dests, out_layer)[0]
        tm = self.timer
        if not fc.known(key):
            kw = {}
            if residual is not None:
                kw = dict(residual=residual, res_alpha=1.0, res_beta=1.0, res_act=res_act)

            def split():
                raw = F.conv2d(xin, w["weights"], None, l.stride, l.padding)
                ops.conv_epilogue_nhwc(raw, y=dest, a=w["a"], b=w["b"], act=l.activation, **kw)

            if fc.tune(key, xin, w["weights"], w["a"], w["b"], dest, residual, split) is None:
                split()                              # the candidates wrote dest after the split form was timed
                T[out_layer.index] = dest
                self.launches += 1
                return True
        s = tm.begin()
        fc.run(key, xin, w["weights"], w["a"], w["b"], dest, residual)
        self.fused_conv_launches += 1
        tm.end(s, "conv+epilogue (cudnn fused)", 0)
        T[out_layer.index] = dest
        return True

    def _conv_epilogue_nhwc(self, st: graph.Step, l: graph.Layer, T, bufs, raw: torch.Tensor, w) -> None:
        """The conv step's epilogue on channels-last tensors."""
        tm = self.timer
        n = raw.numel()
        if st.fused_pool is not None:
            pl = self.model.layers[st.fused_pool]
            pd = self._dest_tensors(bufs, st.pool_dests, pl)
            full = self._dest_tensors(bufs, st.dests, l, dense=raw) if st.keep_full else []
            s = tm.begin()
            ops.conv_epilogue_nhwc(raw, y=full[0] if full else False, a=w["a"], b=w["b"], act=l.activation,
                                   pool=(2, 2, pl.padding), y_pool=pd[0])
            self.launches += 1
            tm.end(s, "epilogue+pool", 4 * n + 4 * pd[0].numel() + (4 * n if full else 0))
            self._extra_copies(pd[0], pd[1:])
            T[st.fused_pool] = pd[0]
            if full:
                self._extra_copies(full[0], full[1:])
                T[l.index] = full[0]
            return
        out_layer = self.model.layers[st.fused_shortcut] if st.fused_shortcut is not None else l
        dests = self._dest_tensors(bufs, st.dests, out_layer, dense=raw)
        kw = {}
        if st.fused_shortcut is not None:
            kw = dict(residual=T[st.inputs[1]], res_alpha=out_layer.alpha, res_beta=out_layer.beta,
                      res_act=out_layer.activation)
        s = tm.begin()
        ops.conv_epilogue_nhwc(raw, y=dests[0], y2=dests[1] if len(dests) > 1 else None, a=w["a"], b=w["b"],
                               act=l.activation, **kw)
        self.launches += 1
        tm.end(s, "epilogue+shortcut" if kw else "epilogue", 4 * n * (1 + min(len(dests), 2) + (1 if kw else 0)))
        self._extra_copies(dests[0], dests[2:])
        T[out_layer.index] = dests[0]

    def _yolo(self, st: graph.Step, l: graph.Layer, T) -> None:
        xin = T[st.inputs[0]]
        if self.nhwc and not st.head_raw:
            # YoloLayer's output() stays NCHW; the raw-head decode below reads the channels-last conv output where it lies
            s = self.timer.begin()
            xin = self._nchw(xin)
            self.timer.end(s, "head->nchw", 8 * xin.numel())
        mask = [int(m) for m in l.params["mask"]]
        anchors = [int(a) for a in l.params["anchors"]]
        classes = l.in_shape[0] // len(mask) - 5
        tm = self.timer
        if st.head_raw:
            conv = self.model.layers[st.inputs[0]]
            s = tm.begin()
            ops.yolo_decode(xin, mask, anchors, classes, self.model.width, self.model.height, self.threshold,
                            self.dets, raw=True, bias=self.w[conv.index]["biases"],
                            batch_id_offset=self.batch_id_offset)
            self.launches += 3
            tm.end(s, "yolo_decode", 4 * xin.numel())
            self.head_marks.append(self.dets.count.clone())
            T[st.layer] = xin
            return
        s = tm.begin()
        act = ops.yolo_activate(xin.contiguous(), len(mask), classes)
        self.launches += 1
        tm.end(s, "yolo_activate", 8 * xin.numel())
        s = tm.begin()
        ops.yolo_decode(act, mask, anchors, classes, self.model.width, self.model.height, self.threshold, self.dets,
                        batch_id_offset=self.batch_id_offset)
        self.launches += 3
        tm.end(s, "yolo_decode", 4 * xin.numel())
        self.head_marks.append(self.dets.count.clone())
        T[st.layer] = act

    # ------------------------------------------------------------------ CUDA graph
    @_on_own_device
    def capture(self, x: torch.Tensor) -> "torch.cuda.CUDAGraph":
        """Captures one forward pass on ``x`` (a device tensor that stays allocated: later replays read whatever
        it holds then) into a CUDA graph and returns it.  At small batches a forward is a few hundred launches of
        a few microseconds each and the host cannot issue them fast enough; a replay issues them all at once.
        The pass must have run at least once before (cuDNN picks its algorithms on first use).  The detection
        buffer, head marks and CenterNet outputs that the captured pass wrote are the ones later replays
        write; read them with the usual accessors after a replay."""
        enabled, self.timer.enabled = self.timer.enabled, False
        try:
            side = torch.cuda.Stream(self.device)
            side.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(side):
                self.forward(x)                      # allocations of the pass settle in the caching allocator
            torch.cuda.current_stream(self.device).wait_stream(side)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self.forward(x)
        finally:
            self.timer.enabled = enabled
        return g

    # ------------------------------------------------------------------ results
    def detections(self):
        """Detections of the last forward in the reference's order (Model::detections):
        (structured array, total count including records dropped for lack of capacity)."""
        recs, total = self.dets.to_host()
        parts = [recs]
        for d, c in self.centernet_out:
            per_image = ops.centernet_to_host(d, c)
            parts.extend(per_image)
            total += sum(len(p) for p in per_image)
        return (np.concatenate(parts) if len(parts) > 1 else recs), total

    def detections_by_head(self):
        """Per-head record arrays of the last forward (input to sharding.merge_shards)."""
        from . import sharding
        recs, _ = self.dets.to_host()
        ends = [min(int(m.item()), len(recs)) for m in self.head_marks]
        heads = sharding.split_heads(recs, ends)
        for d, c in self.centernet_out:
            heads.append(np.concatenate(ops.centernet_to_host(d, c)))
        return heads

    @_on_own_device
    def predict(self, host_batch: torch.Tensor, nms_threshold: Optional[float] = None, nms_on_device: bool = False):
        """The call a user makes: host images in (pinned memory), detections out.  Mirrors
        Model::predictBatchImageList (include/Model.h:951-1060) from the H2D copy on.  With
        ``nms_on_device`` px::nms runs on the device buffer the decodes filled and only the survivors are
        copied to the host (same records, same order as the host form); CenterNet heads, whose records live
        in their own per-image buffers, always take the host form."""
        x = host_batch.to(self.device, non_blocking=True)
        self.forward(x)
        if nms_threshold is not None and nms_on_device and not self.centernet_out:
            total = int(self.dets.count.item())
            n = min(total, self.dets.capacity)
            kept, count = ops.nms_device(self.dets.dets, n, nms_threshold)
            m = int(count.item())
            return kept[:m].cpu().numpy().view(ops.DET_DTYPE).reshape(-1), total
        recs, total = self.detections()
        if nms_threshold is not None:
            recs = ops.nms(recs, nms_threshold)
        return recs, total


class PipelinedPredictor:
    """Keeps the GPU busy across consecutive ``predict`` calls: while batch i runs, batch i+1 is copied to
    the device on a second stream and the detections of batch i-1 are copied back on a third.  Two input
    buffers, two detection buffers and two pinned result buffers alternate.  Every batch still pays its
    own host-to-device and device-to-host copy; they merely overlap the compute of its neighbours.

    Usage: ``submit(host_batch)`` for each batch, in order; each call returns the finished result of the
    batch submitted one call earlier (``None`` for the first), ``drain()`` returns the last one.  A result
    is ``(records, total)`` where ``records`` is a structured view of pinned memory that stays valid
    until two more batches have been submitted.
    """

    def __init__(self, runner: Runner, batch_shape, pinned_capacity: Optional[int] = None, use_graphs: bool = False,
                 nms_threshold: Optional[float] = None):
        """``nms_threshold``: run px::nms on the device (pxe_nms) on each batch's candidates and copy only the
        survivors to the host, as Model::predict does after detections(); None copies every candidate."""
        self.r = runner
        dev = runner.device
        self.compute = torch.cuda.current_stream(dev)
        self.h2d, self.d2h = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        self.nms_threshold = nms_threshold
        self.kept = [None, None]          # per slot: device buffer of NMS survivors
        self.kept_count_host = [torch.zeros(1, dtype=torch.int64).pin_memory() for _ in range(2)]
        self.nms_ws = None
        cap = pinned_capacity or runner.dets.capacity
        self.x = [torch.empty(batch_shape, device=dev) for _ in range(2)]
        self.bufs = [runner.dets, ops.DetectionBuffer(runner.dets.capacity, dev)]
        self.pinned = [torch.empty((cap, 8), dtype=torch.int32).pin_memory() for _ in range(2)]
        self.count_host = [torch.zeros(1, dtype=torch.int64).pin_memory() for _ in range(2)]
        self.x_ready = [None, None]       # event: input slot filled
        self.x_free = [None, None]        # event: the forward that read this input slot finished
        self.out_done = [None, None]      # event: detections of this slot are on the host
        self.pending = None               # (slot, event after forward)
        self.n = 0
        # one CUDA graph per slot (its input buffer and its detection buffer are baked into the graph)
        self.graphs = None
        if use_graphs:
            self.graphs = []
            for slot in range(2):
                runner.dets = self.bufs[slot]
                self.x[slot].zero_()
                self.graphs.append(runner.capture(self.x[slot]))
            runner.dets = self.bufs[0]

    def _device_of(self):
        return self.r.device

    def _stage(self, host_batch, slot):
        with torch.cuda.stream(self.h2d):
            if self.x_free[slot] is not None:
                self.h2d.wait_event(self.x_free[slot])
            self.x[slot].copy_(host_batch, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self.h2d)
            self.x_ready[slot] = ev

    def _retire(self):
        slot, done = self.pending
        self.pending = None
        buf = self.bufs[slot]
        with torch.cuda.stream(self.d2h):
            self.d2h.wait_event(done)
            self.count_host[slot].copy_(buf.count, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self.d2h)
        ev.synchronize()                                  # the next forward is already queued behind this one
        total = int(self.count_host[slot].item())
        n = min(total, buf.capacity, self.pinned[slot].shape[0])
        src = buf.dets
        if self.nms_threshold is not None:
            # NMS of this batch on the copy stream, beside the next batch's forward pass; only survivors leave the GPU
            with torch.cuda.stream(self.d2h):
                need = ops.capi.lib().pxe_nms_workspace_bytes(n)
                if self.nms_ws is None or self.nms_ws.numel() < need:
                    self.nms_ws = torch.empty(max(need, 256), device=buf.dets.device, dtype=torch.uint8)
                if self.kept[slot] is None or self.kept[slot].shape[0] < max(n, 1):
                    self.kept[slot] = torch.empty((max(n, 1), 8), device=buf.dets.device, dtype=torch.int32)
                _, kept_count = ops.nms_device(buf.dets, n, self.nms_threshold, out=self.kept[slot], workspace=self.nms_ws)
                self.kept_count_host[slot].copy_(kept_count, non_blocking=True)
                ev2 = torch.cuda.Event()
                ev2.record(self.d2h)
            ev2.synchronize()
            n = min(int(self.kept_count_host[slot].item()), self.pinned[slot].shape[0])
            src = self.kept[slot]
        with torch.cuda.stream(self.d2h):
            self.pinned[slot][:n].copy_(src[:n], non_blocking=True)
            out = torch.cuda.Event()
            out.record(self.d2h)
        self.out_done[slot] = out
        return slot, n, total

    def _result(self, slot, n, total):
        self.out_done[slot].synchronize()
        return self.pinned[slot][:n].numpy().view(ops.DET_DTYPE).reshape(-1), total

    @_on_own_device
    def submit(self, host_batch: torch.Tensor):
        slot = self.n % 2
        self.n += 1
        self._stage(host_batch, slot)
        self.compute.wait_event(self.x_ready[slot])
        if self.out_done[slot] is not None:
            self.compute.wait_event(self.out_done[slot])  # this slot's previous detections have left the device
        self.r.dets = self.bufs[slot]
        if self.graphs is not None:
            self.graphs[slot].replay()
        else:
            self.r.forward(self.x[slot])
        done = torch.cuda.Event()
        done.record(self.compute)
        self.x_free[slot] = done
        finished = None
        if self.pending is not None:
            finished = self._retire()
        self.pending = (slot, done)
        return self._result(*finished) if finished is not None else None

    @_on_own_device
    def drain(self):
        if self.pending is None:
            return None
        return self._result(*self._retire())
