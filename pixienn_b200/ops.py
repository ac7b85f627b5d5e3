"""The epilogue operators on torch CUDA tensors.

Thin argument marshalling over the C ABI (``include/pxe.h``): torch supplies device memory and
the current stream, every computation runs in ``libpxe.so``.  A tensor argument may be a channel
slice of a wider NCHW buffer (``buf[:, 64:192]``): its batch stride is passed through, which is
how producers write straight into route (concat) buffers.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import numpy as np
import torch

from . import capi
from .capi import ACT, PxeError  # noqa: F401  (re-exported)

DET_DTYPE = np.dtype([("x", "f4"), ("y", "f4"), ("w", "f4"), ("h", "f4"), ("prob", "f4"),
                      ("class_id", "i4"), ("batch_id", "i4"), ("source", "i4")])


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _act(a) -> int:
    return ACT[a] if isinstance(a, str) else int(a)


def _check_device(index: int, name: str) -> None:
    """The library launches on the calling thread's current device and on torch's current stream of that
    device, so a tensor of another GPU must not reach it: without peer access the kernel would fault, with it
    the work would silently run on the wrong GPU.  Callers select the device first (``torch.cuda.device``;
    Runner and PipelinedPredictor do it themselves)."""
    cur = torch.cuda.current_device()
    if index != cur:
        raise ValueError(f"{name} lives on cuda:{index} but the current device is cuda:{cur}; "
                         f"wrap the call in torch.cuda.device({index})")


def _check_f32_cuda(t: torch.Tensor, name: str) -> None:
    if not (isinstance(t, torch.Tensor) and t.is_cuda and t.dtype == torch.float32):
        raise TypeError(f"{name} must be a float32 CUDA tensor")
    _check_device(t.device.index, name)


def _slot(t: Optional[torch.Tensor], name: str):
    """(pointer, batch stride) of a 4-D NCHW tensor whose per-image block is dense."""
    if t is None:
        return None, 0
    _check_f32_cuda(t, name)
    if t.dim() != 4:
        raise ValueError(f"{name} must be 4-D [B,C,H,W], got {tuple(t.shape)}")
    b, c, h, w = t.shape
    st = t.stride()
    if (st[3] != 1 and w > 1) or (st[2] != w and h > 1) or (st[1] != h * w and c > 1):
        raise ValueError(f"{name}: per-image block must be contiguous (strides {st} for shape {tuple(t.shape)})")
    bs = st[0] if b > 1 else c * h * w
    return t.data_ptr(), int(bs)


def _vec(t: Optional[torch.Tensor], n: int, name: str):
    if t is None:
        return None
    _check_f32_cuda(t, name)
    if t.numel() != n or not t.is_contiguous():
        raise ValueError(f"{name} must be a contiguous tensor of {n} elements")
    return t.data_ptr()


def maxpool_out_dim(n: int, kernel: int, stride: int, padding: Optional[int] = None) -> int:
    if padding is None:
        padding = max(0, kernel - 1)
    return capi.lib().pxe_maxpool_out_dim(n, kernel, stride, padding)


def conv_epilogue(x: torch.Tensor, *, y: Optional[torch.Tensor] = None, y2: Optional[torch.Tensor] = None,
                  gamma=None, beta=None, mean=None, var=None, bias=None, act="linear", eps: float = 1e-5,
                  eps_mode: int = capi.EPS_CUDNN, yolo_classes: int = 0,
                  residual: Optional[torch.Tensor] = None, res_alpha: float = 1.0, res_beta: float = 1.0,
                  res_act="linear", pool: Optional[Sequence[int]] = None,
                  y_pool: Optional[torch.Tensor] = None, in_place: bool = True, pool_variant: int = 0,
                  a: Optional[torch.Tensor] = None, b: Optional[torch.Tensor] = None):
    """Fused BN / bias / activation (+ residual, + 2x2 pool, + concat-slot stores).

    Returns ``y`` (or ``(y, y_pool)`` when pooling).  With ``y=None`` the result overwrites ``x``
    (``in_place=True``) or goes to a new tensor; ``y=False`` with pooling skips the
    full-resolution output altogether.  ``a``, ``b``: the layer's coefficients folded once by ``fold_bn`` (then
    gamma / beta / mean / var / bias are not needed); same results, no per-block coefficient table.
    """
    xp, xbs = _slot(x, "x")
    B, Cc, H, W = x.shape
    d = capi.EpilogueDesc()
    d.x, d.x_batch_stride = xp, xbs
    want_full = y is not False
    if y is None:
        y = x if in_place else torch.empty((B, Cc, H, W), device=x.device, dtype=torch.float32)
    if want_full:
        yp, ybs = _slot(y, "y")
        if tuple(y.shape) != (B, Cc, H, W):
            raise ValueError("y shape mismatch")
        d.y, d.y_batch_stride = yp, ybs
    else:
        y = None
    if y2 is not None:
        if tuple(y2.shape) != (B, Cc, H, W):
            raise ValueError("y2 shape mismatch")
        d.y2, d.y2_batch_stride = _slot(y2, "y2")
    d.batch, d.channels, d.height, d.width = B, Cc, H, W
    if gamma is not None:
        d.gamma, d.beta = _vec(gamma, Cc, "gamma"), _vec(beta, Cc, "beta")
        d.mean, d.var = _vec(mean, Cc, "mean"), _vec(var, Cc, "var")
    d.eps, d.eps_mode = eps, eps_mode
    d.bias = _vec(bias, Cc, "bias")
    if a is not None or b is not None:            # coefficients folded once per layer (fold_bn): no per-block table
        d.folded_a, d.folded_b = _vec(a, Cc, "a"), _vec(b, Cc, "b")
    d.act, d.yolo_classes = _act(act), yolo_classes
    if residual is not None:
        if tuple(residual.shape) != (B, Cc, H, W):
            raise ValueError("residual shape mismatch")
        d.residual, d.residual_batch_stride = _slot(residual, "residual")
        d.res_alpha, d.res_beta, d.res_act = res_alpha, res_beta, _act(res_act)
    if pool is not None:
        k, s, pad = pool
        d.pool_kernel, d.pool_stride, d.pool_padding = k, s, pad
        oh, ow = maxpool_out_dim(H, k, s, pad), maxpool_out_dim(W, k, s, pad)
        if y_pool is None:
            y_pool = torch.empty((B, Cc, oh, ow), device=x.device, dtype=torch.float32)
        if tuple(y_pool.shape) != (B, Cc, oh, ow):
            raise ValueError(f"y_pool must be {(B, Cc, oh, ow)}, got {tuple(y_pool.shape)}")
        d.y_pool, d.y_pool_batch_stride = _slot(y_pool, "y_pool")
        d.pool_variant = pool_variant        # capi.POOL_GENERAL: the general pooled kernel whatever the shape (tests)
    capi.check(capi.lib().pxe_conv_epilogue(_stream(), C.byref(d)))
    return (y, y_pool) if pool is not None else y


def activate(kind, x: torch.Tensor) -> torch.Tensor:
    """In-place activation of a contiguous tensor: px::activate (src/Activation.cu:126-133)."""
    _check_f32_cuda(x, "x")
    if not x.is_contiguous():
        raise ValueError("x must be contiguous")
    capi.check(capi.lib().pxe_activate(_stream(), _act(kind), x.data_ptr(), x.numel()))
    return x


def add_bias(out: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """out[b, j, ...] += bias[j] in place: px::addBiasGpu (src/BiasKernels.cu:86-93)."""
    _check_f32_cuda(out, "out")
    if not out.is_contiguous():
        raise ValueError("out must be contiguous")
    B, n = out.shape[0], out.shape[1]
    size = out.numel() // (B * n)
    capi.check(capi.lib().pxe_add_bias(_stream(), out.data_ptr(), _vec(bias, n, "bias"), B, n, size))
    return out


def maxpool(x: torch.Tensor, kernel: int, stride: int, padding: Optional[int] = None,
            out: Optional[torch.Tensor] = None, with_indexes: bool = False):
    """MaxPoolLayer forward.  Returns ``out`` or ``(out, indexes)``."""
    if padding is None:
        padding = max(0, kernel - 1)                       # include/MaxPoolLayer.h:56
    xp, xbs = _slot(x, "x")
    B, Cc, H, W = x.shape
    oh, ow = maxpool_out_dim(H, kernel, stride, padding), maxpool_out_dim(W, kernel, stride, padding)
    if oh <= 0 or ow <= 0:
        raise PxeError(capi.PXE_ERR_BAD_ARG, f"maxpool: empty output {oh}x{ow}")
    if out is None:
        out = torch.empty((B, Cc, oh, ow), device=x.device, dtype=torch.float32)
    if tuple(out.shape) != (B, Cc, oh, ow):
        raise ValueError(f"out must be {(B, Cc, oh, ow)}")
    yp, ybs = _slot(out, "out")
    idx = torch.empty((B, Cc, oh, ow), device=x.device, dtype=torch.int32) if with_indexes else None
    if with_indexes and xbs != Cc * H * W:
        raise ValueError("indexes need a densely packed input")
    capi.check(capi.lib().pxe_maxpool(_stream(), xp, xbs, yp, ybs, idx.data_ptr() if idx is not None else None,
                                      B, Cc, H, W, kernel, stride, padding))
    return (out, idx) if with_indexes else out


def spp(x: torch.Tensor, kernels: Sequence[int], outs: Sequence[torch.Tensor], *, a: Optional[torch.Tensor] = None,
        b: Optional[torch.Tensor] = None, act=None, y_identity: Optional[torch.Tensor] = None) -> Sequence[torch.Tensor]:
    """Stride-1 max pools of one input (default padding kernel-1), one output per kernel size.  With ``act``
    (and optionally the folded coefficients ``a``, ``b`` of fold_bn) ``x`` is a raw convolution output: the
    epilogue is applied as the planes are read, its result goes to ``y_identity`` and into every pool."""
    xp, xbs = _slot(x, "x")
    B, Cc, H, W = x.shape
    n = len(kernels)
    if len(outs) != n:
        raise ValueError("one output per kernel size")
    ptrs, strides = (C.c_void_p * n)(), (C.c_longlong * n)()
    for i, o in enumerate(outs):
        if tuple(o.shape) != (B, Cc, H, W):
            raise ValueError("spp outputs have the input's shape")
        ptrs[i], strides[i] = _slot(o, f"outs[{i}]")
    ks = (C.c_int * n)(*[int(k) for k in kernels])
    if act is None and a is None and y_identity is None:
        capi.check(capi.lib().pxe_spp(_stream(), xp, xbs, B, Cc, H, W, n, ks, ptrs, strides))
        return outs
    if y_identity is not None and tuple(y_identity.shape) != (B, Cc, H, W):
        raise ValueError("y_identity has the input's shape")
    ip, ibs = _slot(y_identity, "y_identity") if y_identity is not None else (None, 0)
    capi.check(capi.lib().pxe_spp_epilogue(_stream(), xp, xbs, B, Cc, H, W, _vec(a, Cc, "a"), _vec(b, Cc, "b"),
                                           _act(act if act is not None else "linear"), ip, ibs, n, ks, ptrs, strides))
    return outs


def upsample(x: torch.Tensor, stride: int = 2, scale: float = 1.0, out: Optional[torch.Tensor] = None):
    xp, xbs = _slot(x, "x")
    B, Cc, H, W = x.shape
    if out is None:
        out = torch.empty((B, Cc, H * stride, W * stride), device=x.device, dtype=torch.float32)
    if tuple(out.shape) != (B, Cc, H * stride, W * stride):
        raise ValueError("out shape mismatch")
    yp, ybs = _slot(out, "out")
    capi.check(capi.lib().pxe_upsample(_stream(), xp, xbs, yp, ybs, B, Cc, H, W, stride, scale))
    return out


def shortcut(x: torch.Tensor, frm: torch.Tensor, alpha: float = 1.0, beta: float = 1.0, act="linear",
             out: Optional[torch.Tensor] = None, out2: Optional[torch.Tensor] = None):
    """out = act(alpha*x + beta*from) for equal shapes (ShortcutLayer forward)."""
    xp, xbs = _slot(x, "x")
    fp, fbs = _slot(frm, "from")
    B, Cc, H, W = x.shape
    if tuple(frm.shape) != (B, Cc, H, W):
        raise ValueError("from shape mismatch")
    if out is None:
        out = torch.empty((B, Cc, H, W), device=x.device, dtype=torch.float32)
    yp, ybs = _slot(out, "out")
    y2p, y2bs = _slot(out2, "out2")
    capi.check(capi.lib().pxe_shortcut(_stream(), xp, xbs, fp, fbs, yp, ybs, y2p, y2bs, B, Cc, H, W,
                                       alpha, beta, _act(act)))
    return out


def shortcut_general(batch, w1, h1, c1, add: torch.Tensor, w2, h2, c2, s1, s2, out: torch.Tensor):
    """px::shortcutGpu for unequal shapes: out = s1*out + s2*add, in place."""
    _check_f32_cuda(add, "add")
    _check_f32_cuda(out, "out")
    capi.check(capi.lib().pxe_shortcut_general(_stream(), batch, w1, h1, c1, add.data_ptr(), w2, h2, c2,
                                               s1, s2, out.data_ptr()))
    return out


def concat(srcs: Sequence[torch.Tensor], out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """RouteLayer forward as one launch."""
    n = len(srcs)
    B, _, H, W = srcs[0].shape
    ch = [int(s.shape[1]) for s in srcs]
    if out is None:
        out = torch.empty((B, sum(ch), H, W), device=srcs[0].device, dtype=torch.float32)
    ptrs, strides = (C.c_void_p * n)(), (C.c_longlong * n)()
    for i, s in enumerate(srcs):
        if s.shape[0] != B or s.shape[2] != H or s.shape[3] != W:
            raise ValueError("route sources must share batch and spatial size")
        ptrs[i], strides[i] = _slot(s, f"srcs[{i}]")
    yp, ybs = _slot(out, "out")
    capi.check(capi.lib().pxe_concat(_stream(), n, ptrs, strides, (C.c_int * n)(*ch), yp, ybs, B, H, W))
    return out


def yolo_activate(x: torch.Tensor, masks: int, classes: int, out: Optional[torch.Tensor] = None):
    _check_f32_cuda(x, "x")
    if not x.is_contiguous():
        raise ValueError("x must be contiguous")
    B = x.shape[0]
    area = x.shape[2] * x.shape[3]
    if out is None:
        out = torch.empty_like(x)
    capi.check(capi.lib().pxe_yolo_activate(_stream(), x.data_ptr(), out.data_ptr(), B, masks, classes, area))
    return out


class DetectionBuffer:
    """Device buffer of detections plus the device-side running count the YOLO decode appends to."""

    def __init__(self, capacity: int, device):
        self.capacity = int(capacity)
        self.dets = torch.empty((self.capacity, 8), device=device, dtype=torch.int32)   # 32-byte records
        self.count = torch.zeros(1, device=device, dtype=torch.int64)
        self._workspace = None

    def reset(self):
        self.count.zero_()

    def workspace(self, nbytes: int) -> torch.Tensor:
        if self._workspace is None or self._workspace.numel() < nbytes:
            self._workspace = torch.empty(max(nbytes, 256), device=self.dets.device, dtype=torch.uint8)
        return self._workspace

    def to_host(self):
        """(structured numpy array of the stored records, total count incl. dropped ones)."""
        total = int(self.count.item())
        n = min(total, self.capacity)
        host = self.dets[:n].cpu().numpy().view(DET_DTYPE).reshape(-1)
        return host, total


def yolo_decode(head: torch.Tensor, mask, anchors, classes: int, net_w: int, net_h: int, threshold: float,
                buf: DetectionBuffer, *, img_w: int = 0, img_h: int = 0, raw: bool = False,
                bias: Optional[torch.Tensor] = None, batch_id_offset: int = 0) -> None:
    """Appends one head's detections to ``buf`` in the reference's emission order.  ``head`` is [B, C, H, W], dense
    NCHW (or a channel slot of a wider NCHW buffer) or dense channels-last; the latter is read where it lies."""
    B, Cc, H, W = head.shape
    d = capi.YoloDecodeDesc()
    nhwc = (not head.is_contiguous()) and head.is_contiguous(memory_format=torch.channels_last) and Cc > 1 and H * W > 1
    if nhwc:
        _check_f32_cuda(head, "head")
        hp, hbs = head.data_ptr(), Cc * H * W
        d.head_channels_last = 1
    else:
        hp, hbs = _slot(head, "head")
    d.head, d.head_batch_stride = hp, hbs
    d.head_is_raw = int(raw)
    d.bias = _vec(bias, Cc, "bias")
    d.batch, d.height, d.width, d.classes = B, H, W, classes
    d.n_masks = len(mask)
    for i, m in enumerate(mask):
        d.mask[i] = int(m)
    d.n_anchor_values = len(anchors)
    for i, a in enumerate(anchors):
        d.anchors[i] = int(a)
    d.net_width, d.net_height = net_w, net_h
    d.image_width, d.image_height = img_w, img_h
    d.threshold, d.batch_id_offset = threshold, batch_id_offset
    if Cc != len(mask) * (classes + 5):
        raise ValueError("head channels must equal masks*(classes+5)")
    need = capi.lib().pxe_yolo_decode_fast_workspace_bytes(B, H, W)
    ws = buf.workspace(need)
    capi.check(capi.lib().pxe_yolo_decode(_stream(), C.byref(d), buf.dets.data_ptr(), buf.capacity,
                                          buf.count.data_ptr(), ws.data_ptr(), ws.numel()))


def centernet_activate(x: torch.Tensor, classes: int, heatmap_bias: float, out: Optional[torch.Tensor] = None):
    _check_f32_cuda(x, "x")
    if not x.is_contiguous():
        raise ValueError("x must be contiguous")
    B = x.shape[0]
    area = x.shape[2] * x.shape[3]
    if out is None:
        out = torch.empty_like(x)
    capi.check(capi.lib().pxe_centernet_activate(_stream(), x.data_ptr(), out.data_ptr(), B, classes, area,
                                                 heatmap_bias))
    return out


def centernet_decode(heat: torch.Tensor, size: torch.Tensor, offset: torch.Tensor, threshold: float,
                     max_detections: int = 100, *, logits: bool = False, heatmap_bias: float = 0.0,
                     img_w: int = 0, img_h: int = 0, batch_id_offset: int = 0, workspace=None,
                     candidate_capacity: int = 0):
    """Returns (dets [B, K, 8] int32 view of 32-byte records, counts [B] int32), both on the device.
    ``candidate_capacity``: see pxe_centernet_decode_desc (0 = default)."""
    hp, hbs = _slot(heat, "heat")
    sp, sbs = _slot(size, "size")
    op, obs = _slot(offset, "offset")
    B, classes, H, W = heat.shape
    d = capi.CenterNetDecodeDesc()
    d.heat, d.heat_batch_stride = hp, hbs
    d.size, d.size_batch_stride = sp, sbs
    d.offset, d.offset_batch_stride = op, obs
    d.heat_is_logit, d.heatmap_bias = int(logits), heatmap_bias
    d.batch, d.classes, d.height, d.width = B, classes, H, W
    d.image_width, d.image_height = img_w, img_h
    d.threshold, d.max_detections, d.batch_id_offset = threshold, max_detections, batch_id_offset
    d.candidate_capacity = candidate_capacity
    need = capi.lib().pxe_centernet_decode_workspace_bytes(B, classes, H, W, max_detections)
    if workspace is None or workspace.numel() < need:
        workspace = torch.empty(max(need, 256), device=heat.device, dtype=torch.uint8)
    dets = torch.empty((B, max_detections, 8), device=heat.device, dtype=torch.int32)
    counts = torch.empty(B, device=heat.device, dtype=torch.int32)
    capi.check(capi.lib().pxe_centernet_decode(_stream(), C.byref(d), dets.data_ptr(), counts.data_ptr(),
                                               workspace.data_ptr(), workspace.numel()))
    return dets, counts


def centernet_to_host(dets: torch.Tensor, counts: torch.Tensor):
    """List of per-image structured arrays."""
    h = dets.cpu().numpy()
    c = counts.cpu().numpy()
    return [h[b, :c[b]].copy().view(DET_DTYPE).reshape(-1) for b in range(h.shape[0])]


def softmax(x: torch.Tensor, groups: int = 1, temperature: float = 1.0, out: Optional[torch.Tensor] = None):
    _check_f32_cuda(x, "x")
    if not x.is_contiguous():
        raise ValueError("x must be contiguous")
    B = x.shape[0]
    inputs = x.numel() // B
    if out is None:
        out = torch.empty_like(x)
    capi.check(capi.lib().pxe_softmax(_stream(), x.data_ptr(), out.data_ptr(), B, inputs, groups, temperature))
    return out


def region_forward(x: torch.Tensor, num: int, coords: int, classes: int, use_softmax: bool = True):
    _check_f32_cuda(x, "x")
    if not x.is_contiguous():
        raise ValueError("x must be contiguous")
    B, _, H, W = x.shape
    out = torch.empty_like(x)
    capi.check(capi.lib().pxe_region_forward(_stream(), x.data_ptr(), out.data_ptr(), B, W, H, num, coords,
                                             classes, int(use_softmax)))
    return out


def nms(dets: np.ndarray, threshold: float) -> np.ndarray:
    """px::nms on host records (structured array of DET_DTYPE)."""
    dets = np.ascontiguousarray(dets, DET_DTYPE)
    out = np.zeros(len(dets), DET_DTYPE)
    n = capi.lib().pxe_nms_host(dets.ctypes.data, len(dets), threshold, out.ctypes.data)
    if n < 0:
        raise PxeError(-n, "pxe_nms_host failed")
    return out[:n].copy()


def nms_device(dets: torch.Tensor, n: int, threshold: float, out: Optional[torch.Tensor] = None,
               workspace: Optional[torch.Tensor] = None):
    """px::nms on the device.  ``dets``: int32 tensor [capacity, 8] of 32-byte records (a DetectionBuffer's
    ``dets``), of which the first ``n`` are valid.  Returns (out [n, 8] int32, count [1] int64), both on the
    device; the first ``count`` records of ``out`` are the survivors in the reference's order."""
    if dets.dtype != torch.int32 or dets.dim() != 2 or dets.shape[1] != 8 or not dets.is_cuda or not dets.is_contiguous():
        raise ValueError("dets must be a contiguous int32 CUDA tensor of shape [capacity, 8]")
    _check_device(dets.device.index, "dets")
    n = int(n)
    if n < 0 or n > dets.shape[0]:
        raise ValueError(f"n = {n} outside 0..{dets.shape[0]}")
    if out is None:
        out = torch.empty((max(n, 1), 8), device=dets.device, dtype=torch.int32)
    count = torch.zeros(1, device=dets.device, dtype=torch.int64)
    need = capi.lib().pxe_nms_workspace_bytes(n)
    if workspace is None or workspace.numel() < need:
        workspace = torch.empty(max(need, 256), device=dets.device, dtype=torch.uint8)
    capi.check(capi.lib().pxe_nms(_stream(), dets.data_ptr(), n, float(threshold), out.data_ptr(), count.data_ptr(),
                                  workspace.data_ptr(), workspace.numel()))
    return out, count


def avgpool(x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Global average pool: [B, C, H, W] -> [B, C, 1, 1]."""
    xp, xbs = _slot(x, "x")
    B, Cc, H, W = x.shape
    if out is None:
        out = torch.empty((B, Cc, 1, 1), device=x.device, dtype=torch.float32)
    capi.check(capi.lib().pxe_avgpool(_stream(), xp, xbs, out.data_ptr(), out.stride(0), B, Cc, H, W))
    return out


def detect_decode(pred: torch.Tensor, side: int, num: int, classes: int, threshold: float, buf: DetectionBuffer, *,
                  coords: int = 4, squared: bool = False, width: float = 1.0, height: float = 1.0,
                  batch_id_offset: int = 0) -> None:
    """Appends a YOLOv1 detection head's boxes to ``buf``.  ``pred``: [B, side*side*(classes + num*(1+coords))]
    (any trailing shape of that many values per image), contiguous."""
    _check_f32_cuda(pred, "pred")
    if not pred.is_contiguous():
        raise ValueError("pred must be contiguous")
    B = pred.shape[0]
    per = pred.numel() // B
    if per != side * side * (classes + num * (1 + coords)):
        raise ValueError(f"pred has {per} values per image, expected {side * side * (classes + num * (1 + coords))}")
    capi.check(capi.lib().pxe_detect_decode(_stream(), pred.data_ptr(), per, B, side, num, classes, coords, int(squared),
                                            float(width), float(height), float(threshold), buf.dets.data_ptr(),
                                            buf.capacity, buf.count.data_ptr(), batch_id_offset))


# ------------------------------------------------------------------------------ backward-side kernels
def activation_gradient(kind, x: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
    """delta *= f'(x) in place: px::gradient (src/Activation.cu:135-143)."""
    _check_f32_cuda(x, "x")
    _check_f32_cuda(delta, "delta")
    if not (x.is_contiguous() and delta.is_contiguous()) or x.numel() != delta.numel():
        raise ValueError("x and delta must be contiguous tensors of the same size")
    capi.check(capi.lib().pxe_activation_gradient(_stream(), _act(kind), x.data_ptr(), x.numel(), delta.data_ptr()))
    return delta


def backward_bias(bias_updates: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
    """bias_updates[f] += sum of delta[:, f] in place: px::backwardBiasGpu (src/BiasKernels.cu:95-111)."""
    _check_f32_cuda(delta, "delta")
    if not delta.is_contiguous():
        raise ValueError("delta must be contiguous")
    B, n = delta.shape[0], delta.shape[1]
    capi.check(capi.lib().pxe_backward_bias(_stream(), _vec(bias_updates, n, "bias_updates"), delta.data_ptr(), B, n,
                                            delta.numel() // (B * n)))
    return bias_updates


def maxpool_backward(delta: torch.Tensor, indexes: torch.Tensor, grad: torch.Tensor) -> torch.Tensor:
    """grad[indexes[i]] += delta[i] in place: px::maxPoolBackwardGpu (src/MaxPoolKernels.cu:61-65)."""
    _check_f32_cuda(delta, "delta")
    _check_f32_cuda(grad, "grad")
    if indexes.dtype != torch.int32 or not indexes.is_cuda or indexes.numel() != delta.numel():
        raise ValueError("indexes must be an int32 CUDA tensor with delta's element count")
    if not (delta.is_contiguous() and indexes.is_contiguous() and grad.is_contiguous()):
        raise ValueError("delta, indexes and grad must be contiguous")
    capi.check(capi.lib().pxe_maxpool_backward(_stream(), delta.data_ptr(), indexes.data_ptr(), grad.data_ptr(), delta.numel()))
    return grad


def upsample_backward(acc: torch.Tensor, out: torch.Tensor, stride: int, scale: float = 1.0) -> torch.Tensor:
    """acc += scale * (sum of the stride x stride block of out above each element): px::upsampleGpu, forward == 0."""
    _check_f32_cuda(acc, "acc")
    _check_f32_cuda(out, "out")
    B, Cc, H, W = acc.shape
    if tuple(out.shape) != (B, Cc, H * stride, W * stride) or not (acc.is_contiguous() and out.is_contiguous()):
        raise ValueError("out must be the contiguous [B, C, H*stride, W*stride] tensor for a contiguous acc [B, C, H, W]")
    capi.check(capi.lib().pxe_upsample_backward(_stream(), acc.data_ptr(), out.data_ptr(), B, Cc, H, W, stride, scale))
    return acc


def constrain(x: torch.Tensor, alpha: float) -> torch.Tensor:
    """x = clamp(x, -alpha, alpha) in place: px::constrainGpu (src/CudaUtils.cu:131-138)."""
    _check_f32_cuda(x, "x")
    if not x.is_contiguous():
        raise ValueError("x must be contiguous")
    capi.check(capi.lib().pxe_constrain(_stream(), x.data_ptr(), x.numel(), alpha))
    return x


def mul(x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    """y = x * y in place: px::mulGpu (src/CudaUtils.cu:140-146)."""
    _check_f32_cuda(x, "x")
    _check_f32_cuda(y, "y")
    if not (x.is_contiguous() and y.is_contiguous()) or x.numel() != y.numel():
        raise ValueError("x and y must be contiguous tensors of the same size")
    capi.check(capi.lib().pxe_mul(_stream(), x.data_ptr(), y.data_ptr(), x.numel()))
    return y


def random_uniform(out: torch.Tensor, a: float = 0.0, b: float = 1.0) -> torch.Tensor:
    """px::randomGpu (src/CudaUtils.cu:77-86)."""
    _check_f32_cuda(out, "out")
    capi.check(capi.lib().pxe_random_uniform(_stream(), out.data_ptr(), out.numel(), a, b))
    return out


def random_normal(out: torch.Tensor, mean: float = 0.0, stddev: float = 1.0) -> torch.Tensor:
    """px::randomNormalGpu (src/CudaUtils.cu:110-120)."""
    _check_f32_cuda(out, "out")
    capi.check(capi.lib().pxe_random_normal(_stream(), out.data_ptr(), out.numel(), mean, stddev))
    return out


def yolo_loss(output: torch.Tensor, delta: torch.Tensor, truths: torch.Tensor, truth_counts: torch.Tensor,
              assigned_classes: torch.Tensor, assigned_anchors: torch.Tensor, assigned_boxes: torch.Tensor,
              masks: torch.Tensor, anchors: torch.Tensor, stats: torch.Tensor, cost: torch.Tensor, net_w: int, net_h: int,
              ignore_thr: float = 0.5, truth_thr: float = 1.0, coord_scale: float = 1.0, object_scale: float = 1.0,
              no_object_scale: float = 1.0, class_scale: float = 1.0) -> None:
    """px::yoloLossGpu as one launch; delta, stats (12 floats) and cost (1 float) are updated in place."""
    _check_f32_cuda(output, "output")
    _check_f32_cuda(delta, "delta")
    B, ch, H, W = output.shape
    d = capi.YoloLossDesc()
    d.output, d.delta, d.truths, d.truth_counts = output.data_ptr(), delta.data_ptr(), truths.data_ptr(), truth_counts.data_ptr()
    d.max_truth = truths.shape[1]
    d.assigned_classes, d.assigned_anchors = assigned_classes.data_ptr(), assigned_anchors.data_ptr()
    d.assigned_boxes, d.masks, d.anchors = assigned_boxes.data_ptr(), masks.data_ptr(), anchors.data_ptr()
    d.stats, d.cost = stats.data_ptr(), cost.data_ptr()
    d.batch, d.mask_count, d.classes, d.width, d.height = B, masks.numel(), ch // masks.numel() - 5, W, H
    d.network_width, d.network_height = net_w, net_h
    d.ignore_threshold, d.truth_threshold, d.coord_scale = ignore_thr, truth_thr, coord_scale
    d.object_scale, d.no_object_scale, d.class_scale = object_scale, no_object_scale, class_scale
    capi.check(capi.lib().pxe_yolo_loss(_stream(), C.byref(d)))


def centernet_loss(output: torch.Tensor, delta: torch.Tensor, target_heat: torch.Tensor, target_size: torch.Tensor,
                   target_offset: torch.Tensor, target_mask: torch.Tensor, costs: torch.Tensor, normalizer: float,
                   alpha: float = 2.0, beta: float = 4.0, size_weight: float = 0.1) -> None:
    """px::centerNetLossGpu; delta and costs (3 floats) are updated in place."""
    _check_f32_cuda(output, "output")
    _check_f32_cuda(delta, "delta")
    B, ch, H, W = output.shape
    capi.check(capi.lib().pxe_centernet_loss(_stream(), output.data_ptr(), delta.data_ptr(), target_heat.data_ptr(),
                                             target_size.data_ptr(), target_offset.data_ptr(), target_mask.data_ptr(),
                                             costs.data_ptr(), B, ch - 4, H * W, normalizer, alpha, beta, size_weight))


# ------------------------------------------------------------------------------ channels-last tier
def _nhwc(t: Optional[torch.Tensor], name: str):
    """(pointer, pixel stride) of a logical [B,C,H,W] tensor stored channels-last: a dense channels-last tensor
    or a channel slice of one."""
    if t is None:
        return None, 0
    _check_f32_cuda(t, name)
    if t.dim() != 4:
        raise ValueError(f"{name} must be 4-D [B,C,H,W], got {tuple(t.shape)}")
    b, c, h, w = t.shape
    st = t.stride()
    ps = st[3] if w > 1 else (st[2] // max(w, 1) if h > 1 else (st[0] // max(h * w, 1) if b > 1 else c))
    if ps < c or (c > 1 and st[1] != 1) or (h > 1 and st[2] != w * ps) or (b > 1 and st[0] != h * w * ps):
        raise ValueError(f"{name} is not channels-last (strides {st} for shape {tuple(t.shape)})")
    return t.data_ptr(), int(ps)


def empty_nhwc(shape, device) -> torch.Tensor:
    return torch.empty(tuple(shape), device=device, dtype=torch.float32, memory_format=torch.channels_last)


def fold_bn(channels: int, device, *, gamma=None, beta=None, mean=None, var=None, bias=None, eps: float = 1e-5,
            eps_mode: int = capi.EPS_CUDNN):
    """Folded per-channel coefficients (a, b) of BN inference + bias, computed once per layer."""
    a = torch.empty(channels, device=device, dtype=torch.float32)
    b = torch.empty(channels, device=device, dtype=torch.float32)
    capi.check(capi.lib().pxe_fold_bn(_stream(), _vec(gamma, channels, "gamma"), _vec(beta, channels, "beta"),
                                      _vec(mean, channels, "mean"), _vec(var, channels, "var"),
                                      _vec(bias, channels, "bias"), eps, eps_mode, channels, a.data_ptr(), b.data_ptr()))
    return a, b


def conv_epilogue_nhwc(x: torch.Tensor, *, y: Optional[torch.Tensor] = None, y2: Optional[torch.Tensor] = None,
                       a: Optional[torch.Tensor] = None, b: Optional[torch.Tensor] = None, act="linear",
                       residual: Optional[torch.Tensor] = None, res_alpha: float = 1.0, res_beta: float = 1.0,
                       res_act="linear", pool: Optional[Sequence[int]] = None, y_pool: Optional[torch.Tensor] = None):
    """Fused epilogue on channels-last tensors; ``y=None`` works in place.  With ``pool=(2, 2, padding)`` the
    2x2 max pool is folded in: returns ``(y, y_pool)``, and ``y=False`` skips the full-resolution output."""
    xp, xps = _nhwc(x, "x")
    B, Cc, H, W = x.shape
    want_full = y is not False
    if y is None:
        y = x
    d = capi.EpilogueNhwcDesc()
    d.x, d.x_pixel_stride = xp, xps
    if want_full:
        d.y, d.y_pixel_stride = _nhwc(y, "y")
    else:
        if pool is None:
            raise ValueError("y=False needs pool")
        y = None
    for t, n in ((y, "y"), (y2, "y2"), (residual, "residual")):
        if t is not None and tuple(t.shape) != (B, Cc, H, W):
            raise ValueError(f"{n} has shape {tuple(t.shape)}, expected {(B, Cc, H, W)}")
    if y2 is not None:
        d.y2, d.y2_pixel_stride = _nhwc(y2, "y2")
    if residual is not None:
        d.residual, d.residual_pixel_stride = _nhwc(residual, "residual")
    d.pixels, d.channels = B * H * W, Cc
    d.a, d.b = _vec(a, Cc, "a"), _vec(b, Cc, "b")
    d.act, d.res_alpha, d.res_beta, d.res_act = _act(act), res_alpha, res_beta, _act(res_act)
    if pool is not None:
        k, st, pad = pool
        d.pool_kernel, d.pool_stride, d.pool_padding = k, st, pad
        d.batch, d.height, d.width = B, H, W
        oh, ow = maxpool_out_dim(H, k, st, pad), maxpool_out_dim(W, k, st, pad)
        if y_pool is None:
            y_pool = empty_nhwc((B, Cc, oh, ow), x.device)
        elif tuple(y_pool.shape) != (B, Cc, oh, ow):
            raise ValueError(f"y_pool has shape {tuple(y_pool.shape)}, expected {(B, Cc, oh, ow)}")
        d.y_pool, d.y_pool_pixel_stride = _nhwc(y_pool, "y_pool")
    capi.check(capi.lib().pxe_conv_epilogue_nhwc(_stream(), C.byref(d)))
    return (y, y_pool) if pool is not None else y


def upsample_nhwc(x: torch.Tensor, stride: int, scale: float = 1.0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    xp, xps = _nhwc(x, "x")
    B, Cc, H, W = x.shape
    if out is None:
        out = empty_nhwc((B, Cc, H * stride, W * stride), x.device)
    op, ops_ = _nhwc(out, "out")
    capi.check(capi.lib().pxe_upsample_nhwc(_stream(), xp, xps, op, ops_, B, Cc, H, W, stride, scale))
    return out


def maxpool_nhwc(x: torch.Tensor, kernel: int, stride: int, padding: Optional[int] = None,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
    xp, xps = _nhwc(x, "x")
    B, Cc, H, W = x.shape
    if padding is None:
        padding = kernel - 1
    oh, ow = maxpool_out_dim(H, kernel, stride, padding), maxpool_out_dim(W, kernel, stride, padding)
    if out is None:
        out = empty_nhwc((B, Cc, oh, ow), x.device)
    op, ops_ = _nhwc(out, "out")
    capi.check(capi.lib().pxe_maxpool_nhwc(_stream(), xp, xps, op, ops_, B, Cc, H, W, kernel, stride, padding))
    return out


def nhwc_to_nchw(x: torch.Tensor) -> torch.Tensor:
    """Dense NCHW copy of a channels-last tensor (for the decoders)."""
    xp, xps = _nhwc(x, "x")
    B, Cc, H, W = x.shape
    out = torch.empty((B, Cc, H, W), device=x.device, dtype=torch.float32)
    capi.check(capi.lib().pxe_nhwc_to_nchw(_stream(), xp, xps, out.data_ptr(), 0, B, Cc, H, W))
    return out


def region_decode(pred: torch.Tensor, width: int, height: int, num: int, coords: int, classes: int, anchors,
                  threshold: float, buf: DetectionBuffer, *, per_image: bool = False, img_w: float = 1.0,
                  img_h: float = 1.0, batch_id_offset: int = 0) -> None:
    """Appends a Region (YOLOv2) head's detections to ``buf``.  ``pred`` is the output of
    :func:`region_forward`.  ``per_image=False`` is the reference's behaviour: every image of the batch decodes
    image 0's predictions (include/RegionLayer.h:363-369)."""
    _check_f32_cuda(pred, "pred")
    if not pred.is_contiguous():
        raise ValueError("pred must be contiguous")
    B = pred.shape[0]
    if pred.numel() != B * width * height * num * (coords + 1 + classes):
        raise ValueError("pred does not have batch * width * height * num * (coords + 1 + classes) values")
    arr = (C.c_float * (2 * num))(*[float(a) for a in list(anchors)[:2 * num]])
    capi.check(capi.lib().pxe_region_decode(_stream(), pred.data_ptr(), B, width, height, num, coords, classes, arr,
                                            int(per_image), float(img_w), float(img_h), float(threshold),
                                            buf.dets.data_ptr(), buf.capacity, buf.count.data_ptr(), batch_id_offset))


def softmax_decode(probs: torch.Tensor, width: float, height: float, threshold: float, buf: DetectionBuffer, *,
                   batch_id_offset: int = 0) -> None:
    """Appends the classifier head's records (SoftmaxLayer::addDetects): one per image whose best class reaches
    the threshold.  ``probs``: [B, classes, ...] contiguous."""
    _check_f32_cuda(probs, "probs")
    if not probs.is_contiguous():
        raise ValueError("probs must be contiguous")
    B = probs.shape[0]
    classes = probs.numel() // B
    capi.check(capi.lib().pxe_softmax_decode(_stream(), probs.data_ptr(), classes, B, classes, float(width), float(height),
                                             float(threshold), buf.dets.data_ptr(), buf.capacity, buf.count.data_ptr(),
                                             batch_id_offset))


def conv_stem(x: torch.Tensor, weights: torch.Tensor, *, a: Optional[torch.Tensor] = None, b: Optional[torch.Tensor] = None,
              act="linear", out: Optional[torch.Tensor] = None, nhwc: bool = False) -> torch.Tensor:
    """First-layer 3x3 / stride 1 / padding 1 convolution fused with its epilogue.  ``x``: NCHW [B, Cin<=4, H, W];
    ``weights``: [Cout, Cin, 3, 3] contiguous; ``a``, ``b``: folded coefficients (:func:`fold_bn`).  The output is
    NCHW, or channels-last with ``nhwc=True``; ``out`` may be a channel slot of a wider buffer of that layout."""
    xp, xbs = _slot(x, "x")
    B, Cin, H, W = x.shape
    _check_f32_cuda(weights, "weights")
    if not weights.is_contiguous() or tuple(weights.shape[1:]) != (Cin, 3, 3):
        raise ValueError(f"weights must be a contiguous [Cout, {Cin}, 3, 3] tensor, got {tuple(weights.shape)}")
    Cout = weights.shape[0]
    if out is None:
        out = empty_nhwc((B, Cout, H, W), x.device) if nhwc else torch.empty((B, Cout, H, W), device=x.device)
    elif tuple(out.shape) != (B, Cout, H, W):
        raise ValueError(f"out has shape {tuple(out.shape)}, expected {(B, Cout, H, W)}")
    d = capi.StemDesc()
    d.x, d.x_batch_stride, d.weights = xp, xbs, weights.data_ptr()
    d.a, d.b = _vec(a, Cout, "a"), _vec(b, Cout, "b")
    d.y, d.y_stride = _nhwc(out, "out") if nhwc else _slot(out, "out")
    d.y_is_nhwc = int(nhwc)
    d.batch, d.in_channels, d.out_channels, d.height, d.width, d.act = B, Cin, Cout, H, W, _act(act)
    capi.check(capi.lib().pxe_conv_stem(_stream(), C.byref(d)))
    return out


def batchnorm_forward_training(x: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor, *, running_mean=None,
                               running_var=None, exp_avg_factor: float = 0.01, eps: float = 1e-5,
                               eps_mode: int = capi.EPS_CUDNN, act=None, y: Optional[torch.Tensor] = None):
    """Batch normalisation with batch statistics (cudnnBatchNormalizationForwardTraining as the reference's CUDA layers
    call it, include/cuda/ConvLayer.h:285-292; CPU twin src/BatchNorm.cpp:44-60).  Returns ``(y, y_act, save_mean,
    save_scale)``: the normalised tensor, its activation (``None`` without ``act``), the batch mean and
    1 / sqrt(var + eps) (``EPS_CUDNN``) or the population variance (``EPS_CPU``).  The running statistics are updated
    in place."""
    _check_f32_cuda(x, "x")
    if not x.is_contiguous():
        raise ValueError("batchnorm_forward_training: x must be dense NCHW")
    B, Cc, H, W = x.shape
    if y is None:
        y = torch.empty_like(x)
    y_act = torch.empty_like(x) if act is not None else None
    save_mean = torch.empty(Cc, device=x.device, dtype=torch.float32)
    save_scale = torch.empty(Cc, device=x.device, dtype=torch.float32)
    nbytes = capi.lib().pxe_batchnorm_workspace_bytes(B, Cc, H, W)
    ws = torch.empty(nbytes, device=x.device, dtype=torch.uint8)
    d = capi.BnTrainDesc()
    d.x, d.y, d.y_act = x.data_ptr(), y.data_ptr(), (y_act.data_ptr() if y_act is not None else None)
    d.act = _act(act if act is not None else "linear")
    d.batch, d.channels, d.height, d.width = B, Cc, H, W
    d.gamma, d.beta = _vec(gamma, Cc, "gamma"), _vec(beta, Cc, "beta")
    d.running_mean = _vec(running_mean, Cc, "running_mean") if running_mean is not None else None
    d.running_var = _vec(running_var, Cc, "running_var") if running_var is not None else None
    d.exp_avg_factor, d.eps, d.eps_mode = exp_avg_factor, eps, eps_mode
    d.save_mean, d.save_scale = save_mean.data_ptr(), save_scale.data_ptr()
    d.workspace, d.workspace_bytes = ws.data_ptr(), nbytes
    capi.check(capi.lib().pxe_batchnorm_forward_training(_stream(), C.byref(d)))
    return y, y_act, save_mean, save_scale


def batchnorm_backward(x: torch.Tensor, dy: torch.Tensor, gamma: torch.Tensor, save_mean: torch.Tensor,
                       save_scale: torch.Tensor, *, dgamma: Optional[torch.Tensor] = None,
                       dbeta: Optional[torch.Tensor] = None, eps: float = 1e-5, eps_mode: int = capi.EPS_CUDNN,
                       dx: Optional[torch.Tensor] = None) -> torch.Tensor:
    """cudnnBatchNormalizationBackward as the reference's CUDA layers call it (include/cuda/ConvLayer.h:327-332; CPU twin
    src/BatchNorm.cpp:68-98): returns dx; ``dgamma`` and ``dbeta`` are added to."""
    _check_f32_cuda(x, "x")
    _check_f32_cuda(dy, "dy")
    if not (x.is_contiguous() and dy.is_contiguous()) or x.shape != dy.shape:
        raise ValueError("batchnorm_backward: x and dy must be dense NCHW of one shape")
    B, Cc, H, W = x.shape
    if dx is None:
        dx = torch.empty_like(x)
    nbytes = capi.lib().pxe_batchnorm_workspace_bytes(B, Cc, H, W)
    ws = torch.empty(nbytes, device=x.device, dtype=torch.uint8)
    d = capi.BnBackwardDesc()
    d.x, d.dy, d.dx = x.data_ptr(), dy.data_ptr(), dx.data_ptr()
    d.batch, d.channels, d.height, d.width = B, Cc, H, W
    d.gamma = _vec(gamma, Cc, "gamma")
    d.dgamma = _vec(dgamma, Cc, "dgamma") if dgamma is not None else None
    d.dbeta = _vec(dbeta, Cc, "dbeta") if dbeta is not None else None
    d.save_mean, d.save_scale = _vec(save_mean, Cc, "save_mean"), _vec(save_scale, Cc, "save_scale")
    d.eps, d.eps_mode = eps, eps_mode
    d.workspace, d.workspace_bytes = ws.data_ptr(), nbytes
    capi.check(capi.lib().pxe_batchnorm_backward(_stream(), C.byref(d)))
    return dx


def adam_update(x: torch.Tensor, m: torch.Tensor, v: torch.Tensor, beta1: float, beta2: float, rate: float, eps: float,
                t: int) -> torch.Tensor:
    """px::adamGpu (src/Adam.cu:26-47): the parameter step from the moment estimates, in place on ``x``."""
    for name, tns in (("x", x), ("m", m), ("v", v)):
        _check_f32_cuda(tns, name)
        if not tns.is_contiguous() or tns.numel() != x.numel():
            raise ValueError("adam_update: x, m, v must be contiguous and of one size")
    capi.check(capi.lib().pxe_adam_update(_stream(), x.numel(), x.data_ptr(), m.data_ptr(), v.data_ptr(), beta1, beta2, rate, eps, t))
    return x


def softmax_cross_entropy(pred: torch.Tensor, truth: torch.Tensor):
    """px::softmaxCrossEntropy (src/SoftmaxKernel.cu:25-48): returns (delta, error)."""
    _check_f32_cuda(pred, "pred")
    _check_f32_cuda(truth, "truth")
    if not (pred.is_contiguous() and truth.is_contiguous()) or pred.numel() != truth.numel():
        raise ValueError("softmax_cross_entropy: pred and truth must be contiguous and of one size")
    delta, error = torch.empty_like(pred), torch.empty_like(pred)
    capi.check(capi.lib().pxe_softmax_cross_entropy(_stream(), pred.numel(), pred.data_ptr(), truth.data_ptr(), delta.data_ptr(),
                                                    error.data_ptr()))
    return delta, error
