"""The workspace-free YOLO decode (pxe_yolo_decode_static) against the ordinary one.

For integrators who cannot hand the decode a scratch buffer -- code running where device memory
was fixed at start-up, or inside a per-frame call that must not allocate -- the library keeps a
4 MiB scratch array of its own.  This test drives both entry points through the C ABI on the same
heads and requires identical records, twice in a row: the second call decodes a different, smaller
head, so whatever the first call left in the shared array must not leak into it.
The file name sorts last on purpose: a run that stops at the first failure has by then run every
other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from pixienn_b200 import capi, ops, synth

pytestmark = pytest.mark.gpu

ANCHORS = [10, 13, 16, 30, 33, 23, 30, 61, 62, 45, 59, 119, 116, 90, 156, 198, 373, 326]


def make_desc(head, mask, classes, thr):
    B, _, H, W = head.shape
    d = capi.YoloDecodeDesc()
    d.head, d.head_batch_stride = head.data_ptr(), 0
    d.head_is_raw, d.bias = 1, None
    d.batch, d.height, d.width, d.classes = B, H, W, classes
    d.n_masks = len(mask)
    for i, m in enumerate(mask):
        d.mask[i] = m
    d.n_anchor_values = len(ANCHORS)
    for i, a in enumerate(ANCHORS):
        d.anchors[i] = a
    d.net_width = d.net_height = 416
    d.threshold = thr
    return d


def decode_both(cuda, seed, B, classes, hw, mask):
    L = capi.lib()
    raw = synth.normal(seed, f"noalloc{hw}", (B, 3 * (classes + 5), hw, hw), 0.0, 1.5)
    raw.reshape(B, 3, classes + 5, hw, hw)[:, :, 4] -= 1.0
    head = torch.from_numpy(raw).to(cuda)
    d = make_desc(head, mask, classes, 0.2)
    cap = B * hw * hw * 3 * classes
    stream = torch.cuda.current_stream().cuda_stream
    out = []
    for static in (False, True):
        dets = torch.zeros((cap, 8), device=cuda, dtype=torch.int32)
        count = torch.zeros(1, device=cuda, dtype=torch.int64)
        if static:
            rc = L.pxe_yolo_decode_static(stream, C.byref(d), dets.data_ptr(), cap, count.data_ptr())
        else:
            need = L.pxe_yolo_decode_workspace_bytes(B, hw, hw)
            ws = torch.empty(need, device=cuda, dtype=torch.uint8)
            rc = L.pxe_yolo_decode(stream, C.byref(d), dets.data_ptr(), cap, count.data_ptr(), ws.data_ptr(), need)
        capi.check(rc)
        torch.cuda.synchronize()
        n = int(count.item())
        out.append(dets[:n].cpu().numpy().view(ops.DET_DTYPE).reshape(-1))
    return out


def test_static_scratch_decode_equals_workspace_decode_twice(cuda):
    first = decode_both(cuda, 101, 4, 6, 26, [3, 4, 5])
    assert len(first[0]) > 100
    assert first[0].tobytes() == first[1].tobytes()
    second = decode_both(cuda, 102, 2, 3, 13, [0, 1, 2])      # smaller head: stale scratch beyond it is ignored
    assert len(second[0]) > 10
    assert second[0].tobytes() == second[1].tobytes()


def test_static_scratch_refuses_heads_beyond_its_size(cuda):
    L = capi.lib()
    B, hw = 2048, 152                                         # 2048 x 152 x 152 cells need about 17 MB > 4 MiB
    assert L.pxe_yolo_decode_workspace_bytes(B, hw, hw) > (4 << 20)
    d = capi.YoloDecodeDesc()
    d.batch, d.height, d.width, d.classes = B, hw, hw, 1
    count = torch.zeros(1, device=cuda, dtype=torch.int64)
    rc = L.pxe_yolo_decode_static(None, C.byref(d), None, 0, count.data_ptr())
    assert rc == capi.PXE_ERR_WORKSPACE
    msg = L.pxe_last_error_string().decode()
    assert "built-in array" in msg and "pxe_yolo_decode" in msg
    torch.cuda.synchronize()
