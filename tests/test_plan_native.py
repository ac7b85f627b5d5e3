"""The library's C++ planner (include/pxe_plan.h) against the Python planner it mirrors: same
steps, destinations, aliases, concat buffers, release points and counters for every preset, fused
and layer-by-layer, and for every model file of the reference when its tree is present."""
import ctypes as C
import glob
import os

import pytest

from oracle.pxoracle import reference_root
from pixienn_b200 import capi, graph, presets

PRESETS = [("yolov3_tiny", 416), ("yolov3", 608), ("yolov7", 640), ("centernet_tiny", 320)]
REFERENCE_MODELS = sorted(glob.glob(os.path.join(reference_root() or "", "resources", "models", "*.yml")))


def same_plan(a: graph.Plan, b: graph.Plan):
    assert len(a.steps) == len(b.steps)
    for x, y in zip(a.steps, b.steps):
        assert x == y, f"step for layer {x.layer}:\n {x}\n {y}"
    assert a.alias == b.alias
    assert a.concat_channels == b.concat_channels
    assert a.last_use == b.last_use
    assert a.stats == b.stats


@pytest.mark.parametrize("name,size", PRESETS)
@pytest.mark.parametrize("fuse,raw_heads", [(True, True), (True, False), (False, True)])
def test_native_plan_equals_python_plan_on_presets(name, size, fuse, raw_heads):
    model = graph.parse_model(getattr(presets, name)(size, size))
    same_plan(graph.plan_native(model, fuse, raw_heads), graph.plan(model, fuse, raw_heads))


@pytest.mark.skipif(not REFERENCE_MODELS, reason="the reference tree is not present")
@pytest.mark.parametrize("path", REFERENCE_MODELS, ids=[os.path.basename(p) for p in REFERENCE_MODELS])
def test_native_plan_equals_python_plan_on_reference_models(path):
    try:
        model = graph.parse_model(graph.load_yaml(path))
    except ValueError as e:                      # a layer type outside the inference path
        pytest.skip(str(e))
    for fuse in (True, False):
        same_plan(graph.plan_native(model, fuse), graph.plan(model, fuse))


def test_plan_entry_points_validate_their_arguments():
    L = capi.lib()
    handle = C.c_void_p()
    assert L.pxe_plan_build(None, 0, 1, 1, C.byref(handle)) == capi.PXE_ERR_BAD_ARG
    d = (capi.LayerDesc * 2)()
    d[0].type, d[0].out_channels, d[0].out_height, d[0].out_width, d[0].n_sources = 0, 8, 4, 4, 1
    d[0].sources[0] = -1
    d[1].type, d[1].out_channels, d[1].out_height, d[1].out_width, d[1].n_sources = 3, 8, 4, 4, 1
    d[1].sources[0] = 1                          # a route that reads itself
    assert L.pxe_plan_build(d, 2, 1, 1, C.byref(handle)) == capi.PXE_ERR_BAD_ARG
    assert b"does not precede" in L.pxe_last_error_string()
    d[1].sources[0] = 0
    assert L.pxe_plan_build(d, 2, 1, 1, C.byref(handle)) == capi.PXE_OK
    assert L.pxe_plan_step_count(handle) == 2 and L.pxe_plan_alias(handle, 1) == 0
    assert not L.pxe_plan_step(handle, 2) and L.pxe_plan_step(handle, 1).contents.op == 1
    assert L.pxe_plan_last_use(handle, -1) == 0 and L.pxe_plan_last_use(handle, 1) == -1
    L.pxe_plan_destroy(handle)
