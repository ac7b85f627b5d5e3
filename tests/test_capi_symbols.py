"""The C-ABI library loads and exports every symbol include/pxe.h declares (no compute calls)."""
import os
import re

from pixienn_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_in_header(name="pxe.h"):
    text = open(os.path.join(ROOT, "include", name)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"PXE_API\s+[\w\s\*]+?\b(pxe_\w+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    names = declared_in_header()
    assert len(names) >= 20
    L = capi.lib()
    for n in names:
        assert hasattr(L, n), f"{n} declared in pxe.h but not exported by libpxe.so"
        assert n in capi.PROTOTYPES, f"{n} has no ctypes prototype"
    assert sorted(capi.PROTOTYPES) == names, "ctypes prototypes and header declarations differ"


def test_planner_symbols_exported_and_bound():
    names = declared_in_header("pxe_plan.h")
    assert len(names) == 8
    L = capi.lib()
    for n in names:
        assert hasattr(L, n), f"{n} declared in pxe_plan.h but not exported by libpxe.so"
    assert sorted(capi.PLAN_PROTOTYPES) == names


def test_debug_symbols_exported_and_answer_unsupported():
    import ctypes as C
    names = declared_in_header("pxe_debug.h")
    assert sorted(capi.DEBUG_PROTOTYPES) == names and len(names) == 3
    L = capi.lib()
    for n in names:
        assert hasattr(L, n), f"{n} declared in pxe_debug.h but not exported by libpxe.so"
    assert L.pxe_debug_bounds_checked() == 0                  # the ordinary build
    rep = capi.BoundsReport()
    assert L.pxe_debug_read_report(C.byref(rep), 0) == capi.PXE_ERR_UNSUPPORTED
    assert L.pxe_debug_set_allocations(None, None, 0) == capi.PXE_ERR_UNSUPPORTED
    assert C.sizeof(capi.BoundsReport) == 80


def test_checked_build_exports_the_same_symbols():
    """libpxe_checked.so (the sources with -DPXE_BOUNDS_CHECK) is the same ABI; only pxe_debug_bounds_checked differs."""
    import ctypes as C
    from pixienn_b200 import debug
    L = C.CDLL(debug.CHECKED_LIB_PATH)
    for header in ("pxe.h", "pxe_plan.h", "pxe_debug.h"):
        for n in declared_in_header(header):
            assert hasattr(L, n), f"{n} declared in {header} but not exported by libpxe_checked.so"
    for n in capi.COMPAT_SYMBOLS:
        assert hasattr(L, n), n
    assert L.pxe_debug_bounds_checked() == 1
    assert L.pxe_debug_read_report(None, 0) == capi.PXE_ERR_BAD_ARG       # argument check comes before any CUDA call


def test_checked_library_is_chosen_before_the_first_load_only():
    """pixienn_b200.debug swaps the library for the bounds-checked one in a fresh process and refuses once libpxe.so is
    loaded; without a CUDA context nothing is armed, and the report reads through the same binding."""
    import subprocess
    import sys
    code = ("from pixienn_b200 import capi, debug\n"
            "debug.use_checked_library()\n"
            "L = capi.lib()\n"
            "assert L.pxe_debug_bounds_checked() == 1 and L.pxe_version() >= 100\n"
            "assert capi.LIB_PATH.endswith('libpxe_checked.so')\n"
            "r = capi.BoundsReport(); r.violations = 3; r.bytes = 16; r.address = 0x7f00; r.line = 96; r.file = b'pxe_nhwc.cu'\n"
            "assert debug.describe(r) == '3 refused accesses; first: 16-byte load at 0x7f00 (outside every allocation), pxe_nhwc.cu:96'\n"
            "print('ok')\n")
    res = subprocess.run([sys.executable, "-c", code], cwd=ROOT, capture_output=True, text=True)
    assert res.returncode == 0 and "ok" in res.stdout, res.stderr[-2000:]
    code = ("from pixienn_b200 import capi, debug\n"
            "capi.lib()\n"
            "try:\n    debug.use_checked_library()\nexcept RuntimeError as e:\n    print('refused:', e)\n")
    res = subprocess.run([sys.executable, "-c", code], cwd=ROOT, capture_output=True, text=True)
    assert res.returncode == 0 and "refused: use_checked_library() must run before" in res.stdout, res.stdout + res.stderr[-2000:]


def test_compat_tier_symbols_exported():
    L = capi.lib()
    for n in capi.COMPAT_SYMBOLS:
        assert hasattr(L, n), n


def test_version_and_status_strings():
    L = capi.lib()
    assert L.pxe_version() >= 100
    assert L.pxe_status_string(capi.PXE_OK) == b"ok"
    assert L.pxe_status_string(capi.PXE_ERR_WORKSPACE) == b"workspace too small"


def test_struct_layouts_match_header_sizes():
    import ctypes as C
    assert C.sizeof(capi.Detection) == 32
    # pointers 8, long long 8, ints/floats 4, natural alignment: same rule the C compiler applies
    assert C.sizeof(capi.EpilogueDesc) % 8 == 0
    assert capi.YoloDecodeDesc.mask.offset % 4 == 0 and capi.YoloDecodeDesc.anchors.size == 256


def test_host_only_entry_points():
    """Argument validation and pure-host helpers can run without a GPU."""
    L = capi.lib()
    assert L.pxe_maxpool_out_dim(416, 2, 2, 1) == 208
    assert L.pxe_maxpool_out_dim(13, 2, 2, 1) == 7
    assert L.pxe_yolo_decode_workspace_bytes(2, 13, 13) > 0
    assert L.pxe_centernet_decode_workspace_bytes(1, 20, 128, 128, 100) >= 20 * 8 * 100 * 8
    assert L.pxe_conv_epilogue(None, None) == capi.PXE_ERR_BAD_ARG
    assert L.pxe_nms_host(None, 0, 0.5, None) == 0
    # batch norm with batch statistics: workspace = per channel one coefficient slot and one partial sum per block
    # that shares the channel; refusals come before any launch
    import ctypes as C
    small = L.pxe_batchnorm_workspace_bytes(2, 8, 16, 16)
    large = L.pxe_batchnorm_workspace_bytes(64, 32, 208, 208)
    assert small >= 8 * 16 and large >= 32 * (16 + 8 * 64) and L.pxe_batchnorm_workspace_bytes(0, 8, 16, 16) == 0
    assert L.pxe_batchnorm_forward_training(None, None) == capi.PXE_ERR_BAD_ARG
    assert L.pxe_batchnorm_backward(None, None) == capi.PXE_ERR_BAD_ARG
    d = capi.BnTrainDesc()
    d.x = d.y = d.gamma = d.beta = d.save_mean = d.save_scale = 0x10000000
    d.batch, d.channels, d.height, d.width, d.eps_mode = 2, 8, 16, 16, 7
    assert L.pxe_batchnorm_forward_training(None, C.byref(d)) == capi.PXE_ERR_BAD_ARG and b"eps_mode" in L.pxe_last_error_string()
    d.eps_mode = capi.EPS_CUDNN
    assert L.pxe_batchnorm_forward_training(None, C.byref(d)) == capi.PXE_ERR_BAD_ARG and b"workspace" in L.pxe_last_error_string()
    assert L.pxe_adam_update(None, 10, None, None, None, 0.9, 0.999, 1e-3, 1e-8, 1) == capi.PXE_ERR_BAD_ARG
    assert L.pxe_adam_update(None, 0, None, None, None, 0.9, 0.999, 1e-3, 1e-8, 1) == capi.PXE_OK          # nothing to do
    assert L.pxe_softmax_cross_entropy(None, 5, None, None, None, None) == capi.PXE_ERR_BAD_ARG
    assert L.pxe_backward_bias(None, None, None, 4, 4, 4) == capi.PXE_ERR_BAD_ARG
    # the bias gradient indexes one filter's terms with an int: batch * size must fit 31 bits (addresses are never touched)
    assert L.pxe_backward_bias(None, 0x10000000, 0x20000000, 70000, 8, 70000) == capi.PXE_ERR_BAD_ARG
    assert b"31 bits" in L.pxe_last_error_string()
    e = capi.EpilogueDesc()
    e.x = e.y = 0x10000000
    e.batch, e.channels, e.height, e.width = 1, 4, 4, 4
    e.folded_a = 0x20000000                      # one of the two folded arrays only
    assert L.pxe_conv_epilogue(None, C.byref(e)) == capi.PXE_ERR_BAD_ARG and b"folded" in L.pxe_last_error_string()


def test_overlapping_tensors_are_refused_before_any_launch():
    """A destination that shares elements with an input or with another destination -- other than being that very
    tensor -- is refused, batch strides or not.  (Channel slots of one buffer interleave without sharing and are
    accepted: the GPU suites store into them.)  Pointers here are never dereferenced: validation fails first."""
    import ctypes as C
    L = capi.lib()
    base = 0x10000000

    def desc(**kw):
        d = capi.EpilogueDesc()
        d.x, d.batch, d.channels, d.height, d.width = base, 4, 6, 10, 10          # 600 floats per image
        d.x_batch_stride = 1000
        for k, v in kw.items():
            setattr(d, k, v)
        return d

    cases = [
        desc(y=base + 4 * 300, y_batch_stride=1000),                       # y starts inside every image of x
        desc(y=base + 4 * 1000, y_batch_stride=1000),                      # image i of y is image i+1 of x
        desc(y=base + 4 * 5000, y2=base + 4 * 100, y2_batch_stride=1000),  # second store into x's images
        desc(y=base + 4 * 5000, y2=base + 4 * 5200),                       # the two stores overlap each other
        desc(y=base + 4 * 5000, residual=base + 4 * 5300),                 # y would overwrite residual values not yet read
        desc(y=base + 4 * 5000, pool_kernel=2, pool_stride=2, pool_padding=0, y_pool=base + 4 * 5100),
        desc(y=None, pool_kernel=2, pool_stride=2, pool_padding=0, y_pool=base, y_pool_batch_stride=1000),
    ]
    for d in cases:
        assert L.pxe_conv_epilogue(None, C.byref(d)) == capi.PXE_ERR_BAD_ARG, L.pxe_last_error_string()
        assert b"overlap" in L.pxe_last_error_string() or b"is y" in L.pxe_last_error_string()
