"""The boundary from the reference's own languages: the public headers compile as strict C99, and a C++
program that includes them (and the px:: declarations of the link-compatible tier) links against
libpxe.so and runs the host-only entry points."""
import os
import shutil
import subprocess

import pytest

from pixienn_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
INC = os.path.join(ROOT, "include")
SRC = os.path.join(ROOT, "tests", "cpp")


@pytest.mark.skipif(shutil.which("gcc") is None, reason="gcc not found")
def test_headers_compile_as_c99(tmp_path):
    obj = tmp_path / "header_is_c.o"
    r = subprocess.run(["gcc", "-std=c99", "-pedantic", "-Wall", "-Wextra", "-Werror", "-I", INC, "-c",
                        os.path.join(SRC, "header_is_c.c"), "-o", str(obj)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr


def test_ctypes_mirrors_have_the_layout_the_c_compiler_gives(tmp_path):
    """sizeof and a few offsetof values of every descriptor, as gcc lays them out from include/pxe.h, against the ctypes
    structures the Python binding passes."""
    import ctypes as C
    exe = tmp_path / "struct_sizes"
    r = subprocess.run(["gcc", "-std=c99", "-I", INC, os.path.join(SRC, "struct_sizes.c"), "-o", str(exe)],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    out = dict(line.rsplit(" ", 1) for line in subprocess.run([str(exe)], capture_output=True, text=True).stdout.splitlines())
    mirrors = {"pxe_detection": capi.Detection, "pxe_epilogue_desc": capi.EpilogueDesc,
               "pxe_epilogue_nhwc_desc": capi.EpilogueNhwcDesc, "pxe_yolo_decode_desc": capi.YoloDecodeDesc,
               "pxe_centernet_decode_desc": capi.CenterNetDecodeDesc, "pxe_yolo_loss_desc": capi.YoloLossDesc,
               "pxe_bn_train_desc": capi.BnTrainDesc, "pxe_bn_backward_desc": capi.BnBackwardDesc,
               "pxe_layer_desc": capi.LayerDesc, "pxe_step": capi.PlanStep, "pxe_bounds_report": capi.BoundsReport}
    for name, cls in mirrors.items():
        assert C.sizeof(cls) == int(out[name]), (name, C.sizeof(cls), out[name])
    for key, value in out.items():
        if "." in key:
            name, field = key.split(".")
            assert getattr(mirrors[name], field).offset == int(value), (key, value)


@pytest.mark.skipif(shutil.which("g++") is None, reason="g++ not found")
def test_cpp_client_links_and_runs(tmp_path):
    capi.lib()                                            # the library exists (raises with build instructions otherwise)
    libdir = os.path.dirname(capi.LIB_PATH)
    exe = tmp_path / "link_client"
    cuda_inc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")   # dim3 (px::cudaGridsize)
    r = subprocess.run(["g++", "-std=c++17", "-Wall", "-Wextra", "-I", INC, "-I", cuda_inc, os.path.join(SRC, "link_client.cpp"),
                        "-L", libdir, "-lpxe", f"-Wl,-rpath,{libdir}", "-o", str(exe)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    run = subprocess.run([str(exe)], capture_output=True, text=True)
    assert run.returncode == 0, (run.returncode, run.stdout, run.stderr)
    assert "steps=4 fused_pool=1 fused_shortcut=1 raw_heads=1" in run.stdout
    assert "nms kept=2" in run.stdout and "px:: symbols resolved" in run.stdout


@pytest.mark.skipif(shutil.which("g++") is None, reason="g++ not found")
def test_shim_fragments_compile_inside_stand_in_layers(tmp_path):
    """include/shim/*.inl are the replacement bodies for the reference's CUDA forward / addDetects members.  They are
    compiled here inside member functions of stand-in classes that carry the reference's member names, with the
    entry points recorded instead of launched; the program then checks which pointers and strides the plan made the
    conv fragment put into pxe_epilogue_desc for a folded shortcut and two concat slots."""
    capi.lib()
    libdir = os.path.dirname(capi.LIB_PATH)
    exe = tmp_path / "shim_standin"
    r = subprocess.run(["g++", "-std=c++17", "-Wall", "-Wextra", "-Werror", "-I", INC, os.path.join(SRC, "shim_standin.cpp"),
                        "-L", libdir, "-lpxe", f"-Wl,-rpath,{libdir}", "-o", str(exe)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    run = subprocess.run([str(exe)], capture_output=True, text=True)
    assert run.returncode == 0 and run.stdout.startswith("ok: epilogues=2 concats=0"), (run.stdout, run.stderr)
    # second graph: a folded pool and the later pools of an SPP block run nothing, the block's first pool makes one pxe_spp
    # call into the route's slots, the upsample writes its route slot, a stand-alone pool and two kinds of shortcut
    assert "ok: pools=1 spp=1 upsamples=1 shortcuts=1 general=1" in run.stdout, run.stdout
    # heads that need no plan: Region forward and addDetects (the reference's image-0 indexing kept), softmax with groups and
    # temperature, the global average pool
    assert "ok: region=1 region_decode=1 softmax=1 avgpool=1" in run.stdout, run.stdout
    # the connected layer's epilogue (a 1x1 map, in place) and the YOLOv1 head decode
    assert "ok: connected=1 detect=1" in run.stdout, run.stdout


@pytest.mark.gpu
@pytest.mark.skipif(shutil.which("g++") is None, reason="g++ not found")
def test_cpp_program_drives_the_c_abi_on_the_gpu(tmp_path):
    """No Python and no torch between the caller and the kernels: a C++ program with the CUDA runtime fills the
    descriptors, launches on its own stream and checks the results itself."""
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    libdir = os.path.dirname(capi.LIB_PATH)
    exe = tmp_path / "epilogue_client"
    r = subprocess.run(["g++", "-std=c++17", "-O1", "-I", INC, "-I", os.path.join(cuda_home, "include"),
                        os.path.join(SRC, "epilogue_client.cpp"), "-L", libdir, "-lpxe", f"-Wl,-rpath,{libdir}",
                        "-L", os.path.join(cuda_home, "lib64"), "-lcudart", f"-Wl,-rpath,{os.path.join(cuda_home, 'lib64')}",
                        "-o", str(exe)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    run = subprocess.run([str(exe)], capture_output=True, text=True)
    assert run.returncode == 0, (run.returncode, run.stdout, run.stderr)
    assert run.stdout.startswith("ok:")


def _nvcc():
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    return None


@pytest.mark.skipif(_nvcc() is None, reason="nvcc not found")
def test_index_division_is_exact(tmp_path):
    """FastDiv (csrc/pxe_common.cuh), the multiply-high division every kernel's index arithmetic uses: the device
    formula with the constructor's constants equals n / d for 7109 divisors (every one up to 5000, powers of two and
    their neighbours, the model shapes, random odd 32-bit values) over 31.7 M values of n -- small ones, the ends of the
    32-bit range, the neighbours of multiples of d, random ones.  A host program; no GPU."""
    exe = tmp_path / "fastdiv_check"
    r = subprocess.run([_nvcc(), "-std=c++17", "-O2", "-gencode", "arch=compute_100a,code=sm_100a", "-I", INC, "-I",
                        os.path.join(ROOT, "pixienn_b200", "csrc"), os.path.join(SRC, "fastdiv_check.cu"), "-o", str(exe)],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    run = subprocess.run([str(exe)], capture_output=True, text=True)
    assert run.returncode == 0 and run.stdout.startswith("ok: 7109 divisors"), run.stdout + run.stderr
