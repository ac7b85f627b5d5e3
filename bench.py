#!/usr/bin/env python
"""Benchmark of the per-layer epilogue path on B200.

  python bench.py --gpus N --steps K --warmup W            the new kernels (one rank per GPU)
  python bench.py --impl reference ...                      the reference's CPU path on the host cores

Workload (default): YOLOv3 on a Darknet-53 backbone, 608x608, 64 images per GPU, fp32, random-init
weights from a seed, inference.  One step = one forward pass of the hot path over one batch:
every convolution on cuDNN (through torch, as the reference keeps it on cuDNN) and everything
between the convolutions -- BN, bias, activation, shortcut, upsample, route, YOLO decode -- on the
kernels of libpxe.so.  `value` is images/s with the input batch resident in HBM; `e2e` is the same
through Runner.predict with a pinned HOST batch in and host detections out.  The batch is sharded
by image across ranks; there is no collective on the data path.

Other workloads (not run by default): --workload sweep (the isolated fused-epilogue sweep),
--workload centernet (the CenterNet head decode), --workload pools (SPP block and stand-alone max pools),
--workload bn-train (batch normalisation with batch statistics, forward and backward),
--workload aux (the kernels no model run or sweep times: generic pools and moves, small heads, NMS, training-side),
--workload yolov3-tiny | yolov7.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

SEED = 1234
CONF = 0.2
NMS = 0.4

# A head that behaves like a trained one, for the end-to-end arm that gathers final detections.  With the plain
# seeded init a deep residual graph drives its heads to logits of magnitude 1e6: every box is certain or absent and
# 228 k candidates per image pass the confidence threshold.  Here the head convolutions' weights are scaled back
# to logits of order one (powers of two, so products stay exact) and the objectness / class biases lowered.
HEAD_VARIANT = {
    "yolov3-608": dict(head_bias=-4.0, class_bias=-1.0, head_gain={81: 2.0 ** -19, 93: 2.0 ** -19, 105: 2.0 ** -18}),
    "yolov3-tiny": dict(head_bias=-4.0, class_bias=-1.0, head_gain=0.5),
    "yolov7": dict(head_bias=-4.0, class_bias=-1.0, head_gain=11.0),
}
HEAD_VARIANT_NOTE = {
    "yolov3-608": "head conv weights x 2^-19 / 2^-19 / 2^-18 (logits of order one), objectness bias -4, class bias -1",
    "yolov3-tiny": "head conv weights x 0.5, objectness bias -4, class bias -1",
    "yolov7": "head conv weights x 11 (about a thousand candidates per image), objectness bias -4, class bias -1",
}

def traffic_ratios():
    """DRAM bytes (ncu dram__bytes_read.sum + dram__bytes_write.sum of one capture) divided by the algorithmic
    bytes of the captured launch, per kind of launch, read from the table in profiles/traffic_ratios.md -- which
    names the kernel and the capture each figure comes from, so a changed kernel shows up as a stale row there
    and not as a constant here.  Traffic grows in proportion to the tensor, so a launch's traffic is this ratio
    times its algorithmic bytes."""
    out = {}
    path = os.path.join(ROOT, "profiles", "traffic_ratios.md")
    if not os.path.exists(path):
        return out
    with open(path) as f:
        for line in f:
            cells = [c.strip() for c in line.strip().strip("|").split("|")]
            if len(cells) >= 4 and cells[0] and not set(cells[0]) <= set("-: ") and cells[0] != "kind":
                try:
                    out[cells[0]] = {"ratio": float(cells[3]), "kernel": cells[1], "capture": cells[2]}
                except ValueError:
                    continue
    return out


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s: no MEASURED_PEAKS.json beside bench.py)"


class ClockSampler:
    """nvidia-smi samples of one GPU while the timed region runs (read-only queries)."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.proc, self.file = gpu_index, None, None

    def start(self):
        try:
            self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        sm, mx, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.file.read().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1])); power.append(float(parts[2]))
            except ValueError:
                continue
            for n, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        name = self.file.name
        self.file.close()
        os.unlink(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "power_w_max": max(power),
                "samples": len(sm), "reasons": sorted(reasons)}


def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


def make_doc(workload: str):
    from pixienn_b200 import presets
    if workload == "yolov3-608":
        return presets.yolov3(608, 608), "YOLOv3 (Darknet-53) 608x608"
    if workload == "yolov3-tiny":
        return presets.yolov3_tiny(416, 416), "YOLOv3-tiny 416x416"
    if workload == "yolov7":
        return presets.yolov7(640, 640), "YOLOv7 640x640"
    raise SystemExit(f"unknown workload {workload}")


def host_batch(model, batch, first_image):
    from pixienn_b200 import synth
    return np.stack([synth.uniform(SEED, f"input/{first_image + b}", (model.channels, model.height, model.width))
                     for b in range(batch)])


# ------------------------------------------------------------------------------------- our arm
def run_model(args):
    import torch
    import torch.distributed as dist
    from pixienn_b200 import capi, graph
    from pixienn_b200.runner import Runner, synth_weights

    rank, local_rank, world = dist_env()
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    capi.lib()                                     # no library, no benchmark: there is no fallback path
    torch.backends.cudnn.benchmark = not args.no_cudnn_benchmark   # the reference picks its conv algorithm with cudnnFind*

    doc, label = make_doc(args.workload)
    model = graph.parse_model(doc)
    B = args.batch
    weights = synth_weights(model, SEED)
    runner = Runner(model, weights, B, dev, det_capacity=args.det_capacity, threshold=CONF,
                    batch_id_offset=rank * B, layout=args.layout, fused_stem=args.fused_stem,
                    conv_fusion=args.conv_fusion and args.layout == "nhwc")
    xh = torch.from_numpy(host_batch(model, B, rank * B)).pin_memory()
    x = xh.to(dev)
    pinned_dets = None

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        runner.forward(x)
    barrier()

    # ---- timed region: K steps, inputs resident in HBM
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    runner.timer.enabled = True
    runner.timer.clear()
    launches = 0
    use_graph = args.cuda_graph != "off"
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t0.record()
    for _ in range(args.steps):
        runner.forward(x)
        launches += runner.launches
    t1.record()
    barrier()
    if use_graph:
        # The eager pass above (kept for the per-kernel event timings of the breakdown and the roofline) pays the
        # host's launch cost and two event records per kernel: 3 % of a step at 64 images, 20 % at 16, 70 % at 1.
        # The reported step time is the same pass replayed as one CUDA graph.
        eager_ms = t0.elapsed_time(t1)
        runner.timer.enabled = False
        cg = runner.capture(x)
        for _ in range(args.warmup):
            cg.replay()
        barrier()
        t0.record()
        for _ in range(args.steps):
            cg.replay()
        t1.record()
        barrier()
        runner.timer.enabled = True
        del cg
    clocks = sampler.stop() if rank == 0 else None
    ms = torch.tensor([t0.elapsed_time(t1)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    total_ms = float(ms.item())
    ops_summary = runner.timer.summary()
    runner.timer.enabled = False
    n_dets = int(runner.dets.count.item())

    # ---- end to end: pinned host batch in, detections on the host out, every step.  Copies of neighbouring
    # steps overlap compute (PipelinedPredictor); each step still moves its own input and its own detections.
    from pixienn_b200.runner import PipelinedPredictor
    del pinned_dets
    pipe = PipelinedPredictor(runner, tuple(xh.shape), use_graphs=use_graph)
    pipe.submit(xh)
    pipe.drain()
    barrier()
    w0 = time.perf_counter()
    n_host = 0
    for _ in range(args.steps):
        res = pipe.submit(xh)
        if res is not None:
            n_host = len(res[0])
    res = pipe.drain()
    n_host = len(res[0])
    torch.cuda.synchronize()
    wall_ms = (time.perf_counter() - w0) * 1e3       # host wall clock: the last result is on the host when it stops
    barrier()
    e2e_ms = torch.tensor([wall_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)
    e2e_total_ms = float(e2e_ms.item())

    # ---- the same forward with channels-last activations (the library's NHWC tier), with cuDNN for every
    # convolution and with the first convolution fused with its epilogue (pxe_conv_stem): reported beside the
    # headline number, which stays on the reference's NCHW layout and cuDNN calls
    def time_runner(r2, x_dev, xh_pinned, nms_threshold=None, prepare=False):
        """(device ms, end-to-end wall ms) for args.steps steps of runner r2, each the max over ranks: resident
        input (one CUDA-graph replay per step unless --cuda-graph off), then host batch in / host records out
        through PipelinedPredictor (with px::nms on the device when nms_threshold is given)."""
        if prepare:
            r2.forward(x_dev)            # the eager pass in which every layer shape times its fused plans once
            torch.cuda.synchronize()
        step2 = r2.capture(x_dev).replay if use_graph else (lambda: r2.forward(x_dev))
        for _ in range(args.warmup):
            step2()
        barrier()
        t0.record()
        for _ in range(args.steps):
            step2()
        t1.record()
        barrier()
        alt_ms = torch.tensor([t0.elapsed_time(t1)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(alt_ms, op=dist.ReduceOp.MAX)
        del step2
        pipe2 = PipelinedPredictor(r2, tuple(xh_pinned.shape), use_graphs=use_graph, nms_threshold=nms_threshold)
        pipe2.submit(xh_pinned)
        pipe2.drain()
        barrier()
        w0 = time.perf_counter()
        for _ in range(args.steps):
            pipe2.submit(xh_pinned)
        last = pipe2.drain()
        torch.cuda.synchronize()
        alt_wall = torch.tensor([(time.perf_counter() - w0) * 1e3], device=dev, dtype=torch.float64)
        barrier()
        if world > 1:
            dist.all_reduce(alt_wall, op=dist.ReduceOp.MAX)
        return float(alt_ms.item()), float(alt_wall.item()), len(last[0]), int(last[1])

    def measure_variant(layout, fused_stem, note, conv_fusion=False):
        r2 = Runner(model, weights, B, dev, det_capacity=args.det_capacity, threshold=CONF, batch_id_offset=rank * B,
                    layout=layout, fused_stem=fused_stem, conv_fusion=conv_fusion)
        r2.dets = runner.dets
        alt_ms, alt_wall, _, _ = time_runner(r2, x, xh, prepare=conv_fusion)
        extra = {}
        if conv_fusion:
            extra = {"conv_fusion": dict(r2.fused_conv.summary(), launches_per_step=r2.fused_conv_launches)}
            if args.fusion_shapes:
                extra["conv_fusion"]["shapes_timed"] = [
                    {"x": list(k[0]), "w": list(k[1]), "stride": k[2], "shortcut": bool(k[7]), "choice": c,
                     "fused_ms": f and round(f, 4), "split_ms": round(sp, 4)} for k, c, f, sp in r2.fused_conv.log]
        return {"layout": layout, "fused_stem": bool(r2.stem is not None), **extra,
                "value": round(B * world * args.steps / (alt_ms / 1e3), 2), "unit": "images/s",
                "ms_per_step": round(alt_ms / args.steps, 3),
                "e2e_value": round(B * world * args.steps / (alt_wall / 1e3), 2),
                "note": note + "; same graph, weights and input; resident input, "
                        + ("one CUDA graph replay per step" if use_graph else "eager launches")}

    # ---- the same model with a head that behaves like a trained one (see HEAD_VARIANT): candidates per image in
    # the thousands instead of 228 k, px::nms on the device, only survivors copied to the host
    def measure_post_nms():
        hw = synth_weights(model, SEED, **HEAD_VARIANT[args.workload])
        r2 = Runner(model, hw, B, dev, det_capacity=args.det_capacity, threshold=CONF, batch_id_offset=rank * B)
        ms2, wall2, kept, total = time_runner(r2, x, xh, nms_threshold=NMS)
        # the decode's own time on this head: eager passes with events around every launch
        r2.timer.enabled = True
        r2.timer.clear()
        for _ in range(3):
            r2.forward(x)
        torch.cuda.synchronize()
        dec = r2.timer.summary().get("yolo_decode", {"ms": 0.0, "bytes": 0})
        r2.timer.enabled = False
        return {"decode_ms": round(dec["ms"] / 3, 4), "decode_head_bytes": int(dec["bytes"] / 3),
                "value": round(B * world * args.steps / (wall2 / 1e3), 2), "unit": "images/s",
                "resident_value": round(B * world * args.steps / (ms2 / 1e3), 2),
                "candidates_per_step_per_gpu": total, "survivors_per_step_per_gpu": kept,
                "d2h_bytes_per_step": kept * 32 + 16,
                "head": HEAD_VARIANT_NOTE[args.workload]}

    # ---- the configured split of the same global batch over the ranks (strong scaling): B / world images per rank
    def measure_strong():
        per = max(1, B // world)
        r2 = Runner(model, weights, per, dev, det_capacity=args.det_capacity, threshold=CONF, batch_id_offset=rank * per)
        xs_h = torch.from_numpy(host_batch(model, per, rank * per)).pin_memory()
        ms2, wall2, _, _ = time_runner(r2, xs_h.to(dev), xs_h)
        return {"per_gpu_batch": per, "global_batch": per * world,
                "value": round(per * world * args.steps / (ms2 / 1e3), 2),
                "e2e": round(per * world * args.steps / (wall2 / 1e3), 2), "ms_per_step": round(ms2 / args.steps, 3)}

    # ---- BASELINE.json's YOLOv7-640 configuration: 16 images per GPU (128 over 8 GPUs)
    def measure_c3():
        doc3, _ = make_doc("yolov7")
        m3 = graph.parse_model(doc3)
        w3 = synth_weights(m3, SEED)
        r3 = Runner(m3, w3, 16, dev, det_capacity=args.det_capacity, threshold=CONF, batch_id_offset=rank * 16)
        x3_h = torch.from_numpy(host_batch(m3, 16, rank * 16)).pin_memory()
        x3 = x3_h.to(dev)
        for _ in range(2):
            r3.forward(x3)
        ms3, wall3, _, _ = time_runner(r3, x3, x3_h)
        out = {"per_gpu_batch": 16, "global_batch": 16 * world, "value": round(16 * world * args.steps / (ms3 / 1e3), 2),
               "e2e": round(16 * world * args.steps / (wall3 / 1e3), 2), "ms_per_step": round(ms3 / args.steps, 3)}
        # the same with the trained-like head, NMS on the device and only the survivors copied (e2e.post_nms_* above)
        del r3
        torch.cuda.empty_cache()
        r4 = Runner(m3, synth_weights(m3, SEED, **HEAD_VARIANT["yolov7"]), 16, dev, det_capacity=args.det_capacity,
                    threshold=CONF, batch_id_offset=rank * 16)
        for _ in range(2):
            r4.forward(x3)
        _, wall4, kept4, total4 = time_runner(r4, x3, x3_h, nms_threshold=NMS)
        out.update(post_nms_e2e=round(16 * world * args.steps / (wall4 / 1e3), 2), post_nms_candidates_per_step_per_gpu=total4,
                   post_nms_survivors_per_step_per_gpu=kept4)
        return out

    alt = alt_stem = nchw_stem = alt_fusion = None
    if args.layout == "nchw" and not args.no_alt_layout:
        del pipe
        torch.cuda.empty_cache()
        if not args.fused_stem:
            nchw_stem = measure_variant("nchw", True, "the reference's layout, and the first convolution + its epilogue as one "
                                                      "launch of this library instead of cuDNN + epilogue")
            torch.cuda.empty_cache()
        alt = measure_variant("nhwc", False, "activations channels-last between layers, so cuDNN converts no layouts around "
                                             "its convolutions")
        torch.cuda.empty_cache()
        alt_stem = measure_variant("nhwc", True, "channels-last, and the first convolution + its epilogue as one launch of "
                                                 "this library instead of cuDNN + epilogue")
        torch.cuda.empty_cache()
        if not args.no_conv_fusion:
            try:
                alt_fusion = measure_variant(
                    "nhwc", True, "channels-last, fused first layer, and every other convolution whose cuDNN runtime-fusion "
                                  "plan (conv + scale + bias + activation + shortcut in one launch) measured faster than "
                                  "cuDNN convolution + this library's epilogue", conv_fusion=True)
            except Exception as e:                     # e.g. an image without the cuDNN frontend: reported, not hidden
                alt_fusion = {"unavailable": f"{type(e).__name__}: {str(e)[:200]}"}
            torch.cuda.empty_cache()

    post_nms = strong = c3 = None
    if args.workload == "yolov3-608" and not args.no_extras:
        try:
            del pipe
        except NameError:
            pass
        torch.cuda.empty_cache()
        post_nms = measure_post_nms()
        torch.cuda.empty_cache()
        strong = measure_strong() if world > 1 else None
        torch.cuda.empty_cache()
        c3 = measure_c3()
        torch.cuda.empty_cache()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    images = B * world * args.steps
    value = images / (total_ms / 1e3)
    peak, peak_src = measured_peaks()
    ratios = traffic_ratios()
    mine = {k: v for k, v in ops_summary.items() if "cudnn" not in k}       # this library's kernels only
    dom = max(mine, key=lambda k: mine[k]["ms"])
    d = mine[dom]
    achieved = d["bytes"] / (d["ms"] / 1e3) / 1e9
    breakdown = {k: {"launches_per_step": v["launches"] // args.steps, "ms_per_step": round(v["ms"] / args.steps, 4),
                     "GBps": (round(v["bytes"] / (v["ms"] / 1e3) / 1e9, 1) if v["bytes"] and v["ms"] > 0 else None)}
                 for k, v in ops_summary.items()}
    epi_ms = sum(v["ms"] for v in mine.values()) / args.steps
    epi_bytes = sum(v["bytes"] for v in mine.values()) / args.steps

    line = {
        "metric": "YOLOv3 608x608 inference throughput" if args.workload == "yolov3-608" else f"{label} inference throughput",
        "value": round(value, 2), "unit": "images/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(total_ms / args.steps, 3),
        "eager_ms_per_step": round(eager_ms / args.steps, 3) if use_graph else None,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{label}, {B} images per GPU, global batch {B * world}, fp32 {args.layout.upper()}, random-init weights "
                               f"(seed {SEED}), conf {CONF}; conv on cuDNN (TF32 allowed, cuDNN's default math mode), "
                               "epilogue/shortcut/upsample/route/decode on libpxe.so",
                   "per_gpu_batch": B, "global_batch": B * world, "sharding": "by image, no collectives",
                   "l2": "inputs larger than L2: every timed tensor is 24 MB-3 GB and is produced/consumed once per step",
                   "detections_per_step_per_gpu": n_dets, "plan": runner.plan.stats,
                   "launch": ("one CUDA graph replay per step (eager pass with per-kernel events: "
                              f"{eager_ms / args.steps:.3f} ms/step)") if use_graph else "eager, per-kernel CUDA events inside the timed region"},
        "clocks": clocks,
        "e2e": {"value": round(images / (e2e_total_ms / 1e3), 2), "unit": "images/s",
                "h2d_bytes_per_step": int(xh.numel() * 4), "d2h_bytes_per_step": int(n_host * 32 + 8),
                "api": "pixienn_b200.runner.PipelinedPredictor.submit: pinned host batch -> device, forward, detections -> pinned host, copies of neighbouring steps overlapped with compute; host wall clock"},
        "gpu_launches": launches,
        "roofline": {"bound": "hbm", "kernel": dom, "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                     "frac": round(achieved / peak, 4), "frac_of_nominal_8000": round(achieved / 8000.0, 4),
                     "peak_source": peak_src,
                     "traffic": (int(ratios[dom]["ratio"] * d["bytes"] / d["launches"]) if dom in ratios else None),
                     "traffic_note": ("bytes per launch (average over the timed launches): ncu DRAM read+write of a smaller "
                                      f"capture ({ratios[dom]['kernel']}, {ratios[dom]['capture']}: x{ratios[dom]['ratio']} of its "
                                      "algorithmic bytes), scaled by algorithmic bytes") if dom in ratios else "no capture on record",
                     "algorithmic_bytes_per_launch": int(d["bytes"] / d["launches"]),
                     "launches_timed": d["launches"], "avg_launch_ms": round(d["ms"] / d["launches"], 4),
                     "algorithmic_bytes_per_step": int(d["bytes"] / args.steps)},
        "epilogue": {"ms_per_step": round(epi_ms, 3), "algorithmic_GB_per_step": round(epi_bytes / 1e9, 3),
                     "GBps": round(epi_bytes / (epi_ms / 1e3) / 1e9, 1), "images_per_s_epilogue_only": round(B / (epi_ms / 1e3), 1)},
        "breakdown": breakdown,
    }
    if alt is not None:
        line["channels_last"] = alt
        line["channels_last_fused_stem"] = alt_stem
        if nchw_stem is not None:
            line["nchw_fused_stem"] = nchw_stem
        if alt_fusion is not None:
            line["channels_last_conv_fusion"] = alt_fusion
    if post_nms is not None:
        line["e2e"].update(post_nms_value=post_nms["value"], post_nms_resident_value=post_nms["resident_value"],
                           post_nms_d2h_bytes_per_step=post_nms["d2h_bytes_per_step"],
                           post_nms_candidates_per_step_per_gpu=post_nms["candidates_per_step_per_gpu"],
                           post_nms_survivors_per_step_per_gpu=post_nms["survivors_per_step_per_gpu"],
                           post_nms_head=post_nms["head"], post_nms_decode_ms=post_nms["decode_ms"],
                           post_nms_api="PipelinedPredictor(nms_threshold=0.4): decode, px::nms on the device, survivors -> pinned host")
        line["config"].update(
            strong_value=strong["value"] if strong else line["value"],
            strong_e2e=strong["e2e"] if strong else line["e2e"]["value"],
            strong_per_gpu_batch=strong["per_gpu_batch"] if strong else B,
            strong_global_batch=strong["global_batch"] if strong else B,
            strong_note="the same model with the global batch of one GPU's share split over the ranks (BASELINE.json's "
                        "64 / 32 / 16 / 8 images per GPU)",
            c3_value=c3["value"], c3_e2e=c3["e2e"], c3_per_gpu_batch=16, c3_global_batch=c3["global_batch"],
            c3_ms_per_step=c3["ms_per_step"], c3_post_nms_e2e=c3["post_nms_e2e"],
            c3_post_nms_candidates_per_step_per_gpu=c3["post_nms_candidates_per_step_per_gpu"],
            c3_post_nms_survivors_per_step_per_gpu=c3["post_nms_survivors_per_step_per_gpu"],
            c3_note="YOLOv7 640x640, 16 images per GPU, same measurement; c3_e2e copies every candidate of the random-init heads "
                    "to the host, c3_post_nms_e2e runs the trained-like head (" + HEAD_VARIANT_NOTE["yolov7"] + ") with NMS on "
                    "the device and copies the survivors")
    if post_nms is not None and "yolo_decode" in ops_summary:
        rd = ops_summary["yolo_decode"]
        line["roofline"].update(
            yolo_decode_ms=round(rd["ms"] / args.steps, 4),
            yolo_decode_frac=round(rd["bytes"] / (rd["ms"] / 1e3) / 1e9 / peak, 4),
            yolo_decode_trained_like_ms=post_nms["decode_ms"],
            yolo_decode_trained_like_frac=round(post_nms["decode_head_bytes"] / (post_nms["decode_ms"] / 1e3) / 1e9 / peak, 4)
            if post_nms["decode_ms"] > 0 else None,
            yolo_decode_note="three heads of one step; frac = 4 bytes per head element / time / peak.  Random-init heads emit "
                             "228 k records per image (466 MB written per step); the trained-like head (e2e.post_nms_head) "
                             "about a thousand")
    if world == 1 and not args.no_extras and args.workload == "yolov3-608":
        # the path's other stated targets, measured after every timed region above, on this GPU
        del runner
        torch.cuda.empty_cache()
        try:
            ours_ms, ref_ms, _, _ = epilogue_compare(args, "yolov3-608", B)
            line["roofline"].update(epilogue_ms=round(ours_ms, 3), ref_cuda_epilogue_ms=round(ref_ms, 3) if ref_ms else None,
                                    vs_ref_cuda=round(ref_ms / ours_ms, 2) if ref_ms else None,
                                    ref_cuda_kind="reference-cuda: the reference's own src/*.cu for sm_100a (oracle/_ref/"
                                                  "libpxref_cuda.so) replaying Layer<CUDA>::forward's epilogue calls on "
                                                  f"YOLOv3-608, {B} images, beside this library's planned launches; no convolutions")
        except Exception as e:
            line["roofline"]["ref_cuda_error"] = f"{type(e).__name__}: {str(e)[:160]}"
        torch.cuda.empty_cache()
        sw_args = argparse.Namespace(**vars(args))
        sw_args.sweep_shapes, sw_args.sweep_shape_index, sw_args.sweep_residual, sw_args.layout = 0, -1, False, "nchw"
        sw_args.sweep_folded = True                    # coefficients folded once per layer, as the runner passes them
        sw_args.steps = max(args.steps, 10)
        rows = sweep_rows(sw_args, [(a, k) for a in ("leaky", "mish") for k in ("plain", "pool", "shortcut")])
        worst = min(rows, key=lambda r: r["frac_measured"])
        vs_copy = [r["GBps"] / r["copy_GBps"] for r in rows]
        line["roofline"].update(
            sweep_cells=len(rows), sweep_min_frac=worst["frac_measured"],
            sweep_median_frac=round(statistics.median(r["frac_measured"] for r in rows), 3),
            sweep_max_frac=max(r["frac_measured"] for r in rows),
            sweep_worst_cell=f"{'x'.join(map(str, worst['shape']))} {worst['act']} "
                             f"{'pool' if worst['pool'] else ('shortcut' if worst['residual'] else 'plain')}",
            sweep_worst_cell_copy_frac=round(worst["copy_GBps"] / peak, 3),
            sweep_min_vs_copy=round(min(vs_copy), 3), sweep_median_vs_copy=round(statistics.median(vs_copy), 3),
            sweep_note="isolated fused epilogue (BN + bias folded once per layer by pxe_fold_bn, as the runner calls it), "
                       "[64,C,H,W] x {leaky, mish} x {plain, +2x2 pool, +shortcut}: fraction of the "
                       "measured peak on algorithmic bytes; *_vs_copy = against a device copy of the same tensor timed the same way")
        torch.cuda.empty_cache()
        cn_ms, _ = centernet_time(args, 256)
        line["roofline"].update(centernet_ms=round(cn_ms, 4), centernet_batch=256,
                                centernet_frac=round(4 * 256 * 20 * 128 * 128 / cn_ms / 1e6 / peak, 4),
                                centernet_note="CenterNet head decode, [256,20,128,128] logits, K=100: heat-map bytes / time / peak")
        torch.cuda.empty_cache()
        try:
            pc = pool_cells(sw_args, ["spp", "maxpool"], compact=True)
            bc = bn_train_cells(sw_args, [(128, 52, 52)])[0]
            line["roofline"].update(
                spp_us=pc[0]["us_median"], spp_frac=pc[0]["frac_measured"], maxpool_k2s1_us=pc[1]["us_median"],
                maxpool_k2s1_frac=pc[1]["frac_measured"],
                pools_note="SPP 5/9/13 with its conv epilogue and pass-through slot on [16,512,20,20]; kernel-2 stride-1 pool on "
                           "[64,512,13,13]: algorithmic bytes / time / peak",
                bn_train_forward_frac=bc["forward_frac_measured"], bn_train_backward_frac=bc["backward_frac_measured"],
                bn_train_vs_cudnn_sequence=bc["vs_cudnn_sequence"],
                bn_train_note="batch norm with batch statistics on [64,128,52,52]: forward 16 B / element (statistics, y, "
                              "leaky(y)), backward 20 B; cudnn_sequence = copy + cuDNN training batch norm + copy + activation")
        except Exception as e:
            line["roofline"]["pools_error"] = f"{type(e).__name__}: {str(e)[:160]}"
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_reference(args, steps=1, warmup=0)
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ------------------------------------------------------------------------------- reference arm
def cpu_reference(args, steps: int, warmup: int):
    """The reference's CPU path for the same model on the host cores: a bounded sample of
    `args.cpu_images` image(s) per step."""
    from oracle import pxoracle as po
    from oracle.pxmodel import CpuModel
    from pixienn_b200 import graph
    from pixienn_b200.runner import synth_weights
    doc, label = make_doc(args.workload)
    model = graph.parse_model(doc)
    weights = synth_weights(model, SEED)
    ref = po.ref_cpu()
    cores = os.cpu_count() or 1
    if ref is not None:
        cores = ref.set_threads(cores)
    cpu = CpuModel(doc, weights, eps_mode=1, keep_outputs=False)
    x = host_batch(model, args.cpu_images, 0)
    for _ in range(warmup):
        cpu.forward(x)
    t = time.perf_counter()
    for _ in range(steps):
        cpu.forward(x)
        cpu.detections(CONF)
    sec = time.perf_counter() - t
    single = None
    if ref is not None and args.cpu_single_core and cores > 1:
        # the same path on one host thread: one image, once (about ten seconds for YOLOv3-608)
        ref.set_threads(1)
        x1 = x[:1]
        t1 = time.perf_counter()
        cpu.forward(x1)
        cpu.detections(CONF)
        single = round(1.0 / (time.perf_counter() - t1), 4)
        ref.set_threads(cores)
    return {"value": round(args.cpu_images * steps / sec, 4), "unit": "images/s", "cores": cores,
            "single_core_value": single,
            "kind": "reference" if ref is not None else "port",
            "sample": f"{args.cpu_images} image(s) of the {label} batch per step, {steps} step(s): conv (im2col + OpenBLAS "
                      "sgemm), BN, bias, activation in the reference's own compiled CpuUtil.cpp / BatchNorm.cpp / "
                      "Activation.h" + ("" if ref is not None else " (not available: C restatement used)")
                      + "; maxpool / upsample / shortcut / route / YOLO decode loops restated in C (oracle/px_oracle.c)",
            "ms_per_image": round(sec / (args.cpu_images * steps) * 1e3, 1)}


def run_reference(args):
    rank, _, world = dist_env()
    if rank != 0:
        return
    base = cpu_reference(args, steps=args.steps, warmup=min(args.warmup, 1))
    doc, label = make_doc(args.workload)
    line = {
        "impl": "reference",
        "metric": "YOLOv3 608x608 inference throughput" if args.workload == "yolov3-608" else f"{label} inference throughput",
        "value": base["value"], "unit": "images/s", "n_gpus": world, "steps": args.steps, "warmup": min(args.warmup, 1),
        "ms_per_step": round(args.cpu_images / base["value"] * 1e3, 2), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{label}, reference CPU forward path (OpenBLAS) on the host cores, "
                               f"{args.cpu_images} image(s) per step of the {args.batch}-image batch",
                   "per_gpu_batch": args.batch, "global_batch": args.batch * world},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------ other workloads
def sweep_rows(args, variants=None):
    """Times the cells of the isolated fused-epilogue sweep.  ``variants``: list of (act, kind) with kind in
    {"plain", "pool", "shortcut"}; None = the cells the command line asks for."""
    import torch
    from pixienn_b200 import ops, synth
    dev = torch.device("cuda", torch.cuda.current_device())
    peak, peak_src = measured_peaks()
    shapes = [(32, 208, 208), (64, 104, 104), (128, 52, 52), (256, 26, 26), (512, 13, 13)]
    if args.sweep_shapes:
        shapes = shapes[:args.sweep_shapes]
    if args.sweep_shape_index >= 0:
        shapes = [shapes[args.sweep_shape_index]]
    rows = []
    for (C, H, W) in shapes:
        B = args.batch
        n = B * C * H * W
        sets = max(3, int(400e6 // (n * 4)) + 1)          # rotate so that no iteration finds its data in L2
        g, b, m, v = (torch.from_numpy(t).to(dev) for t in synth.bn_params(SEED, f"sweep{C}", C))
        bias = torch.from_numpy(synth.normal(SEED, f"sweepb{C}", C, 0, 0.1)).to(dev)
        base = torch.randn((B, C, H, W), device=dev, generator=torch.Generator(dev).manual_seed(SEED))
        nhwc = args.layout == "nhwc"
        folded = getattr(args, "sweep_folded", False)
        if nhwc:                      # the same cells on channels-last tensors, coefficients folded once
            base = base.contiguous(memory_format=torch.channels_last)
        if nhwc or folded:
            fa, fb = ops.fold_bn(C, dev, gamma=g, beta=b, mean=m, var=v, bias=bias)
        bnkw = dict(a=fa, b=fb) if folded else dict(gamma=g, beta=b, mean=m, var=v, bias=bias)
        xs = [base.clone() for _ in range(sets)]
        want_res = args.sweep_residual or (variants is not None and any(k == "shortcut" for _, k in variants))
        frm_sets = [base.clone() for _ in range(sets)] if want_res else None

        def graph_time(call):
            """Median / min device time (ms) of one call: a CUDA graph holds one launch per rotating input set;
            replays are timed with events, so no Python / ctypes launch cost sits between the launches."""
            for i in range(max(args.warmup, sets)):
                call(i)
            torch.cuda.synchronize()
            cg = torch.cuda.CUDAGraph()
            with torch.cuda.graph(cg):
                for i in range(sets):
                    call(i)
            cg.replay()
            ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
            torch.cuda.synchronize()
            for a, z in ev:
                a.record(); cg.replay(); z.record()
            torch.cuda.synchronize()
            ts = sorted(a.elapsed_time(z) / sets for a, z in ev)
            return ts[len(ts) // 2], ts[0]

        # the floor at this size: a plain device-to-device copy of the same tensor (4 B read + 4 B written per element)
        dsts = [torch.empty_like(base) for _ in range(sets)]
        copy_med, _ = graph_time(lambda i: dsts[i % sets].copy_(xs[i % sets]))
        del dsts
        if variants is None:
            cells = [(act, "pool" if pool else ("shortcut" if args.sweep_residual else "plain"))
                     for act in args.sweep_acts.split(",")
                     for pool in {"none": (False,), "pool": (True,), "both": (False, True)}[args.sweep_pool]
                     if not (pool and args.sweep_residual)]
        else:
            cells = list(variants)
        for act, kind in cells:
            pool = kind == "pool"
            frm = frm_sets if kind == "shortcut" else None
            oh = ops.maxpool_out_dim(H, 2, 2, 1)
            yps = [torch.empty((B, C, oh, ops.maxpool_out_dim(W, 2, 2, 1)), device=dev) for _ in range(sets)] if pool else None
            if nhwc and pool:
                yps = [t.contiguous(memory_format=torch.channels_last) for t in yps]

            def call(i):
                if nhwc:
                    if pool:
                        ops.conv_epilogue_nhwc(xs[i % sets], y=False, a=fa, b=fb, act=act, pool=(2, 2, 1), y_pool=yps[i % sets])
                    elif frm is not None:
                        ops.conv_epilogue_nhwc(xs[i % sets], a=fa, b=fb, act=act, residual=frm[i % sets], res_act="linear")
                    else:
                        ops.conv_epilogue_nhwc(xs[i % sets], a=fa, b=fb, act=act)
                elif pool:
                    ops.conv_epilogue(xs[i % sets], y=False, act=act, pool=(2, 2, 1), y_pool=yps[i % sets], **bnkw)
                elif frm is not None:      # conv epilogue + the shortcut layer that follows it: 12 B / element
                    ops.conv_epilogue(xs[i % sets], act=act, residual=frm[i % sets], res_act="linear", **bnkw)
                else:
                    ops.conv_epilogue(xs[i % sets], act=act, **bnkw)
            med, tmin = graph_time(call)
            nbytes = (4 * n + 4 * yps[0].numel()) if pool else (12 * n if frm is not None else 8 * n)
            rows.append({"shape": [B, C, H, W], "act": act, "pool": pool, "residual": frm is not None, "MB": round(nbytes / 1e6, 1),
                         "us_median": round(med * 1e3, 2), "us_min": round(tmin * 1e3, 2),
                         "copy_us": round(copy_med * 1e3, 2), "copy_GBps": round(8 * n / copy_med / 1e6, 1),
                         "GBps": round(nbytes / med / 1e6, 1), "frac_measured": round(nbytes / med / 1e6 / peak, 3),
                         "frac_8000": round(nbytes / med / 1e6 / 8000, 3)})
        del xs, frm_sets
    return rows


def run_sweep(args):
    """Isolated fused-epilogue sweep: [64,C,H,W] x {leaky, mish, swish, logistic} x {no pool, 2x2/2 pool}."""
    peak, peak_src = measured_peaks()
    rows = sweep_rows(args)
    for r in rows:
        print(json.dumps(r), file=sys.stderr)
    fr = [r["frac_measured"] for r in rows]
    print(json.dumps({"metric": "fused-epilogue HBM bandwidth, isolated sweep", "value": round(statistics.median(r["GBps"] for r in rows), 1),
                      "unit": "GB/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "higher_is_better": True,
                      "dtype": "f32", "data": "synthetic", "peak": peak, "peak_source": peak_src,
                      "frac_min": min(fr), "frac_median": statistics.median(fr), "frac_max": max(fr),
                      "config": {"workload": f"isolated fused epilogue sweep, {args.layout.upper()}", "l2": "rotating input sets > 400 MB", "timing": "CUDA events around a CUDA-graph replay of one launch per input set"},
                      "cells": rows}), flush=True)


def centernet_time(args, B):
    """CenterNet head decode: [B,20,128,128] heat logits N(-4,2) + Gaussian peaks, K = 100.  Returns
    (median ms per decode, mean records kept per image)."""
    import torch
    from pixienn_b200 import ops, synth
    dev = torch.device("cuda", torch.cuda.current_device())
    classes, H, W, K = 20, 128, 128, 100
    rng = np.random.default_rng(SEED)
    heat = synth.normal(SEED, "c4/heat", (B, classes, H, W), -4.0, 2.0)
    yy, xx = np.mgrid[0:H, 0:W]
    for bi in range(B):
        for _ in range(int(rng.integers(1, 31))):
            c, y, x = int(rng.integers(classes)), int(rng.integers(H)), int(rng.integers(W))
            y0, y1, x0, x1 = max(0, y - 6), min(H, y + 7), max(0, x - 6), min(W, x + 7)
            heat[bi, c, y0:y1, x0:x1] += (8.0 * np.exp(-((yy[y0:y1, x0:x1] - y) ** 2 + (xx[y0:y1, x0:x1] - x) ** 2) / 4.5)).astype(np.float32)
    sets = 3
    hs = [torch.from_numpy(heat).to(dev) for _ in range(sets)]
    size = torch.from_numpy(synth.uniform(SEED, "c4/wh", (B, 2, H, W))).to(dev)
    off = torch.from_numpy(synth.uniform(SEED, "c4/off", (B, 2, H, W))).to(dev)
    need = ops.capi.lib().pxe_centernet_decode_workspace_bytes(B, classes, H, W, K)
    ws = torch.empty(need, device=dev, dtype=torch.uint8)
    for i in range(max(args.warmup, 3)):
        ops.centernet_decode(hs[i % sets], size, off, CONF, K, logits=True, heatmap_bias=0.0, workspace=ws)
    steps = max(args.steps, 10)
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    torch.cuda.synchronize()
    for i, (a, z) in enumerate(ev):
        a.record()
        d, c = ops.centernet_decode(hs[i % sets], size, off, CONF, K, logits=True, heatmap_bias=0.0, workspace=ws)
        z.record()
    torch.cuda.synchronize()
    ts = sorted(a.elapsed_time(z) for a, z in ev)
    return ts[len(ts) // 2], float(c.float().mean().item())


def run_centernet(args):
    peak, peak_src = measured_peaks()
    B = args.batch
    med, kept = centernet_time(args, B)
    nbytes = 4 * B * 20 * 128 * 128
    print(json.dumps({"metric": "CenterNet head decode", "value": round(B / (med / 1e3), 1), "unit": "images/s", "n_gpus": 1,
                      "steps": max(args.steps, 10), "warmup": max(args.warmup, 3), "ms_per_step": round(med, 4), "higher_is_better": True,
                      "dtype": "f32", "data": "synthetic",
                      "config": {"workload": f"CenterNet decode B={B}, 20x128x128 heat + 2x wh + 2x offset, K=100, thr {CONF}",
                                 "l2": "3 rotating heat maps", "kept_per_image_mean": kept},
                      "roofline": {"bound": "hbm", "achieved": round(nbytes / med / 1e6, 1), "peak": peak, "unit": "GB/s",
                                   "frac": round(nbytes / med / 1e6 / peak, 4), "peak_source": peak_src, "traffic": None}}),
          flush=True)


def run_nms(args):
    """px::nms on the device (pxe_nms) against the same rule on the host (pxe_nms_host): `--batch` images with
    `--nms-boxes` candidate boxes each over 80 classes, clustered around 12 objects per image so that
    suppression has real work to do."""
    import torch
    from pixienn_b200 import ops
    dev = torch.device("cuda", 0)
    rng = np.random.default_rng(SEED)
    B, per = args.batch, args.nms_boxes
    n = B * per
    d = np.zeros(n, ops.DET_DTYPE)
    centres = rng.random((B, 12, 2)) * 0.8 + 0.1
    sizes = rng.random((B, 12, 2)) * 0.25 + 0.05
    obj = rng.integers(0, 12, n)
    img = np.repeat(np.arange(B), per)
    d["w"] = sizes[img, obj, 0] * (1 + rng.normal(0, 0.08, n))
    d["h"] = sizes[img, obj, 1] * (1 + rng.normal(0, 0.08, n))
    d["x"] = centres[img, obj, 0] + rng.normal(0, 0.01, n) - d["w"] / 2
    d["y"] = centres[img, obj, 1] + rng.normal(0, 0.01, n) - d["h"] / 2
    d["prob"] = rng.random(n).astype(np.float32) * 0.8 + 0.2
    d["class_id"] = (obj * 5 + rng.integers(0, 2, n)) % 80
    d["batch_id"] = img
    d["source"] = np.arange(n)
    t = torch.from_numpy(d.view(np.int32).reshape(-1, 8).copy()).to(dev)
    ws = torch.empty(ops.capi.lib().pxe_nms_workspace_bytes(n), device=dev, dtype=torch.uint8)
    out = torch.empty_like(t)
    for _ in range(args.warmup):
        o, c = ops.nms_device(t, n, 0.4, out=out, workspace=ws)
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    torch.cuda.synchronize()
    for a, z in ev:
        a.record()
        o, c = ops.nms_device(t, n, 0.4, out=out, workspace=ws)
        z.record()
    torch.cuda.synchronize()
    ts = sorted(a.elapsed_time(z) for a, z in ev)
    kept = int(c.item())
    h0 = time.perf_counter()
    want = ops.nms(d, 0.4)
    host_ms = (time.perf_counter() - h0) * 1e3
    got = o[:kept].cpu().numpy().view(ops.DET_DTYPE).reshape(-1)
    print(json.dumps({"metric": "px::nms on the device", "value": round(ts[len(ts) // 2], 4), "unit": "ms", "higher_is_better": False,
                      "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "dtype": "f32", "data": "synthetic",
                      "config": {"workload": f"NMS of {B} images x {per} boxes, 80 classes, threshold 0.4", "records": n, "kept": kept},
                      "host_ms": round(host_ms, 2), "identical_to_host": bool(got.tobytes() == want.tobytes())}), flush=True)


def epilogue_compare(args, model_name, B):
    """Epilogue path only (no convolutions), layer by layer over the model graph, on scratch buffers of
    each layer's shape: the reference's own CUDA call sequences (its src/*.cu compiled for sm_100a in
    oracle/_ref/libpxref_cuda.so: fills, cuDNN BN inference, preActivation copy, thrust activation, per-image
    route copies, shortcut copy + kernel + activation, YOLO activate + full device-to-host copy) against
    this library's planned launches.  Returns (ms per batch here, ms per batch of the reference's kernels or None
    when that library is not built, label, plan statistics)."""
    import torch
    from oracle import pxoracle as po
    from pixienn_b200 import graph, ops
    from pixienn_b200.runner import synth_weights
    dev = torch.device("cuda", torch.cuda.current_device())
    doc, label = make_doc(model_name)
    model = graph.parse_model(doc)
    L = model.layers
    ref = po.ref_cuda()
    weights = synth_weights(model, SEED)
    wd = {i: {k: torch.from_numpy(v).to(dev) for k, v in d.items() if k != "weights"} for i, d in weights.items()}
    # the same scratch data is transformed in place by every layer and every repetition: neutral BN statistics keep
    # it bounded, and a negative head bias keeps the decode at the few-detections regime of a trained network
    for i, d in wd.items():
        if "scales" in d:
            d["scales"].fill_(1.0); d["biases"].zero_(); d["rolling_mean"].zero_(); d["rolling_var"].fill_(1.0)
        else:
            d["biases"].fill_(-6.0)
    biggest = max(l.out_elems for l in L) * B
    big = [torch.empty(biggest, device=dev) for _ in range(5)]       # out, delta, preact, scratch, other
    for t in big:
        t.normal_()
    host = torch.empty(max(l.out_elems for l in L if l.type == "yolo") * B).pin_memory()
    idx = torch.empty(biggest // 4 + 1, device=dev, dtype=torch.int32)
    ptr = lambda t: t.data_ptr()

    def reference_pass():
        for l in L:
            c, h, w = l.out_shape
            n = B * c * h * w
            if l.type == "conv":
                p = wd[l.index]
                if l.batch_norm:
                    ref.call("conv_epilogue_replay", ptr(big[0]), ptr(big[1]), ptr(big[2]), ptr(big[3]), B, c, h, w,
                             ptr(p["scales"]), ptr(p["biases"]), ptr(p["rolling_mean"]), ptr(p["rolling_var"]), None,
                             po.ACT[l.activation])
                else:
                    ref.call("conv_epilogue_replay", ptr(big[0]), ptr(big[1]), ptr(big[2]), ptr(big[3]), B, c, h, w,
                             None, None, None, None, ptr(p["biases"]), po.ACT[l.activation])
            elif l.type == "shortcut":
                ref.call("shortcut_replay", ptr(big[0]), ptr(big[4]), ptr(big[2]), ptr(big[1]), B, c, h, w, l.alpha, l.beta,
                         po.ACT[l.activation])
            elif l.type == "upsample":
                ic, ih, iw = l.in_shape
                ref.call("upsample_replay", ptr(big[0]), ptr(big[2]), ptr(big[1]), B, ic, ih, iw, l.stride, l.alpha)
            elif l.type == "maxpool":
                ic, ih, iw = l.in_shape
                ref.call("maxpool_replay", ptr(big[0]), ptr(big[2]), ptr(big[1]), ptr(idx), B, ic, ih, iw, h, w, l.kernel,
                         l.stride, l.padding)
            elif l.type == "route":
                srcs = (C.c_void_p * len(l.sources))(*[ptr(big[0]) for _ in l.sources])
                outs = (C.c_int * len(l.sources))(*[L[s].out_elems for s in l.sources])
                ref.call("route_replay", len(l.sources), srcs, outs, ptr(big[2]), ptr(big[1]), B)
            elif l.type == "yolo":
                masks = len(l.params["mask"])
                ref.call("yolo_replay", ptr(big[0]), ptr(big[2]), ptr(big[1]), ptr(host), B, masks, c // masks - 5, h * w)

    plan = graph.plan(model)
    dets = ops.DetectionBuffer(args.det_capacity, dev)

    def view(i, layer):
        c, h, w = layer.out_shape
        return big[i][:B * c * h * w].view(B, c, h, w)

    def our_pass():
        dets.reset()
        for st in plan.steps:
            l = L[st.layer]
            if st.op == "conv":
                p = wd[l.index]
                x = view(0, l)
                if st.head_raw:
                    continue
                if "a" not in p:                   # folded once per layer, as the runner does at load time
                    p["a"], p["b"] = ops.fold_bn(l.filters, dev, **(dict(gamma=p["scales"], beta=p["biases"], mean=p["rolling_mean"],
                                                                       var=p["rolling_var"]) if l.batch_norm else dict(bias=p["biases"])))
                bn = dict(a=p["a"], b=p["b"])
                if st.fused_pool is not None:
                    ops.conv_epilogue(x, y=x if st.keep_full else False, act=l.activation, pool=(2, 2, L[st.fused_pool].padding),
                                      y_pool=view(2, L[st.fused_pool]), **bn)
                elif st.fused_shortcut is not None:
                    ops.conv_epilogue(x, y2=view(2, l) if len(st.dests) > 1 else None, act=l.activation, residual=view(4, l), **bn)
                else:
                    ops.conv_epilogue(x, y2=view(2, l) if len(st.dests) > 1 else None, act=l.activation, **bn)
            elif st.op == "shortcut":
                ops.shortcut(view(0, l), view(4, l), l.alpha, l.beta, l.activation, out=view(2, l))
            elif st.op == "upsample":
                src = big[0][:B * l.in_shape[0] * l.in_shape[1] * l.in_shape[2]].view(B, *l.in_shape)
                ops.upsample(src, l.stride, l.alpha, out=view(2, l))
            elif st.op == "maxpool":
                src = big[0][:B * l.in_shape[0] * l.in_shape[1] * l.in_shape[2]].view(B, *l.in_shape)
                ops.maxpool(src, l.kernel, l.stride, l.padding, out=view(2, l))
            elif st.op == "spp":
                src = big[0][:B * l.in_shape[0] * l.in_shape[1] * l.in_shape[2]].view(B, *l.in_shape)
                outs = [big[2][k * src.numel():(k + 1) * src.numel()].view_as(src) for k in range(len(st.spp_layers))]
                ops.spp(src, [L[g].kernel for g in st.spp_layers], outs)
            elif st.op == "yolo":
                conv = L[st.inputs[0]]
                ops.yolo_decode(view(0, l), l.params["mask"], l.params["anchors"], l.in_shape[0] // len(l.params["mask"]) - 5,
                                model.width, model.height, CONF, dets, raw=True, bias=wd[conv.index]["biases"])

    def timed(fn):
        for _ in range(max(1, args.warmup // 2)):
            fn()
        torch.cuda.synchronize()
        a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.steps):
            fn()
        z.record()
        torch.cuda.synchronize()
        return a.elapsed_time(z) / args.steps

    ours = timed(our_pass)
    refms = timed(reference_pass) if ref is not None else None
    return ours, refms, label, plan.stats


def run_epilogue_compare(args):
    B = args.batch
    ours, refms, label, stats = epilogue_compare(args, args.model, B)
    print(json.dumps({"metric": f"{label} epilogue path only, ms per {B}-image batch", "value": round(ours, 3), "unit": "ms",
                      "higher_is_better": False, "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "dtype": "f32",
                      "data": "synthetic", "reference_cuda_ms": round(refms, 3) if refms else None,
                      "speedup_vs_reference_cuda": round(refms / ours, 2) if refms else None,
                      "images_per_s": round(B / ours * 1e3, 1),
                      "reference_cuda_images_per_s": round(B / refms * 1e3, 1) if refms else None,
                      "config": {"workload": f"{label}, {B} images, epilogue launches only (no convolution), scratch buffers of each "
                                             "layer's shape; reference = its own src/*.cu for sm_100a replaying Layer<CUDA>::forward",
                                 "plan": stats}}), flush=True)


def pool_cells(args, which, compact=False):
    """The stand-alone pooling kernels on the shapes the preset graphs run them on: the SPP block (with the conv
    epilogue folded in, as YOLOv7's does, and on its own), the kernel-2 stride-1 pool of YOLOv3-tiny, single
    stride-1 pools.  Buffers rotate past L2; CUDA events around a CUDA-graph replay of one launch per buffer set."""
    import torch
    from pixienn_b200 import ops
    dev = torch.device("cuda", torch.cuda.current_device())
    peak, peak_src = measured_peaks()
    gen = torch.Generator(dev).manual_seed(SEED)

    def graph_time(call, sets):
        for i in range(max(args.warmup, sets)):
            call(i)
        torch.cuda.synchronize()
        cg = torch.cuda.CUDAGraph()
        with torch.cuda.graph(cg):
            for i in range(sets):
                call(i)
        cg.replay()
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
        torch.cuda.synchronize()
        for a, z in ev:
            a.record(); cg.replay(); z.record()
        torch.cuda.synchronize()
        ts = sorted(a.elapsed_time(z) / sets for a, z in ev)
        return ts[len(ts) // 2]

    cells = []

    def record(kind, shape, ms, nbytes):
        cells.append({"kernel": kind, "shape": list(shape), "MB": round(nbytes / 1e6, 1), "us_median": round(ms * 1e3, 2),
                      "GBps": round(nbytes / ms / 1e6, 1), "frac_measured": round(nbytes / ms / 1e6 / peak, 3)})

    def spp_case(B, C, H, W, fused, act="swish"):
        n = B * C * H * W
        sets = max(3, int(500e6 // (n * 20)) + 1)
        xs = [torch.randn((B, C, H, W), device=dev, generator=gen) for _ in range(sets)]
        cats = [torch.empty((B, 4 * C, H, W), device=dev) for _ in range(sets)]
        a, b = torch.rand(C, device=dev, generator=gen) + 0.5, torch.randn(C, device=dev, generator=gen)

        def call(i):
            cat = cats[i % sets]
            outs = [cat[:, 0:C], cat[:, C:2 * C], cat[:, 2 * C:3 * C]]
            if fused:
                ops.spp(xs[i % sets], [13, 9, 5], outs, a=a, b=b, act=act, y_identity=cat[:, 3 * C:])
            else:
                ops.spp(xs[i % sets], [13, 9, 5], outs)
        record(f"spp 5/9/13{' + epilogue (' + act + ') + pass-through slot' if fused else ''}", (B, C, H, W),
               graph_time(call, sets), n * 4 * (5 if fused else 4))

    def maxpool_case(B, C, H, W, k, s):
        n = B * C * H * W
        sets = max(3, int(500e6 // (n * 8)) + 1)
        xs = [torch.randn((B, C, H, W), device=dev, generator=gen) for _ in range(sets)]
        oh, ow = ops.maxpool_out_dim(H, k, s, k - 1), ops.maxpool_out_dim(W, k, s, k - 1)
        ys = [torch.empty((B, C, oh, ow), device=dev) for _ in range(sets)]
        record(f"maxpool k{k}/s{s}", (B, C, H, W), graph_time(lambda i: ops.maxpool(xs[i % sets], k, s, out=ys[i % sets]), sets),
               4 * n + 4 * B * C * oh * ow)

    if "spp" in which:
        spp_case(16, 512, 20, 20, True)               # YOLOv7-640 at 16 images
        if not compact:
            spp_case(16, 512, 20, 20, False)
            spp_case(64, 512, 19, 19, True, "leaky")  # YOLOv3-SPP / YOLOv4 at 608
            spp_case(64, 512, 13, 13, False)
    if "maxpool" in which:
        maxpool_case(64, 512, 13, 13, 2, 1)           # YOLOv3-tiny-416, layer 11
        if not compact:
            maxpool_case(64, 512, 19, 19, 2, 1)       # the same at 608
            maxpool_case(16, 512, 20, 20, 5, 1)
            maxpool_case(64, 256, 26, 26, 3, 2)
    return cells


def run_pools(args):
    cells = pool_cells(args, args.pool_cases.split(","))
    peak, peak_src = measured_peaks()
    fr = sorted(c["frac_measured"] for c in cells)
    print(json.dumps({"metric": "stand-alone pooling kernels, HBM bandwidth", "value": cells[0]["GBps"], "unit": "GB/s", "n_gpus": 1,
                      "steps": args.steps, "warmup": args.warmup, "higher_is_better": True, "dtype": "f32", "data": "synthetic",
                      "peak": peak, "peak_source": peak_src, "frac_min": fr[0], "frac_max": fr[-1],
                      "config": {"workload": "SPP block and stand-alone max pools, NCHW", "l2": "rotating buffer sets > 400 MB",
                                 "timing": "CUDA events around a CUDA-graph replay of one launch per buffer set"},
                      "cells": cells}), flush=True)


def bn_train_cells(args, shapes):
    """Batch normalisation in training mode on shapes of the epilogue sweep: this library's forward (statistics +
    one pass that writes the normalised tensor and the activated output) and backward, beside the sequence the
    reference's CUDA conv layer runs around cuDNN (copy of the conv output, cudnnBatchNormalizationForwardTraining,
    copy to preActivation_, activation in place: include/cuda/ConvLayer.h:284-307), here through PyTorch's cuDNN
    batch norm.  Buffers rotate past L2; CUDA events around a CUDA-graph replay of one call per buffer set."""
    import torch
    import torch.nn.functional as F
    from pixienn_b200 import ops
    dev = torch.device("cuda", torch.cuda.current_device())
    peak, peak_src = measured_peaks()
    gen = torch.Generator(dev).manual_seed(SEED)
    B = args.batch
    cells = []
    for (Cc, H, W) in shapes:
        n = B * Cc * H * W
        sets = max(2, int(400e6 // (n * 4)) + 1)
        xs = [torch.randn((B, Cc, H, W), device=dev, generator=gen) for _ in range(sets)]
        dys = [torch.randn((B, Cc, H, W), device=dev, generator=gen) for _ in range(sets)]
        g, b = torch.rand(Cc, device=dev, generator=gen) + 0.5, torch.randn(Cc, device=dev, generator=gen)
        rm, rv = torch.zeros(Cc, device=dev), torch.ones(Cc, device=dev)
        ys = [torch.empty_like(xs[0]) for _ in range(sets)]
        saved = {}

        def graph_time(call):
            for i in range(max(args.warmup, sets)):
                call(i)
            torch.cuda.synchronize()
            cg = torch.cuda.CUDAGraph()
            with torch.cuda.graph(cg):
                for i in range(sets):
                    call(i)
            cg.replay()
            ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
            torch.cuda.synchronize()
            for a, z in ev:
                a.record(); cg.replay(); z.record()
            torch.cuda.synchronize()
            ts = sorted(a.elapsed_time(z) / sets for a, z in ev)
            return ts[len(ts) // 2]

        def ours_fwd(i):
            saved[i % sets] = ops.batchnorm_forward_training(xs[i % sets], g, b, running_mean=rm, running_var=rv, act="leaky",
                                                            y=ys[i % sets])

        def ours_bwd(i):
            _, _, sm, ss = saved[i % sets]
            ops.batchnorm_backward(xs[i % sets], dys[i % sets], g, sm, ss, dx=dys[i % sets])

        def ref_seq(i):
            x_saved = xs[i % sets].clone()                                       # x_.copy(output_)
            y = F.batch_norm(x_saved, rm, rv, g, b, training=True, momentum=0.01, eps=1e-5)
            pre = y.clone()                                                      # preActivation_.copy(output_)
            F.leaky_relu(y, 0.1, inplace=True)
            return pre

        with torch.no_grad():
            t_fwd, t_ref = graph_time(ours_fwd), graph_time(ref_seq)
            t_bwd = graph_time(ours_bwd)
        fwd_bytes, bwd_bytes = 16 * n, 20 * n
        cells.append({"shape": [B, Cc, H, W], "forward_us": round(t_fwd * 1e3, 1), "forward_GBps": round(fwd_bytes / t_fwd / 1e6, 1),
                      "forward_frac_measured": round(fwd_bytes / t_fwd / 1e6 / peak, 3),
                      "cudnn_sequence_us": round(t_ref * 1e3, 1), "vs_cudnn_sequence": round(t_ref / t_fwd, 2),
                      "backward_us": round(t_bwd * 1e3, 1), "backward_GBps": round(bwd_bytes / t_bwd / 1e6, 1),
                      "backward_frac_measured": round(bwd_bytes / t_bwd / 1e6 / peak, 3)})
        del xs, dys, ys, saved
        torch.cuda.empty_cache()
    return cells


def run_bn_train(args):
    shapes = [(32, 208, 208), (64, 104, 104), (128, 52, 52), (256, 26, 26), (512, 13, 13)]
    if args.sweep_shapes:
        shapes = shapes[:args.sweep_shapes]
    if args.bn_shapes:
        shapes = [tuple(int(v) for v in s.split("x")) for s in args.bn_shapes.split(",")]
    cells = bn_train_cells(args, shapes)
    peak, peak_src = measured_peaks()
    B = args.batch
    print(json.dumps({"metric": "batch-norm training forward, HBM bandwidth", "value": cells[0]["forward_GBps"], "unit": "GB/s",
                      "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "higher_is_better": True, "dtype": "f32",
                      "data": "synthetic", "peak": peak, "peak_source": peak_src,
                      "config": {"workload": f"batch norm with batch statistics, {B} images, NCHW; forward = statistics + y + leaky(y) "
                                             "(16 B per element), backward = sums + dx (20 B per element); cudnn_sequence = copy, "
                                             "cuDNN batch-norm training, copy, activation in place as the reference's conv layer does",
                                 "l2": "rotating buffer sets > 400 MB",
                                 "timing": "CUDA events around a CUDA-graph replay of one call per buffer set"},
                      "cells": cells}), flush=True)


def run_aux(args):
    """The kernels no model benchmark and no sweep times: the generic pools and moves, the small heads, device NMS and the
    training-side kernels, each at a model-size shape.  Two buffer sets alternate (every set is larger than L2 or the
    pair is); CUDA events around bursts of eight calls, median of `steps` bursts; algorithmic bytes per call as stated in
    each cell."""
    import torch
    from pixienn_b200 import capi, ops
    dev = torch.device("cuda", torch.cuda.current_device())
    peak, peak_src = measured_peaks()
    gen = torch.Generator(dev).manual_seed(SEED)
    B = args.batch
    rnd = lambda *shape: torch.randn(shape, device=dev, generator=gen)
    cells = []

    def timed(name, shape, nbytes, make, call, note=""):
        sets = [make() for _ in range(2)]
        for i in range(max(args.warmup, 2)):
            call(sets[i % 2])
        torch.cuda.synchronize()
        burst = 8                                          # calls per event pair: launch gaps do not count as kernel time
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
        for a, z in ev:
            a.record()
            for i in range(burst):
                call(sets[i % 2])
            z.record()
        torch.cuda.synchronize()
        ts = sorted(a.elapsed_time(z) / burst for a, z in ev)
        ms = ts[len(ts) // 2]
        cell = {"kernel": name, "shape": shape, "us": round(ms * 1e3, 1)}
        if nbytes:
            cell.update(MB=round(nbytes / 1e6, 1), GBps=round(nbytes / ms / 1e6, 1), frac_measured=round(nbytes / ms / 1e6 / peak, 3))
        if note:
            cell["note"] = note
        cells.append(cell)
        del sets
        torch.cuda.empty_cache()

    C1, H1 = 64, 104                                    # [B, 64, 104, 104]: 177 MB at 64 images
    n1 = B * C1 * H1 * H1
    big = [B, C1, H1, H1]
    for act in ("leaky", "mish"):
        timed(f"activation gradient ({act})", big, 12 * n1, lambda: (rnd(*big), rnd(*big)),
              lambda t, act=act: ops.activation_gradient(act, t[0], t[1]), "x and delta read, delta written")
    timed("bias gradient", big, 4 * n1, lambda: (torch.zeros(C1, device=dev), rnd(*big)), lambda t: ops.backward_bias(t[0], t[1]),
          "delta read once")
    timed("connected-layer bias gradient", [4096, 1000], 4 * 4096 * 1000, lambda: (torch.zeros(1000, device=dev), rnd(4096, 1000)),
          lambda t: ops.backward_bias(t[0], t[1]))

    def pool_case():
        x = rnd(*big)
        y, idx = ops.maxpool(x, 2, 2, 1, with_indexes=True)
        return rnd(*y.shape), idx, torch.zeros_like(x)
    half = [B, C1, H1 // 2, H1 // 2]
    timed("max-pool backward (2x2 / 2)", half, 16 * (n1 // 4), pool_case, lambda t: ops.maxpool_backward(t[0], t[1], t[2]),
          "delta and index read, one float added in place per output")
    timed("upsample backward (x2)", half, 4 * n1 + 8 * (n1 // 4), lambda: (rnd(*half), rnd(*big)),
          lambda t: ops.upsample_backward(t[0], t[1], 2, 1.0), "four outputs read, one input updated")
    timed("clip", big, 8 * n1, lambda: (rnd(*big),), lambda t: ops.constrain(t[0], 1.0))
    timed("product", big, 12 * n1, lambda: (rnd(*big), rnd(*big)), lambda t: ops.mul(t[0], t[1]))
    timed("Adam step", big, 16 * n1, lambda: (rnd(*big), rnd(*big), rnd(*big).abs_()),
          lambda t: ops.adam_update(t[0], t[1], t[2], 0.9, 0.999, 1e-3, 1e-8, 10))
    timed("uniform fill", big, 4 * n1, lambda: (torch.empty(big, device=dev),), lambda t: ops.random_uniform(t[0], 0.0, 1.0))
    timed("normal fill", big, 4 * n1, lambda: (torch.empty(big, device=dev),), lambda t: ops.random_normal(t[0], 0.0, 1.0))
    timed("softmax cross entropy", [n1], 16 * n1, lambda: (torch.rand(n1, device=dev, generator=gen), (rnd(n1) > 1.5).float()),
          lambda t: ops.softmax_cross_entropy(t[0], t[1]), "prediction and truth read, delta and error written (allocated per call)")

    # YOLO loss on the three heads of YOLOv3-608 and CenterNet loss on a 128x128 head
    def yolo_case(hw):
        out = torch.rand((B, 255, hw, hw), device=dev, generator=gen)
        slots = B * 3 * hw * hw
        truths = torch.rand((B, 30, 5), device=dev, generator=gen) * 0.8 + 0.1
        truths[:, :, 4] = torch.randint(0, 80, (B, 30), device=dev, generator=gen).float()
        cls = torch.full((slots,), -1, device=dev, dtype=torch.int32)
        pick = torch.randint(0, slots, (B * 10,), device=dev, generator=gen)
        cls[pick] = torch.randint(0, 80, (B * 10,), device=dev, generator=gen).int()
        return (out, torch.zeros_like(out), truths, torch.full((B,), 10, device=dev, dtype=torch.int32), cls,
                torch.randint(0, 9, (slots,), device=dev, generator=gen).int(), torch.rand((slots, 4), device=dev, generator=gen) * 0.8 + 0.1,
                torch.tensor([0, 1, 2], device=dev, dtype=torch.int32),
                torch.tensor([10, 13, 16, 30, 33, 23, 30, 61, 62, 45, 59, 119, 116, 90, 156, 198, 373, 326], device=dev, dtype=torch.float32),
                torch.zeros(12, device=dev), torch.zeros(1, device=dev))
    for hw in (76, 38):
        timed("YOLO loss", [B, 255, hw, hw], 8 * B * 255 * hw * hw, lambda hw=hw: yolo_case(hw),
              lambda t: ops.yolo_loss(*t, 608, 608, ignore_thr=0.7, truth_thr=1.0), "head read, delta written; 10 truths per image")

    def cn_case():
        out = torch.rand((B, 24, 128, 128), device=dev, generator=gen)
        return (out, torch.zeros_like(out), torch.rand((B, 20, 128, 128), device=dev, generator=gen) ** 8,
                torch.rand((B, 2, 128, 128), device=dev, generator=gen), torch.rand((B, 2, 128, 128), device=dev, generator=gen),
                (torch.rand((B, 128, 128), device=dev, generator=gen) > 0.999).float(), torch.zeros(3, device=dev))
    ncn = B * 128 * 128
    timed("CenterNet loss", [B, 24, 128, 128], 4 * ncn * (20 * 3 + 1), cn_case, lambda t: ops.centernet_loss(*t, 1.0 / B),
          "heat map, target and delta of the 20 classes; the mask; size / offset terms only where the mask is set")

    # generic pools and moves
    for k, st in ((3, 2), (3, 1)):
        pad = k - 1
        oh = ops.maxpool_out_dim(H1, k, st, pad)
        for widx in (False, True):
            timed(f"generic max pool {k}x{k} / {st}" + (" with indexes" if widx else ""), big, 4 * n1 + (8 if widx else 4) * B * C1 * oh * oh,
                  lambda: (rnd(*big),), lambda t, k=k, st=st, pad=pad, widx=widx: ops.maxpool(t[0], k, st, pad, with_indexes=widx),
                  "output allocated per call")
    timed("global average pool", [B, 1024, 19, 19], 4 * B * 1024 * 361, lambda: (rnd(B, 1024, 19, 19),), lambda t: ops.avgpool(t[0]))
    q = [B, C1, 52, 52]
    nq = B * C1 * 52 * 52
    timed("upsample x3 (scalar form)", q, 4 * nq * 10, lambda: (rnd(*q), torch.empty((B, C1, 156, 156), device=dev)),
          lambda t: ops.upsample(t[0], 3, 1.0, out=t[1]))
    timed("shortcut across shapes", [B, 128, 52, 52], 12 * B * 64 * 52 * 52, lambda: (rnd(*big), rnd(B, 128, 52, 52)),
          lambda t: ops.shortcut_general(B, H1, H1, C1, t[0], 52, 52, 128, 1.0, 1.0, t[1]),
          "[B,64,104,104] sampled with stride 2 into the first 64 channels of [B,128,52,52]")
    timed("route copy (two sources)", [B, 384, 52, 52], 8 * B * 384 * 52 * 52,
          lambda: ([rnd(B, 128, 52, 52), rnd(B, 256, 52, 52)], torch.empty((B, 384, 52, 52), device=dev)),
          lambda t: ops.concat(t[0], out=t[1]))
    timed("CenterNet head activation", [B, 24, 128, 128], 8 * B * 24 * 128 * 128, lambda: (rnd(B, 24, 128, 128), torch.empty((B, 24, 128, 128), device=dev)),
          lambda t: ops.centernet_activate(t[0], 20, -2.19, out=t[1]))
    timed("softmax layer", [B * 64, 1000], 8 * B * 64 * 1000, lambda: (rnd(B * 64, 1000), torch.empty((B * 64, 1000), device=dev)),
          lambda t: ops.softmax(t[0], out=t[1]), "rows of 1000; the row is read three times, twice from L1 / L2")
    timed("Region head forward", [B, 425, 19, 19], 8 * B * 425 * 361, lambda: (rnd(B, 425, 19, 19),),
          lambda t: ops.region_forward(t[0], 5, 4, 80), "NCHW in, per-box records out (allocated per call)")

    # device NMS: 1000 candidates per image
    def nms_case():
        n = B * 1000
        d = torch.zeros((n, 8), device=dev, dtype=torch.float32)
        d[:, 0:2] = torch.rand((n, 2), device=dev, generator=gen) * 500
        d[:, 2:4] = torch.rand((n, 2), device=dev, generator=gen) * 100 + 10
        d[:, 4] = torch.rand(n, device=dev, generator=gen)
        di = d.view(torch.int32).clone()
        di[:, 5] = torch.randint(0, 80, (n,), device=dev, generator=gen).int()
        di[:, 6] = torch.arange(n, device=dev, dtype=torch.int32) // 1000
        ws = torch.empty(max(int(capi.lib().pxe_nms_workspace_bytes(n)), 256), device=dev, dtype=torch.uint8)
        return di, torch.empty((n, 8), device=dev, dtype=torch.int32), ws
    timed("device NMS", [B, 1000], 0, nms_case, lambda t: ops.nms_device(t[0], t[0].shape[0], 0.4, out=t[1], workspace=t[2]),
          "1000 candidates per image, 80 classes: every launch of pxe_nms")
    print(json.dumps({"metric": "auxiliary kernels, HBM bandwidth", "value": cells[0]["GBps"], "unit": "GB/s", "n_gpus": 1,
                      "steps": args.steps, "warmup": args.warmup, "higher_is_better": True, "dtype": "f32", "data": "synthetic",
                      "peak": peak, "peak_source": peak_src,
                      "config": {"workload": f"kernels outside the model benchmarks and the sweeps, {B} images", "l2": "two buffer sets alternate",
                                 "timing": "CUDA events around bursts of 8 calls, median of steps"},
                      "cells": cells}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="yolov3-608")
    ap.add_argument("--batch", type=int, default=None, help="images per GPU (default 64; 256 for --workload centernet)")
    ap.add_argument("--cpu-images", type=int, default=2, help="images per step of the CPU reference sample")
    ap.add_argument("--det-capacity", type=int, default=24 * (1 << 20))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-cpu-single-core", dest="cpu_single_core", action="store_false",
                    help="skip timing the CPU reference on one host thread as well (one image, a few seconds)")
    ap.add_argument("--no-extras", action="store_true",
                    help="only the headline: skip the post-NMS end-to-end arm, the configured split, YOLOv7 and (at one "
                         "GPU) the reference-CUDA epilogue comparison, the compact sweep and the CenterNet decode")
    ap.add_argument("--fusion-shapes", action="store_true", help="list every layer shape the conv-fusion variant timed")
    ap.add_argument("--sweep-shapes", type=int, default=0, help="only the first N shapes of the sweep")
    ap.add_argument("--sweep-shape-index", type=int, default=-1, help="only this shape of the sweep (0..4)")
    ap.add_argument("--sweep-acts", default="leaky,mish,swish,logistic")
    ap.add_argument("--sweep-pool", default="both", choices=["none", "pool", "both"])
    ap.add_argument("--sweep-residual", action="store_true", help="sweep the epilogue fused with a shortcut add")
    ap.add_argument("--sweep-folded", action="store_true",
                    help="sweep with the layer's coefficients folded once (pxe_fold_bn) instead of the raw BN parameters per launch")
    ap.add_argument("--model", default="yolov3-608", help="model graph for --workload epilogue-compare")
    ap.add_argument("--pool-cases", default="spp,maxpool", help="kernel families for --workload pools")
    ap.add_argument("--bn-shapes", default="", help="--workload bn-train: CxHxW[,CxHxW...] instead of the sweep's five shapes")
    ap.add_argument("--nms-boxes", type=int, default=1000, help="candidate boxes per image for --workload nms")
    ap.add_argument("--no-cudnn-benchmark", action="store_true", help="skip cuDNN's algorithm search (profiling runs)")
    ap.add_argument("--layout", default="nchw", choices=["nchw", "nhwc"],
                    help="activation layout between layers: nchw = the reference's (BASELINE.json's configs); nhwc = "
                         "channels-last, which lets cuDNN skip its layout conversions (the library's NHWC tier)")
    ap.add_argument("--no-alt-layout", action="store_true", help="skip the extra channels-last measurement")
    ap.add_argument("--conv-fusion", action="store_true",
                    help="with --layout nhwc: the measured runner itself uses cuDNN conv + epilogue fusion (per-kernel breakdown "
                         "of that form); with the default layout the fused variant is measured beside the headline anyway")
    ap.add_argument("--no-conv-fusion", action="store_true",
                    help="skip the channels-last measurement with conv + epilogue as one cuDNN runtime-fusion launch per "
                         "layer where that is faster (it adds about a minute of plan compilation and timing)")
    ap.add_argument("--fused-stem", action="store_true",
                    help="first convolution + epilogue as one launch of the library (pxe_conv_stem) instead of cuDNN + epilogue")
    ap.add_argument("--cuda-graph", default="auto", choices=["auto", "on", "off"],
                    help="auto / on: the reported step is one CUDA-graph replay of the forward pass (the eager pass "
                         "with per-kernel events is still run and timed for the breakdown); off: eager only")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    if args.batch is None:
        args.batch = 256 if args.workload == "centernet" else 64
    _, _, world = dist_env()
    if args.gpus != world and world == 1 and args.gpus > 1 and args.impl == "ours":
        raise SystemExit("for --gpus N > 1 launch with: python -m torch.distributed.run --nnodes=1 --nproc-per-node N "
                         "--master-addr 127.0.0.1 --master-port P bench.py --gpus N ...")
    if args.impl == "reference":
        return run_reference(args)
    if args.workload == "sweep":
        return run_sweep(args)
    if args.workload == "centernet":
        return run_centernet(args)
    if args.workload == "nms":
        return run_nms(args)
    if args.workload == "epilogue-compare":
        return run_epilogue_compare(args)
    if args.workload == "pools":
        return run_pools(args)
    if args.workload == "bn-train":
        return run_bn_train(args)
    if args.workload == "aux":
        return run_aux(args)
    return run_model(args)


if __name__ == "__main__":
    # Native libraries (NCCL's version banner, cuDNN) write to file descriptor 1; the contract is ONE JSON line on
    # stdout. Python's own stdout keeps the real descriptor, everything else that writes to fd 1 lands on stderr.
    _real_stdout = os.dup(1)
    os.dup2(2, 1)
    sys.stdout = os.fdopen(_real_stdout, "w")
    main()
