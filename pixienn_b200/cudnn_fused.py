"""Convolution and its epilogue as ONE cuDNN launch, for channels-last tensors.

The reference runs ``cudnnConvolutionForward`` and then its epilogue passes over the output
(include/cuda/ConvLayer.h:278-307).  The library's fused epilogue removes all of those passes but one read
and one write of the conv output; this module removes that last pass too, where cuDNN can: the layer becomes
a cuDNN operation graph  conv -> * a[k] -> + b[k] -> activation (-> + residual)  built with the cuDNN frontend
and executed by one of cuDNN's runtime-fusion engines, so the convolution's result never visits HBM before the
epilogue has been applied.  ``a``/``b`` are the folded batch-norm coefficients of ``pxe_fold_bn``.

This is library code on both sides of the fusion (cuDNN owns the convolution in the reference as well); it is
optional (``Runner(conv_fusion=True)``), chosen per layer by measurement: at construction of a layer's graph
every candidate plan is timed against the split form (cuDNN convolution + ``pxe_conv_epilogue_nhwc``) on the
layer's real tensors, and the layer keeps whichever is faster.  cuDNN's first heuristic choice is not always
the fastest plan and for some shapes no fused plan beats the split form.

Needs the ``cudnn`` Python frontend; there is no fallback: asking for fusion without it raises.
"""
from __future__ import annotations

from typing import Callable, Dict, Optional, Tuple

import torch

_ACT_OPS = ("linear", "leaky", "relu", "logistic", "swish")


def _frontend():
    try:
        import cudnn  # noqa: WPS433
    except Exception as e:  # pragma: no cover - depends on the image
        raise RuntimeError("conv fusion needs the cuDNN Python frontend (module 'cudnn'): %s" % e)
    return cudnn


def _pixel_stride(t: torch.Tensor) -> Optional[int]:
    """Channel count of the buffer a channels-last tensor (or a channel slot of one) lives in."""
    B, C, H, W = t.shape
    if t.stride(1) != 1:
        return None
    if W > 1:
        ps = t.stride(3)
    elif H > 1:
        ps = t.stride(2)
    else:
        return None
    if ps < C or (H > 1 and t.stride(2) != W * ps) or (B > 1 and t.stride(0) != H * W * ps):
        return None
    return ps


class FusedConv:
    """One layer shape: the cuDNN graph, its tensors and the plan that won the timing."""

    def __init__(self, graph, tensors, plan: int, workspace: torch.Tensor, name: str, ms: float, split_ms: float):
        self.graph, self.tensors, self.plan, self.workspace = graph, tensors, plan, workspace
        self.name, self.ms, self.split_ms = name, ms, split_ms


class FusedConvPlanner:
    """Builds, times and caches the fused graphs of one device."""

    max_candidates = 6      # plans compiled and timed per layer shape (runtime compilation costs ~0.3 s each)
    prefer_fused = False    # True: keep the best fused plan even where the split form timed faster (tests)

    def __init__(self, device):
        self.cudnn = _frontend()
        self.device = device
        with torch.cuda.device(device):
            self.handle = self.cudnn.create_handle()
        self.cache: Dict[Tuple, Optional[FusedConv]] = {}
        self.log = []           # (key, chosen plan name or "split", fused ms, split ms)

    # ------------------------------------------------------------------ keys
    @staticmethod
    def key(x, weight, stride, padding, act, out, residual, res_act) -> Optional[Tuple]:
        if act not in _ACT_OPS or res_act not in ("linear", "leaky"):
            return None
        if not x.is_contiguous(memory_format=torch.channels_last) or x.shape[2] * x.shape[3] == 1:
            return None
        ops_ = _pixel_stride(out)
        rps = _pixel_stride(residual) if residual is not None else 0
        if ops_ is None or rps is None or out.shape[1] < 2:
            return None
        return (tuple(x.shape), tuple(weight.shape), int(stride), int(padding), act, tuple(out.shape), ops_, rps, res_act)

    def known(self, key) -> bool:
        return key in self.cache

    # ------------------------------------------------------------------ build
    def _build(self, key):
        cudnn = self.cudnn
        (N, C, H, W), (K, _, R, S), stride, pad, act, (_, _, OH, OW), ops_, rps, res_act = key
        f32 = cudnn.data_type.FLOAT
        g = cudnn.pygraph(io_data_type=f32, intermediate_data_type=f32, compute_data_type=f32, handle=self.handle)
        X = g.tensor(name="x", dim=[N, C, H, W], stride=[C * H * W, 1, W * C, C], data_type=f32)
        Wt = g.tensor(name="w", dim=[K, C, R, S], stride=[C * R * S, 1, S * C, C], data_type=f32)
        A = g.tensor(name="a", dim=[1, K, 1, 1], stride=[K, 1, K, K], data_type=f32)
        Bv = g.tensor(name="b", dim=[1, K, 1, 1], stride=[K, 1, K, K], data_type=f32)
        y = g.conv_fprop(image=X, weight=Wt, padding=[pad, pad], stride=[stride, stride], dilation=[1, 1])
        y = g.bias(input=g.scale(input=y, scale=A), bias=Bv)
        y = self._activation(g, y, act)
        Rt = None
        if rps:
            Rt = g.tensor(name="r", dim=[N, K, OH, OW], stride=[OH * OW * rps, 1, OW * rps, rps], data_type=f32)
            y = self._activation(g, g.add(a=y, b=Rt), res_act)
        y.set_output(True).set_data_type(f32).set_dim([N, K, OH, OW]).set_stride([OH * OW * ops_, 1, OW * ops_, ops_])
        g.validate()
        g.build_operation_graph()
        g.create_execution_plans([cudnn.heur_mode.A, cudnn.heur_mode.FALLBACK])
        g.check_support()
        return g, (X, Wt, A, Bv, Rt, y)

    @staticmethod
    def _activation(g, y, act):
        if act == "leaky":
            return g.leaky_relu(input=y, negative_slope=0.1)
        if act == "relu":
            return g.relu(input=y)
        if act == "logistic":
            return g.sigmoid(input=y)
        if act == "swish":
            return g.mul(a=y, b=g.sigmoid(input=y))      # x * sigmoid(x), as the reference's functor (include/Activation.h)
        return y

    # ------------------------------------------------------------------ run
    def _args(self, fc_tensors, x, weight, a, b, out, residual):
        X, Wt, A, Bv, Rt, Y = fc_tensors
        args = {X: x, Wt: weight, A: a.view(1, -1, 1, 1), Bv: b.view(1, -1, 1, 1), Y: out}
        if Rt is not None:
            args[Rt] = residual
        return args

    def _time(self, fn: Callable[[], None], reps: int = 3) -> float:
        fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        e1.synchronize()
        return e0.elapsed_time(e1) / reps

    def tune(self, key, x, weight, a, b, out, residual, split: Callable[[], None]) -> Optional[FusedConv]:
        """Times the split form and the candidate fused plans on the layer's own tensors; caches the winner
        (None = the split form stays)."""
        cudnn = self.cudnn
        cudnn.set_stream(handle=self.handle, stream=torch.cuda.current_stream().cuda_stream)
        split_ms = self._time(split)
        best: Optional[FusedConv] = None
        try:
            g, tensors = self._build(key)
            args = self._args(tensors, x, weight, a, b, out, residual)
            tried = 0
            for pi in range(g.get_execution_plan_count()):
                if tried >= self.max_candidates:
                    break
                try:
                    g.build_plan_at_index(pi)
                    ws = torch.empty(max(int(g.get_workspace_size_plan_at_index(pi)), 16), device=self.device, dtype=torch.uint8)
                    name = g.get_plan_name_at_index(pi)
                except Exception:
                    continue
                tried += 1

                def one(pi=pi, ws=ws):
                    g.execute_plan_at_index(args, ws, pi, handle=self.handle)

                one()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(); one(); e1.record(); e1.synchronize()
                if e0.elapsed_time(e1) > 4.0 * split_ms:
                    continue
                ms = self._time(one)
                if best is None or ms < best.ms:
                    best = FusedConv(g, tensors, pi, ws, name, ms, split_ms)
        except Exception as e:  # an unsupported graph: the split form stays
            self.log.append((key, "unsupported: %s" % str(e)[:120], None, split_ms))
            self.cache[key] = None
            return None
        if best is not None and best.ms >= split_ms and not self.prefer_fused:
            self.log.append((key, "split (best fused %s %.3f ms)" % (best.name, best.ms), best.ms, split_ms))
            best = None
        elif best is not None:
            self.log.append((key, best.name, best.ms, split_ms))
        else:
            self.log.append((key, "split (no fused plan)", None, split_ms))
        self.cache[key] = best
        return best

    def run(self, key, x, weight, a, b, out, residual) -> bool:
        """Executes the cached fused plan of ``key``; False when the layer keeps the split form."""
        fc = self.cache.get(key)
        if fc is None:
            return False
        self.cudnn.set_stream(handle=self.handle, stream=torch.cuda.current_stream().cuda_stream)
        fc.graph.execute_plan_at_index(self._args(fc.tensors, x, weight, a, b, out, residual), fc.workspace, fc.plan,
                                       handle=self.handle)
        return True

    def summary(self) -> Dict[str, float]:
        fused = [e for e in self.log if e[2] is not None and not str(e[1]).startswith("split")]
        return {"shapes": len(self.log), "fused": len(fused),
                "fused_ms": round(sum(e[2] for e in fused), 3), "split_ms_of_fused": round(sum(e[3] for e in fused), 3)}
