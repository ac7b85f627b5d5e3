"""PixieNN model graphs: YAML -> layer list with shapes, and the fusion plan for the epilogue path.

Shape propagation follows the reference's ``Model<D>::parseModel`` (include/Model.h:1596-1641) and
the layer constructors (ConvLayer.h:74-123, MaxPoolLayer.h:51-71, UpsampleLayer.h:49-63,
RouteLayer.h:40-80, ShortcutLayer.h:45-75, YoloLayer.h:115-147, CenterNetLayer.h:49-69,
RegionLayer.h, SoftmaxLayer.h:60-79), so the same YAML files drive this package unchanged.

``plan()`` decides, once per model, what the reference does layer by layer at run time:
which conv epilogues absorb the shortcut or 2x2 max pool that follows them, which producers store
straight into a route's concat buffer (so the route itself runs nothing), which stride-1 pools
form an SPP block that reads its input once, and which YOLO heads are decoded from the raw conv
output.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import yaml


@dataclass
class Layer:
    index: int
    type: str
    params: dict
    in_shape: Tuple[int, int, int]           # channels, height, width of the layer's input
    out_shape: Tuple[int, int, int]
    sources: List[int]                       # layer indices read (-1 = the network input)
    # conv
    filters: int = 0
    kernel: int = 1
    stride: int = 1
    padding: int = 0
    dilation: int = 1
    groups: int = 1
    batch_norm: bool = False
    activation: str = "linear"
    # shortcut
    alpha: float = 1.0
    beta: float = 1.0

    @property
    def out_elems(self) -> int:
        c, h, w = self.out_shape
        return c * h * w


@dataclass
class Model:
    channels: int
    height: int
    width: int
    layers: List[Layer]
    classes: Optional[int] = None

    def consumers(self) -> Dict[int, List[int]]:
        cons: Dict[int, List[int]] = {i: [] for i in range(-1, len(self.layers))}
        for l in self.layers:
            for s in l.sources:
                cons[s].append(l.index)
        return cons


def load_yaml(path: str) -> dict:
    with open(path) as f:
        return yaml.safe_load(f)


def parse_model(doc: dict, height: Optional[int] = None, width: Optional[int] = None,
                classes: Optional[int] = None) -> Model:
    """``doc`` is the parsed model YAML (with or without the top-level ``model`` key)."""
    m = doc.get("model", doc)
    C, H, W = int(m["channels"]), int(height or m["height"]), int(width or m["width"])
    layers: List[Layer] = []
    c, h, w = C, H, W
    for i, ld in enumerate(m.get("layers") or []):
        t = ld["type"]
        L = Layer(i, t, dict(ld), (c, h, w), (c, h, w), [i - 1])
        if t == "conv":
            L.activation = ld.get("activation", "logistic")                   # ConvLayer.h:77
            L.batch_norm = bool(ld.get("batch_normalize", False))
            L.dilation = int(ld.get("dilation", 1))
            L.filters = int(ld.get("filters", 1))
            L.kernel = int(ld.get("kernel", 1))
            eff = L.dilation * (L.kernel - 1) + 1
            L.padding = eff // 2 if ld.get("pad", False) else 0
            L.stride = int(ld.get("stride", 1))
            L.groups = max(1, int(ld.get("groups", 1)))
            L.out_shape = (L.filters, (h + 2 * L.padding - eff) // L.stride + 1,
                           (w + 2 * L.padding - eff) // L.stride + 1)
        elif t == "maxpool":
            L.kernel = int(ld.get("kernel", 1))
            L.stride = int(ld.get("stride", 1))
            L.padding = int(ld.get("padding", max(0, L.kernel - 1)))          # MaxPoolLayer.h:56
            L.out_shape = (c, _cdiv(h + L.padding - L.kernel, L.stride) + 1,
                           _cdiv(w + L.padding - L.kernel, L.stride) + 1)
        elif t == "upsample":
            L.stride = int(ld.get("stride", 2))
            L.alpha = float(ld.get("scale", 1.0))
            L.out_shape = (c, h * L.stride, w * L.stride)
        elif t == "route":
            srcs = [(s if s >= 0 else i + s) for s in ld["layers"]]
            for s in srcs:
                if not 0 <= s < i:
                    raise ValueError(f"layer {i}: route source {s} out of range")
            L.sources = srcs
            first = layers[srcs[0]].out_shape
            for s in srcs[1:]:
                if layers[s].out_shape[1:] != first[1:]:
                    raise ValueError(f"layer {i}: route layers must have matching spatial dimensions")
            L.out_shape = (sum(layers[s].out_shape[0] for s in srcs), first[1], first[2])
        elif t == "shortcut":
            frm = int(ld["from"])
            frm = frm if frm >= 0 else i + frm
            if not 0 <= frm < i:
                raise ValueError(f"layer {i}: shortcut source {frm} out of range")
            L.sources = [i - 1, frm]
            L.activation = ld.get("activation", "linear")                     # ShortcutLayer.h:49
            L.alpha, L.beta = float(ld.get("alpha", 1.0)), float(ld.get("beta", 1.0))
        elif t in ("yolo", "centernet", "region", "softmax", "dropout", "detection"):
            pass
        elif t == "avgpool":
            L.out_shape = (c, 1, 1)
        elif t in ("connected", "conn"):
            L.filters = int(ld.get("output", ld.get("outputs", 1)))
            L.activation = ld.get("activation", "logistic")
            L.batch_norm = bool(ld.get("batch_normalize", False))
            L.out_shape = (L.filters, 1, 1)
        else:
            raise ValueError(f"layer {i}: unsupported layer type {t!r}")
        layers.append(L)
        c, h, w = L.out_shape
    model = Model(C, H, W, layers, classes)
    if model.classes is None:
        model.classes = _infer_classes(model)
    return model


def _cdiv(a: int, b: int) -> int:
    """C integer division (truncation toward zero)."""
    q = abs(a) // abs(b)
    return q if (a >= 0) == (b > 0) else -q


def _infer_classes(model: Model) -> Optional[int]:
    for l in model.layers:
        if l.type == "yolo":
            return l.in_shape[0] // len(l.params["mask"]) - 5
        if l.type == "centernet":
            return l.in_shape[0] - 4
        if l.type == "region":
            return int(l.params.get("classes", 20))
        if l.type == "detection":
            side, num = int(l.params.get("side", 7)), int(l.params.get("num", 1))
            coords = int(l.params.get("coords", 4))
            return l.in_shape[0] * l.in_shape[1] * l.in_shape[2] // (side * side) - num * (1 + coords)
        if l.type == "softmax":
            return l.in_shape[0] * l.in_shape[1] * l.in_shape[2]
    return None


# ------------------------------------------------------------------------------------------ plan
@dataclass
class Dest:
    """Where a produced tensor is stored: a dense tensor of its own, or a channel slot of a route's
    concat buffer."""
    kind: str                  # "dense" | "slot"
    route: int = -1            # concat buffer id (the route layer index) for kind == "slot"
    offset: int = 0            # first channel of the slot


@dataclass
class Step:
    """One launch (or one convolution + its fused epilogue)."""
    op: str                    # conv | maxpool | spp | upsample | shortcut | concat | yolo | centernet |
    #                            region | softmax | avgpool | alias
    layer: int                 # the layer whose output this step produces (for spp: the first pool)
    inputs: List[int] = field(default_factory=list)
    dests: List[Dest] = field(default_factory=list)
    fused_shortcut: Optional[int] = None      # shortcut layer absorbed into this conv's epilogue
    fused_pool: Optional[int] = None          # maxpool layer absorbed
    pool_dests: List[Dest] = field(default_factory=list)
    keep_full: bool = True                    # with fused_pool: is the full-resolution output needed too
    spp_layers: List[int] = field(default_factory=list)
    spp_dests: List[List[Dest]] = field(default_factory=list)
    head_raw: bool = False                    # yolo: decode the raw conv output (conv step skipped its epilogue)
    produces: List[int] = field(default_factory=list)   # every layer index whose value this step defines


@dataclass
class Plan:
    model: Model
    steps: List[Step]
    alias: Dict[int, int]                     # layer -> layer whose tensor it shares (fan-in-1 routes, fused layers)
    concat_channels: Dict[int, int]           # route id -> total channels
    last_use: Dict[int, int]                  # layer -> index of the last step that reads it
    stats: Dict[str, int] = field(default_factory=dict)


def plan(model: Model, fuse: bool = True, raw_heads: bool = True) -> Plan:
    """Builds the launch list.  ``fuse=False`` gives the layer-by-layer schedule (one step per layer,
    every route a real concat) used as the unfused comparison."""
    L = model.layers
    n = len(L)
    cons = model.consumers()
    alias: Dict[int, int] = {}

    def resolve(i: int) -> int:
        while i in alias:
            i = alias[i]
        return i

    # 1. fan-in-1 routes are pure aliases
    for l in L:
        if l.type == "route" and len(l.sources) == 1 and fuse:
            alias[l.index] = l.sources[0]

    # consumers seen through aliases: who really reads tensor t
    def real_consumers(t: int) -> List[int]:
        out = []
        for c in cons[t]:
            if c in alias and alias[c] == t:
                out.extend(real_consumers(c))
            else:
                out.append(c)
        return out

    # 2. slots: for each fan-in>1 route, each source tensor gets a channel range
    slots: Dict[int, List[Tuple[int, int]]] = {}        # tensor -> [(route, channel offset)]
    concat_channels: Dict[int, int] = {}
    if fuse:
        for l in L:
            if l.type == "route" and len(l.sources) > 1:
                off = 0
                for s in l.sources:
                    slots.setdefault(resolve(s), []).append((l.index, off))
                    off += L[s].out_shape[0]
                concat_channels[l.index] = off

    absorbed = set()
    steps: List[Step] = []
    stats = {"fused_shortcut": 0, "fused_pool": 0, "routes_eliminated": 0, "routes_aliased": 0, "spp_blocks": 0,
             "raw_heads": 0, "concat_copies": 0}

    def needs_dense(t: int, readers: List[int]) -> bool:
        """A dense copy is needed when a reader cannot take a strided channel slot (the cuDNN
        convolution and the heads read dense tensors) or when the tensor has no slot at all."""
        if t not in slots:
            return True
        for r in readers:
            if L[r].type in ("conv", "connected", "conn", "yolo", "centernet", "region", "softmax", "avgpool", "dropout",
                             "detection"):
                return True
        return False

    def dests_for(t: int, readers: List[int]) -> List[Dest]:
        ds: List[Dest] = []
        if needs_dense(t, readers):
            ds.append(Dest("dense"))
        for (r, off) in slots.get(t, []):
            ds.append(Dest("slot", r, off))
        return ds

    i = 0
    while i < n:
        l = L[i]
        if i in absorbed:
            i += 1
            continue
        if i in alias:
            steps.append(Step("alias", i, [alias[i]], produces=[i]))
            stats["routes_aliased"] += 1
            i += 1
            continue
        if l.type == "conv":
            st = Step("conv", i, [resolve(l.sources[0])], produces=[i])
            out_t = i
            readers = real_consumers(i)
            nxt = L[i + 1] if i + 1 < n else None
            if fuse and nxt is not None and readers == [i + 1]:
                if nxt.type == "shortcut" and nxt.sources[0] == i and L[nxt.sources[1]].out_shape == l.out_shape:
                    st.fused_shortcut = i + 1
                    st.inputs.append(resolve(nxt.sources[1]))
                    absorbed.add(i + 1)
                    alias[i] = i + 1            # the conv's own value is never materialised
                    out_t = i + 1
                    st.produces = [i + 1]
                    stats["fused_shortcut"] += 1
                elif raw_heads and nxt.type == "yolo" and not l.batch_norm and l.activation == "linear":
                    st.head_raw = True
                    stats["raw_heads"] += 1
            if fuse and st.fused_shortcut is None and nxt is not None and nxt.type == "maxpool" \
                    and nxt.kernel == 2 and nxt.stride == 2 and nxt.padding in (0, 1) and (i + 1) in readers:
                others = [r for r in readers if r != i + 1]
                covered = 2 * nxt.out_shape[1] >= l.out_shape[1] and 2 * nxt.out_shape[2] >= l.out_shape[2]
                if covered or not others:
                    st.fused_pool = i + 1
                    st.keep_full = bool(others) or i in slots
                    st.pool_dests = dests_for(i + 1, real_consumers(i + 1))
                    absorbed.add(i + 1)
                    st.produces.append(i + 1)
                    stats["fused_pool"] += 1
                    readers = others
            st.dests = dests_for(out_t, real_consumers(out_t) if out_t != i else readers)
            if st.fused_pool is not None and not st.keep_full:
                st.dests = []
            steps.append(st)
        elif l.type == "maxpool":
            src = resolve(l.sources[0])
            group = [i]
            if fuse and l.stride == 1 and l.padding == l.kernel - 1:
                # SPP: later stride-1 pools of the same tensor, separated only by alias routes
                j = i + 1
                while j < n:
                    if j in alias:
                        j += 1
                        continue
                    lj = L[j]
                    if lj.type == "maxpool" and lj.stride == 1 and lj.padding == lj.kernel - 1 \
                            and resolve(lj.sources[0]) == src and len(group) < 4:
                        group.append(j)
                        j += 1
                        continue
                    break
            if len(group) > 1:
                st = Step("spp", i, [src], spp_layers=group, produces=list(group))
                st.spp_dests = [dests_for(g, real_consumers(g)) for g in group]
                for g in group[1:]:
                    absorbed.add(g)
                steps.append(st)
                stats["spp_blocks"] += 1
            else:
                steps.append(Step("maxpool", i, [src], dests_for(i, real_consumers(i)), produces=[i]))
        elif l.type == "upsample":
            steps.append(Step("upsample", i, [resolve(l.sources[0])], dests_for(i, real_consumers(i)), produces=[i]))
        elif l.type == "shortcut":
            steps.append(Step("shortcut", i, [resolve(l.sources[0]), resolve(l.sources[1])],
                              dests_for(i, real_consumers(i)), produces=[i]))
        elif l.type == "route":
            if fuse:
                # every source already stored into this route's buffer
                # (if this route is itself a source of a later route, its buffer is copied into that slot)
                steps.append(Step("alias", i, [], [Dest("slot", r, off) for (r, off) in slots.get(i, [])],
                                  produces=[i]))
                stats["routes_eliminated"] += 1
            else:
                steps.append(Step("concat", i, list(l.sources), [Dest("dense")], produces=[i]))
                stats["concat_copies"] += 1
        elif l.type in ("yolo", "centernet", "region", "softmax", "avgpool", "dropout", "connected", "conn", "detection"):
            # a dense tensor of its own, plus a copy into every route buffer that concatenates it
            st = Step(l.type, i, [resolve(l.sources[0])],
                      [Dest("dense")] + [Dest("slot", r, off) for (r, off) in slots.get(i, [])], produces=[i])
            if l.type == "yolo" and steps and steps[-1].op == "conv" and steps[-1].head_raw:
                st.head_raw = True
            steps.append(st)
        else:
            raise ValueError(f"cannot plan layer type {l.type}")
        i += 1

    # a slot consumer that reads a concat buffer which is itself a source of another route needs a copy:
    # handled at run time by treating route outputs as ordinary tensors with slots (dests_for is
    # consulted when the route's buffer is complete).
    last_use: Dict[int, int] = {}
    for si, st in enumerate(steps):
        for t in st.inputs:
            last_use[t] = si
    return Plan(model, steps, alias, concat_channels, last_use, stats)


# ------------------------------------------------------------------------- the library's planner
_LAYER_TYPE = {"conv": 0, "maxpool": 1, "upsample": 2, "route": 3, "shortcut": 4, "yolo": 5, "centernet": 6,
               "region": 7, "softmax": 8, "avgpool": 9, "dropout": 10, "connected": 11, "conn": 11, "detection": 12}
_STEP_OP = {0: "conv", 1: "alias", 2: "maxpool", 3: "spp", 4: "upsample", 5: "shortcut", 6: "concat"}


def layer_descs(model: Model):
    """The model as the array of ``pxe_layer_desc`` records that ``pxe_plan_build`` takes
    (include/pxe_plan.h): what a C++ caller fills from its own layer objects."""
    from . import capi
    arr = (capi.LayerDesc * len(model.layers))()
    for l, d in zip(model.layers, arr):
        d.type = _LAYER_TYPE[l.type]
        d.out_channels, d.out_height, d.out_width = l.out_shape
        d.kernel, d.stride, d.padding = l.kernel, l.stride, l.padding
        d.batch_norm = int(l.batch_norm)
        d.activation = capi.ACT.get(l.activation, capi.ACT["linear"])
        if len(l.sources) > capi.PLAN_MAX_SOURCES:
            raise ValueError(f"layer {l.index}: {len(l.sources)} sources exceed {capi.PLAN_MAX_SOURCES}")
        d.n_sources = len(l.sources)
        for k, s in enumerate(l.sources):
            d.sources[k] = s
    return arr


def plan_native(model: Model, fuse: bool = True, raw_heads: bool = True) -> Plan:
    """The same plan as :func:`plan`, built by the library's C++ planner (``pxe_plan_build``) and
    converted to the Python records the runner walks."""
    import ctypes as C
    from . import capi
    L = capi.lib()
    descs = layer_descs(model)
    handle = C.c_void_p()
    capi.check(L.pxe_plan_build(descs, len(model.layers), int(fuse), int(raw_heads), C.byref(handle)))
    try:
        def dests(arr, n):
            return [Dest("slot", arr[k].route, arr[k].channel_offset) if arr[k].kind else Dest("dense") for k in range(n)]

        steps: List[Step] = []
        for si in range(L.pxe_plan_step_count(handle)):
            s = L.pxe_plan_step(handle, si).contents
            layer = model.layers[s.layer]
            op = _STEP_OP.get(s.op) or ("connected" if layer.type == "conn" else layer.type)
            st = Step(op, s.layer, [s.inputs[k] for k in range(s.n_inputs)], dests(s.dests, s.n_dests))
            if op == "concat":
                st.inputs = list(layer.sources)
            st.fused_shortcut = s.fused_shortcut if s.fused_shortcut >= 0 else None
            st.fused_pool = s.fused_pool if s.fused_pool >= 0 else None
            st.keep_full = bool(s.keep_full)
            st.pool_dests = dests(s.pool_dests, s.n_pool_dests)
            st.head_raw = bool(s.head_raw)
            st.spp_layers = [s.spp_layers[g] for g in range(s.n_spp)]
            st.spp_dests = [dests(s.spp_dests[g], s.n_spp_dests[g]) for g in range(s.n_spp)]
            if st.spp_layers:
                st.produces = list(st.spp_layers)
            elif st.fused_shortcut is not None:
                st.produces = [st.fused_shortcut]
            else:
                st.produces = [s.layer] + ([st.fused_pool] if st.fused_pool is not None else [])
            steps.append(st)
        n = len(model.layers)
        alias = {i: L.pxe_plan_alias(handle, i) for i in range(n) if L.pxe_plan_alias(handle, i) >= 0}
        concat = {i: L.pxe_plan_concat_channels(handle, i) for i in range(n) if L.pxe_plan_concat_channels(handle, i) > 0}
        last_use = {i: L.pxe_plan_last_use(handle, i) for i in range(-1, n) if L.pxe_plan_last_use(handle, i) >= 0}
        stats = capi.PlanStats()
        L.pxe_plan_get_stats(handle, C.byref(stats))
        return Plan(model, steps, alias, concat, last_use, {name: getattr(stats, name) for name, _ in stats._fields_})
    finally:
        L.pxe_plan_destroy(handle)
