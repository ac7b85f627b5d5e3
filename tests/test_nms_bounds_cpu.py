"""The two cheap upper bounds the device NMS puts in front of the exact IoU (csrc/pxe_nms_gpu.cu, cross-class pass)
never reject a pair that the exact single-precision expression would count as overlapping by more than 0.9.

Everything here is float32 numpy arithmetic, operation by operation as the kernel evaluates it (every product, sum and
quotient rounded once): `iou32` restates rect_intersect / rect_iou (cv::Rect2f's `&` and the reference's IoU,
src/Box.cpp:25-54), `maybe32` the bounds with their "plain box" switch.  No GPU, no library call.
"""
import numpy as np

F = np.float32


def iou32(a, b):
    """rect_iou(a, b) of the kernel for arrays of boxes [n, 4] = x, y, w, h (float32)."""
    ax, ay, aw, ah = (a[:, i] for i in range(4))
    bx, by, bw, bh = (b[:, i] for i in range(4))
    empty = (aw <= 0) | (ah <= 0) | (bw <= 0) | (bh <= 0)
    a_first_x, a_first_y = ax < bx, ay < by
    xmin_x, xmin_w = np.where(a_first_x, ax, bx), np.where(a_first_x, aw, bw)
    xmax_x, xmax_w = np.where(a_first_x, bx, ax), np.where(a_first_x, bw, aw)
    ymin_y, ymin_h = np.where(a_first_y, ay, by), np.where(a_first_y, ah, bh)
    ymax_y, ymax_h = np.where(a_first_y, by, ay), np.where(a_first_y, bh, ah)
    apart = ((xmin_x < 0) & ((xmin_x + xmin_w) < xmax_x)) | ((ymin_y < 0) & ((ymin_y + ymin_h) < ymax_y))
    rw = np.minimum(xmin_w - (xmax_x - xmin_x), xmax_w)
    rh = np.minimum(ymin_h - (ymax_y - ymin_y), ymax_h)
    none = empty | apart | (rw <= 0) | (rh <= 0)
    inter = np.where(none, F(0), rw * rh).astype(F)
    uni = np.maximum(F(0), (aw * ah + bw * bh) - inter).astype(F)
    with np.errstate(divide="ignore", invalid="ignore"):
        r = (inter / uni).astype(F)
    return np.where(np.isfinite(r), r, F(0)).astype(F)


def area_or_nan(r):
    x, y, w, h = (r[:, i] for i in range(4))
    plain = (np.abs(x) + w <= F(16384) * w) & (np.abs(y) + h <= F(16384) * h)
    return np.where(plain, w * h, F(np.nan)).astype(F)


def maybe32(q, p):
    """True where the kernel goes on to the exact expression for the pair (q later than p in the order)."""
    aq, ap = area_or_nan(q), area_or_nan(p)
    with np.errstate(invalid="ignore"):
        maybe = ~((aq < F(0.8) * ap) | (ap < F(0.8) * aq))
        both = maybe & (aq == aq) & (ap == ap)
        wi = np.minimum(q[:, 0] + q[:, 2], p[:, 0] + p[:, 2]) - np.maximum(q[:, 0], p[:, 0])
        hi = np.minimum(q[:, 1] + q[:, 3], p[:, 1] + p[:, 3]) - np.maximum(q[:, 1], p[:, 1])
        near = ~((wi < F(0.8) * q[:, 2]) | (hi < F(0.8) * q[:, 3]))
    return np.where(both, near, maybe)


def boxes(rng, n, origin, size):
    xy = (rng.random((n, 2)) * 2 - 1) * origin
    wh = rng.random((n, 2)) * size + size * 1e-3
    return np.concatenate([xy, wh], 1).astype(F)


def nudged(rng, p, rel):
    """Boxes close to p: corners moved and sizes scaled by up to `rel` of the size."""
    q = p.copy()
    q[:, 0:2] += ((rng.random((len(p), 2)) * 2 - 1) * rel).astype(F) * p[:, 2:4]
    q[:, 2:4] *= (1 + (rng.random((len(p), 2)) * 2 - 1) * rel).astype(F)
    return q.astype(F)


def test_bounds_never_hide_an_overlap_above_the_threshold():
    rng = np.random.default_rng(2024)
    n = 200_000
    hits = 0
    cases = []
    for origin, size in ((500.0, 100.0), (1.0, 0.3), (4096.0, 8.0), (1e6, 1e-2), (1e7, 1.0), (0.0, 50.0), (3e4, 1.0)):
        p = boxes(rng, n, origin, size)
        cases.append((boxes(rng, n, origin, size), p))                      # unrelated boxes
        for rel in (0.3, 0.1, 0.03, 0.005):
            cases.append((nudged(rng, p, rel), p))                          # near-duplicates on both sides of 0.9
    for q, p in cases:
        exact = iou32(q, p) > F(0.9)
        kept = maybe32(q, p)
        assert not np.any(exact & ~kept), "a bound rejected a pair whose exact IoU exceeds 0.9"
        hits += int(exact.sum())
    assert hits > 100_000                                                   # the near-duplicates do cross the threshold


def test_bounds_do_spare_unrelated_pairs_the_exact_expression():
    rng = np.random.default_rng(7)
    q, p = boxes(rng, 100_000, 250.0, 100.0), boxes(rng, 100_000, 250.0, 100.0)
    assert maybe32(q, p).mean() < 0.01
    # boxes whose coordinates dwarf their size are never rejected by the bounds: their areas are NaNs
    far = boxes(rng, 1000, 1e7, 1e-2)
    assert np.isnan(area_or_nan(far)).mean() > 0.95 and maybe32(far, far[::-1].copy()).all()


def test_matrix_then_in_order_resolution_equals_the_pivot_loop():
    """The cross-class pass finds every "q would fall to p" pair first and then walks the rows in order; the reference
    walks the pivots in order (src/Box.cpp:80-96): p discards q only while p itself stands.  Same survivors."""
    rng = np.random.default_rng(11)
    for n, density in ((40, 0.05), (64, 0.2), (33, 0.5), (100, 0.01), (7, 1.0)):
        for _ in range(50):
            falls_to = np.tril(rng.random((n, n)) < density, -1)            # [q, p], p < q
            dead_ref = np.zeros(n, bool)
            for p in range(n):                                              # the pivot loop
                if dead_ref[p]:
                    continue
                dead_ref |= falls_to[:, p] & (np.arange(n) > p)
            dead = np.zeros(n, bool)
            for q in range(1, n):                                           # rows in order, as the resolving warp does
                if falls_to[q].any() and (falls_to[q] & ~dead).any():
                    dead[q] = True
            assert np.array_equal(dead, dead_ref)
