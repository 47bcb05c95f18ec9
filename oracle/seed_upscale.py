"""CPU oracle for the seed + incremental-upscale quantiser.  TEST INFRASTRUCTURE ONLY.

A numpy / plain-Python restatement of what the reference project computes per weight row in
any_precision/quantization/quantize.py:85-187 (``_seed_and_upscale_layer``) and :13-76
(``_upscale_group``, ``_increment_group``):

* sample weights are the sensitivities with the entries of zero weights masked out (:118-120);
* the row is sorted by value, prefix sums of ``w``, ``w * x`` (and ``w * x * x``) are taken in fp64;
  a row whose sample weights sum to zero is treated as unweighted (:124-143);
* a ``2**seed_bit``-cluster 1-D k-means on the sorted row gives the seed table and the cluster
  borders (:145-157, centroids cast to fp32);
* every further bit splits every cluster in two with a 2-cluster 1-D k-means; an empty cluster hands
  its centroid to both children (:43-74); tables are fp32 at every level;
* the parent-precision cluster index of every weight, un-sorted, is the stored code (:171-180); the
  tables go to fp16 when saved (:205-207).

Parity status: UNPINNED for the two k-means primitives.  The reference takes them from the package
``flash1dkmeans`` (requirements.txt:14, ``>=0.2.3``), which is neither vendored in the reference nor
installed on the build machine, and its k-cluster routine starts from a randomised k-means++ draw
(``random_state=None`` by default, quantize.py:262), so no bit-level agreement with a run of the
reference exists even in principle.  ``kmeans_k_cluster`` and ``kmeans_two_cluster`` below restate
the package's published approach (Lloyd iterations and a binary search for the split, both on prefix
sums of the sorted row) with a deterministic start.  Everything around the two primitives IS pinned:
``tests/golden/make_quantizer_fixture.py`` runs the reference's own ``_seed_and_upscale_layer`` with
these two functions standing in for the missing package and stores its output; the tests compare
``seed_and_upscale_row`` with it.

The two primitives are written as scalar loops over plain arrays so that the fixture script can hand
the very same source to ``numba.njit``.

Nothing that ships imports this module.
"""
from __future__ import annotations

import numpy as np

THREADS = 1024      # the CUDA kernel's block size: its prefix sums add in this blocked order


# ----------------------------------------------------------------------------- the two primitives
def _range_sum(prefix, a, b):
    """Sum over sorted positions [a, b) from an inclusive prefix-sum array."""
    if b <= a:
        return 0.0
    if a > 0:
        return prefix[b - 1] - prefix[a - 1]
    return prefix[b - 1]


def _count_le(sorted_X, start, stop, v):
    """start + number of sorted_X[start:stop] that are <= v (bisect right)."""
    lo = start
    hi = stop
    while lo < hi:
        m = (lo + hi) // 2
        if np.float64(sorted_X[m]) <= v:
            lo = m + 1
        else:
            hi = m
    return lo


def kmeans_k_cluster(sorted_X, n_clusters, max_iter, weights_prefix_sum, weighted_X_prefix_sum, start_idx, stop_idx):
    """Deterministic 1-D k-means on ``sorted_X[start_idx:stop_idx]``.

    Start: clusters of equal weight mass (border j = number of positions whose inclusive weight prefix is
    <= total * j / k), centroids = their weighted means (a cluster without weight takes the value at its
    first position).  Then Lloyd iterations on the prefix sums: a value goes to the left of two
    neighbouring centroids if it is <= their midpoint; a cluster without weight keeps its centroid; stop
    when the borders repeat or after ``max_iter`` assignments.  Returns fp64 centroids ``[k]`` and int32
    borders ``[k + 1]`` (cluster j = sorted positions [borders[j], borders[j + 1])).
    """
    k = n_clusters
    n = stop_idx - start_idx
    centroids = np.empty(k, dtype=np.float64)
    borders = np.empty(k + 1, dtype=np.int32)
    base = 0.0
    if start_idx > 0:
        base = weights_prefix_sum[start_idx - 1]
    total = weights_prefix_sum[stop_idx - 1] - base
    borders[0] = start_idx
    borders[k] = stop_idx
    for j in range(1, k):
        target = base + total * np.float64(j) / np.float64(k)
        lo = start_idx
        hi = stop_idx
        while lo < hi:
            m = (lo + hi) // 2
            if weights_prefix_sum[m] <= target:
                lo = m + 1
            else:
                hi = m
        borders[j] = lo
    for j in range(1, k):
        if borders[j] < borders[j - 1]:
            borders[j] = borders[j - 1]
    for j in range(k):
        wsum = _range_sum(weights_prefix_sum, borders[j], borders[j + 1])
        if wsum > 0.0:
            centroids[j] = _range_sum(weighted_X_prefix_sum, borders[j], borders[j + 1]) / wsum
        else:
            at = borders[j]
            if at > stop_idx - 1:
                at = stop_idx - 1
            centroids[j] = np.float64(sorted_X[at])
    new_borders = np.empty(k + 1, dtype=np.int32)
    for _ in range(max_iter):
        new_borders[0] = start_idx
        new_borders[k] = stop_idx
        for j in range(1, k):
            mid = (centroids[j - 1] + centroids[j]) * 0.5
            new_borders[j] = _count_le(sorted_X, start_idx, stop_idx, mid)
        for j in range(1, k):
            if new_borders[j] < new_borders[j - 1]:
                new_borders[j] = new_borders[j - 1]
        same = True
        for j in range(k + 1):
            if new_borders[j] != borders[j]:
                same = False
        if same:
            break
        for j in range(k + 1):
            borders[j] = new_borders[j]
        for j in range(k):
            wsum = _range_sum(weights_prefix_sum, borders[j], borders[j + 1])
            if wsum > 0.0:
                centroids[j] = _range_sum(weighted_X_prefix_sum, borders[j], borders[j + 1]) / wsum
    return centroids, borders


def kmeans_two_cluster(sorted_X, weights_prefix_sum, weighted_X_prefix_sum, start_idx, stop_idx):
    """2-cluster 1-D k-means of the non-empty range ``[start_idx, stop_idx)`` of a sorted row.

    One element: both centroids are it, and it stays in the left cluster.  Otherwise a binary search over
    the split position d in [start + 1, stop - 1] for the first d whose element belongs to the right
    cluster, i.e. lies above the midpoint of the weighted means of [start, d) and [d, stop) (a side
    without weight pulls the split towards itself).  Both means rise with d, so the first such d is a
    fixed point of the Lloyd iteration.  A side without weight takes the value next to the split as its
    centroid.  Returns fp64 centroids ``[2]`` and int32 borders ``[start, d, stop]``.
    """
    centroids = np.empty(2, dtype=np.float64)
    borders = np.empty(3, dtype=np.int32)
    borders[0] = start_idx
    borders[2] = stop_idx
    if stop_idx - start_idx == 1:
        centroids[0] = np.float64(sorted_X[start_idx])
        centroids[1] = centroids[0]
        borders[1] = stop_idx
        return centroids, borders
    lo = start_idx + 1
    hi = stop_idx - 1
    while lo < hi:
        d = (lo + hi) // 2
        wl = _range_sum(weights_prefix_sum, start_idx, d)
        wr = _range_sum(weights_prefix_sum, d, stop_idx)
        if wl <= 0.0:
            move_right = True
        elif wr <= 0.0:
            move_right = False
        else:
            mid = (_range_sum(weighted_X_prefix_sum, start_idx, d) / wl +
                   _range_sum(weighted_X_prefix_sum, d, stop_idx) / wr) * 0.5
            move_right = np.float64(sorted_X[d]) <= mid
        if move_right:
            lo = d + 1
        else:
            hi = d
    d = lo
    wl = _range_sum(weights_prefix_sum, start_idx, d)
    wr = _range_sum(weights_prefix_sum, d, stop_idx)
    if wl > 0.0:
        centroids[0] = _range_sum(weighted_X_prefix_sum, start_idx, d) / wl
    else:
        centroids[0] = np.float64(sorted_X[d - 1])
    if wr > 0.0:
        centroids[1] = _range_sum(weighted_X_prefix_sum, d, stop_idx) / wr
    else:
        centroids[1] = np.float64(sorted_X[d])
    borders[1] = d
    return centroids, borders


# ----------------------------------------------------------------------------- a row, a layer
def _cumsum(v, blocked):
    """Inclusive fp64 prefix sums: plain left-to-right (the reference's ``np.cumsum``), or in the CUDA
    kernel's order: THREADS consecutive runs summed left to right, the runs' totals summed left to
    right, offset + local sum."""
    if not blocked:
        return np.cumsum(v)
    n = len(v)
    run = -(-n // THREADS)
    pad = np.zeros(THREADS * run, dtype=np.float64)
    pad[:n] = v
    local = np.cumsum(pad.reshape(THREADS, run), axis=1)
    totals = local[:, -1]
    offset = np.concatenate([[0.0], np.cumsum(totals)[:-1]])
    return (offset[:, None] + local).reshape(-1)[:n]


def prepare_row(x, sensitivity, blocked=False):
    """Sorted row, permutation and the fp64 prefix sums of quantize.py:118-143.  ``-0.0`` counts as ``0.0``
    and equal values keep their original order (the reference's ``np.argsort`` leaves that order open)."""
    x = np.asarray(x, dtype=np.float32) + np.float32(0.0)
    w = np.asarray(sensitivity, dtype=np.float32) * (x != 0)
    order = np.argsort(x, kind="stable")
    sx = x[order]
    sw = w[order].astype(np.float64)
    sx64 = sx.astype(np.float64)
    wp = _cumsum(sw, blocked)
    if wp[-1] == 0:
        wp = np.arange(1, len(sx) + 1, dtype=np.float64)
        wxp = _cumsum(sx64, blocked)
    else:
        wxp = _cumsum(sx64 * sw, blocked)
    return sx, order, wp, wxp


def seed_and_upscale_row(x, sensitivity, seed_bit, parent_bit, max_iter=50, blocked=False):
    """``(luts, codes)`` of one row: ``luts[i]`` is the fp32 table ``[2**(seed_bit + i)]``, ``codes`` the
    uint8 parent-precision cluster index of every weight in its original position."""
    sx, order, wp, wxp = prepare_row(x, sensitivity, blocked)
    n = len(sx)
    cent, borders = kmeans_k_cluster(sx, 1 << seed_bit, max_iter, wp, wxp, 0, n)
    luts = [cent.astype(np.float32)]
    for bit in range(seed_bit, parent_bit):
        old = luts[-1]
        new = np.empty(2 << bit, dtype=np.float32)
        nb = np.empty((2 << bit) + 1, dtype=np.int32)
        for c in range(1 << bit):
            a, b = int(borders[c]), int(borders[c + 1])
            if a == b:
                new[2 * c] = new[2 * c + 1] = old[c]
                nb[2 * c] = nb[2 * c + 1] = a
                continue
            cc, lb = kmeans_two_cluster(sx, wp, wxp, a, b)
            new[2 * c], new[2 * c + 1] = cc[0], cc[1]
            nb[2 * c], nb[2 * c + 1] = a, lb[1]
        nb[-1] = borders[-1]
        luts.append(new)
        borders = nb
    labels = np.empty(n, dtype=np.uint8)
    for c in range(1 << parent_bit):
        labels[borders[c]:borders[c + 1]] = c
    codes = np.empty(n, dtype=np.uint8)
    codes[order] = labels
    return luts, codes


def seed_and_upscale_layer(weight, sensitivity, seed_bit, parent_bit, max_iter=50, blocked=False):
    """Row by row over ``weight[N, K]``: ``({bit: fp16 table [N, 2**bit]}, uint8 codes [N, K])``."""
    weight = np.asarray(weight, dtype=np.float32)
    sensitivity = np.asarray(sensitivity, dtype=np.float32)
    N, K = weight.shape
    luts = {b: np.empty((N, 1 << b), dtype=np.float16) for b in range(seed_bit, parent_bit + 1)}
    codes = np.empty((N, K), dtype=np.uint8)
    for r in range(N):
        row_luts, codes[r] = seed_and_upscale_row(weight[r], sensitivity[r], seed_bit, parent_bit, max_iter, blocked)
        for i, b in enumerate(range(seed_bit, parent_bit + 1)):
            luts[b][r] = row_luts[i].astype(np.float16)
    return luts, codes


def weighted_error(weight, sensitivity, lut, codes):
    """Sum over a layer of sensitivity * (weight - table[code])**2 in fp64 (the k-means objective)."""
    w = np.asarray(weight, dtype=np.float64)
    deq = np.take_along_axis(np.asarray(lut, dtype=np.float64), codes.astype(np.int64), axis=1)
    return float((np.asarray(sensitivity, dtype=np.float64) * (w - deq) ** 2).sum())
