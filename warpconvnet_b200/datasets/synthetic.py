"""Seeded synthetic voxel scenes standing in for indoor scans and LiDAR sweeps.

Pure NumPy, deterministic for a given seed.  Every generator returns int32
coordinates ``[N, 3]`` of DISTINCT voxels; batching (the leading batch column,
offsets) is done by the caller or by :func:`batch_scenes`.

Scenes
------
``random_cells``   N distinct cells of a cube, uniformly without replacement.
``room_scene``     a 10 x 10 x 3 m room (floor + 4 walls) holding 40 random
                   axis-aligned boxes, voxelised either by rasterising every
                   face completely and cropping a room-centred, room-proportional
                   box to the requested voxel count (``mode="raster_crop"``:
                   solid, scan-like surfaces) or by area-weighted random surface
                   points (``mode="sample"``: porous surfaces).
``lidar_scene``    returns of a spinning 64-beam sensor against a ground plane
                   and random boxes, accumulated over several poses.

The literal room at 2 cm is about 1.4 M voxels and one 64 x 2048 sweep is at
most 131 k returns, so the requested counts are reached by cropping (rooms) or
by raising the number of sweeps / azimuth steps (LiDAR); the realised counts are
returned with the data.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import numpy as np

ROOM = np.array([10.0, 10.0, 3.0])


def random_cells(n: int, extent: int = 64, seed: int = 0) -> np.ndarray:
    rng = np.random.default_rng(seed)
    cells = rng.choice(extent**3, n, replace=False)
    return np.stack(np.unravel_index(cells, (extent, extent, extent)), axis=1).astype(np.int32)


def _unique_rows_first_occurrence(c: np.ndarray) -> np.ndarray:
    mins = c.min(axis=0).astype(np.int64)
    span = (c.max(axis=0).astype(np.int64) - mins + 1)
    key = ((c[:, 0] - mins[0]) * span[1] + (c[:, 1] - mins[1])) * span[2] + (c[:, 2] - mins[2])
    _, first = np.unique(key, return_index=True)
    first.sort()
    return c[first]


def _room_faces(rng) -> List[Tuple[int, float, np.ndarray, np.ndarray]]:
    """(fixed axis, fixed value, lo[3], hi[3]) rectangles: floor, 4 walls, 6 faces x 40 boxes."""
    faces = []
    lo, hi = np.zeros(3), ROOM.copy()
    faces.append((2, 0.0, lo, hi))  # floor
    for ax in (0, 1):
        faces.append((ax, 0.0, lo, hi))
        faces.append((ax, ROOM[ax] - 1e-6, lo, hi))
    for _ in range(40):
        side = rng.uniform(0.2, 2.0, size=3)
        c_lo = rng.uniform(0.0, 1.0, size=3) * (ROOM - side)
        c_hi = c_lo + side
        for ax in range(3):
            faces.append((ax, c_lo[ax], c_lo, c_hi))
            faces.append((ax, c_hi[ax], c_lo, c_hi))
    return faces


def _raster_face(ax, val, lo, hi, voxel):
    others = [a for a in range(3) if a != ax]
    rng0 = np.arange(int(np.floor(lo[others[0]] / voxel)), int(np.floor((hi[others[0]] - 1e-9) / voxel)) + 1)
    rng1 = np.arange(int(np.floor(lo[others[1]] / voxel)), int(np.floor((hi[others[1]] - 1e-9) / voxel)) + 1)
    g0, g1 = np.meshgrid(rng0, rng1, indexing="ij")
    out = np.empty((g0.size, 3), dtype=np.int32)
    out[:, ax] = int(np.floor(val / voxel))
    out[:, others[0]] = g0.reshape(-1)
    out[:, others[1]] = g1.reshape(-1)
    return out


def room_scene(target_voxels: int, voxel: float = 0.02, seed: int = 100, mode: str = "raster_crop",
               order: str = "random") -> np.ndarray:
    """One room; ``order`` in {"random", "raster"} is the row order of the result
    (a real scan has no useful order, so "random" is the default)."""
    rng = np.random.default_rng(seed)
    faces = _room_faces(rng)
    if mode == "raster_crop":
        # A room-centred box of the room's proportions, grown until it holds the
        # target count.  Only faces that can intersect a generously sized crop
        # are rasterised (the full room at 1 cm is ~5.6 M voxels).
        parts = [_raster_face(ax, val, lo, hi, voxel) for ax, val, lo, hi in faces]
        c = _unique_rows_first_occurrence(np.concatenate(parts, axis=0))
        centre = (c.astype(np.float64) + 0.5) * voxel - ROOM / 2.0
        s = np.max(np.abs(centre) / (ROOM / 2.0), axis=1)
        if target_voxels < len(c):
            keep = np.argsort(s, kind="stable")[:target_voxels]
            keep.sort()
            c = c[keep]
    elif mode == "sample":
        areas = []
        for ax, val, lo, hi in faces:
            o = [a for a in range(3) if a != ax]
            areas.append((hi[o[0]] - lo[o[0]]) * (hi[o[1]] - lo[o[1]]))
        areas = np.array(areas)
        budget = int(target_voxels * 1.13)
        c = np.zeros((0, 3), dtype=np.int32)
        for _ in range(6):  # grow the point budget until the unique count reaches the target
            which = rng.choice(len(faces), size=budget, p=areas / areas.sum())
            pts = np.empty((budget, 3))
            lo_a = np.stack([f[2] for f in faces])[which]
            hi_a = np.stack([f[3] for f in faces])[which]
            pts[:] = lo_a + rng.uniform(size=(budget, 3)) * (hi_a - lo_a)
            ax_a = np.array([f[0] for f in faces])[which]
            val_a = np.array([f[1] for f in faces])[which]
            pts[np.arange(budget), ax_a] = val_a
            c = _unique_rows_first_occurrence(np.floor(pts / voxel).astype(np.int32))
            if len(c) >= target_voxels:
                break
            budget = int(budget * 1.15)
        c = c[:target_voxels]
    else:
        raise ValueError(f"unknown mode {mode!r}")
    if order == "random":
        c = c[rng.permutation(len(c))]
    elif order != "raster":
        raise ValueError(f"unknown order {order!r}")
    return np.ascontiguousarray(c, dtype=np.int32)


def lidar_scene(target_voxels: Optional[int] = None, sweeps: int = 4, azimuth_steps: int = 2048,
                voxel: float = 0.05, seed: int = 500, max_sweeps: int = 512) -> Tuple[np.ndarray, dict]:
    """Spinning 64-beam sensor: elevations -25..+3 deg, ground plane 1.7 m below
    the sensor, 300 random boxes within 80 m, 0.5 % Gaussian range noise, random-walk
    poses.  With ``target_voxels`` the sweep count is raised (up to ``max_sweeps``)
    until the distinct-voxel count reaches it."""
    rng = np.random.default_rng(seed)
    nb = 300
    foot = rng.uniform(1.0, 6.0, size=(nb, 2))
    height = rng.uniform(1.0, 4.0, size=nb)
    r = 80.0 * np.sqrt(rng.uniform(0.01, 1.0, size=nb))
    th = rng.uniform(0, 2 * np.pi, size=nb)
    centre = np.stack([r * np.cos(th), r * np.sin(th)], axis=1)
    blo = np.concatenate([centre - foot / 2, np.full((nb, 1), -1.7)], axis=1)
    bhi = np.concatenate([centre + foot / 2, (-1.7 + height)[:, None]], axis=1)
    elev = np.deg2rad(np.linspace(-25.0, 3.0, 64))
    azim = np.linspace(0, 2 * np.pi, azimuth_steps, endpoint=False)
    el, az = np.meshgrid(elev, azim, indexing="ij")
    dirs_local = np.stack([np.cos(el) * np.cos(az), np.cos(el) * np.sin(az), np.sin(el)], -1).reshape(-1, 3)

    pos = np.zeros(3)
    yaw = 0.0
    chunks = []
    total = np.zeros((0, 3), dtype=np.int32)
    n_sweeps = 0
    n_el, n_az = len(elev), azimuth_steps
    d_az = 2 * np.pi / n_az
    corners = np.stack([np.stack([blo[:, 0], blo[:, 1]], 1), np.stack([blo[:, 0], bhi[:, 1]], 1),
                        np.stack([bhi[:, 0], blo[:, 1]], 1), np.stack([bhi[:, 0], bhi[:, 1]], 1)], 1)  # [nb,4,2]
    while True:
        cy, sy = np.cos(yaw), np.sin(yaw)
        R = np.array([[cy, -sy, 0], [sy, cy, 0], [0, 0, 1.0]])
        d = dirs_local @ R.T
        t_hit = np.full(len(d), np.inf)
        down = d[:, 2] < -1e-6
        t_hit[down] = (-1.7 - pos[2]) / d[down, 2]
        t2 = t_hit.reshape(n_el, n_az)
        d3 = d.reshape(n_el, n_az, 3)
        # every box only meets the rays inside the azimuth interval its footprint subtends
        rel = corners - pos[None, None, :2]
        caz = np.arctan2(rel[:, :, 1], rel[:, :, 0])
        cen = np.arctan2((blo[:, 1] + bhi[:, 1]) / 2 - pos[1], (blo[:, 0] + bhi[:, 0]) / 2 - pos[0])
        dd = (caz - cen[:, None] + np.pi) % (2 * np.pi) - np.pi
        inside = (blo[:, 0] <= pos[0]) & (pos[0] <= bhi[:, 0]) & (blo[:, 1] <= pos[1]) & (pos[1] <= bhi[:, 1])
        for b0 in range(nb):
            if inside[b0]:
                cols = np.arange(n_az)
            else:
                a0 = cen[b0] + dd[b0].min() - yaw
                a1 = cen[b0] + dd[b0].max() - yaw
                c0 = int(np.floor(a0 / d_az)) - 1
                c1 = int(np.ceil(a1 / d_az)) + 1
                cols = np.arange(c0, c1 + 1) % n_az
            dv = d3[:, cols, :]
            inv = 1.0 / np.where(np.abs(dv) < 1e-12, 1e-12, dv)
            lo = (blo[b0] - pos) * inv
            hi = (bhi[b0] - pos) * inv
            tmin = np.minimum(lo, hi).max(axis=2)
            tmax = np.maximum(lo, hi).min(axis=2)
            ok = tmax >= np.maximum(tmin, 0.0)
            tb = np.where(ok, np.maximum(tmin, 0.0), np.inf)
            t2[:, cols] = np.minimum(t2[:, cols], tb)
        t_hit = t2.reshape(-1)
        rng_noise = 1.0 + 0.005 * rng.standard_normal(len(d))
        t = t_hit * rng_noise
        good = np.isfinite(t) & (t <= 80.0) & (t > 0.5)
        pts = pos + d[good] * t[good, None]
        chunks.append(np.floor(pts / voxel).astype(np.int32))
        n_sweeps += 1
        pos = pos + np.array([np.cos(yaw), np.sin(yaw), 0.0]) * rng.uniform(0.5, 2.0)
        yaw += np.deg2rad(rng.normal(0.0, 5.0))
        if target_voxels is None:
            if n_sweeps >= sweeps:
                break
        elif n_sweeps >= sweeps and (n_sweeps % 8 == 0 or n_sweeps >= max_sweeps):
            total = _unique_rows_first_occurrence(np.concatenate(chunks, axis=0))
            chunks = [total]
            if len(total) >= target_voxels or n_sweeps >= max_sweeps:
                break
    total = _unique_rows_first_occurrence(np.concatenate(chunks, axis=0))
    if target_voxels is not None and len(total) > target_voxels:
        total = total[:target_voxels]
    info = {"sweeps": n_sweeps, "azimuth_steps": azimuth_steps, "voxels": int(len(total)), "voxel_m": voxel}
    return np.ascontiguousarray(total, dtype=np.int32), info


def batch_scenes(scenes: Sequence[np.ndarray]) -> Tuple[np.ndarray, np.ndarray]:
    """Concatenate scenes into batch-indexed coordinates ``[N, 4]`` (b, x, y, z)
    and ``offsets [B+1]``."""
    rows = [np.concatenate([np.full((len(s), 1), b, dtype=np.int32), s], axis=1) for b, s in enumerate(scenes)]
    offsets = np.concatenate([[0], np.cumsum([len(s) for s in scenes])]).astype(np.int64)
    return np.concatenate(rows, axis=0), offsets
