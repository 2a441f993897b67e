"""Turn policy outputs into robot commands: rotation conversions (6-D, quaternion, Euler, matrix), end-effector delta
integration, joint targets with limits, gripper thresholding (reference: loongforge/embodied/eval/action_decoders/*)."""
from __future__ import annotations

from typing import Optional

import numpy as np


def rot6d_to_matrix(r6: np.ndarray) -> np.ndarray:
    """Gram-Schmidt on the two 3-vectors of the 6-D rotation representation -> [..., 3, 3] (columns b1, b2, b3)."""
    a1, a2 = r6[..., :3], r6[..., 3:6]
    b1 = a1 / np.linalg.norm(a1, axis=-1, keepdims=True).clip(1e-8)
    a2 = a2 - (b1 * a2).sum(-1, keepdims=True) * b1
    b2 = a2 / np.linalg.norm(a2, axis=-1, keepdims=True).clip(1e-8)
    return np.stack([b1, b2, np.cross(b1, b2)], axis=-1)


def matrix_to_rot6d(m: np.ndarray) -> np.ndarray:
    return np.concatenate([m[..., :, 0], m[..., :, 1]], axis=-1)


def quat_to_matrix(q: np.ndarray) -> np.ndarray:
    """Quaternion (w, x, y, z) -> rotation matrix."""
    q = q / np.linalg.norm(q, axis=-1, keepdims=True).clip(1e-8)
    w, x, y, z = (q[..., i] for i in range(4))
    return np.stack([
        np.stack([1 - 2 * (y * y + z * z), 2 * (x * y - z * w), 2 * (x * z + y * w)], -1),
        np.stack([2 * (x * y + z * w), 1 - 2 * (x * x + z * z), 2 * (y * z - x * w)], -1),
        np.stack([2 * (x * z - y * w), 2 * (y * z + x * w), 1 - 2 * (x * x + y * y)], -1)], -2)


def matrix_to_quat(m: np.ndarray) -> np.ndarray:
    """Rotation matrix -> quaternion (w, x, y, z) with w >= 0."""
    t = np.trace(m, axis1=-2, axis2=-1)
    w = np.sqrt(np.clip(1 + t, 0, None)) / 2
    x = np.sqrt(np.clip(1 + m[..., 0, 0] - m[..., 1, 1] - m[..., 2, 2], 0, None)) / 2
    y = np.sqrt(np.clip(1 - m[..., 0, 0] + m[..., 1, 1] - m[..., 2, 2], 0, None)) / 2
    z = np.sqrt(np.clip(1 - m[..., 0, 0] - m[..., 1, 1] + m[..., 2, 2], 0, None)) / 2
    x = np.copysign(x, m[..., 2, 1] - m[..., 1, 2])
    y = np.copysign(y, m[..., 0, 2] - m[..., 2, 0])
    z = np.copysign(z, m[..., 1, 0] - m[..., 0, 1])
    return np.stack([w, x, y, z], -1)


def euler_to_matrix(e: np.ndarray) -> np.ndarray:
    """Roll, pitch, yaw (XYZ extrinsic) -> matrix = Rz(yaw) Ry(pitch) Rx(roll)."""
    r, p, y = e[..., 0], e[..., 1], e[..., 2]
    cr, sr, cp, sp, cy, sy = np.cos(r), np.sin(r), np.cos(p), np.sin(p), np.cos(y), np.sin(y)
    return np.stack([
        np.stack([cy * cp, cy * sp * sr - sy * cr, cy * sp * cr + sy * sr], -1),
        np.stack([sy * cp, sy * sp * sr + cy * cr, sy * sp * cr - cy * sr], -1),
        np.stack([-sp, cp * sr, cp * cr], -1)], -2)


def decode_ee_delta(actions: np.ndarray, ee_pos: np.ndarray, ee_rot: np.ndarray, space: str = "ee_delta_6d",
                    gripper_threshold: Optional[float] = 0.5):
    """Integrates a chunk of end-effector deltas from the current pose. Action layout: [dx, dy, dz, rotation..., gripper]
    with a 6-D / quaternion / Euler rotation. Returns (positions [H, 3], rotations [H, 3, 3], gripper [H])."""
    n_rot = {"ee_delta_6d": 6, "ee_delta_quat": 4, "ee_delta_euler": 3}[space]
    conv = {"ee_delta_6d": rot6d_to_matrix, "ee_delta_quat": quat_to_matrix, "ee_delta_euler": euler_to_matrix}[space]
    pos, rot = [], []
    p, R = ee_pos.astype(np.float64), ee_rot.astype(np.float64)
    for a in actions:
        p = p + a[:3]
        R = conv(a[3:3 + n_rot].astype(np.float64)) @ R
        pos.append(p)
        rot.append(R)
    g = actions[:, 3 + n_rot]
    if gripper_threshold is not None:
        g = (g > gripper_threshold).astype(np.float32)
    return np.stack(pos), np.stack(rot), g


def decode_joint(actions: np.ndarray, current: np.ndarray, *, delta: bool = False, lower=None, upper=None) -> np.ndarray:
    """Joint targets (absolute, or cumulative deltas from `current`), clipped to limits."""
    out = current[None] + np.cumsum(actions, 0) if delta else actions.copy()
    if lower is not None or upper is not None:
        out = np.clip(out, lower, upper)
    return out
