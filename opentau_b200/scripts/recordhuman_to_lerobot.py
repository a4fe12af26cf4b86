"""Convert a headset recording (egocentric video + per-frame head and hand-joint poses) into a LeRobot episode.

Data contract of the reference tool (``src/opentau/scripts/recordhuman_to_lerobot.py:102-703``):

* pose file: ``{"frames": [{"t": seconds, "head_pos": [3], "head_rot": [x,y,z,w], "left_joints": [26*7],
  "left_tracked": bool, "right_joints": [26*7], "right_tracked": bool}, ...]}`` with joints as position + quaternion in
  tracking space;
* state (364): both hands' 26 joints x (position, quaternion) expressed in the camera frame of that instant
  (``p_cam = R_head^T (p - eye)``, ``q_cam = q_head^-1 * q``); an untracked hand is zeros;
* action (371): the NEXT frame's state followed by the head motion to it (position difference and relative rotation
  ``q_{t+1} * q_t^-1``); the last frame repeats its state with a zero step and the identity rotation;
* every output frame takes the pose sample nearest in time to its video frame (plus ``--time-offset``); ``--fps`` below
  the video rate resamples the frames.

An optional overlay video draws the projected hand skeletons on the frames (pinhole model from the vertical FOV).

    python -m opentau_b200.scripts.recordhuman_to_lerobot --video rec.mp4 --poses rec.json --output ds --prompt "..."
"""

from __future__ import annotations

import argparse
import json
from pathlib import Path

import numpy as np

JOINTS_PER_HAND, FLOATS_PER_JOINT = 26, 7
STATE_DIM_PER_HAND = JOINTS_PER_HAND * FLOATS_PER_JOINT
STATE_DIM = 2 * STATE_DIM_PER_HAND
ACTION_DIM = STATE_DIM + 7
# wrist (1) to palm (0); thumb 1-2-3-4-5; the other four fingers 1-s-(s+1)-...-(s+4) with s = 6, 11, 16, 21
SKELETON_BONES = [(1, 0), (1, 2), (2, 3), (3, 4), (4, 5)] + [
    bone for s0 in (6, 11, 16, 21) for bone in [(1, s0)] + [(s0 + i, s0 + i + 1) for i in range(4)]]


def quat_to_rotation_matrix(q) -> np.ndarray:
    """(x, y, z, w) -> 3x3 matrix taking local column vectors to the world frame."""
    x, y, z, w = np.asarray(q, float) / np.linalg.norm(q)
    return np.array([[1 - 2 * (y * y + z * z), 2 * (x * y - w * z), 2 * (x * z + w * y)],
                     [2 * (x * y + w * z), 1 - 2 * (x * x + z * z), 2 * (y * z - w * x)],
                     [2 * (x * z - w * y), 2 * (y * z + w * x), 1 - 2 * (x * x + y * y)]])


def quat_inverse(q) -> np.ndarray:
    x, y, z, w = q
    return np.array([-x, -y, -z, w])


def quat_multiply(q1, q2) -> np.ndarray:
    """``q1 * q2``: rotate by q2 first, then by q1; (x, y, z, w) order."""
    x1, y1, z1, w1 = q1
    x2, y2, z2, w2 = q2
    return np.array([w1 * x2 + x1 * w2 + y1 * z2 - z1 * y2, w1 * y2 - x1 * z2 + y1 * w2 + z1 * x2,
                     w1 * z2 + x1 * y2 - y1 * x2 + z1 * w2, w1 * w2 - x1 * x2 - y1 * y2 - z1 * z2])


def world_to_camera(points, head_pos, head_rot, eye_offset=None) -> np.ndarray:
    R = quat_to_rotation_matrix(head_rot)
    eye = head_pos if eye_offset is None else head_pos + R @ eye_offset
    return (np.asarray(points, float) - eye) @ R            # row vectors: (p - eye) R == R^T (p - eye)


def project_camera_to_pixel(points_cam, fx, fy, cx, cy):
    """Camera frame with Z forward and Y up; points with Z <= 0.01 are invalid (NaN)."""
    valid = points_cam[:, 2] > 0.01
    px, py = np.full(len(points_cam), np.nan), np.full(len(points_cam), np.nan)
    z = points_cam[valid, 2]
    px[valid] = fx * points_cam[valid, 0] / z + cx
    py[valid] = -fy * points_cam[valid, 1] / z + cy
    return px, py, valid


def compute_frame_state(pf: dict, head_pos, head_rot, eye_offset=None):
    """-> ``(state (364,), left camera-space joints | None, right | None)``."""
    state = np.zeros(STATE_DIM, np.float32)
    cams = [None, None]
    q_inv = quat_inverse(head_rot)
    for h, (jk, tk) in enumerate((("left_joints", "left_tracked"), ("right_joints", "right_tracked"))):
        if not pf.get(tk, False):
            continue
        joints = np.asarray(pf[jk], float).reshape(JOINTS_PER_HAND, FLOATS_PER_JOINT)
        pos = world_to_camera(joints[:, :3], head_pos, head_rot, eye_offset)
        quat = np.stack([quat_multiply(q_inv, q) for q in joints[:, 3:]])
        state[h * STATE_DIM_PER_HAND:(h + 1) * STATE_DIM_PER_HAND] = np.hstack([pos, quat]).ravel()
        cams[h] = pos
    return state, cams[0], cams[1]


def nearest_pose_index(pose_t: np.ndarray, t: float) -> int:
    i = int(np.clip(np.searchsorted(pose_t, t), 0, len(pose_t) - 1))
    return i - 1 if i > 0 and abs(pose_t[i - 1] - t) < abs(pose_t[i] - t) else i


def build_actions(states: list[np.ndarray], head_poses: list[np.ndarray]) -> list[np.ndarray]:
    acts = []
    for i in range(len(states) - 1):
        dpos = head_poses[i + 1][:3] - head_poses[i][:3]
        drot = quat_multiply(head_poses[i + 1][3:], quat_inverse(head_poses[i][3:]))
        acts.append(np.concatenate([states[i + 1], dpos, drot]).astype(np.float32))
    acts.append(np.concatenate([states[-1], [0, 0, 0, 0, 0, 0, 1]]).astype(np.float32))
    return acts


def draw_hand(frame, px, py, valid, colour) -> None:
    import cv2
    for a, b in SKELETON_BONES:
        if valid[a] and valid[b]:
            cv2.line(frame, (int(px[a]), int(py[a])), (int(px[b]), int(py[b])), colour, 2)
    for i in range(len(px)):
        if valid[i]:
            cv2.circle(frame, (int(px[i]), int(py[i])), 4, colour, -1)


def convert(video: str | Path, poses: str | Path, output: str | Path, prompt: str, fps: float | None = None,
            time_offset: float = 0.0, tracking_origin=(-0.32, 2.0276, 0.0), eye_offset: float = 0.06,
            overlay: str | Path | None = None, fov_deg: float = 90.0) -> dict:
    import cv2
    from ..datasets.lerobot_dataset import LeRobotDataset
    frames_data = json.loads(Path(poses).read_text())["frames"]
    pose_t = np.array([f["t"] for f in frames_data])
    cap = cv2.VideoCapture(str(video))
    if not cap.isOpened():
        raise FileNotFoundError(f"cannot open video {video}")
    vfps = float(cap.get(cv2.CAP_PROP_FPS)) or 30.0
    w, h = int(cap.get(cv2.CAP_PROP_FRAME_WIDTH)), int(cap.get(cv2.CAP_PROP_FRAME_HEIGHT))
    total = int(cap.get(cv2.CAP_PROP_FRAME_COUNT))
    target = fps or vfps
    n_out = max(1, int(round(total * target / vfps)))
    sampled = [min(int(round(i * vfps / target)), total - 1) for i in range(n_out)]
    origin = np.asarray(tracking_origin, float)
    eye = np.array([eye_offset, 0.0, 0.0]) if eye_offset else None
    fy = (h / 2) / np.tan(np.radians(fov_deg) / 2)
    writer = cv2.VideoWriter(str(overlay), cv2.VideoWriter_fourcc(*"mp4v"), vfps, (w, h)) if overlay else None
    wanted = {f: i for i, f in reversed(list(enumerate(sampled)))}
    images, states, head_poses = {}, {}, {}
    for fidx in range(total):
        ok, frame = cap.read()
        if not ok:
            break
        if fidx not in wanted and writer is None:
            continue
        pf = frames_data[nearest_pose_index(pose_t, fidx / vfps + time_offset)]
        head_pos, head_rot = np.asarray(pf["head_pos"], float) - origin, np.asarray(pf["head_rot"], float)
        state, lc, rc = compute_frame_state(pf, head_pos, head_rot, eye)
        if fidx in wanted:
            images[fidx], states[fidx] = np.ascontiguousarray(frame[:, :, ::-1]), state
            head_poses[fidx] = np.concatenate([head_pos, head_rot])
        if writer is not None:
            for pts, colour in ((lc, (255, 150, 50)), (rc, (50, 150, 255))):
                if pts is not None:
                    draw_hand(frame, *project_camera_to_pixel(pts, fy, fy, w / 2, h / 2), colour)
            writer.write(frame)
    cap.release()
    if writer is not None:
        writer.release()
    order = [f for f in sampled if f in states]
    if not order:
        raise ValueError("no frame processed")
    st = [states[f] for f in order]
    acts = build_actions(st, [head_poses[f] for f in order])
    out = Path(output)
    ds = LeRobotDataset.create(out.name, fps=int(round(target)) or 30, root=out, robot_type="human", features={
        "observation.images.camera": {"dtype": "video", "shape": (h, w, 3), "names": ["height", "width", "channel"]},
        "observation.state": {"dtype": "float32", "shape": (STATE_DIM,), "names": None},
        "action": {"dtype": "float32", "shape": (ACTION_DIM,), "names": None}}, use_videos=True, image_writer_threads=2)
    for f, s, a in zip(order, st, acts):
        ds.add_frame({"observation.images.camera": images[f], "observation.state": s, "action": a, "task": prompt})
    ds.save_episode()
    ds.stop_image_writer()
    return {"frames": len(order), "fps": int(round(target)) or 30}


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--video", required=True)
    ap.add_argument("--poses", required=True)
    ap.add_argument("--output", required=True)
    ap.add_argument("--prompt", required=True)
    ap.add_argument("--overlay", default=None)
    ap.add_argument("--fov", type=float, default=90.0)
    ap.add_argument("--time-offset", type=float, default=0.0)
    ap.add_argument("--tracking-origin", type=float, nargs=3, default=[-0.32, 2.0276, 0.0])
    ap.add_argument("--eye-offset", type=float, default=0.06)
    ap.add_argument("--fps", type=float, default=None)
    a = ap.parse_args(argv)
    print(convert(a.video, a.poses, a.output, a.prompt, a.fps, a.time_offset, a.tracking_origin, a.eye_offset,
                  a.overlay, a.fov))


if __name__ == "__main__":
    main()
