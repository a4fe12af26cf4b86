"""``opentau-so101-record``: teleoperated episodes written in the LeRobot v2.1 layout."""

import argparse
import time

import numpy as np

from ...datasets.lerobot_dataset import LeRobotDataset
from .devices import CameraConfig, SOArmConfig, SOFollower, SOLeader, busy_wait
from .motors_bus import SO101_MOTORS


def features(cameras: dict[str, CameraConfig]) -> dict:
    names = [f"{n}.pos" for n in SO101_MOTORS]
    f = {"observation.state": {"dtype": "float32", "shape": (len(names),), "names": names},
         "action": {"dtype": "float32", "shape": (len(names),), "names": names}}
    for n, c in cameras.items():
        f[f"observation.images.{n}"] = {"dtype": "video", "shape": (c.height, c.width, 3), "names": ["height", "width", "channel"]}
    return f


def record_episode(rec, leader: SOLeader, follower: SOFollower, task: str, seconds: float, fps: int) -> int:
    n = int(seconds * fps)
    for _ in range(n):
        t0 = time.perf_counter()
        action = leader.get_action()
        follower.send_action(action)
        obs = follower.get_observation()
        frame = {"observation.state": np.array([obs[f"{m}.pos"] for m in SO101_MOTORS], np.float32),
                 "action": np.array([action[f"{m}.pos"] for m in SO101_MOTORS], np.float32), "task": task}
        for cam in follower.cameras:
            frame[f"observation.images.{cam}"] = obs[cam]
        rec.add_frame(frame)
        busy_wait(max(0.0, 1 / fps - (time.perf_counter() - t0)))
    rec.save_episode()
    return n


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--leader-port", required=True)
    ap.add_argument("--follower-port", required=True)
    ap.add_argument("--repo-id", required=True)
    ap.add_argument("--root", default=None)
    ap.add_argument("--task", required=True)
    ap.add_argument("--episodes", type=int, default=1)
    ap.add_argument("--episode-time", type=float, default=30.0)
    ap.add_argument("--fps", type=int, default=30)
    ap.add_argument("--camera", action="append", default=[], help="name:index")
    a = ap.parse_args(argv)
    cams = {c.split(":")[0]: CameraConfig(int(c.split(":")[1])) for c in a.camera}
    leader = SOLeader(SOArmConfig(port=a.leader_port, id="leader"))
    follower = SOFollower(SOArmConfig(port=a.follower_port, id="follower", cameras=cams))
    leader.connect()
    follower.connect()
    rec = LeRobotDataset.create(a.repo_id, a.fps, root=a.root, robot_type="so101", features=features(cams),
                                use_videos=True, image_writer_threads=4)
    try:
        for e in range(a.episodes):
            input(f"episode {e}: press Enter to start")
            record_episode(rec, leader, follower, a.task, a.episode_time, a.fps)
    finally:
        rec.stop_image_writer()
        leader.disconnect()
        follower.disconnect()


if __name__ == "__main__":
    main()
