"""``opentau-so101-record``: teleoperated episodes written in the LeRobot v2.1 layout
(reference ``src/opentau/scripts/so101/record.py:15-328``).

A session records ``--episodes`` episodes of at most ``--episode-time`` seconds each, with a reset pause between them,
and can be steered while it runs (arrow keys when ``pynput`` and a display are there; the same three flags can be set
by any other front end through the ``events`` dict):

    right arrow  end the current episode (or the reset pause) now
    left arrow   throw the current episode away and record it again
    escape       stop after this episode

``--resume`` appends to an existing dataset; a dataset that already has the requested number of episodes records
nothing.  The dataset's ``info.json`` is marked ``control_mode: joint`` (the leader arm commands joint positions).
"""

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


def new_events() -> dict:
    return {"exit_early": False, "rerecord_episode": False, "stop_recording": False}


def init_keyboard_listener(events: dict):
    """Arrow-key control of the session through ``pynput``; ``None`` (and a note in the log) without it / headless."""
    try:
        from pynput import keyboard
    except Exception:  # noqa: BLE001 - missing package or no display
        import logging
        logging.warning("pynput is not usable here (headless?): keyboard controls are off")
        return None

    def on_press(key):
        if key == keyboard.Key.right:
            events["exit_early"] = True
        elif key == keyboard.Key.left:
            events["rerecord_episode"] = events["exit_early"] = True
        elif key == keyboard.Key.esc:
            events["stop_recording"] = events["exit_early"] = True

    listener = keyboard.Listener(on_press=on_press)
    listener.start()
    return listener


def open_dataset_for_append(repo_id: str, root, image_writer_threads: int = 0, image_writer_processes: int = 0):
    """A recorder over an EXISTING local dataset: the next episode continues its numbering."""
    from ...datasets.lerobot_dataset import LeRobotDatasetMetadata, LeRobotRecorder
    meta = LeRobotDatasetMetadata(repo_id, root=root)
    if meta.version != "v2.1":
        raise ValueError(f"recording appends to the v2.1 layout; {repo_id} is {meta.version}")
    return LeRobotRecorder(meta, image_writer_threads, image_writer_processes=image_writer_processes)


def record_episode(rec, leader: SOLeader, follower: SOFollower, task: str, seconds: float, fps: int,
                   events: dict | None = None, save: bool = True) -> int:
    """Frames until ``seconds`` have passed or ``events["exit_early"]`` is raised (cleared on return); with ``save`` the
    episode is written, otherwise it stays in the buffer for the caller to save or discard."""
    n = int(seconds * fps)
    done = 0
    for _ in range(n):
        if events is not None and events["exit_early"]:
            break
        t0 = time.perf_counter()
        action = leader.get_action()
        follower.send_action(action)
        obs = follower.get_observation()
        frame = {"observation.state": np.array([obs[f"{m}.pos"] for m in SO101_MOTORS], np.float32),
                 "action": np.array([action[f"{m}.pos"] for m in SO101_MOTORS], np.float32), "task": task}
        for cam in follower.cameras:
            frame[f"observation.images.{cam}"] = obs[cam]
        rec.add_frame(frame)
        done += 1
        busy_wait(max(0.0, 1 / fps - (time.perf_counter() - t0)))
    if events is not None:
        events["exit_early"] = False
    if save:
        rec.save_episode()
    return done


def reset_pause(leader: SOLeader, follower: SOFollower, seconds: float, fps: int, events: dict) -> None:
    """Between episodes the operator puts the scene back; teleoperation stays live, nothing is recorded."""
    t_end = time.perf_counter() + seconds
    while time.perf_counter() < t_end and not events["exit_early"]:
        t0 = time.perf_counter()
        follower.send_action(leader.get_action())
        busy_wait(max(0.0, 1 / fps - (time.perf_counter() - t0)))
    events["exit_early"] = False


def record_session(rec, leader: SOLeader, follower: SOFollower, task: str, num_episodes: int, episode_time_s: float,
                   reset_time_s: float, fps: int, events: dict | None = None, say=print) -> int:
    """Records until the DATASET holds ``num_episodes`` episodes (so a resumed session only adds what is missing) or a
    stop is asked for; returns the number of episodes this call saved."""
    events = events if events is not None else new_events()
    have, saved = rec.meta.total_episodes, 0
    if have >= num_episodes:
        say(f"the dataset already has {have} episode(s) >= {num_episodes}: nothing to record")
    while have < num_episodes and not events["stop_recording"]:
        say(f"recording episode {have + 1} of {num_episodes}")
        frames = record_episode(rec, leader, follower, task, episode_time_s, fps, events, save=False)
        if events["rerecord_episode"] or frames == 0:
            say("re-recording the episode")
            events["rerecord_episode"] = False
            if rec.image_writer is not None:
                rec.image_writer.wait_until_done()
            rec.clear_episode_buffer()
            if frames == 0 and events["stop_recording"]:
                break
            continue
        rec.save_episode()
        have, saved = have + 1, saved + 1
        if have < num_episodes and not events["stop_recording"] and reset_time_s > 0:
            say("reset the environment")
            reset_pause(leader, follower, reset_time_s, fps, events)
    return saved



def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--leader-port", required=True)
    ap.add_argument("--follower-port", required=True)
    ap.add_argument("--repo-id", required=True)
    ap.add_argument("--root", default=None)
    ap.add_argument("--task", required=True)
    ap.add_argument("--episodes", type=int, default=50)
    ap.add_argument("--episode-time", type=float, default=60.0)
    ap.add_argument("--reset-time", type=float, default=10.0)
    ap.add_argument("--fps", type=int, default=30)
    ap.add_argument("--camera", action="append", default=[], help="name:index")
    ap.add_argument("--resume", action="store_true", help="append to the existing dataset at --root")
    ap.add_argument("--no-video", action="store_true", help="keep the frames as images")
    ap.add_argument("--image-writer-processes", type=int, default=0)
    ap.add_argument("--image-writer-threads-per-camera", type=int, default=4)
    ap.add_argument("--push-to-hub", action="store_true")
    ap.add_argument("--private", action="store_true")
    a = ap.parse_args(argv)
    cams = {c.split(":")[0]: CameraConfig(int(c.split(":")[1])) for c in a.camera}
    leader = SOLeader(SOArmConfig(port=a.leader_port, id="leader"))
    follower = SOFollower(SOArmConfig(port=a.follower_port, id="follower", cameras=cams))
    threads = a.image_writer_threads_per_camera * max(len(cams), 1)
    if a.resume:
        rec = open_dataset_for_append(a.repo_id, a.root, threads, a.image_writer_processes)
    else:
        rec = LeRobotDataset.create(a.repo_id, a.fps, root=a.root, robot_type="so101", features=features(cams),
                                    use_videos=not a.no_video, image_writer_threads=threads,
                                    image_writer_processes=a.image_writer_processes)
        from ...datasets.utils import INFO_PATH, write_json
        rec.meta.info["control_mode"] = "joint"
        write_json({**rec.meta.info, "features": {k: {**v, "shape": list(v["shape"])} for k, v in rec.meta.info["features"].items()}},
                   rec.meta.root / INFO_PATH)
    leader.connect()
    follower.connect()
    events = new_events()
    listener = init_keyboard_listener(events)
    try:
        record_session(rec, leader, follower, a.task, a.episodes, a.episode_time, a.reset_time, a.fps, events)
    finally:
        rec.stop_image_writer()
        leader.disconnect()
        follower.disconnect()
        if listener is not None:
            listener.stop()
    if a.push_to_hub:
        from ...datasets.lerobot_dataset import LeRobotDatasetMetadata
        LeRobotDatasetMetadata(a.repo_id, root=a.root).push_to_hub(private=a.private, tags=["so101"])


if __name__ == "__main__":
    main()
