"""Convert a directory of ROS 2 bags into one LeRobot dataset, one episode per bag.

Flow of the reference tool (``src/opentau/scripts/convert_ros_to_lerobot.py:100-242``): every ``<input>/<bag>/recording``
is read once; messages on the topics named by ``dataset_features`` go through the extractor that the feature's
``enum_values`` selects (``state`` / ``action`` / ``image``), stamped with the header time when there is one; each
stream is resampled to ``fps`` from the bag's start time; frames are added up to the shortest stream; the task string
comes from the bag's ``metadata.yaml``.  A bag that fails is logged and skipped without corrupting the next episode.

Reading bag files needs the ``rosbags`` package (not in this image); ``convert`` also accepts any iterable of
``(topic, stamp, message)`` per bag, which is what the tests feed it.

    python -m opentau_b200.scripts.convert_ros_to_lerobot --config_path ros2lerobot.json
"""

from __future__ import annotations

import logging
from collections import defaultdict
from pathlib import Path
from typing import Any, Callable, Iterable

import numpy as np

from ..configs import parser
from ..configs.ros2lerobot import RosToLeRobotConfig
from ..utils.ros2lerobot import EXTRACTORS, synchronize_sensor_data


def read_bag(path: Path) -> Iterable[tuple[str, Any, Any]]:  # pragma: no cover - needs rosbags and a bag file
    try:
        from rosbags.highlevel import AnyReader
    except ImportError as e:
        raise ImportError("reading ROS 2 bags needs the `rosbags` package") from e
    with AnyReader([path]) as reader:
        for conn, stamp, raw in reader.messages(connections=reader.connections):
            yield conn.topic, stamp, reader.deserialize(raw, conn.msgtype)


def extract_topics(cfg: RosToLeRobotConfig, messages: Iterable[tuple[str, Any, Any]]) -> dict[tuple[str, str], list]:
    """``{(topic, attribute): [(stamp, value), ...]}`` for the topics the features ask for."""
    wanted: dict[str, list[tuple[str, str]]] = defaultdict(list)
    for f in cfg.dataset_features.values():
        wanted[f.ros_topic].append((f.topic_attribute, f.enum_values))
    extractors = {k: v(cfg) for k, v in EXTRACTORS.items()}
    out: dict[tuple[str, str], list] = defaultdict(list)
    for topic, stamp, msg in messages:
        for attribute, kind in wanted.get(topic, ()):
            if kind not in extractors:
                raise KeyError(f"no extractor for {kind!r} (feature on {topic})")
            header = getattr(getattr(msg, "header", None), "stamp", None)
            value = extractors[kind](msg, topic, attribute)
            if value is None or (isinstance(value, (list, np.ndarray)) and len(value) == 0):
                continue
            out[(topic, attribute)].append((header if header is not None else stamp, value))
    return out


def bag_info(bag: Path) -> tuple[str, float]:
    import yaml
    meta = yaml.safe_load((bag / "metadata.yaml").read_text())
    return meta.get("task") or "", meta["rosbag2_bagfile_information"]["starting_time"]["nanoseconds_since_epoch"] / 1e9


def convert(cfg: RosToLeRobotConfig, reader: Callable[[Path], Iterable[tuple[str, Any, Any]]] = read_bag,
            info: Callable[[Path], tuple[str, float]] = bag_info) -> dict[str, int]:
    from ..datasets.lerobot_dataset import LeRobotDataset
    out = Path(cfg.output_path)
    features = {k: {"dtype": v.dtype, "shape": tuple(v.shape),
                    "names": (cfg.joint_order or None) if ("state" in k or "action" in k) else None}
                for k, v in cfg.dataset_features.items()}
    ds = LeRobotDataset.create(out.name, fps=cfg.fps, root=out, robot_type=cfg.robot_type, features=features,
                               use_videos=True, image_writer_threads=2)
    done = {"episodes": 0, "frames": 0, "failed": 0}
    for bag in sorted(p for p in Path(cfg.input_path).iterdir() if p.is_dir()):
        rec = bag / "recording"
        try:
            streams = extract_topics(cfg, reader(rec))
            task, start = info(rec)
            synced = {k: synchronize_sensor_data(v, cfg.fps, start) for k, v in streams.items()}
            keys = [(f.ros_topic, f.topic_attribute) for f in cfg.dataset_features.values()]
            n = min((len(synced.get(k, [])) for k in keys), default=0)
            if n == 0:
                raise ValueError("a required topic has no message")
            for i in range(n):
                frame = {"task": task}
                for name, f in cfg.dataset_features.items():
                    val = synced[(f.ros_topic, f.topic_attribute)][i]
                    frame[name] = np.asarray(val) if f.dtype in ("image", "video") else np.asarray(val, dtype=f.dtype)
                ds.add_frame(frame)
            ds.save_episode()
            done["episodes"] += 1
            done["frames"] += n
        except Exception as e:  # noqa: BLE001 - one bad bag must not end the batch
            logging.exception("bag %s not converted: %s", bag.name, e)
            ds.episode_buffer = ds.create_episode_buffer()
            done["failed"] += 1
    ds.stop_image_writer()
    return done


@parser.wrap()
def batch_convert_ros_bags(cfg: RosToLeRobotConfig) -> None:
    logging.basicConfig(level=logging.INFO)
    logging.info("converted: %s", convert(cfg))


def main() -> None:
    batch_convert_ros_bags()


if __name__ == "__main__":
    main()
