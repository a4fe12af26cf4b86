"""SO-101 stack on a simulated Feetech bus: packet framing, sign-magnitude registers, calibration, normalised IO,
teleoperation mirroring, motor renumbering, episode recording."""

import numpy as np
import pytest

from opentau_b200.scripts.so101.devices import SOArmConfig, SOFollower, SOLeader, teleoperate_step
from opentau_b200.scripts.so101.feetech import (FakeFeetechPort, FeetechError, FeetechProtocol, build_packet, checksum,
                                                 decode_sign, encode_sign)
from opentau_b200.scripts.so101.setup_motors import setup_motor

IDS = [1, 2, 3, 4, 5, 6]


def test_packet_framing_and_sign_magnitude():
    assert build_packet(1, 0x02, bytes([56, 2])) == bytes([0xFF, 0xFF, 1, 4, 2, 56, 2, (~(1 + 4 + 2 + 56 + 2)) & 0xFF])
    assert checksum(bytes([1, 2, 1])) == 0xFB
    assert encode_sign("Homing_Offset", -100) == 100 | (1 << 11) and decode_sign("Homing_Offset", 100 | (1 << 11)) == -100
    with pytest.raises(ValueError):
        encode_sign("Homing_Offset", 5000)
    port = FakeFeetechPort(IDS)
    p = FeetechProtocol(port)
    assert p.ping(3) and not p.ping(9)
    p.write(2, "Homing_Offset", -77)
    assert p.read(2, "Homing_Offset") == -77
    port.regs[4][56:58] = (1234).to_bytes(2, "little")
    assert p.sync_read("Present_Position", IDS)[4] == 1234
    with pytest.raises(FeetechError):
        p.read(9, "ID")


def test_calibration_normalised_io_and_teleoperation(tmp_path):
    lp, fp = FakeFeetechPort(IDS), FakeFeetechPort(IDS)
    leader = SOLeader(SOArmConfig(port=lp, id="l", calibration_dir=str(tmp_path)))
    follower = SOFollower(SOArmConfig(port=fp, id="f", calibration_dir=str(tmp_path), max_relative_target=None))
    ranges = {n: (1024, 3072) for n in leader.bus.motors}
    for arm in (leader, follower):
        arm.bus.connect()
        arm.calibrate(ranges)
        arm.configure()
    assert follower.calibration_path.exists() and fp._get(1, "Torque_Enable") == 1 and lp._get(1, "Torque_Enable") == 0
    a = leader.get_action()
    assert abs(a["shoulder_pan.pos"]) < 0.1 and abs(a["gripper.pos"] - 50.0) < 0.1      # mid range
    lp._set(1, "Present_Position", 3072)                  # the operator moves the leader's first joint to its limit
    lp._set(6, "Present_Position", 1024)
    obs, sent = teleoperate_step(leader, follower)
    assert abs(sent["shoulder_pan.pos"] - 100.0) < 0.1 and abs(obs["shoulder_pan.pos"] - 100.0) < 0.1
    assert fp._get(1, "Goal_Position") == 3072 and fp._get(6, "Goal_Position") == 1024
    # a reloaded arm picks the saved calibration up
    again = SOFollower(SOArmConfig(port=FakeFeetechPort(IDS), id="f", calibration_dir=str(tmp_path)))
    again.connect()
    assert again.is_calibrated and again.bus.calibration["elbow_flex"].range_max == 3072
    # the safety clamp limits the per-step move
    follower.cfg.max_relative_target = 5.0
    lp._set(1, "Present_Position", 1024)
    _, sent = teleoperate_step(leader, follower)
    assert abs(sent["shoulder_pan.pos"] - 95.0) < 0.2


def test_setup_motor_renumbers_the_single_motor_on_the_bus():
    port = FakeFeetechPort([1])
    assert setup_motor(FeetechProtocol(port), 4, scan=range(0, 8)) == 1
    assert list(port.regs) == [4] and port._get(4, "ID") == 4
    with pytest.raises(RuntimeError, match="exactly one"):
        setup_motor(FeetechProtocol(FakeFeetechPort([1, 2])), 3, scan=range(0, 8))


def test_record_episode_writes_a_lerobot_dataset(tmp_path):
    from opentau_b200.datasets.lerobot_dataset import LeRobotDataset, LeRobotDatasetMetadata
    from opentau_b200.scripts.so101.record import features, record_episode
    leader = SOLeader(SOArmConfig(port=FakeFeetechPort(IDS), id="l", calibration_dir=str(tmp_path / "c")))
    follower = SOFollower(SOArmConfig(port=FakeFeetechPort(IDS), id="f", calibration_dir=str(tmp_path / "c")))
    for arm in (leader, follower):
        arm.bus.connect()
        arm.calibrate({n: (0, 4095) for n in arm.bus.motors})
        arm.configure()
    rec = LeRobotDataset.create("local/so101", 50, root=tmp_path / "ds", robot_type="so101", features=features({}))
    assert record_episode(rec, leader, follower, "wave", seconds=0.1, fps=50) == 5
    meta = LeRobotDatasetMetadata("local/so101", root=tmp_path / "ds")
    assert meta.total_frames == 5 and meta.robot_type == "so101" and meta.tasks == {0: "wave"}
    assert np.allclose(meta.stats["action"]["mean"][:5], 0.0, atol=0.1)


def test_bimanual_pair_prefixes_keys_and_keeps_one_calibration_per_side(tmp_path):
    from opentau_b200.scripts.so101.devices import BiSOArmConfig, BiSOFollower, BiSOLeader
    ports = {k: FakeFeetechPort(IDS) for k in ("ll", "lr", "fl", "fr")}
    leader = BiSOLeader(BiSOArmConfig(SOArmConfig(port=ports["ll"]), SOArmConfig(port=ports["lr"]), id="lead",
                                      calibration_dir=str(tmp_path)))
    follower = BiSOFollower(BiSOArmConfig(SOArmConfig(port=ports["fl"]), SOArmConfig(port=ports["fr"]), id="follow",
                                          calibration_dir=str(tmp_path)))
    ranges = {n: (1024, 3072) for n in leader.left_arm.bus.motors}
    for pair in (leader, follower):
        for _, arm in pair.arms:
            arm.bus.connect()
        pair.calibrate({"left": ranges, "right": ranges})
        pair.configure()
    assert follower.is_calibrated and follower.left_arm.calibration_path.name == "follow_left.json"
    assert follower.right_arm.calibration_path.exists() and leader.right_arm.calibration_path.name == "lead_right.json"
    ports["ll"]._set(1, "Present_Position", 3072)          # only the LEFT leader moves
    obs, sent = teleoperate_step(leader, follower)
    assert set(sent) == {f"{s}_{n}.pos" for s in ("left", "right") for n in ranges}
    assert abs(sent["left_shoulder_pan.pos"] - 100.0) < 0.1 and abs(sent["right_shoulder_pan.pos"]) < 0.1
    assert ports["fl"]._get(1, "Goal_Position") == 3072 and ports["fr"]._get(1, "Goal_Position") == 2048
    assert abs(obs["left_shoulder_pan.pos"] - 100.0) < 0.1 and "right_gripper.pos" in obs


def test_stable_device_aliases(tmp_path):
    from opentau_b200.scripts.so101.device_paths import stable_link_map, stable_serial_path, stable_video_path
    dev = tmp_path / "dev"
    by_id = dev / "serial" / "by-id"
    by_path = dev / "v4l" / "by-path"
    by_id.mkdir(parents=True)
    by_path.mkdir(parents=True)
    (dev / "ttyACM0").write_text("")
    (dev / "video0").write_text("")
    (by_id / "usb-1a86_USB_Single_Serial_5A46-if00").symlink_to(dev / "ttyACM0")
    (by_path / "pci-0000:00:14.0-usb-0:2:1.0-video-index0").symlink_to(dev / "video0")
    (by_path / "pci-0000:00:14.0-usbv2-0:2:1.0-video-index0").symlink_to(dev / "video0")
    assert stable_serial_path(str(dev / "ttyACM0"), by_id).endswith("usb-1a86_USB_Single_Serial_5A46-if00")
    # two aliases of one node: the first in sorted order, every time
    assert stable_video_path(str(dev / "video0"), by_path).endswith("-usb-0:2:1.0-video-index0")
    assert len(stable_link_map(by_path)) == 1
    assert stable_video_path(0, by_path) is None and stable_serial_path(str(dev / "ttyACM9"), by_id) is None
    assert stable_link_map(tmp_path / "missing") == {}


def test_record_session_rerecord_stop_and_resume(tmp_path):
    from opentau_b200.datasets.lerobot_dataset import LeRobotDataset, LeRobotDatasetMetadata
    from opentau_b200.scripts.so101.record import (features, new_events, open_dataset_for_append, record_episode,
                                                   record_session)
    leader = SOLeader(SOArmConfig(port=FakeFeetechPort(IDS), id="l", calibration_dir=str(tmp_path / "c")))
    follower = SOFollower(SOArmConfig(port=FakeFeetechPort(IDS), id="f", calibration_dir=str(tmp_path / "c")))
    for arm in (leader, follower):
        arm.bus.connect()
        arm.calibrate({n: (0, 4095) for n in arm.bus.motors})
        arm.configure()
    rec = LeRobotDataset.create("local/so101", 50, root=tmp_path / "ds", robot_type="so101", features=features({}))
    events, said = new_events(), []

    class Script(dict):
        """Plays the operator: throws the first take away, ends the second early, asks to stop during the third."""
        takes = 0

    def say(msg):
        said.append(msg)
        if msg.startswith("recording episode"):
            Script.takes += 1
            if Script.takes == 1:
                events["rerecord_episode"] = True
            if Script.takes == 3:
                events["stop_recording"] = True
    saved = record_session(rec, leader, follower, "wave", num_episodes=5, episode_time_s=0.06, reset_time_s=0.02, fps=50,
                           events=events, say=say)
    assert saved == 2 and Script.takes == 3 and "re-recording the episode" in said and "reset the environment" in said
    meta = LeRobotDatasetMetadata("local/so101", root=tmp_path / "ds")
    assert meta.total_episodes == 2 and meta.total_frames == 6
    # an early exit keeps what was recorded so far
    ev = new_events()
    ev["exit_early"] = True
    assert record_episode(rec, leader, follower, "wave", 1.0, 50, ev, save=False) == 0 and ev["exit_early"] is False
    rec.clear_episode_buffer()
    # a resumed session only adds what is missing, and continues the numbering
    again = open_dataset_for_append("local/so101", tmp_path / "ds")
    assert record_session(again, leader, follower, "wave", 3, 0.04, 0.0, 50, new_events(), say=lambda m: None) == 1
    assert record_session(again, leader, follower, "wave", 3, 0.04, 0.0, 50, new_events(), say=said.append) == 0
    assert "nothing to record" in said[-1]
    meta = LeRobotDatasetMetadata("local/so101", root=tmp_path / "ds")
    assert meta.total_episodes == 3 and sorted(meta.episodes) == [0, 1, 2]
