"""``opentau-so101-calibrate --role follower|leader --port /dev/ttyACM0 --id my_arm``"""

import argparse

from .devices import SOArmConfig, SOFollower, SOLeader


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--role", choices=["follower", "leader"], required=True)
    ap.add_argument("--port", required=True)
    ap.add_argument("--id", default="so101")
    a = ap.parse_args(argv)
    arm = (SOFollower if a.role == "follower" else SOLeader)(SOArmConfig(port=a.port, id=a.id))
    arm.bus.connect()
    input("Move the arm to the middle of its range of motion and press Enter...")
    cal = arm.calibrate()
    print(f"calibration saved to {arm.calibration_path}")
    arm.disconnect()
    return cal


if __name__ == "__main__":
    main()
